// tcgen05 weight-only GEMM: out[tok, n] = sum_k x[tok, k] * dequant(W)[n, k].
//
// The 128 weight rows of a CTA's strip are the MMA's M dimension and the tokens its N
// dimension ("swap-AB"), so one kernel serves decode (16..64 tokens) and prefill (256-token
// tiles).  Warp roles, one CTA of 11 to 19 warps per output tile:
//   warp 0     TMA producer of raw quantised weight tiles (runs up to RS stages ahead: this
//              is the HBM stream)
//   warp 1     tensor-memory owner and the single thread that issues tcgen05.mma
//   warp 2     TMA producer of activation tiles [TOK x 64] (128-byte swizzle)
//   the rest   transform (two groups of four warps, four groups for the 256-token tile; decode tiles
//              have a second MMA issuer in front of them): raw int4 / fp8 -> 16-bit values written straight into the
//              128-byte-swizzled K-major operand layout the MMA reads; afterwards the same
//              warps drain the fp32 accumulator from tensor memory, apply per-row scales and
//              store out[tok, n].
// Every mbarrier wait is bounded; on expiry the CTA records a code in a status word, releases
// its tensor memory and returns.
//
// Reference counterparts: GEMM_int4_pgrp_kernel (csrc/xpu/esimd_kernels/int4_GEMM.h:81-270),
// FP8_GEMM_DPAS_V9 (fp8_GEMM_pert.h:2940-3150), moe_prefill_up/down_forward_kernel
// (csrc/moe_prefill/moe_prefill_int4.sycl:121-395), moe_gemm_block_prefill_kernel
// (fp8_moe_gemm_blockscale.h:187-302).
#include <atomic>
#include "umma_gemm.cuh"
#include "sm100.cuh"
#include "smallm.cuh"   // nib2_to_act / fp8x2_to_act / lds128
#include "peer_reduce.cuh"

namespace b2q {

using namespace sm100;

__device__ int g_umma_status = 0;
constexpr int SK_BANKS = 64, SK_MAX_STRIPS = 1024;
__device__ int g_sk_counters[SK_BANKS * SK_MAX_STRIPS];     // arrival counters of cut strips (see "balanced mode" below)

enum { WK_W4N = 0, WK_W4K = 1, WK_W8 = 2 };
enum { ST_XFULL = 101, ST_AFULL = 102, ST_EMPTY = 103, ST_RAWFULL = 104, ST_RAWEMPTY = 105, ST_ACCUM = 106, ST_ACCEMPTY = 107, ST_FIXUP = 108, ST_SCALERANGE = 109 };

// One piece of a CTA's work: 64-k chunks [c_begin, c_begin + nk) of the strip of 128 weight rows at n0.
// part = the strip's other chunks belong to other CTAs; slot = which of the CTA's two partial-sum slots it uses.
struct Segment { int n0, c_begin, nk, strip, part, slot; };

// constants of the fp16 magic-number nibble decode, handed to the kernel as parameters (see w4_word_magic)
struct MagicConsts { uint32_t magic_lo, magic_hi, m72; };
// twos: the nibbles are two's complement (value, not value + 8).  Flipping their sign bits gives the offset form; the
// flip is folded into the constant that is merged in: (w & m) ^ (0x6400 ^ flip) is 0x6400 | ((w ^ flip) & m) because
// the 0x6400 bits and the nibble bits do not overlap.  No extra operation, no branch in the decode.
__host__ __device__ inline MagicConsts magic_consts(bool twos) {
  return MagicConsts{0x64006400u ^ (twos ? 0x00080008u : 0u), 0x64006400u ^ (twos ? 0x00800080u : 0u), 0xD480D480u};
}

struct UmmaWoParams {
  const void* scale; int scale_dtype; int scale_mode;      // scale_mode: B2Q_SCALE_* (fp8) ; ignored for int4
  int64_t s_stride_n, s_stride_g, s_expert_elems;
  void* out; int64_t ldo;
  int M, N, K;
  int marlin; uint32_t xor_mask; int e5m2;
  int sk_sps, sk_units;      // balanced mode: raw stages per strip and in total (0 = one CTA per token tile and strip)
  float* sk_partials;        // balanced mode: [2 * grid][TOK][128] fp32 partial sums of cut strips
  int* sk_counters;          // balanced mode: arrivals per strip, zero between launches
  int sk_grid;               // host side only: CTAs of a balanced launch
  int tiles_on_y;            // grouped launches: tile index on blockIdx.y, strip on blockIdx.x (see the kernel)
  int magic;                 // INT4: fp16 magic-number transform; x was permuted / scaled by the pre-pass
  const int32_t* tiles; const int32_t* expert_offsets; const int32_t* out_map;
  int w_rows_per_expert;     // tensor-map rows per expert: N (N-major) or K/8 (K-major)
  const float* tok_scale;    // optional per-token output multiplier (undoes the activation pre-scale)
  int out_bf16;              // output element type (may differ from the MMA input type)
  int overlap_ok;            // host side only: launch with programmatic stream serialization
  int* status;
  MagicConsts mk;            // constants of the fp16 magic-number nibble decode (see w4_word_magic)
  int peer_on;               // decode tiles only: the output tile goes to the owner ranks' reduction slots (peer memory)
  PeerEpilogue peer;
};

template <bool BF16> __device__ __forceinline__ uint32_t pack2f(float a, float b) {
  uint32_t r;
  if constexpr (BF16) asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
  else asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
  return r;
}
template <bool BF16> __device__ __forceinline__ uint32_t mul2(uint32_t a, uint32_t b) {
  if constexpr (BF16) {
    __nv_bfloat162 r = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
  } else {
    __half2 r = __hmul2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
  }
}
__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}

// One int32 of eight nibbles -> eight 16-bit values (q - 8) * s in k order (one 16-byte chunk).
// FAST: the scale has the activation dtype, so a packed 16-bit multiply rounds exactly like
// ((q - 8).float() * s.float()).to(dtype).  Otherwise the product is formed in fp32.
template <bool BF16, bool FAST>
__device__ __forceinline__ void w4_word(uint32_t w, uint32_t s2, float sf, bool marlin, uint32_t (&o)[4]) {
  if constexpr (FAST) {
    uint32_t p0 = mul2<BF16>(nib2_to_act<BF16>(w), s2);
    uint32_t p1 = mul2<BF16>(nib2_to_act<BF16>(w >> 4), s2);
    uint32_t p2 = mul2<BF16>(nib2_to_act<BF16>(w >> 8), s2);
    uint32_t p3 = mul2<BF16>(nib2_to_act<BF16>(w >> 12), s2);
    if (marlin) { const uint32_t t = p1; p1 = p2; p2 = t; }
    const uint32_t q0 = __byte_perm(p0, p1, 0x5410), q1 = __byte_perm(p0, p1, 0x7632);
    const uint32_t q2 = __byte_perm(p2, p3, 0x5410), q3 = __byte_perm(p2, p3, 0x7632);
    o[0] = q0; o[1] = marlin ? q1 : q2; o[2] = marlin ? q2 : q1; o[3] = q3;
  } else {
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int slot = marlin ? ((j & 3) * 2 + (j >> 2)) : j;
      v[j] = (float)((int)((w >> (4 * slot)) & 0xFu) - 8) * sf;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) o[j] = pack2f<BF16>(v[2 * j], v[2 * j + 1]);
  }
}

// fp16 magic-number variant: 0x6400 | q is 1024 + q and 0x6400 | (q << 4) is 1024 + 16 q, so the nibbles at
// bits 0-3 / 4-7 of each half-word need no shift; one shift by 8 reaches the other four.  The result
// (q - 8) * s is rounded to fp16 once.  Output pair order: (n0,n4) (n1,n5) (n2,n6) (n3,n7) where n_i is the
// nibble at bits 4i; the activation pre-pass stores x in the matching order.  Integer work per word: one
// shift and four LOP3 (the ALU pipe, not the FP pipes, is what bounds the int4 transform).
// Where the constants live matters more than the arithmetic.  All of them as literals: the compiler folds them into
// immediates, and since an instruction takes one immediate at most it then spends two logic operations per
// mask-and-merge and a register move per fused multiply-add (measured: 82 logic operations and 61 moves per 64 k of a
// row where 32 and a handful are needed).  All of them as kernel parameters: seven registers held through a loop that
// has none to spare.  Hence one of each instruction's two constants as an immediate, the other in a register
// (and_xor_lo / and_xor_hi / w4_word_magic below).

// a, b, c or d for i = 0, 1, 2, anything else: three compares and three selects, never a branch (written as a
// conditional expression the selection of a chunk's prefetched scale became a jump table with a dozen register moves)
__device__ __forceinline__ uint32_t sel4(int i, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  uint32_t r;
  asm("{\n\t.reg .pred p0, p1, p2;\n\tsetp.eq.s32 p0, %1, 0;\n\tsetp.eq.s32 p1, %1, 1;\n\tsetp.eq.s32 p2, %1, 2;\n\t"
      "selp.u32 %0, %4, %5, p2;\n\tselp.u32 %0, %3, %0, p1;\n\tselp.u32 %0, %2, %0, p0;\n\t}"
      : "=&r"(r) : "r"(i), "r"(a), "r"(b), "r"(c), "r"(d));
  return r;
}
__device__ __forceinline__ uint32_t and_xor_lo(uint32_t a, uint32_t c) {      // (a & 0x000F000F) ^ c: the mask as an immediate, c in a register
  uint32_t d;
  asm("lop3.b32 %0, %1, 0x000F000F, %2, 0x6A;" : "=r"(d) : "r"(a), "r"(c));
  return d;
}
__device__ __forceinline__ uint32_t and_xor_hi(uint32_t a, uint32_t c) {      // (a & 0x00F000F0) ^ c
  uint32_t d;
  asm("lop3.b32 %0, %1, 0x00F000F0, %2, 0x6A;" : "=r"(d) : "r"(a), "r"(c));
  return d;
}
// An instruction takes ONE immediate: the masks, 1032 and 1/16 are written as literals, the merge constants (which depend
// on the nibble encoding) and -72 come in registers.  Three registers of constants instead of seven.
__device__ __forceinline__ void w4_word_magic(uint32_t w, uint32_t s2, const MagicConsts& k, uint32_t (&o)[4]) {
  const uint32_t w8 = w >> 8;
  uint32_t v[4] = {and_xor_lo(w, k.magic_lo), and_xor_hi(w, k.magic_hi), and_xor_lo(w8, k.magic_lo), and_xor_hi(w8, k.magic_hi)};
  const __half2 sc = *reinterpret_cast<const __half2*>(&s2);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __half2 h = *reinterpret_cast<__half2*>(&v[i]);
    const uint32_t c_r16 = 0x2C002C00u, c_1032 = 0x64086408u;
    if (i & 1) h = __hfma2(h, *reinterpret_cast<const __half2*>(&c_r16), *reinterpret_cast<const __half2*>(&k.m72));      // h / 16 - 72
    else h = __hsub2(h, *reinterpret_cast<const __half2*>(&c_1032));                                                     // h - 1032
    h = __hmul2(h, sc);
    o[i] = *reinterpret_cast<uint32_t*>(&h);
  }
}

// Four fp8 bytes -> four 16-bit values in k order.  SCALED folds an fp32 scale in (one rounding);
// otherwise bf16 results carry an exact 2^-112 that the epilogue removes.
template <bool BF16, bool SCALED>
__device__ __forceinline__ void w8_word(uint32_t w, bool e5m2, float sf, uint32_t& o0, uint32_t& o1) {
  if constexpr (!SCALED) {
    if (e5m2) { o0 = fp8x2_to_act<BF16, true>(w); o1 = fp8x2_to_act<BF16, true>(w >> 16); }
    else { o0 = fp8x2_to_act<BF16, false>(w); o1 = fp8x2_to_act<BF16, false>(w >> 16); }
  } else {
    uint32_t h0, h1;
    if (e5m2) { h0 = fp8x2_to_act<false, true>(w); h1 = fp8x2_to_act<false, true>(w >> 16); }
    else { h0 = fp8x2_to_act<false, false>(w); h1 = fp8x2_to_act<false, false>(w >> 16); }
    const float2 f0 = __half22float2(*reinterpret_cast<__half2*>(&h0));
    const float2 f1 = __half22float2(*reinterpret_cast<__half2*>(&h1));
    o0 = pack2f<BF16>(f0.x * sf, f0.y * sf);
    o1 = pack2f<BF16>(f1.x * sf, f1.y * sf);
  }
}

template <int TOK> struct UmmaCfg {
  // The dequantised weight operand lives in tensor memory, not shared memory: a 64-k chunk of 128
  // rows is 128 lanes x 32 columns, written by the transform warps with tcgen05.st and read by the
  // MMA as its A operand.  Shared memory then carries only the raw quantised stream (written by TMA,
  // read once by the transform) and the activation tiles, i.e. about twice the HBM traffic instead
  // of six (fp8) to ten (int4) times, which is what capped the shared-memory variant near 3 TB/s.
  // transform groups of 4 warps.  The 256-token tile runs one CTA per SM: four groups give it the sixteen converting
  // warps the narrower tiles get from two CTAs (prefill layer -3.4 %, FP8 block GEMM -2.7 %).
  static constexpr int NG = TOK == 256 ? 4 : 2;
  static constexpr int CTAS = TOK <= 128 ? 2 : 1;                    // two CTAs per SM except for the 256-token prefill tile: a second CTA hides fill and epilogue of short K loops (MoE) and doubles the issuers for decode
  // activation stages (64 k each).  Up to 128 tokens there are as many as operand stages, and one barrier per stage
  // releases both (see SHARED_EMPTY in the kernel): one tcgen05.commit less per chunk for the issuing thread.
  static constexpr int XS = TOK <= 128 ? 4 : 5;
  // Issuing tcgen05.mma is a serial job of one thread and costs it several hundred cycles per 64-k
  // chunk regardless of the tile width; decode tiles therefore use two issuer warps on alternate
  // chunks, each with its own accumulator (summed in the epilogue).
  static constexpr int NMMA = TOK <= 64 ? 2 : 1;
  static constexpr int CW = 2 + NMMA;                                // control warps: raw TMA, X TMA, MMA issuer(s)
  static constexpr int THREADS = CW * 32 + NG * 128;                 // + transform / epilogue warps
  static constexpr int X_BYTES = TOK * 128;
  static constexpr int RAW_BYTES = 16384;
  static constexpr int SMEM_BUDGET = CTAS == 2 ? 114688 : 230400;    // per CTA, leaving room for the driver's reserve
  static constexpr int RS_FIT = (SMEM_BUDGET - 1536 - XS * X_BYTES) / RAW_BYTES;
  static constexpr int RS = RS_FIT > 8 ? 8 : RS_FIT;                 // raw weight stages (16 KB each)
  static constexpr int SMEM = XS * X_BYTES + RS * RAW_BYTES + 1024 /*align*/ + 512 /*barriers*/;
  static constexpr int ACC_COLS = TOK < 32 ? 32 : TOK;               // fp32 accumulator columns
  static constexpr int A_COL0 = NMMA * ACC_COLS;                     // first operand column
  static constexpr int TMEM_COLS = CTAS == 2 ? 256 : 512;            // the SM's 512 columns split over resident CTAs
  // Operand stages (32 columns each) fill the rest of the allocation: a stage is only reusable once
  // the MMAs that read it have completed and signalled, a round trip of a couple of microseconds, so
  // the ring has to be deep for the transform warps to stay busy.
  static constexpr int S = (TMEM_COLS - A_COL0) / 32 > 12 ? 12 : (TMEM_COLS - A_COL0) / 32;
};

// MAGIC: INT4 weights behind the activation pre-pass (fp16 activations in the nibble decode's pair order): its own
// instantiation so that the decode loop carries none of the other routes' code or registers.
template <int WK, bool BF16, int TOK, bool FAST, bool MAGIC>
__global__ void __launch_bounds__(UmmaCfg<TOK>::THREADS, UmmaCfg<TOK>::CTAS)
umma_wo_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x, const UmmaWoParams p) {
  using Cfg = UmmaCfg<TOK>;
  constexpr int S = Cfg::S, RS = Cfg::RS, NG = Cfg::NG, XS = Cfg::XS;
  constexpr int CPR = (WK == WK_W8) ? 2 : 4;          // 64-k chunks per raw stage
  constexpr int GPR = CPR < NG ? CPR : NG;            // transform groups that touch one raw stage
  // With equally deep rings chunk g uses operand stage g % S and activation stage g % XS = the same index, and the MMAs
  // that free one free the other: the activation producer waits on the operand stage's barrier, the issuer commits once
  // (MoE pipeline 676 -> 664 us; the decode tiles are indifferent).
  constexpr bool SHARED_EMPTY = S == XS;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t x_smem = base;
  const uint32_t raw_smem = x_smem + XS * Cfg::X_BYTES;
  const uint32_t bar = raw_smem + RS * Cfg::RAW_BYTES;
  // barrier map (8 bytes each)
  const uint32_t x_full = bar, x_empty = x_full + 8 * XS, a_full = x_empty + 8 * XS, ab_empty = a_full + 8 * S;
  const uint32_t raw_full = ab_empty + 8 * S, raw_empty = raw_full + 8 * RS, accum_full = raw_empty + 8 * RS;
  const uint32_t accum_empty = accum_full + 8, fix_bar = accum_full + 16;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen + (accum_full + 24 - base));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + (accum_full + 32 - base));
  volatile int* last_flag = reinterpret_cast<volatile int*>(gen + (accum_full + 36 - base));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // ---- which work ----
  // Dense launches let the next kernel of the stream begin at once and themselves wait for the kernels
  // before them only where they first touch activations (the X producer below): the weight stream, the
  // conversion into tensor memory and all set-up overlap the tail of whatever ran before.
  // Grouped launches read a tile list the previous kernel built, so they wait here.
  grid_dep_release();
  // Grid axes: dense launches put the token tile on x (neighbouring CTAs share a weight strip), grouped launches
  // the strip (neighbouring CTAs share an expert's activation tile, whose rows would otherwise be re-read from
  // DRAM once per strip: the gathered activations of a MoE layer do not fit in L2 next to the weights).
  const int tile_idx = p.tiles_on_y ? blockIdx.y : blockIdx.x, strip_idx = p.tiles_on_y ? blockIdx.x : blockIdx.y;
  int tok0 = tile_idx * TOK, xrow0 = 0, M = p.M, expert = 0;
  if (p.tiles) {
    grid_dep_wait();
    if (tile_idx >= p.tiles[0]) return;
    const int2 td = reinterpret_cast<const int2*>(p.tiles + 4)[tile_idx];
    expert = td.x; tok0 = td.y;
    xrow0 = p.expert_offsets[expert];
    M = p.expert_offsets[expert + 1] - xrow0;
  }
  // A CTA works through a list of segments = (strip of 128 weight rows, range of 64-k chunks).  Normally that
  // is one whole strip, blockIdx.y.  Balanced mode (decode shapes, one token tile): the launch is a 1-D grid
  // that fills the machine exactly, the work is cut into units of one raw stage, and CTA b takes the units
  // [b U / G, (b + 1) U / G): up to two partial strips around any number of whole ones.  Every role below walks
  // the same list with its own copy of this cursor.
  constexpr bool BAL = TOK <= 64;               // only decode tiles carry the multi-segment / partial-sum code
  const bool balanced = BAL && p.sk_sps > 0;
  int u = 0, u0 = 0, u1 = 1;
  if (balanced) {
    tok0 = 0;
    u0 = (int)((int64_t)blockIdx.x * p.sk_units / gridDim.x);
    u1 = (int)((int64_t)(blockIdx.x + 1) * p.sk_units / gridDim.x);
    u = u0;
  }
  auto next_segment = [&](Segment& sg) -> bool {
    if (u >= u1) return false;
    if (!balanced) {
      sg.n0 = strip_idx * 128; sg.c_begin = 0; sg.nk = p.K / 64; sg.strip = strip_idx; sg.part = 0; sg.slot = 0;
      u = u1;
      return true;
    }
    const int strip = u / p.sk_sps, r0 = u - strip * p.sk_sps;
    const int take = min(p.sk_sps - r0, u1 - u);
    sg.n0 = strip * 128; sg.c_begin = r0 * CPR; sg.nk = take * CPR; sg.strip = strip;
    sg.part = take != p.sk_sps; sg.slot = (u == u0) ? 0 : 1;
    u += take;
    return true;
  };
  const int64_t sbase = (int64_t)expert * p.s_expert_elems;

  if (threadIdx.x == 0) {
    for (int i = 0; i < S; ++i) { mbar_init(a_full + 8 * i, 128); mbar_init(ab_empty + 8 * i, 1); }
    for (int i = 0; i < XS; ++i) { mbar_init(x_full + 8 * i, 1); mbar_init(x_empty + 8 * i, 1); }
    for (int i = 0; i < RS; ++i) { mbar_init(raw_full + 8 * i, 1); mbar_init(raw_empty + 8 * i, GPR * 128); }
    mbar_init(accum_full, Cfg::NMMA);
    mbar_init(accum_empty, NG * 128);
    mbar_init(fix_bar, NG * 128);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), Cfg::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  Segment sg;

  if (warp == 0) {
    // ---------------- raw weight producer ----------------
    if (lane == 0) {
      tma_prefetch_desc(&tm_w);
      int grb = 0;                       // raw stages issued so far: ring position and phase carry across segments
      int issued = 0;
      bool ok = true;
      while (ok && next_segment(sg)) {
        const int nraw = (sg.nk + CPR - 1) / CPR;
        for (int r = 0; r < nraw; ++r) {
          const int gr = grb + r, rs = gr % RS;
          { if (gr >= RS && !mbar_wait(raw_empty + 8 * rs, ((gr / RS) - 1) & 1, abort_flag, p.status, ST_RAWEMPTY)) { ok = false; break; } }
          issued = gr + 1;
          mbar_expect_tx(raw_full + 8 * rs, Cfg::RAW_BYTES);
          if constexpr (WK == WK_W4K)
            tma_load_2d(raw_smem + rs * Cfg::RAW_BYTES, &tm_w, sg.n0, expert * p.w_rows_per_expert + (sg.c_begin / CPR + r) * 32, raw_full + 8 * rs);
          else
            tma_load_2d(raw_smem + rs * Cfg::RAW_BYTES, &tm_w, (sg.c_begin / CPR + r) * 128, expert * p.w_rows_per_expert + sg.n0, raw_full + 8 * rs);
        }
        grb += nraw;
      }
      if (!ok) drain_issued(raw_full, RS, issued);
    }
  } else if (warp == 2) {
    // ---------------- activation producer ----------------
    if (lane == 0) {
      tma_prefetch_desc(&tm_x);
      if (!p.tiles) grid_dep_wait();
      int gb = 0, issued = 0;
      bool ok = true;
      while (ok && next_segment(sg)) {
        for (int c = 0; c < sg.nk; ++c) {
          const int g = gb + c, s = g % XS;
          { if (g >= XS && !mbar_wait((SHARED_EMPTY ? ab_empty : x_empty) + 8 * s, ((g / XS) - 1) & 1, abort_flag, p.status, ST_EMPTY)) { ok = false; break; } }
          issued = g + 1;
          mbar_expect_tx(x_full + 8 * s, Cfg::X_BYTES);
          tma_load_2d(x_smem + s * Cfg::X_BYTES, &tm_x, (sg.c_begin + c) * 64, xrow0 + tok0, x_full + 8 * s);
        }
        gb += sg.nk;
      }
      if (!ok) drain_issued(x_full, XS, issued);
    }
  } else if (warp == 1 || (Cfg::NMMA == 2 && warp == 3)) {
    // ---------------- MMA issuer(s) ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc(BF16 ? 1u : 0u, BF16 ? 1u : 0u, 128, TOK);
      const int me = warp == 1 ? 0 : 1;
      const uint32_t dacc = tmem + me * Cfg::ACC_COLS;
      const uint64_t db0 = smem_desc_sw128(x_smem);
      bool ok = true;
      int gb = 0, si = 0;
      while (ok && next_segment(sg)) {
        // the accumulators are reused: wait until the epilogue warps have read the previous segment's
        if (BAL && si > 0) { ok = mbar_wait(accum_empty, (si - 1) & 1, abort_flag, p.status, ST_ACCEMPTY); if (!ok) break; tc_fence_after(); }
#pragma unroll 1
        for (int c = me; c < sg.nk; c += Cfg::NMMA) {
          const int g = gb + c, s = g % S, xs = g % XS;
          { ok = mbar_wait(x_full + 8 * xs, (g / XS) & 1, abort_flag, p.status, ST_XFULL); }
          if (ok) { ok = mbar_wait(a_full + 8 * s, (g / S) & 1, abort_flag, p.status, ST_AFULL); }
          if (!ok) break;
          tc_fence_after();
          const uint32_t ta = tmem + Cfg::A_COL0 + 32 * s;
          const uint64_t db = db0 + (uint64_t)(xs * (Cfg::X_BYTES >> 4));
          mma_f16_ts(dacc, ta, db, idesc, c >= Cfg::NMMA ? 1u : 0u);
          mma_f16_ts(dacc, ta + 8, db + 2, idesc, 1u);
          mma_f16_ts(dacc, ta + 16, db + 4, idesc, 1u);
          mma_f16_ts(dacc, ta + 24, db + 6, idesc, 1u);
          tc_commit(ab_empty + 8 * s);
          if constexpr (!SHARED_EMPTY) tc_commit(x_empty + 8 * xs);
        }
        if (ok) tc_commit(accum_full);
        gb += sg.nk; ++si;
      }
    }
  } else {
    // ---------------- transform, then epilogue (the NG x 4 warps after the control warps) ----------------
    // NG groups of four warps; group g converts the 64-k chunks with c % NG == g, one weight row
    // (N-major / fp8) or column (K-major) per thread, so NG chunks are always in flight.
    const int t = (warp & 3) * 32 + lane;        // row of the strip == tensor-memory lane this thread may write
    const int grp = (threadIdx.x - Cfg::CW * 32) >> 7;
    const int sw = t & 7;
    const bool blockscale = (WK == WK_W8) && (p.scale_mode == B2Q_SCALE_BLOCK128);
    const int kblocks = (p.K + 127) >> 7;
    bool ok = true;
    int gb = 0, grb = 0, si = 0, fixn = 0;       // chunks / raw stages / segments / fix-up barrier phases so far
    while (ok && next_segment(sg)) {
    const int n0 = sg.n0, nk = sg.nk, c_begin = sg.c_begin;
    int nrow = n0 + t; if (nrow >= p.N) nrow = p.N - 1;
    // The scale of a chunk (one per weight row for INT4, one per CTA for block-scaled FP8) comes from global memory,
    // usually from DRAM (scales are read once per launch): about a thousand cycles.  Scales are requested four to
    // eight of this group's chunks ahead, four at a time, and nothing touches a requested register before its chunk
    // is converted: decoding a value to fp32 where it is loaded, or rotating a freshly requested register into the
    // next variable, makes the warp wait for the load right there, on every chunk (measured: 1800 of the 2900
    // cycles a chunk cost a transform group).  Hence two sets of four raw values: the set in use, loaded at least
    // four chunks ago, and the set in flight, which replaces it every fourth chunk.
    auto chunk_scale_raw = [&](int c) -> uint32_t {
      if (c >= nk) return 0u;
      if constexpr (WK == WK_W4N || WK == WK_W4K) {
        const int64_t i = sbase + (int64_t)nrow * p.s_stride_n + (int64_t)((c_begin + c) >> 1) * p.s_stride_g;
        if (p.scale_dtype == B2Q_F32) return __ldg(reinterpret_cast<const uint32_t*>(p.scale) + i);
        return (uint32_t)__ldg(reinterpret_cast<const unsigned short*>(p.scale) + i);
      } else {
        return blockscale ? __ldg(reinterpret_cast<const uint32_t*>(p.scale) + sbase + (int64_t)(n0 >> 7) * kblocks + ((c_begin + c) >> 1)) : 0u;
      }
    };
    auto scale_value = [&](uint32_t raw) -> float {
      if constexpr (WK == WK_W4N || WK == WK_W4K) {
        // all three readings, then two selects: no branch per chunk
        const float as_f32 = __uint_as_float(raw), as_bf16 = __uint_as_float(raw << 16);
        const float as_f16 = __half2float(__ushort_as_half((unsigned short)raw));
        return p.scale_dtype == B2Q_F32 ? as_f32 : (p.scale_dtype == B2Q_BF16 ? as_bf16 : as_f16);
      } else {
        return __uint_as_float(raw);
      }
    };
    uint32_t sq0 = chunk_scale_raw(grp), sq1 = chunk_scale_raw(grp + NG), sq2 = chunk_scale_raw(grp + 2 * NG),
             sq3 = chunk_scale_raw(grp + 3 * NG);
    uint32_t sn0 = chunk_scale_raw(grp + 4 * NG), sn1 = chunk_scale_raw(grp + 5 * NG), sn2 = chunk_scale_raw(grp + 6 * NG),
             sn3 = chunk_scale_raw(grp + 7 * NG);
    int it4 = 0;                                   // position of the current chunk in its set of four
    int pend = -1;                                 // MAGIC: operand stage whose tensor-memory stores are still in flight
    int saturated = 0;                             // MAGIC: a scale had to be clamped (reported once, behind the loop)
    // fp16 magic route with bf16 / fp32 scales: the group scale is rounded to fp16, whose normal range starts at
    // 6.1e-5.  Every row of a segment therefore carries its own power of two, taken from the scale of the segment's
    // first group: the row's scales are multiplied by 2^row_e so that this first one lands in [0.5, 1), and the fp32
    // accumulator row is multiplied by 2^-row_e when it is read ((q - 8) * s needs 11 bits at most, so the fp16
    // operand stays exact).  Groups within 2^13 of the first one, either way, are exact; one further above would
    // overflow fp16 and is saturated and reported through the status word (ST_SCALERANGE).
    float row_mul = 1.f, row_post = 1.f;
    if constexpr (MAGIC) {
      if (p.scale_dtype != B2Q_F16) {
        const int ex = (int)((__float_as_uint(scale_value(chunk_scale_raw(0))) >> 23) & 0xFFu);   // biased exponent; 0 = zero / subnormal, 255 = inf / nan
        if (ex != 0 && ex != 255) {
          int k = 126 - ex;
          k = k > 120 ? 120 : (k < -120 ? -120 : k);
          row_mul = __uint_as_float((uint32_t)(127 + k) << 23);
          row_post = __uint_as_float((uint32_t)(127 - k) << 23);
        }
      }
    }
    // Position in the raw ring: by counting (this group converts CPG chunks of every raw stage, a segment starts on a
    // stage boundary, jj counts them) or by dividing the chunk number by the stage count for every chunk.  Which is
    // faster is a matter of what the register allocator makes of the loop, measured per tile width on one GPU: the
    // 128-token grouped tiles gain 3 % from counting (MoE pipeline 693 -> 672 us), the decode tiles lose 2 %
    // (gate_up at M = 64: 133 -> 136 us).
    constexpr bool COUNTED = TOK > 64 && NG <= CPR;      // counting assumes every group has a chunk in every raw stage
    constexpr int CPG = CPR / NG > 0 ? CPR / NG : 1;
    int jj = 0, rs = grb % RS;
    uint32_t rpar = (uint32_t)(grb / RS) & 1u;
#pragma unroll 1
    for (int c = grp; c < nk; c += NG) {
      if (it4 == 4) {
        it4 = 0;
        sq0 = sn0; sq1 = sn1; sq2 = sn2; sq3 = sn3;                       // requested at least four chunks ago
        sn0 = chunk_scale_raw(c + 4 * NG); sn1 = chunk_scale_raw(c + 5 * NG);
        sn2 = chunk_scale_raw(c + 6 * NG); sn3 = chunk_scale_raw(c + 7 * NG);
      }
      const uint32_t sr_cur = sel4(it4, sq0, sq1, sq2, sq3);
      ++it4;
      int j;
      if constexpr (COUNTED) {
        j = grp + jj * NG;                           // == c % CPR
      } else {
        const int gr = grb + c / CPR;
        j = c % CPR; rs = gr % RS; rpar = (uint32_t)(gr / RS) & 1u;
      }
      ok = mbar_wait(raw_full + 8 * rs, rpar, abort_flag, p.status, ST_RAWFULL);
      if (!ok) break;
      const float sc_cur = scale_value(sr_cur);
      const uint32_t rawrow = raw_smem + rs * Cfg::RAW_BYTES + t * 128;     // N-major / fp8: this thread's row
      const uint32_t rawcol = raw_smem + rs * Cfg::RAW_BYTES + t * 4;       // K-major: this thread's column
      {
        const int g = gb + c, s = g % S;
        // no test for the ring's first round: a wait for the phase before a fresh barrier's first one returns at once
        { ok = mbar_wait(ab_empty + 8 * s, ((g / S) + 1) & 1, abort_flag, p.status, ST_EMPTY); if (!ok) break; }
        tc_fence_after();
        const uint32_t ta = tmem + ((uint32_t)((warp & 3) * 32) << 16) + Cfg::A_COL0 + 32 * s;
        if constexpr (MAGIC) {
          // fp16 magic-number route.  The chunk goes to tensor memory in two halves of 32 k (16 registers each): with
          // all 64 values of a row live at once the loop ran out of registers, and the decode's masks and fp16
          // constants were re-created for every use.
          float ss = sc_cur * row_mul;
          const bool too_big = fabsf(ss) > 8188.f;            // 8 * scale would leave fp16: saturate, and say so (after the loop)
          ss = too_big ? copysignf(8188.f, ss) : ss;
          saturated |= too_big ? 1 : 0;
          const uint32_t hv = __half_as_ushort(__float2half_rn(ss));
          const uint32_t m2 = hv | (hv << 16);
          const MagicConsts mk = p.mk;
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
            uint32_t w0, w1, w2, w3;
            if constexpr (WK == WK_W4N) {
              const uint4 rr = lds128(rawrow + (((2 * j + hf) ^ sw) << 4));
              w0 = rr.x; w1 = rr.y; w2 = rr.z; w3 = rr.w;
            } else {
              w0 = lds32(rawcol + (8 * j + 4 * hf + 0) * 512); w1 = lds32(rawcol + (8 * j + 4 * hf + 1) * 512);
              w2 = lds32(rawcol + (8 * j + 4 * hf + 2) * 512); w3 = lds32(rawcol + (8 * j + 4 * hf + 3) * 512);
            }
            uint32_t a16[16];
            { uint32_t o[4]; w4_word_magic(w0, m2, mk, o); a16[0] = o[0]; a16[1] = o[1]; a16[2] = o[2]; a16[3] = o[3]; }
            { uint32_t o[4]; w4_word_magic(w1, m2, mk, o); a16[4] = o[0]; a16[5] = o[1]; a16[6] = o[2]; a16[7] = o[3]; }
            { uint32_t o[4]; w4_word_magic(w2, m2, mk, o); a16[8] = o[0]; a16[9] = o[1]; a16[10] = o[2]; a16[11] = o[3]; }
            { uint32_t o[4]; w4_word_magic(w3, m2, mk, o); a16[12] = o[0]; a16[13] = o[1]; a16[14] = o[2]; a16[15] = o[3]; }
            // The previous chunk's stores have had this half's conversion to complete: only now are they waited for and
            // the chunk handed to the MMA warp.  Waiting right behind the store would leave the warp idle for the
            // store's whole latency, once per chunk.
            if (hf == 0 && pend >= 0) { tmem_st_wait(); tc_fence_before(); mbar_arrive(a_full + 8 * pend); }
            tmem_st16(ta + 16 * hf, a16);
          }
          pend = s;
        } else {
        uint32_t av[32];                         // this row's 64 values of the chunk, two per register, k ascending
        if constexpr (WK == WK_W4N || WK == WK_W4K) {
          uint32_t s2 = 0; float sf = 0.f;
          if constexpr (FAST) {
            // the scale has the activation's 16-bit type here, so float -> 16 bit gives back its stored bits
            if (!p.magic) { const uint32_t sv = BF16 ? __bfloat16_as_ushort(__float2bfloat16_rn(sc_cur)) : __half_as_ushort(__float2half_rn(sc_cur)); s2 = sv | (sv << 16); }
          } else sf = sc_cur;
          uint32_t ww[8];
          bool marlin = false;
          if constexpr (WK == WK_W4N) {
            const uint4 r0 = lds128(rawrow + (((2 * j) ^ sw) << 4));
            const uint4 r1 = lds128(rawrow + (((2 * j + 1) ^ sw) << 4));
            ww[0] = r0.x ^ p.xor_mask; ww[1] = r0.y ^ p.xor_mask; ww[2] = r0.z ^ p.xor_mask; ww[3] = r0.w ^ p.xor_mask;
            ww[4] = r1.x ^ p.xor_mask; ww[5] = r1.y ^ p.xor_mask; ww[6] = r1.z ^ p.xor_mask; ww[7] = r1.w ^ p.xor_mask;
          } else {
            marlin = p.marlin != 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) ww[i] = lds32(rawcol + (8 * j + i) * 512);
          }
          {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              uint32_t o[4];
              w4_word<BF16, FAST>(ww[i], s2, sf, marlin, o);
              av[4 * i] = o[0]; av[4 * i + 1] = o[1]; av[4 * i + 2] = o[2]; av[4 * i + 3] = o[3];
            }
          }
        } else {
          uint4 rv[4];
#pragma unroll
          for (int c4 = 0; c4 < 4; ++c4) rv[c4] = lds128(rawrow + (((4 * j + c4) ^ sw) << 4));
          uint32_t (&o)[32] = av;
          if (blockscale) {
            const float sf = sc_cur;
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) {
              w8_word<BF16, true>(rv[c4].x, p.e5m2, sf, o[8 * c4 + 0], o[8 * c4 + 1]);
              w8_word<BF16, true>(rv[c4].y, p.e5m2, sf, o[8 * c4 + 2], o[8 * c4 + 3]);
              w8_word<BF16, true>(rv[c4].z, p.e5m2, sf, o[8 * c4 + 4], o[8 * c4 + 5]);
              w8_word<BF16, true>(rv[c4].w, p.e5m2, sf, o[8 * c4 + 6], o[8 * c4 + 7]);
            }
          } else if (p.e5m2) {
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) {
              o[8 * c4 + 0] = fp8x2_to_act<BF16, true>(rv[c4].x); o[8 * c4 + 1] = fp8x2_to_act<BF16, true>(rv[c4].x >> 16);
              o[8 * c4 + 2] = fp8x2_to_act<BF16, true>(rv[c4].y); o[8 * c4 + 3] = fp8x2_to_act<BF16, true>(rv[c4].y >> 16);
              o[8 * c4 + 4] = fp8x2_to_act<BF16, true>(rv[c4].z); o[8 * c4 + 5] = fp8x2_to_act<BF16, true>(rv[c4].z >> 16);
              o[8 * c4 + 6] = fp8x2_to_act<BF16, true>(rv[c4].w); o[8 * c4 + 7] = fp8x2_to_act<BF16, true>(rv[c4].w >> 16);
            }
          } else {
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) {
              o[8 * c4 + 0] = fp8x2_to_act<BF16, false>(rv[c4].x); o[8 * c4 + 1] = fp8x2_to_act<BF16, false>(rv[c4].x >> 16);
              o[8 * c4 + 2] = fp8x2_to_act<BF16, false>(rv[c4].y); o[8 * c4 + 3] = fp8x2_to_act<BF16, false>(rv[c4].y >> 16);
              o[8 * c4 + 4] = fp8x2_to_act<BF16, false>(rv[c4].z); o[8 * c4 + 5] = fp8x2_to_act<BF16, false>(rv[c4].z >> 16);
              o[8 * c4 + 6] = fp8x2_to_act<BF16, false>(rv[c4].w); o[8 * c4 + 7] = fp8x2_to_act<BF16, false>(rv[c4].w >> 16);
            }
          }
        }
        tmem_st32(ta, av);
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(a_full + 8 * s);
        }
      }
      // release the raw stage once this group's last chunk in it is converted
      if constexpr (COUNTED) {
        const bool stage_done = jj == CPG - 1;
        if (stage_done || c + NG >= nk) mbar_arrive(raw_empty + 8 * rs);
        if (stage_done) {
          jj = 0;
          if (++rs == RS) { rs = 0; rpar ^= 1u; }
        } else {
          ++jj;
        }
      } else {
        if (c + NG >= nk || (c + NG) / CPR != c / CPR) mbar_arrive(raw_empty + 8 * rs);
      }
    }
    if (pend >= 0) { tmem_st_wait(); tc_fence_before(); mbar_arrive(a_full + 8 * pend); pend = -1; }
    if (saturated) atomicCAS(p.status, 0, ST_SCALERANGE);
    if (!ok) break;

    // ---------------- epilogue of this segment ----------------
    { ok = mbar_wait(accum_full, si & 1, abort_flag, p.status, ST_ACCUM); }
    if (!ok) break;
    tc_fence_after();
    const int quad = warp & 3;                   // tensor-memory lane quadrant this warp may read
    const int cgrp = (warp - Cfg::CW) >> 2;      // the NG warps of a quadrant take column blocks in turn
    const int n = n0 + quad * 32 + lane;
    float post = 1.f;
    if constexpr (WK == WK_W8) {
      if (p.scale_mode != B2Q_SCALE_BLOCK128) {
        post = (BF16 ? 5192296858534827628530496329220096.0f : 1.0f);   // 2^112 undoes the bf16 bit trick
        const int nn = n < p.N ? n : p.N - 1;
        post *= load_scalar(p.scale, sbase + (p.scale_mode == B2Q_SCALE_CHANNEL ? nn : 0), p.scale_dtype);
      }
    }
    uint16_t* outp = reinterpret_cast<uint16_t*>(p.out);
    constexpr int CB = TOK >= 32 ? 32 : 16;
    // Row-parallel layer of a tensor-parallel stack: this strip of 128 output columns belongs to one owner rank and
    // one 128-column block of that rank's slice; the tile is stored into this rank's slot of the owner's buffer
    // ([block][row][128 columns]) with plain peer stores, and the owner is told through flag1 when the strip is done.
    uint16_t* peer_dst = nullptr;
    uint32_t* peer_flag = nullptr;
    if constexpr (BAL) {
      if (p.peer_on) {
        const int owner = n0 / p.peer.slice, blk = (n0 - owner * p.peer.slice) >> 7;
        uint8_t* ob = p.peer.bufs[owner];
        peer_dst = reinterpret_cast<uint16_t*>(ob + p.peer.slot_off + (size_t)p.peer.rank * p.peer.slot_bytes +
                                               (size_t)blk * p.peer.M * (PR_CB * 2)) + quad * 32 + lane;
        peer_flag = &reinterpret_cast<PeerCtrl*>(ob)->flag1[p.peer.rank][blk];
      }
    }
    auto write_out = [&](const uint32_t (&r)[32], int cb) {
      // per-token scales of this column block: one load per lane, read past L1 (it may still hold the previous
      // call's scales at this address), handed round the warp by shuffle
      float ts_lane = 1.f;
      if (p.tok_scale && lane < CB && tok0 + cb + lane < M) ts_lane = __ldcg(p.tok_scale + xrow0 + tok0 + cb + lane);
#pragma unroll
      for (int i = 0; i < CB; ++i) {
        const float ts = __shfl_sync(0xffffffffu, ts_lane, i);
        const int tok = tok0 + cb + i;
        if (tok < M && n < p.N) {
          int64_t orow = xrow0 + tok;
          if (p.out_map) orow = p.out_map[orow];
          const float v = __uint_as_float(r[i]) * post * ts;
          uint16_t* dst = outp + orow * p.ldo + n;
          if constexpr (BAL) { if (peer_dst) dst = peer_dst + (size_t)tok * PR_CB; }
          *dst = p.out_bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(v)) : __half_as_ushort(__float2half_rn(v));
        }
      }
    };
    // partial sums of a cut strip: [CTA][slot][token][row of the strip] fp32, raw accumulator values
    float* const my_part = balanced ? p.sk_partials + ((size_t)(blockIdx.x * 2 + sg.slot) * TOK) * 128 + quad * 32 + lane : nullptr;
    bool freed = false;
#pragma unroll 1
    for (int cb = cgrp * CB; cb < TOK; cb += NG * CB) {
      if (tok0 + cb >= M) break;
      uint32_t r[32];
      if constexpr (CB == 32) tmem_ld32(tmem + ((uint32_t)(quad * 32) << 16) + cb, r);
      else { uint32_t r16[16]; tmem_ld16(tmem + ((uint32_t)(quad * 32) << 16) + cb, r16);
#pragma unroll
             for (int i = 0; i < 16; ++i) r[i] = r16[i]; }
      tmem_ld_wait();
      if (Cfg::NMMA == 2 && nk >= 2) {
        uint32_t q[32];
        if constexpr (CB == 32) tmem_ld32(tmem + ((uint32_t)(quad * 32) << 16) + Cfg::ACC_COLS + cb, q);
        else { uint32_t q16[16]; tmem_ld16(tmem + ((uint32_t)(quad * 32) << 16) + Cfg::ACC_COLS + cb, q16);
#pragma unroll
               for (int i = 0; i < 16; ++i) q[i] = q16[i]; }
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < CB; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) + __uint_as_float(q[i]));
      }
      if constexpr (MAGIC) {
        if (row_post != 1.f) {
#pragma unroll
          for (int i = 0; i < CB; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * row_post);
        }
      }
      // balanced mode has one column block per thread at most: the accumulators are free for the next segment now
      if (BAL && balanced && !freed) { tc_fence_before(); mbar_arrive(accum_empty); freed = true; }
      if (!BAL || !sg.part) {
        write_out(r, cb);
      } else {
#pragma unroll
        for (int i = 0; i < CB; ++i)
          if (cb + i < M) __stcg(my_part + (cb + i) * 128, __uint_as_float(r[i]));
      }
    }
    if (BAL && balanced && !freed) { tc_fence_before(); mbar_arrive(accum_empty); }
    if constexpr (BAL) {
      if (peer_flag && !sg.part) {
        // all epilogue threads have issued their stores of this strip; one of them publishes it
        mbar_arrive(fix_bar);
        ok = mbar_wait(fix_bar, fixn & 1, abort_flag, p.status, ST_FIXUP); ++fixn;
        if (!ok) break;
        if (threadIdx.x == Cfg::CW * 32) {
          __threadfence_system();
          st_release_sys(peer_flag, reinterpret_cast<const PeerCtrl*>(p.peer.bufs[p.peer.rank])->epoch + 1);
        }
      }
    }
    if (BAL && sg.part) {
      // Whoever delivers a strip's last partial sums adds all of them up, always in CTA order, and writes the
      // result: no CTA ever waits for another one, and the sum does not depend on who came last.
      const int64_t U = p.sk_units, G = gridDim.x;
      const int64_t us = (int64_t)sg.strip * p.sk_sps, ue = us + p.sk_sps - 1;
      const int b_lo = (int)(((us + 1) * G + U - 1) / U) - 1, b_hi = (int)(((ue + 1) * G + U - 1) / U) - 1;
      // the barrier hands every thread's partial sums to the leader (release / acquire at CTA scope); the leader's one
      // device-scope fence then orders all of them before the count.  A fence per thread in front of the barrier adds
      // nothing to that and cost 0.7 % of a decode layer.
      mbar_arrive(fix_bar);
      ok = mbar_wait(fix_bar, fixn & 1, abort_flag, p.status, ST_FIXUP); ++fixn;
      if (!ok) break;
      if (threadIdx.x == Cfg::CW * 32) {
        __threadfence();                               // orders the partial sums of all epilogue threads before the count
        const int old = atomicAdd(p.sk_counters + sg.strip, 1);
        const int last = old == b_hi - b_lo;
        if (last) p.sk_counters[sg.strip] = 0;       // every contributor has arrived: ready for the next launch
        *last_flag = last;
      }
      mbar_arrive(fix_bar);
      ok = mbar_wait(fix_bar, fixn & 1, abort_flag, p.status, ST_FIXUP); ++fixn;
      if (!ok) break;
      const int cb = cgrp * CB;
      if (*last_flag && cb < TOK && cb < M) {
        __threadfence();
        uint32_t r[32];
#pragma unroll
        for (int i = 0; i < CB; ++i) r[i] = 0u;
        for (int b = b_lo; b <= b_hi; ++b) {
          const int64_t bu0 = (int64_t)b * U / G;
          const float* src = p.sk_partials + ((size_t)(b * 2 + (bu0 >= us ? 0 : 1)) * TOK) * 128 + quad * 32 + lane;
#pragma unroll
          for (int i = 0; i < CB; ++i)
            if (cb + i < M) r[i] = __float_as_uint(__uint_as_float(r[i]) + __ldcg(src + (cb + i) * 128));
        }
        write_out(r, cb);
      }
      if (*last_flag && peer_flag) {
        mbar_arrive(fix_bar);
        ok = mbar_wait(fix_bar, fixn & 1, abort_flag, p.status, ST_FIXUP); ++fixn;
        if (!ok) break;
        if (threadIdx.x == Cfg::CW * 32) {
          __threadfence_system();
          st_release_sys(peer_flag, reinterpret_cast<const PeerCtrl*>(p.peer.bufs[p.peer.rank])->epoch + 1);
        }
      }
    }
    gb += nk; grb += (nk + CPR - 1) / CPR; ++si;
    }   // segments
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, Cfg::TMEM_COLS); }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
PFN_tensorMapEncodeTiled tensor_map_encoder() {
  static PFN_tensorMapEncodeTiled fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_tensorMapEncodeTiled>(p);
  }
  return fn;
}

int make_tmap_2d(CUtensorMap* out, CUtensorMapDataType dt, int elem_bytes, const void* base, uint64_t rows, uint64_t cols,
                 uint64_t pitch_bytes, uint32_t box_rows, uint32_t box_cols, CUtensorMapSwizzle swz) {
  PFN_tensorMapEncodeTiled enc = tensor_map_encoder();
  if (!enc) return B2Q_ERR_CUDA;
  if ((reinterpret_cast<uintptr_t>(base) & 15u) || (pitch_bytes & 15u)) return B2Q_ERR_ALIGN;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  (void)elem_bytes;
  return r == CUDA_SUCCESS ? B2Q_OK : B2Q_ERR_CUDA;
}

static int* status_ptr() {
  static thread_local int* ptr[16] = {nullptr};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 16) return nullptr;
  if (!ptr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_umma_status) != cudaSuccess) return nullptr;
    ptr[dev] = reinterpret_cast<int*>(p);
  }
  return ptr[dev];
}

// Self-test of the bounded-wait machinery: one CTA waits on an mbarrier that nobody ever arrives on, with a limit of
// about a millisecond instead of two seconds.  The wait must give up, record `code` in the status word and return;
// the context stays usable.  Nothing here faults or spins without bound.
__global__ void bounded_wait_selftest_kernel(int* status, int code, long long limit_ticks, int* gave_up) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) { sm100::mbar_init(sm100::smem_u32(&bar), 1); abort_flag = 0; sm100::fence_barrier_init(); }
  __syncthreads();
  const bool ok = sm100::mbar_wait(sm100::smem_u32(&bar), 0, &abort_flag, status, code, limit_ticks);
  if (threadIdx.x == 0) *gave_up = ok ? 0 : 1;
}

int w8a8_read_status(int* out);
int w8d_read_status(int* out);
int w4i_read_status(int* out);

int umma_selftest_bounded_wait(int code, int* gave_up_dev, cudaStream_t st) {
  int* p = status_ptr();
  if (!p) return B2Q_ERR_CUDA;
  bounded_wait_selftest_kernel<<<1, 64, 0, st>>>(p, code, 2000000LL, gave_up_dev);     // ~1 ms at 1.9 GHz
  note_launch("bounded_wait_selftest");
  return launch_status();
}

int w8a8_reset_state();
int w8d_reset_state();
int w4i_reset_state();

// Clears, on the current device, the status word of every tcgen05 kernel family and the arrival counters of cut
// strips.  A CTA that gave up on a wait never delivered its arrival, so its strip's counter is left non-zero and the
// next launch that takes the same bank would finish that strip one arrival early: status and counters go together.
// The device must be idle (the call synchronises it first).
int umma_reset_status() {
  int* p = status_ptr();
  if (!p) return B2Q_ERR_CUDA;
  if (cudaDeviceSynchronize() != cudaSuccess) return B2Q_ERR_CUDA;
  if (cudaMemset(p, 0, sizeof(int)) != cudaSuccess) return B2Q_ERR_CUDA;
  void* c = nullptr;
  if (cudaGetSymbolAddress(&c, g_sk_counters) != cudaSuccess) return B2Q_ERR_CUDA;
  if (cudaMemset(c, 0, sizeof(int) * SK_BANKS * SK_MAX_STRIPS) != cudaSuccess) return B2Q_ERR_CUDA;
  int rc = w8a8_reset_state();
  if (!rc) rc = w8d_reset_state();
  if (!rc) rc = w4i_reset_state();
  return rc;
}

int umma_read_status(int* out) {
  int* p = status_ptr();
  if (!p) return B2Q_ERR_CUDA;
  int rc = cuda_status(cudaMemcpy(out, p, sizeof(int), cudaMemcpyDeviceToHost));
  if (rc || *out) return rc;
  rc = w8a8_read_status(out);
  if (rc || *out) return rc;
  rc = w8d_read_status(out);
  if (rc || *out) return rc;
  return w4i_read_status(out);
}


// ---- balanced mode (decode shapes) ----------------------------------------------------------------
// Arrival counters of cut strips.  They are zero whenever no launch is in flight (the last arriver of a
// strip resets its counter), so nothing has to be cleared per launch; launches take one of 64 banks in turn
// so that launches overlapping in time (other streams, programmatic dependent launch) do not share counters.

static int* sk_counter_bank() {
  static thread_local int* basep[16] = {nullptr};
  static std::atomic<unsigned> next_bank{0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 16) return nullptr;
  if (!basep[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_sk_counters) != cudaSuccess) return nullptr;
    basep[dev] = reinterpret_cast<int*>(p);
  }
  return basep[dev] + (size_t)(next_bank.fetch_add(1, std::memory_order_relaxed) % SK_BANKS) * SK_MAX_STRIPS;
}

static int device_slots() {
  static thread_local int sms[16] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 16) return 296;
  if (!sms[dev]) {
    cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
    if (sms[dev] <= 0) sms[dev] = 148;
  }
  return 2 * sms[dev];                     // decode tiles run two CTAs per SM
}

static int pick_tok(int m);

size_t umma_balanced_ws_bytes(int64_t M) {
  if (M > 64) return 0;
  return (size_t)2 * device_slots() * pick_tok((int)M) * 128 * sizeof(float);
}

// Fills the balanced-mode fields of p when the shape profits: one token tile, whole raw stages, and a grid of
// one CTA per strip that would leave more than a twentieth of the machine idle in its last wave.
static int plan_balanced(UmmaWoParams& p, const UmmaGroupArgs& a, int M, int N, int K, int cpr, int tok) {
  p.sk_sps = 0; p.sk_units = 0; p.sk_partials = nullptr; p.sk_counters = nullptr;
  if (tls().force_kernel == 4) return 0;       // benchmarking: one CTA per strip
  if (a.expert_offsets || tok > 64 || M > tok || !a.sk_ws || a.sk_ws_bytes < umma_balanced_ws_bytes(M)) return 0;
  if ((K % (64 * cpr)) != 0 || (reinterpret_cast<uintptr_t>(a.sk_ws) & 15u)) return 0;
  const int strips = (N + 127) / 128, slots = device_slots();
  if (strips > SK_MAX_STRIPS) return 0;
  const double eff = (double)strips / ((double)((strips + slots - 1) / slots) * slots);
  if (eff > 0.95) return 0;
  const int sps = K / (64 * cpr);
  const int64_t units = (int64_t)strips * sps;
  if (units > INT32_MAX) return 0;
  int* counters = sk_counter_bank();
  if (!counters) return 0;
  p.sk_sps = sps; p.sk_units = (int)units;
  p.sk_partials = reinterpret_cast<float*>(a.sk_ws); p.sk_counters = counters;
  return (int)(units < slots ? units : slots);
}

static int pick_tok(int m) { return m <= 16 ? 16 : (m <= 32 ? 32 : (m <= 64 ? 64 : (m <= 128 ? 128 : 256))); }

template <int WK, bool BF16, int TOK, bool FAST, bool MAGIC>
static int launch_one(const CUtensorMap& tw, const CUtensorMap& tx, const UmmaWoParams& p_in, int token_tiles, cudaStream_t st) {
  UmmaWoParams p = p_in;
  p.tiles_on_y = (p.tiles && token_tiles <= 65535) ? 1 : 0;      // gridDim.y is limited to 65535
  using Cfg = UmmaCfg<TOK>;
  auto kern = umma_wo_kernel<WK, BF16, TOK, FAST, MAGIC>;
  static thread_local bool configured[16] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 16 || !configured[dev]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM) != cudaSuccess) return B2Q_ERR_CUDA;
    if (dev < 16) configured[dev] = true;
  }
  dim3 grid(token_tiles, (p.N + 127) / 128, 1);
  if (p.tiles_on_y) grid = dim3((p.N + 127) / 128, token_tiles, 1);
  if (p.sk_sps > 0) grid = dim3(p.sk_grid, 1, 1);
  const bool overlap = tls().overlap_mode > 0 && p.overlap_ok;
  if (launch_overlapped(kern, grid, dim3(Cfg::THREADS), Cfg::SMEM, st, overlap, tw, tx, p) != cudaSuccess) return B2Q_ERR_CUDA;
  note_launch("umma_wo");
  return launch_status();
}

template <int WK, bool BF16, bool FAST, bool MAGIC = false>
static int launch_tok(int tok, const CUtensorMap& tw, const CUtensorMap& tx, const UmmaWoParams& p, int tiles, cudaStream_t st) {
  switch (tok) {
    case 16: return launch_one<WK, BF16, 16, FAST, MAGIC>(tw, tx, p, tiles, st);
    case 32: return launch_one<WK, BF16, 32, FAST, MAGIC>(tw, tx, p, tiles, st);
    case 64: return launch_one<WK, BF16, 64, FAST, MAGIC>(tw, tx, p, tiles, st);
    case 128: return launch_one<WK, BF16, 128, FAST, MAGIC>(tw, tx, p, tiles, st);
    default: return launch_one<WK, BF16, 256, FAST, MAGIC>(tw, tx, p, tiles, st);
  }
}

template <int WK>
static int launch_wk(bool bf16, bool fast, int tok, const CUtensorMap& tw, const CUtensorMap& tx, const UmmaWoParams& p,
                     int tiles, cudaStream_t st) {
  if (bf16) return fast ? launch_tok<WK, true, true>(tok, tw, tx, p, tiles, st) : launch_tok<WK, true, false>(tok, tw, tx, p, tiles, st);
  return fast ? launch_tok<WK, false, true>(tok, tw, tx, p, tiles, st) : launch_tok<WK, false, false>(tok, tw, tx, p, tiles, st);
}

static int grouped_tok(int rows, int E) {
  const int avg = E > 0 ? (rows + E - 1) / E : rows;
  return avg <= 16 ? 16 : (avg <= 32 ? 32 : (avg <= 96 ? 64 : 128));
}

bool umma_w4_supported(const UmmaW4Args& a) {
  if (a.K % 128 != 0 || a.K < 64) return false;
  if (!aligned16(a.x) || !aligned16(a.w) || ((a.ldx * 2) & 15)) return false;
  const bool kmajor = a.layout == B2Q_W4_KMAJOR || a.layout == B2Q_W4_KMAJOR_MARLIN;
  if (kmajor && (a.N % 4) != 0) return false;              // tensor-map pitch must be a multiple of 16 bytes
  if (a.act != B2Q_ACT_NONE) return false;                 // activation is applied by a separate kernel
  if (a.row_map) return false;                             // rows are gathered by the caller first
  return tensor_map_encoder() != nullptr && status_ptr() != nullptr;
}
int umma_w4_token_tile(const UmmaW4Args& a) { return a.expert_offsets ? grouped_tok(a.M, a.E) : pick_tok(a.M); }

int umma_w4_linear(const UmmaW4Args& a, cudaStream_t st) {
  const bool kmajor = a.layout == B2Q_W4_KMAJOR || a.layout == B2Q_W4_KMAJOR_MARLIN;
  const bool grouped = a.expert_offsets != nullptr;
  const int E = grouped ? a.E : 1;
  const int tok = umma_w4_token_tile(a);
  CUtensorMap tw, tx;
  int rc;
  if (kmajor)
    rc = make_tmap_2d(&tw, CU_TENSOR_MAP_DATA_TYPE_INT32, 4, a.w, (uint64_t)E * (a.K / 8), a.N, (uint64_t)a.N * 4, 32, 128,
                      CU_TENSOR_MAP_SWIZZLE_NONE);
  else
    rc = make_tmap_2d(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.w, (uint64_t)E * a.N, a.K / 2, (uint64_t)a.K / 2, 128, 128,
                      CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  rc = make_tmap_2d(&tx, a.bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, a.x, a.M, a.K,
                    (uint64_t)a.ldx * 2, tok, 64, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  UmmaWoParams p{};
  p.scale = a.scale; p.scale_dtype = a.scale_dtype; p.scale_mode = 0;
  p.s_stride_n = a.s_stride_n; p.s_stride_g = a.s_stride_g;
  p.s_expert_elems = (int64_t)a.N * (a.K / 128);
  p.out = a.out; p.ldo = a.ldo; p.M = a.M; p.N = a.N; p.K = a.K;
  p.marlin = a.layout == B2Q_W4_KMAJOR_MARLIN; p.xor_mask = a.layout == B2Q_W4_NMAJOR_S4 ? 0x88888888u : 0u;
  p.tiles = grouped ? a.tiles : nullptr; p.expert_offsets = a.expert_offsets; p.out_map = a.out_map;
  p.w_rows_per_expert = kmajor ? a.K / 8 : a.N;
  p.tok_scale = a.tok_scale; p.out_bf16 = a.out_bf16 ? 1 : 0; p.magic = a.magic ? 1 : 0;
  p.mk = magic_consts(p.xor_mask != 0);
  p.status = status_ptr();
  p.overlap_ok = (a.after_prep || tls().overlap_mode == 2) ? 1 : 0;
  p.sk_grid = plan_balanced(p, a, a.M, a.N, a.K, 4, tok);
  if (a.peer) {
    if (tok > 64 || grouped || (a.N % 128) != 0 || (a.peer->slice % 128) != 0 || a.peer->M != a.M) return B2Q_ERR_UNSUPPORTED;
    p.peer_on = 1; p.peer = *a.peer;
  }
  const bool fast = a.magic || (a.scale_dtype == (a.bf16 ? B2Q_BF16 : B2Q_F16));
  const int tiles = grouped ? a.tile_cap : (a.M + tok - 1) / tok;
  if (a.magic) {
    if (a.bf16) return B2Q_ERR_UNSUPPORTED;       // the pre-pass always hands over fp16
    return kmajor ? launch_tok<WK_W4K, false, true, true>(tok, tw, tx, p, tiles, st)
                  : launch_tok<WK_W4N, false, true, true>(tok, tw, tx, p, tiles, st);
  }
  return kmajor ? launch_wk<WK_W4K>(a.bf16, fast, tok, tw, tx, p, tiles, st)
                : launch_wk<WK_W4N>(a.bf16, fast, tok, tw, tx, p, tiles, st);
}

bool umma_w8_supported(const UmmaW8Args& a) {
  if (a.K % 64 != 0) return false;
  if (!aligned16(a.x) || !aligned16(a.w) || ((a.ldx * 2) & 15)) return false;
  if (a.scale_mode == B2Q_SCALE_BLOCK128 && ((a.N % 128) != 0 || (a.K % 128) != 0) && a.expert_offsets) return false;
  if (a.act != B2Q_ACT_NONE || a.row_map) return false;
  return tensor_map_encoder() != nullptr && status_ptr() != nullptr;
}
int umma_w8_token_tile(const UmmaW8Args& a) { return a.expert_offsets ? grouped_tok(a.M, a.E) : pick_tok(a.M); }

int umma_w8_linear(const UmmaW8Args& a, cudaStream_t st) {
  const bool grouped = a.expert_offsets != nullptr;
  const int E = grouped ? a.E : 1;
  const int tok = umma_w8_token_tile(a);
  CUtensorMap tw, tx;
  int rc = make_tmap_2d(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.w, (uint64_t)E * a.N, a.K, (uint64_t)a.K, 128, 128,
                        CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  rc = make_tmap_2d(&tx, a.bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, a.x, a.M, a.K,
                    (uint64_t)a.ldx * 2, tok, 64, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  UmmaWoParams p{};
  p.scale = a.scale; p.scale_dtype = a.scale_dtype; p.scale_mode = a.scale_mode;
  p.s_expert_elems = a.s_expert_elems;
  p.out = a.out; p.ldo = a.ldo; p.M = a.M; p.N = a.N; p.K = a.K;
  p.e5m2 = a.fmt == B2Q_E5M2;
  p.tiles = grouped ? a.tiles : nullptr; p.expert_offsets = a.expert_offsets; p.out_map = a.out_map;
  p.w_rows_per_expert = a.N;
  p.tok_scale = a.tok_scale; p.out_bf16 = a.out_bf16 ? 1 : 0;
  p.status = status_ptr();
  p.overlap_ok = (a.after_prep || tls().overlap_mode == 2) ? 1 : 0;
  p.sk_grid = plan_balanced(p, a, a.M, a.N, a.K, 2, tok);
  const int tiles = grouped ? a.tile_cap : (a.M + tok - 1) / tok;
  return launch_wk<WK_W8>(a.bf16, true, tok, tw, tx, p, tiles, st);
}


}  // namespace b2q
