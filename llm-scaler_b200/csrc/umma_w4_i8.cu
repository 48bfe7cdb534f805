// INT4 (group 128) decode GEMM on the 8-bit integer tensor-core path:
//     out[m, n] = sum_g s[n, g] * sum_{k in g} (q[n, k] - 8) * x[m, k].
//
// Turning a packed nibble into a 16-bit float costs several integer operations per weight and doubles the
// MMA count (K = 16 per instruction); that, not bandwidth, bounds the 16-bit decode path.  Here a word of
// eight nibbles becomes two words of unsigned bytes with one AND, one shift and one AND, the bytes go into
// tensor memory as the A operand of tcgen05.mma kind::i8 (K = 32 per instruction), and the activations come
// in as signed bytes: a pre-pass scales each token row by a power of two and splits it into three int8 terms,
//     x * 2^e = t0 + t1 / 128 + t2 / 16384,
// stacked as extra token columns of the MMA's N (an MMA with N <= 64 costs the same whatever N is).  Products
// and sums are exact integers.  The group scale varies along k, so every group of 128 k gets its own s32
// accumulator in tensor memory and four promotion warps add s[n, g] * (partial - 8 * sum_k x) into fp32
// registers while the MMA already works on the next groups (the -8 of the nibble offset is folded into that
// step through the pre-pass's per-group activation sums).
// Work is shared out like in umma_w8_direct.cu: one CTA per strip of h <= 128 rows, h chosen for equal load
// per SM, or, when there are few strips, strips cut along k with ordered partial sums.
//
// Status: measured on B200 it streams 1.2-1.9 TB/s, on a level with the two 16-bit kernels and ahead of them only
// for few rows and a long k ([8192 x 28672] at M <= 8), which is where it is dispatched (umma_w4_i8_preferred): with
// one accumulator per group of 128 k, only four groups (32 KB of weights) fit in a CTA's tensor memory between the
// transform and the promotion warps, and the barrier hand-offs along that chain, not arithmetic, set the pace.
// b2q_set_force_kernel(5) selects it for every decode shape.
//
// Reference counterpart: esimd_gemv_int4 / esimd_gemm_int4_pgrp
// (vllm/custom-esimd-kernels-vllm/csrc/xpu/esimd_kernels/gemv_int4.h, gemm_int4_pgrp.h), GGML N-major weights.
#include <atomic>
#include "umma_gemm.cuh"
#include "sm100.cuh"
#include "smallm.cuh"   // lds128

namespace b2q {

using namespace sm100;

__device__ int g_w4i_status = 0;
constexpr int W4I_BANKS = 64, W4I_MAX_STRIPS = 2048;
__device__ int g_w4i_counters[W4I_BANKS * W4I_MAX_STRIPS];

namespace w4i {
enum { ST_RAWFULL = 401, ST_RAWEMPTY = 402, ST_XFULL = 403, ST_XEMPTY = 404, ST_AFULL = 405, ST_AEMPTY = 406,
       ST_ACCFULL = 407, ST_ACCEMPTY = 408, ST_FIXUP = 409 };

template <int NTOK> struct Cfg {
  static constexpr int RAW_BYTES = 16384;                       // 128 rows x 256 k of nibbles = two groups
  static constexpr int X_BYTES = NTOK * 128;                    // NTOK term rows x 128 k of int8 = one group
  static constexpr int RS = NTOK <= 32 ? 5 : 4;                 // raw stages
  static constexpr int XS = NTOK <= 32 ? 6 : 5;                 // activation stages
  static constexpr int SMEM = RS * RAW_BYTES + XS * X_BYTES + 1024 + 512;
  static constexpr int SA = NTOK <= 32 ? 4 : 2;                 // operand slots in tensor memory (32 columns = 128 k each)
  static constexpr int NB = NTOK <= 32 ? 4 : 3;                 // group accumulators (NTOK columns each)
  static constexpr int ACC0 = SA * 32;
  static constexpr int TMEM_COLS = 256;                         // two CTAs per SM
  static constexpr int THREADS = 16 * 32;   // warps: 0 raw TMA, 1 MMA, 2 X TMA, 3 idle, 4-7 promotion, 8-15 transform
};

// groups [g_begin, g_end) of the strip at row n0, taken in the order g_begin + (j + rot) % (g_end - g_begin)
struct Segment { int n0, strip, g_begin, g_end, part, slot, rot; };
}  // namespace w4i

struct W4IParams {
  const void* scale; int scale_dtype; int64_t s_stride_n, s_stride_g;
  const float* inv_scale;            // [M] 2^-e of the pre-pass
  const float* xsum;                 // [K/128][Mp] per-group sums of the scaled activations
  void* out; int64_t ldo; int out_bf16;
  int M, Mp, N, K;
  uint32_t xor_mask;                 // 0x88888888 for two's-complement nibbles
  int h;                             // weight rows per strip
  int sps, ust, units;               // units per strip, raw stages per unit, units in total
  float* partials; int* counters;
  int* status;
};

template <int NTOK>
__global__ void __launch_bounds__(w4i::Cfg<NTOK>::THREADS, 2)
umma_w4_i8_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x, const W4IParams p) {
  using C = w4i::Cfg<NTOK>;
  using namespace w4i;
  constexpr int RS = C::RS, XS = C::XS, SA = C::SA, NB = C::NB;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t raw_smem = base, x_smem = base + RS * C::RAW_BYTES;
  const uint32_t bar = x_smem + XS * C::X_BYTES;
  const uint32_t raw_full = bar, raw_empty = raw_full + 8 * RS, x_full = raw_empty + 8 * RS, x_empty = x_full + 8 * XS;
  const uint32_t a_full = x_empty + 8 * XS, a_empty = a_full + 8 * SA, acc_full = a_empty + 8 * SA, acc_empty = acc_full + 8 * NB;
  const uint32_t fix_bar = acc_empty + 8 * NB;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen + (fix_bar + 8 - base));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + (fix_bar + 16 - base));
  volatile int* last_flag = reinterpret_cast<volatile int*>(gen + (fix_bar + 20 - base));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ngroups = p.K >> 7;

  grid_dep_release();      // the next kernel may start; this one waits for earlier ones only before it reads activations

  // every role walks the same list of segments with its own copy of this cursor
  const int u0 = (int)((int64_t)blockIdx.x * p.units / gridDim.x), u1 = (int)((int64_t)(blockIdx.x + 1) * p.units / gridDim.x);
  int u = u0;
  auto next_segment = [&](Segment& sg) -> bool {
    if (u >= u1) return false;
    const int strip = u / p.sps, r0 = u - strip * p.sps;
    const int take = min(p.sps - r0, u1 - u);
    sg.strip = strip; sg.n0 = strip * p.h;
    sg.g_begin = r0 * p.ust * 2; sg.g_end = min(ngroups, (r0 + take) * p.ust * 2);
    sg.part = take != p.sps; sg.slot = (u == u0) ? 0 : 1;
    // Every CTA starts at a different group: all CTAs read the same small activation array, and in step they would
    // all ask the same L2 lines for it at the same moment.  (Whole raw stages only, so an odd tail is not rotated.)
    const int ng = sg.g_end - sg.g_begin;
    sg.rot = (ng & 1) ? 0 : (int)((2u * (blockIdx.x * 5u + (unsigned)strip)) % (unsigned)ng);
    u += take;
    return true;
  };

  if (threadIdx.x == 0) {
    for (int i = 0; i < RS; ++i) { mbar_init(raw_full + 8 * i, 1); mbar_init(raw_empty + 8 * i, 256); }
    for (int i = 0; i < XS; ++i) { mbar_init(x_full + 8 * i, 1); mbar_init(x_empty + 8 * i, 1); }
    for (int i = 0; i < SA; ++i) { mbar_init(a_full + 8 * i, 128); mbar_init(a_empty + 8 * i, 1); }
    for (int i = 0; i < NB; ++i) { mbar_init(acc_full + 8 * i, 1); mbar_init(acc_empty + 8 * i, 128); }
    mbar_init(fix_bar, 128);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), C::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  Segment sg;

  if (warp == 0) {
    // ---- raw weight producer: one box of h rows x 128 bytes (256 k) per stage ----
    if (lane == 0) {
      tma_prefetch_desc(&tm_w);
      int gr = 0;
      bool ok = true;
      while (ok && next_segment(sg)) {
        const int ng = sg.g_end - sg.g_begin;
        for (int j = 0; j < ng; j += 2, ++gr) {
          const int g = sg.g_begin + (j + sg.rot) % ng;
          const int rs = gr % RS;
          if (gr >= RS && !mbar_wait(raw_empty + 8 * rs, ((gr / RS) - 1) & 1, abort_flag, p.status, ST_RAWEMPTY)) { ok = false; break; }
          mbar_expect_tx(raw_full + 8 * rs, p.h * 128);
          tma_load_2d(raw_smem + rs * C::RAW_BYTES, &tm_w, (g >> 1) * 128, sg.n0, raw_full + 8 * rs);
        }
      }
      if (!ok) drain_issued(raw_full, RS, gr);
    }
  } else if (warp == 2) {
    // ---- activation producer: the NTOK term rows of one group per stage ----
    if (lane == 0) {
      tma_prefetch_desc(&tm_x);
      grid_dep_wait();
      int gc = 0;
      bool ok = true;
      while (ok && next_segment(sg)) {
        const int ng = sg.g_end - sg.g_begin;
        for (int j = 0; j < ng; ++j, ++gc) {
          const int g = sg.g_begin + (j + sg.rot) % ng;
          const int s = gc % XS;
          if (gc >= XS && !mbar_wait(x_empty + 8 * s, ((gc / XS) - 1) & 1, abort_flag, p.status, ST_XEMPTY)) { ok = false; break; }
          mbar_expect_tx(x_full + 8 * s, C::X_BYTES);
          tma_load_2d(x_smem + s * C::X_BYTES, &tm_x, g * 128, 0, x_full + 8 * s);
        }
      }
      if (!ok) drain_issued(x_full, XS, gc);
    }
  } else if (warp == 1) {
    // ---- MMA issuer: one group (128 k) = four MMAs into that group's own accumulator ----
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc_i8(0u, 1u, 128, NTOK);       // u8 weights x s8 activations -> s32
      int gc = 0;
      bool ok = true;
      while (ok && next_segment(sg)) {
#pragma unroll 1
        for (int g = sg.g_begin; g < sg.g_end; ++g, ++gc) {
          const int sa = gc % SA, xs = gc % XS, nb = gc % NB;
          { ok = mbar_wait(x_full + 8 * xs, (gc / XS) & 1, abort_flag, p.status, ST_XFULL); }
          if (ok) { ok = mbar_wait(a_full + 8 * sa, (gc / SA) & 1, abort_flag, p.status, ST_AFULL); }
          if (ok && gc >= NB) { ok = mbar_wait(acc_empty + 8 * nb, ((gc / NB) - 1) & 1, abort_flag, p.status, ST_ACCEMPTY); }
          if (!ok) break;
          tc_fence_after();
          const uint32_t d = tmem + C::ACC0 + nb * NTOK, ta = tmem + sa * 32;
          const uint64_t db = smem_desc_sw128(x_smem + xs * C::X_BYTES);
          mma_i8_ts(d, ta, db, idesc, 0u);
          mma_i8_ts(d, ta + 8, db + 2, idesc, 1u);
          mma_i8_ts(d, ta + 16, db + 4, idesc, 1u);
          mma_i8_ts(d, ta + 24, db + 6, idesc, 1u);
          tc_commit(a_empty + 8 * sa);
          tc_commit(x_empty + 8 * xs);
          tc_commit(acc_full + 8 * nb);
        }
      }
    }
  } else if (warp >= 8) {
    // ---- transform: two teams of four warps on alternate groups; a thread owns one weight row ----
    const int team = (warp - 8) >> 2;
    const int t = (warp & 3) * 32 + lane;            // row of the strip == tensor-memory lane
    const int sw = t & 7;
    const uint32_t trow = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    int gc = 0, gr = 0;
    bool ok = true;
    while (ok && next_segment(sg)) {
      const int ng = sg.g_end - sg.g_begin;
#pragma unroll 1
      for (int j = 0; j < ng; ++j) {
        const int c = gc + j, r = gr + (j >> 1), rs = r % RS;
        const bool mine = (j & 1) == team;
        if (mine) {
          { ok = mbar_wait(raw_full + 8 * rs, (r / RS) & 1, abort_flag, p.status, ST_RAWFULL); }
          if (!ok) break;
          const int sa = c % SA;
          if (c >= SA) { ok = mbar_wait(a_empty + 8 * sa, ((c / SA) - 1) & 1, abort_flag, p.status, ST_AEMPTY); if (!ok) break; }
          tc_fence_after();
          const uint32_t rawrow = raw_smem + rs * C::RAW_BYTES + t * 128;
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            uint32_t av[16];
#pragma unroll
            for (int q4 = 0; q4 < 2; ++q4) {
              const uint4 v = lds128(rawrow + ((((j & 1) * 4 + half * 2 + q4) ^ sw) << 4));
              const uint32_t w[4] = {v.x ^ p.xor_mask, v.y ^ p.xor_mask, v.z ^ p.xor_mask, v.w ^ p.xor_mask};
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                av[q4 * 8 + 2 * i] = w[i] & 0x0F0F0F0Fu;                  // k 0, 2, 4, 6 of the word
                av[q4 * 8 + 2 * i + 1] = (w[i] >> 4) & 0x0F0F0F0Fu;       // k 1, 3, 5, 7
              }
            }
            tmem_st16(trow + sa * 32 + half * 16, av);
          }
          tmem_st_wait();
          tc_fence_before();
          mbar_arrive(a_full + 8 * sa);
          mbar_arrive(raw_empty + 8 * rs);      // a raw stage holds two groups, one per team
        }
      }
      if (!ok) break;
      // a segment with an odd number of groups leaves the last raw stage with one group only: the team without a
      // group in it still has to release the stage
      if ((ng & 1) && team == 1) mbar_arrive(raw_empty + 8 * ((gr + (ng >> 1)) % RS));
      gc += ng; gr += (ng + 1) >> 1;
    }
  } else if (warp >= 4) {
    // ---- promotion + epilogue: warps 4..7, lane quadrant = warp & 3; a thread owns one weight row ----
    constexpr int MPMAX = NTOK <= 32 ? 8 : 16;        // tokens (rounded up to 8) a launch of this width can carry
    const int quad = warp & 3, rowi = quad * 32 + lane;
    const uint32_t trow = tmem + ((uint32_t)(quad * 32) << 16) + C::ACC0;
    uint16_t* outp = reinterpret_cast<uint16_t*>(p.out);
    int gc = 0, fixn = 0;
    bool ok = true;
    grid_dep_wait();                                   // reads what the pre-pass wrote (activation sums, token scales)
    while (ok && next_segment(sg)) {
      const int n = sg.n0 + rowi;
      const int nn = n < p.N ? n : p.N - 1;
      float acc[MPMAX];
#pragma unroll
      for (int i = 0; i < MPMAX; ++i) acc[i] = 0.f;
      // group scales of this row, fetched four groups ahead of their use
      // (as raw bits: decoding a value at its load would make the warp wait for DRAM there, once per group)
      uint32_t sc_nxt[4];
      const int ng = sg.g_end - sg.g_begin;
      auto group_scale = [&](int j) -> uint32_t {   // raw scale of the j-th group in processing order
        if (j >= ng) return 0u;
        const int g = sg.g_begin + (j + sg.rot) % ng;
        return load_scalar_raw(p.scale, (int64_t)nn * p.s_stride_n + (int64_t)g * p.s_stride_g, p.scale_dtype);
      };
#pragma unroll
      for (int j = 0; j < 4; ++j) sc_nxt[j] = group_scale(j);
#pragma unroll 1
      for (int gb = 0; gb < ng && ok; gb += 4) {
        uint32_t sc_raw[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          sc_raw[j] = sc_nxt[j];
          sc_nxt[j] = group_scale(gb + 4 + j);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (gb + j < ng && ok) {
            const int nb = gc % NB;
            // the group's activation sums (a few floats shared by the whole CTA): requested before the wait so that the
            // L2 round trip overlaps it; read past L1, which may still hold the previous call's values at this address
            const float* xs_g = p.xsum + (int64_t)(sg.g_begin + (gb + j + sg.rot) % ng) * p.Mp;
            float xv[MPMAX];
#pragma unroll
            for (int mb = 0; mb < MPMAX / 8; ++mb) {
              if (mb * 8 < p.Mp) {
                const float4 x0 = __ldcg(reinterpret_cast<const float4*>(xs_g + mb * 8));
                const float4 x1 = __ldcg(reinterpret_cast<const float4*>(xs_g + mb * 8 + 4));
                xv[mb * 8 + 0] = x0.x; xv[mb * 8 + 1] = x0.y; xv[mb * 8 + 2] = x0.z; xv[mb * 8 + 3] = x0.w;
                xv[mb * 8 + 4] = x1.x; xv[mb * 8 + 5] = x1.y; xv[mb * 8 + 6] = x1.z; xv[mb * 8 + 7] = x1.w;
              }
            }
            { ok = mbar_wait(acc_full + 8 * nb, (gc / NB) & 1, abort_flag, p.status, ST_ACCFULL); }
            if (ok) {
              tc_fence_after();
              const float scj = scalar_from_raw(sc_raw[j], p.scale_dtype);
#pragma unroll
              for (int mb = 0; mb < MPMAX / 8; ++mb) {
                if (mb * 8 < p.Mp) {
                  uint32_t a[8], b[8], c[8];
                  tmem_ld8(trow + nb * NTOK + mb * 8, a);
                  tmem_ld8(trow + nb * NTOK + p.Mp + mb * 8, b);
                  tmem_ld8(trow + nb * NTOK + 2 * p.Mp + mb * 8, c);
                  tmem_ld_wait();
#pragma unroll
                  for (int i = 0; i < 8; ++i) {
                    const float v = (float)(int)a[i] + (float)(int)b[i] * 0.0078125f + (float)(int)c[i] * 6.103515625e-05f -
                                    8.f * xv[mb * 8 + i];
                    acc[mb * 8 + i] = fmaf(scj, v, acc[mb * 8 + i]);
                  }
                }
              }
              tc_fence_before();
              mbar_arrive(acc_empty + 8 * nb);
              ++gc;
            }
          }
        }
      }
      if (!ok) break;
      auto write_out = [&](const float (&v)[MPMAX]) {
        if (n >= p.N || rowi >= p.h) return;
#pragma unroll
        for (int m = 0; m < MPMAX; ++m)
          if (m < p.M) {
            const float o = v[m] * __ldcg(p.inv_scale + m);
            outp[(int64_t)m * p.ldo + n] = p.out_bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(o)) : __half_as_ushort(__float2half_rn(o));
          }
      };
      if (!sg.part) {
        write_out(acc);
      } else {
        // a strip cut between CTAs: whoever delivers its partial sums last adds them up in CTA order and writes
        float* const my_part = p.partials + ((size_t)(blockIdx.x * 2 + sg.slot) * MPMAX) * 128 + rowi;
#pragma unroll
        for (int m = 0; m < MPMAX; ++m)
          if (m < p.Mp) __stcg(my_part + m * 128, acc[m]);
        const int64_t U = p.units, G = gridDim.x;
        const int64_t us = (int64_t)sg.strip * p.sps, ue = us + p.sps - 1;
        const int b_lo = (int)(((us + 1) * G + U - 1) / U) - 1, b_hi = (int)(((ue + 1) * G + U - 1) / U) - 1;
        mbar_arrive(fix_bar);          // hands this thread's partial sums to the leader, whose fence orders them before the count
        ok = mbar_wait(fix_bar, fixn & 1, abort_flag, p.status, ST_FIXUP); ++fixn;
        if (!ok) break;
        if (threadIdx.x == 4 * 32) {
          __threadfence();
          const int old = atomicAdd(p.counters + sg.strip, 1);
          const int last = old == b_hi - b_lo;
          if (last) p.counters[sg.strip] = 0;
          *last_flag = last;
        }
        mbar_arrive(fix_bar);
        ok = mbar_wait(fix_bar, fixn & 1, abort_flag, p.status, ST_FIXUP); ++fixn;
        if (!ok) break;
        if (*last_flag) {
          __threadfence();
          float v[MPMAX];
#pragma unroll
          for (int m = 0; m < MPMAX; ++m) v[m] = 0.f;
          for (int b = b_lo; b <= b_hi; ++b) {
            const int64_t bu0 = (int64_t)b * U / G;
            const float* src = p.partials + ((size_t)(b * 2 + (bu0 >= us ? 0 : 1)) * MPMAX) * 128 + rowi;
#pragma unroll
            for (int m = 0; m < MPMAX; ++m)
              if (m < p.Mp) v[m] += __ldcg(src + m * 128);
          }
          write_out(v);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, C::TMEM_COLS); }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
static int w4i_sm_count() {
  static thread_local int sms[16] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 16) return 148;
  if (!sms[dev]) {
    cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
    if (sms[dev] <= 0) sms[dev] = 148;
  }
  return sms[dev];
}

static int* w4i_counter_bank() {
  static thread_local int* basep[16] = {nullptr};
  static std::atomic<unsigned> next_bank{0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 16) return nullptr;
  if (!basep[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_w4i_counters) != cudaSuccess) return nullptr;
    basep[dev] = reinterpret_cast<int*>(p);
  }
  return basep[dev] + (size_t)(next_bank.fetch_add(1, std::memory_order_relaxed) % W4I_BANKS) * W4I_MAX_STRIPS;
}

// term rows of the activation buffer: three terms x (M rounded up to 8), as a legal MMA N
int umma_w4_i8_rows(int64_t M) { return M <= 8 ? 32 : 64; }

// Shapes on which this kernel measured faster than both 16-bit kernels: few rows (strips get cut along k, which the
// mma.sync kernel cannot do) and a long k.  [8192 x 28672] at M <= 8: 58-65 us against 94 us (mma.sync) and 71 us (tcgen05, 16 bit).
bool umma_w4_i8_preferred(int64_t M, int64_t N, int64_t K) {
  return M <= 8 && ((N + 127) / 128) * 2 <= w4i_sm_count() && N * K >= ((int64_t)1 << 27);
}
// fp32 partial sums of cut strips: [two CTAs per SM][2 slots][16][128]
size_t umma_w4_i8_partial_bytes() { return (size_t)w4i_sm_count() * 2 * 2 * 16 * 128 * sizeof(float); }

static int w4i_pick_strip_rows(int N, int sms) {
  int best = 128;
  int64_t best_load = INT64_MAX;
  for (int h = 128; h >= 32; h -= 8) {
    const int n = (N + h - 1) / h;
    const int64_t load = (int64_t)h * ((n + sms - 1) / sms);
    if (load < best_load) { best_load = load; best = h; }
  }
  return best;
}

template <int NTOK>
static int launch_w4i(const CUtensorMap& tw, const CUtensorMap& tx, const W4IParams& p, int grid, bool overlap, cudaStream_t st) {
  using C = w4i::Cfg<NTOK>;
  auto kern = umma_w4_i8_kernel<NTOK>;
  static thread_local bool configured[16] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 16 || !configured[dev]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM) != cudaSuccess) return B2Q_ERR_CUDA;
    if (dev < 16) configured[dev] = true;
  }
  if (launch_overlapped(kern, dim3(grid), dim3(C::THREADS), C::SMEM, st, overlap, tw, tx, p) != cudaSuccess) return B2Q_ERR_CUDA;
  note_launch("umma_w4_i8");
  return launch_status();
}

int umma_w4_i8_linear(const UmmaW4I8Args& a, cudaStream_t st) {
  if (a.M <= 0 || a.M > 16 || (a.K % 128) != 0) return B2Q_ERR_SHAPE;
  if (!tensor_map_encoder()) return B2Q_ERR_CUDA;
  const int ntok = umma_w4_i8_rows(a.M);
  W4IParams p{};
  p.scale = a.scale; p.scale_dtype = a.scale_dtype; p.s_stride_n = a.s_stride_n; p.s_stride_g = a.s_stride_g;
  p.inv_scale = a.inv_scale; p.xsum = a.xsum; p.out = a.out; p.ldo = a.ldo; p.out_bf16 = a.out_bf16 ? 1 : 0;
  p.M = a.M; p.Mp = (a.M + 7) / 8 * 8; p.N = a.N; p.K = a.K; p.xor_mask = a.xor_mask;
  void* sym = nullptr;
  if (cudaGetSymbolAddress(&sym, g_w4i_status) != cudaSuccess) return B2Q_ERR_CUDA;
  p.status = reinterpret_cast<int*>(sym);
  const int sms = w4i_sm_count(), slots = 2 * sms, nst = (a.K + 255) / 256;
  const bool cut = ((a.N + 127) / 128) * 2 <= sms && a.partials && a.partial_bytes >= umma_w4_i8_partial_bytes() &&
                   (a.N + 127) / 128 <= W4I_MAX_STRIPS;
  p.h = cut ? 128 : w4i_pick_strip_rows(a.N, sms);
  const int strips = (a.N + p.h - 1) / p.h;
  p.ust = cut ? 1 : nst; p.sps = cut ? nst : 1; p.units = strips * p.sps;
  p.partials = reinterpret_cast<float*>(a.partials);
  p.counters = cut ? w4i_counter_bank() : nullptr;
  if (cut && !p.counters) return B2Q_ERR_CUDA;
  const int grid = cut ? (p.units < slots ? p.units : slots) : strips;
  CUtensorMap tw, tx;
  int rc = make_tmap_2d(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.w, a.N, a.K / 2, (uint64_t)a.K / 2, p.h, 128, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  rc = make_tmap_2d(&tx, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.xq, ntok, a.K, (uint64_t)a.K, ntok, 128, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  const bool overlap = tls().overlap_mode > 0;     // always directly behind its own pre-pass
  return ntok == 32 ? launch_w4i<32>(tw, tx, p, grid, overlap, st) : launch_w4i<64>(tw, tx, p, grid, overlap, st);
}


int w4i_reset_state() {
  void* p = nullptr;
  if (cudaGetSymbolAddress(&p, g_w4i_status) != cudaSuccess) return B2Q_ERR_CUDA;
  if (cudaMemset(p, 0, sizeof(int)) != cudaSuccess) return B2Q_ERR_CUDA;
  if (cudaGetSymbolAddress(&p, g_w4i_counters) != cudaSuccess) return B2Q_ERR_CUDA;
  return cuda_status(cudaMemset(p, 0, sizeof(int) * W4I_BANKS * W4I_MAX_STRIPS));
}
int w4i_read_status(int* out) { return cuda_status(cudaMemcpyFromSymbol(out, g_w4i_status, sizeof(int))); }

}  // namespace b2q
