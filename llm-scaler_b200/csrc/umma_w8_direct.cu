// FP8-weight decode GEMM without any weight conversion:  out[m, n] = s_w[n] * sum_k w_q[n, k] * x[m, k].
//
// The e4m3 / e5m2 weights go from TMA straight into the tensor core (tcgen05.mma kind::f8f6f4, K = 32 per
// instruction).  That MMA kind wants both operands in an 8-bit format, while the activations are 16-bit and
// have to stay exact.  So a pre-pass splits every activation row into a short sum of e4m3 terms,
//     x * 2^e  =  t0 + t1 / 16 (+ t2 / 256),
// each term holding the next four significant bits (two terms cover bf16's eight bits, three cover fp16's
// eleven), and stacks the terms as extra token columns of the MMA's N dimension: N = terms x M.  An MMA with
// N <= 64 costs the same 45 cycles whatever N is, so the extra columns are free, every product is exact in
// the fp32 accumulator, and the epilogue adds the term columns of a token with their powers of two.
// Compared with dequantising the weights to 16 bit this needs half the MMA instructions per byte of weight
// (K = 32 instead of 16), no conversion warps and no operand staging in tensor memory: the kernel is a TMA
// producer, an MMA issuer and an epilogue.
//
// Reference counterpart: the per-channel / per-tensor FP8 GEMV and GEMM of
// vllm/custom-esimd-kernels-vllm/csrc/xpu/esimd_kernels.sycl (esimd_gemv_fp8_pern, esimd_gemv_fp8_pert,
// esimd_gemm_fp8_pern), which dequantise in registers and keep the activation in 16 bit.
#include <atomic>
#include "umma_gemm.cuh"
#include "sm100.cuh"

namespace b2q {

using namespace sm100;

__device__ int g_w8d_status = 0;

// Arrival counters of strips that are cut between CTAs: zero whenever no launch is in flight (the last
// arriver of a strip resets its counter); launches take one of 64 banks in turn so that launches that
// overlap in time (other streams, programmatic dependent launch) never share counters.
constexpr int W8D_BANKS = 64, W8D_MAX_STRIPS = 2048;
__device__ int g_w8d_counters[W8D_BANKS * W8D_MAX_STRIPS];

namespace w8d {
enum { ST_FULL = 301, ST_EMPTY = 302, ST_ACCUM = 303, ST_ACCEMPTY = 304, ST_FIXUP = 305 };

template <int NTOK> struct Cfg {
  static constexpr int W_BYTES = 16384;                                 // up to 128 rows x 128 k
  static constexpr int X_BYTES = NTOK * 128;
  static constexpr int STAGE = W_BYTES + X_BYTES;
  // measured: two CTAs per SM with about 100 KB of ring each stream fastest and leave room for the CTAs of the
  // next launch to start (programmatic dependent launch) while this one drains
  static constexpr int NS = NTOK <= 16 ? 6 : (NTOK == 32 ? 5 : (NTOK == 64 ? 4 : (NTOK == 128 ? 3 : 4)));
  static constexpr int SMEM = NS * STAGE + 1024 + 256;
  static constexpr int CTAS = NTOK <= 128 ? 2 : 1;
  static constexpr int ACC_COLS = NTOK < 32 ? 32 : NTOK;                // two accumulators: the epilogue of one segment
  static constexpr int TMEM_COLS = 2 * ACC_COLS;                        // runs under the MMAs of the next
  static constexpr int THREADS = 7 * 32;                                // W TMA, MMA, X TMA, four epilogue warps
};

// One piece of a CTA's work: stages [st_begin, st_end) of 128 k of the strip of 128 weight rows at n0.
struct Segment { int n0, strip, st_begin, st_end, part, slot, rot; };   // stage order: st_begin + (i + rot) % count
}  // namespace w8d

struct W8DParams {
  const void* scale; int scale_dtype; int scale_per_channel;
  const float* inv_scale;            // [M]: 2^-e of the activation pre-pass
  void* out; int64_t ldo; int out_bf16;
  int M, Mp, NT, N, K;
  int e5m2;
  int sps, ust, units;               // work units: units per strip, stages per unit, units in total
  float* partials;                   // [grid][2 slots][Mp][128] fp32 sums of cut strips (terms already combined)
  int* counters;                     // [strips]
  int h;                             // weight rows per strip (a multiple of 8, at most 128)
  int* status;
};

// A persistent grid of one CTA per SM.  The work, (strips) x (stages of 128 k), is cut into equal contiguous
// runs, so a CTA streams up to two partial strips around any number of whole ones and every SM moves the same
// number of bytes with all of its shared memory as the ring.  A strip that is cut is completed by whichever of
// its CTAs delivers last: it adds the partial sums up in CTA order (so the result does not depend on who that
// is) and writes the output.  Nobody waits for another CTA.
template <int NTOK>
__global__ void __launch_bounds__(w8d::Cfg<NTOK>::THREADS, w8d::Cfg<NTOK>::CTAS)
umma_w8_direct_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x, const W8DParams p) {
  using C = w8d::Cfg<NTOK>;
  using namespace w8d;
  constexpr int NS = C::NS;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bar = base + NS * C::STAGE;
  const uint32_t full = bar, empty = bar + 8 * NS, accum_full = bar + 16 * NS, accum_empty = accum_full + 16;
  const uint32_t fix_bar = accum_empty + 16;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen + (fix_bar + 8 - base));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + (fix_bar + 16 - base));
  volatile int* last_flag = reinterpret_cast<volatile int*>(gen + (fix_bar + 20 - base));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nst = (p.K + 127) >> 7;

  // the next kernel of the stream may start; this one waits for its predecessors only before it reads activations
  grid_dep_release();

  // every role walks the same list of segments with its own copy of this cursor
  const int u0 = (int)((int64_t)blockIdx.x * p.units / gridDim.x), u1 = (int)((int64_t)(blockIdx.x + 1) * p.units / gridDim.x);
  int u = u0;
  auto next_segment = [&](Segment& sg) -> bool {
    if (u >= u1) return false;
    const int strip = u / p.sps, r0 = u - strip * p.sps;
    const int take = min(p.sps - r0, u1 - u);
    sg.strip = strip; sg.n0 = strip * p.h;
    sg.st_begin = r0 * p.ust; sg.st_end = min(nst, (r0 + take) * p.ust);
    sg.part = take != p.sps; sg.slot = (u == u0) ? 0 : 1;
    // Every CTA starts at a different stage: all CTAs read the same small activation array, and in step they would
    // all ask the same L2 lines for it at the same moment.
    sg.rot = (int)((blockIdx.x * 5u + (unsigned)strip) % (unsigned)(sg.st_end - sg.st_begin));
    u += take;
    return true;
  };

  if (threadIdx.x == 0) {
    for (int i = 0; i < NS; ++i) { mbar_init(full + 8 * i, 2); mbar_init(empty + 8 * i, 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(accum_full + 8 * i, 1); mbar_init(accum_empty + 8 * i, 128); }
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
    // ---- weight producer: one 128 x 128 box per stage ----
    if (lane == 0) {
      tma_prefetch_desc(&tm_w);
      int g = 0;
      bool ok = true;
      while (ok && next_segment(sg)) {
        const int cnt = sg.st_end - sg.st_begin;
        for (int i = 0; i < cnt; ++i, ++g) {
          const int r = sg.st_begin + (i + sg.rot) % cnt;
          const int s = g % NS;
          if (g >= NS && !mbar_wait(empty + 8 * s, ((g / NS) - 1) & 1, abort_flag, p.status, ST_EMPTY)) { ok = false; break; }
          mbar_expect_tx(full + 8 * s, p.h * 128);
          tma_load_2d(base + s * C::STAGE, &tm_w, r * 128, sg.n0, full + 8 * s);
        }
      }
      if (!ok) drain_issued(full, NS, g);
    }
  } else if (warp == 2) {
    // ---- activation producer: the NTOK term rows of the same 128 k ----
    if (lane == 0) {
      tma_prefetch_desc(&tm_x);
      grid_dep_wait();
      int g = 0;
      bool ok = true;
      while (ok && next_segment(sg)) {
        const int cnt = sg.st_end - sg.st_begin;
        for (int i = 0; i < cnt; ++i, ++g) {
          const int r = sg.st_begin + (i + sg.rot) % cnt;
          const int s = g % NS;
          if (g >= NS && !mbar_wait(empty + 8 * s, ((g / NS) - 1) & 1, abort_flag, p.status, ST_EMPTY)) { ok = false; break; }
          mbar_expect_tx(full + 8 * s, C::X_BYTES);
          tma_load_2d(base + s * C::STAGE + C::W_BYTES, &tm_x, r * 128, 0, full + 8 * s);
        }
      }
      if (!ok) drain_issued(full, NS, g);
    }
  } else if (warp == 1) {
    // ---- MMA issuer ----
    if (lane == 0) {
      const uint32_t idesc = instr_desc(p.e5m2 ? 1u : 0u, 0u, 128, NTOK);
      bool ok = true;
      int g = 0, si = 0;
      while (ok && next_segment(sg)) {
        const int buf = si & 1;
        if (si >= 2) { ok = mbar_wait(accum_empty + 8 * buf, ((si >> 1) - 1) & 1, abort_flag, p.status, ST_ACCEMPTY); if (!ok) break; }
        const uint32_t d = tmem + buf * C::ACC_COLS;
#pragma unroll 1
        for (int r = sg.st_begin; r < sg.st_end; ++r, ++g) {
          const int s = g % NS;
          ok = mbar_wait(full + 8 * s, (g / NS) & 1, abort_flag, p.status, ST_FULL);
          if (!ok) break;
          tc_fence_after();
          const uint64_t da = smem_desc_sw128(base + s * C::STAGE);
          const uint64_t db = smem_desc_sw128(base + s * C::STAGE + C::W_BYTES);
          mma_f8(d, da, db, idesc, r > sg.st_begin ? 1u : 0u);
          mma_f8(d, da + 2, db + 2, idesc, 1u);
          mma_f8(d, da + 4, db + 4, idesc, 1u);
          mma_f8(d, da + 6, db + 6, idesc, 1u);
          tc_commit(empty + 8 * s);
        }
        if (ok) tc_commit(accum_full + 8 * buf);
        ++si;
      }
    }
  } else {
    // ---- epilogue: warps 3..6, lane quadrant = warp & 3; a thread owns one weight row ----
    const int quad = warp & 3, rowi = quad * 32 + lane;
    uint16_t* outp = reinterpret_cast<uint16_t*>(p.out);
    bool ok = true;
    int si = 0, fixn = 0;
    while (ok && next_segment(sg)) {
      const int buf = si & 1;
      ok = mbar_wait(accum_full + 8 * buf, (si >> 1) & 1, abort_flag, p.status, ST_ACCUM);
      if (!ok) break;
      tc_fence_after();
      const int n = sg.n0 + rowi;
      const int nn = n < p.N ? n : p.N - 1;
      const float sw = load_scalar(p.scale, p.scale_per_channel ? nn : 0, p.scale_dtype);
      const uint32_t trow = tmem + ((uint32_t)(quad * 32) << 16) + buf * C::ACC_COLS;
      float* const my_part = p.partials + ((size_t)(blockIdx.x * 2 + sg.slot) * p.Mp) * 128 + rowi;
      auto write_out = [&](const float (&v)[8], int m0) {
        // token scales of this block of eight: one load per lane, past L1 (it may still hold the previous call's
        // scales at this address), handed round the warp by shuffle
        float ts_lane = 1.f;
        if (lane < 8 && m0 + lane < p.M) ts_lane = __ldcg(p.inv_scale + m0 + lane);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float ts = __shfl_sync(0xffffffffu, ts_lane, i);
          const int m = m0 + i;
          if (m < p.M && n < p.N && rowi < p.h) {
            const float o = v[i] * sw * ts;
            outp[(int64_t)m * p.ldo + n] = p.out_bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(o)) : __half_as_ushort(__float2half_rn(o));
          }
        }
      };
#pragma unroll 1
      for (int m0 = 0; m0 < p.M; m0 += 8) {
        uint32_t a[8], b[8], c[8];
        tmem_ld8(trow + m0, a);
        tmem_ld8(trow + p.Mp + m0, b);
        if (p.NT == 3) tmem_ld8(trow + 2 * p.Mp + m0, c);
        tmem_ld_wait();
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          v[i] = __uint_as_float(a[i]) + __uint_as_float(b[i]) * 0.0625f;
          if (p.NT == 3) v[i] += __uint_as_float(c[i]) * 0.00390625f;
        }
        if (!sg.part) {
          write_out(v, m0);
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) __stcg(my_part + (m0 + i) * 128, v[i]);
        }
      }
      tc_fence_before();
      mbar_arrive(accum_empty + 8 * buf);          // the MMAs of the segment after next may overwrite this accumulator
      if (sg.part) {
        const int64_t U = p.units, G = gridDim.x;
        const int64_t us = (int64_t)sg.strip * p.sps, ue = us + p.sps - 1;
        const int b_lo = (int)(((us + 1) * G + U - 1) / U) - 1, b_hi = (int)(((ue + 1) * G + U - 1) / U) - 1;
        mbar_arrive(fix_bar);          // hands this thread's partial sums to the leader, whose fence orders them before the count
        ok = mbar_wait(fix_bar, fixn & 1, abort_flag, p.status, ST_FIXUP); ++fixn;
        if (!ok) break;
        if (threadIdx.x == 3 * 32) {
          __threadfence();                             // orders the partial sums of all 128 threads before the count
          const int old = atomicAdd(p.counters + sg.strip, 1);
          const int last = old == b_hi - b_lo;
          if (last) p.counters[sg.strip] = 0;        // every contributor has arrived: ready for the next launch
          *last_flag = last;
        }
        mbar_arrive(fix_bar);
        ok = mbar_wait(fix_bar, fixn & 1, abort_flag, p.status, ST_FIXUP); ++fixn;
        if (!ok) break;
        if (*last_flag) {
          __threadfence();
#pragma unroll 1
          for (int m0 = 0; m0 < p.M; m0 += 8) {
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = 0.f;
            for (int b = b_lo; b <= b_hi; ++b) {
              const int64_t bu0 = (int64_t)b * U / G;
              const float* src = p.partials + ((size_t)(b * 2 + (bu0 >= us ? 0 : 1)) * p.Mp) * 128 + rowi;
#pragma unroll
              for (int i = 0; i < 8; ++i) v[i] += __ldcg(src + (m0 + i) * 128);
            }
            write_out(v, m0);
          }
        }
      }
      ++si;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, C::TMEM_COLS); }
}

// Term rows the pre-pass writes for M tokens: terms x (M rounded up to 8), rounded up to a legal MMA N.
int umma_w8_direct_rows(int64_t M, bool bf16) {
  const int mp = (int)((M + 7) / 8 * 8), need = (bf16 ? 2 : 3) * mp;
  return need <= 16 ? 16 : (need <= 32 ? 32 : (need <= 64 ? 64 : (need <= 128 ? 128 : 256)));
}

static int sm_count() {
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

static int* w8d_counter_bank() {
  static thread_local int* basep[16] = {nullptr};
  static std::atomic<unsigned> next_bank{0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 16) return nullptr;
  if (!basep[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_w8d_counters) != cudaSuccess) return nullptr;
    basep[dev] = reinterpret_cast<int*>(p);
  }
  return basep[dev] + (size_t)(next_bank.fetch_add(1, std::memory_order_relaxed) % W8D_BANKS) * W8D_MAX_STRIPS;
}

// fp32 partial sums: [up to two CTAs per SM][2 slots][M rounded up to 8][128 rows]
size_t umma_w8_direct_partial_bytes(int64_t M) {
  return (size_t)sm_count() * 2 * 2 * (size_t)((M + 7) / 8 * 8) * 128 * sizeof(float);
}

// Rows per strip (a multiple of 8 up to 128) that minimise the rows the busiest SM has to stream when the
// strips are dealt out evenly; ties go to the taller strip.
static int pick_strip_rows(int N, int sms) {
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
static int launch_direct(const CUtensorMap& tw, const CUtensorMap& tx, const W8DParams& p, int grid, bool overlap, cudaStream_t st) {
  using C = w8d::Cfg<NTOK>;
  auto kern = umma_w8_direct_kernel<NTOK>;
  static thread_local bool configured[16] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 16 || !configured[dev]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM) != cudaSuccess) return B2Q_ERR_CUDA;
    if (dev < 16) configured[dev] = true;
  }
  if (launch_overlapped(kern, dim3(grid), dim3(C::THREADS), C::SMEM, st, overlap, tw, tx, p) != cudaSuccess) return B2Q_ERR_CUDA;
  note_launch("umma_w8_direct");
  return launch_status();
}

int umma_w8_direct_linear(const UmmaW8DirectArgs& a, cudaStream_t st) {
  if (a.M <= 0 || a.M > 80 || (a.K % 16) != 0) return B2Q_ERR_SHAPE;
  if (!tensor_map_encoder()) return B2Q_ERR_CUDA;
  const int ntok = umma_w8_direct_rows(a.M, a.terms == 2);
  CUtensorMap tw, tx;
  int rc = make_tmap_2d(&tx, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.xq, ntok, a.K, (uint64_t)a.K, ntok, 128, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  W8DParams p{};
  p.scale = a.scale; p.scale_dtype = a.scale_dtype; p.scale_per_channel = a.scale_mode == B2Q_SCALE_CHANNEL ? 1 : 0;
  p.inv_scale = a.inv_scale; p.out = a.out; p.ldo = a.ldo; p.out_bf16 = a.out_bf16 ? 1 : 0;
  p.M = a.M; p.Mp = (a.M + 7) / 8 * 8; p.NT = a.terms; p.N = a.N; p.K = a.K; p.e5m2 = a.fmt == B2Q_E5M2;
  void* sym = nullptr;
  if (cudaGetSymbolAddress(&sym, g_w8d_status) != cudaSuccess) return B2Q_ERR_CUDA;
  p.status = reinterpret_cast<int*>(sym);
  const int sms = sm_count(), slots = sms * (ntok <= 128 ? 2 : 1), nst = (a.K + 127) / 128;
  // Few rows (less than one strip for every other SM): strips of 128 rows are cut along k into equal runs, which
  // needs the scratch for partial sums.  Otherwise one CTA per strip, and the strip height is chosen so that the
  // SMs end up with equal numbers of rows: the MMA always works on 128 rows, a lower strip just loads fewer.
  const bool cut = ((a.N + 127) / 128) * 2 <= sms && a.partials && a.partial_bytes >= umma_w8_direct_partial_bytes(a.M);
  p.h = cut ? 128 : pick_strip_rows(a.N, sms);
  const int strips = (a.N + p.h - 1) / p.h;
  rc = make_tmap_2d(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.w, a.N, a.K, (uint64_t)a.K, p.h, 128, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  p.ust = cut ? 1 : nst; p.sps = cut ? nst : 1; p.units = strips * p.sps;
  p.partials = reinterpret_cast<float*>(a.partials);
  p.counters = cut ? w8d_counter_bank() : nullptr;
  if (cut && !p.counters) return B2Q_ERR_CUDA;
  const int grid = cut ? (p.units < slots ? p.units : slots) : strips;
  const bool overlap = tls().overlap_mode > 0;     // always directly behind its own pre-pass
  switch (ntok) {
    case 16: return launch_direct<16>(tw, tx, p, grid, overlap, st);
    case 32: return launch_direct<32>(tw, tx, p, grid, overlap, st);
    case 64: return launch_direct<64>(tw, tx, p, grid, overlap, st);
    case 128: return launch_direct<128>(tw, tx, p, grid, overlap, st);
    default: return launch_direct<256>(tw, tx, p, grid, overlap, st);
  }
}

int w8d_reset_state() {
  void* p = nullptr;
  if (cudaGetSymbolAddress(&p, g_w8d_status) != cudaSuccess) return B2Q_ERR_CUDA;
  if (cudaMemset(p, 0, sizeof(int)) != cudaSuccess) return B2Q_ERR_CUDA;
  if (cudaGetSymbolAddress(&p, g_w8d_counters) != cudaSuccess) return B2Q_ERR_CUDA;
  return cuda_status(cudaMemset(p, 0, sizeof(int) * W8D_BANKS * W8D_MAX_STRIPS));
}
int w8d_read_status(int* out) { return cuda_status(cudaMemcpyFromSymbol(out, g_w8d_status, sizeof(int))); }

}  // namespace b2q
