// W8A8 block-scaled FP8 GEMM on tcgen05:  out[tok, n] = sum_kb xs[tok, kb] * ws[n/128, kb] * (xq[tok, kb-block] . wq[n, kb-block]).
//
// Both operands are e4m3 and go from TMA straight into the tensor core (kind::f8f6f4, K = 32 per
// instruction); nothing is dequantised in shared memory.  The hardware block-scaling MMA only takes
// power-of-two scales, while these scales are arbitrary fp32 (amax / 448), so every 128-deep K block is
// accumulated into its own tensor-memory buffer and promoted by the epilogue warps:
// acc[n, tok] += partial[n, tok] * xs[tok, kb] * ws[n/128, kb] in fp32 registers, while the MMA already
// works on the next K blocks (four accumulator buffers rotate through the 512 TMEM columns).
// The 128 weight rows of a strip are the MMA's M dimension, a 128-token tile its N dimension, so
// ws is one scalar per (CTA, kb) and the scale varies only along the columns a thread owns.
//
// Reference counterpart: the block-scaled linear of vllm/patches/vllm_for_multi_arc.patch:2651-2691 with the
// (1,128) dynamic activation quantisation its capability key asks for (:2628-2634); the reference itself
// keeps the activation in 16 bit, which b2q_linear_fp8 reproduces.
#include "umma_gemm.cuh"
#include "sm100.cuh"

namespace b2q {

using namespace sm100;

__device__ int g_w8a8_status = 0;

namespace w8a8 {
constexpr int THREADS = 64 + 512;   // TMA warp, MMA warp, 16 promotion / epilogue warps (4 lane quadrants x 4 column groups)
constexpr int MAX_KB = 128;         // K <= 16384
enum { ST_FULL = 201, ST_EMPTY = 202, ST_ACCFULL = 203, ST_ACCEMPTY = 204 };

// TOK = token tile (MMA N), 128 or 256.  Measured on B200 at [4096 x 17408 x 5120]: 128 -> 1.21 PFLOP/s, 256 ->
// 1.13 PFLOP/s (only two accumulator buffers fit, so MMA and promotion overlap less); 128 is what is launched.
template <int TOK> struct Cfg {
  static constexpr int NBUF = 512 / TOK;                     // accumulator buffers of TOK columns (all of tensor memory)
  static constexpr int STAGE_BYTES = 16384 + TOK * 128;      // one K block of W + one of X
  static constexpr int S = TOK == 128 ? 4 : 3;               // operand stages
  static constexpr int CPT = TOK / 4;                        // token columns per promotion thread
  static constexpr int SC_PITCH = TOK + 4;   // scale-table row pitch in floats: float4 rows stay aligned, transposing writes spread over banks
  static constexpr int smem_bytes(int nkb) { return S * STAGE_BYTES + nkb * SC_PITCH * 4 + 1024 + 256; }
};
}  // namespace w8a8

struct W8A8Params {
  const float* xs; const float* ws;     // [M, K/128], [ceil(N/128), K/128]
  void* out; int64_t ldo; int out_bf16;
  int M, N, K;
  int* status;
};

template <int TOK>
__global__ void __launch_bounds__(w8a8::THREADS, 1)
umma_w8a8_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x, const W8A8Params p) {
  using namespace w8a8;
  using C = Cfg<TOK>;
  constexpr int S = C::S, NBUF = C::NBUF, STAGE_BYTES = C::STAGE_BYTES, SC_PITCH = C::SC_PITCH, CPT = C::CPT;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  const int nkb = p.K >> 7;
  // layout: [S stages of (W tile, X tile)] [scale table nkb x SC_PITCH fp32] [barriers]
  const uint32_t sc_off = S * STAGE_BYTES;
  float* sc = reinterpret_cast<float*>(gen + sc_off);
  const uint32_t bar = base + sc_off + nkb * SC_PITCH * 4;
  const uint32_t full = bar, empty = bar + 8 * S, acc_full = bar + 16 * S, acc_empty = acc_full + 8 * NBUF;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen + (acc_empty + 8 * NBUF - base));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + (acc_empty + 8 * NBUF + 8 - base));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tok0 = blockIdx.x * TOK, n0 = blockIdx.y * 128;

  if (threadIdx.x == 0) {
    for (int i = 0; i < S; ++i) { mbar_init(full + 8 * i, 1); mbar_init(empty + 8 * i, 1); }
    for (int i = 0; i < NBUF; ++i) { mbar_init(acc_full + 8 * i, 1); mbar_init(acc_empty + 8 * i, 16); }   // one arrival per promotion warp
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tm_w);
      tma_prefetch_desc(&tm_x);
      int kb = 0;
      for (; kb < nkb; ++kb) {
        const int s = kb % S;
        if (kb >= S && !mbar_wait(empty + 8 * s, ((kb / S) - 1) & 1, abort_flag, p.status, ST_EMPTY)) break;
        mbar_expect_tx(full + 8 * s, STAGE_BYTES);
        tma_load_2d(base + s * STAGE_BYTES, &tm_w, kb * 128, n0, full + 8 * s);
        tma_load_2d(base + s * STAGE_BYTES + 16384, &tm_x, kb * 128, tok0, full + 8 * s);
      }
      if (kb < nkb) drain_issued(full, S, kb);       // gave up: let the copies already issued land first
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc(0u, 0u, 128, TOK);       // e4m3 x e4m3 -> fp32
      for (int kb = 0; kb < nkb; ++kb) {
        const int s = kb % S, b = kb % NBUF;
        if (!mbar_wait(full + 8 * s, (kb / S) & 1, abort_flag, p.status, ST_FULL)) break;
        if (kb >= NBUF && !mbar_wait(acc_empty + 8 * b, ((kb / NBUF) - 1) & 1, abort_flag, p.status, ST_ACCEMPTY)) break;
        tc_fence_after();
        const uint64_t da = smem_desc_sw128(base + s * STAGE_BYTES);
        const uint64_t db = smem_desc_sw128(base + s * STAGE_BYTES + 16384);
        const uint32_t d = tmem + b * TOK;
        mma_f8(d, da, db, idesc, 0u);
        mma_f8(d, da + 2, db + 2, idesc, 1u);
        mma_f8(d, da + 4, db + 4, idesc, 1u);
        mma_f8(d, da + 6, db + 6, idesc, 1u);
        tc_commit(empty + 8 * s);
        tc_commit(acc_full + 8 * b);
      }
    }
  } else {
    // ---- promotion + epilogue: 16 warps, lane quadrant = warp & 3, column group = (warp - 2) >> 2 ----
    // A thread owns one weight row and CPT token columns.
    const int quad = warp & 3, cgroup = (warp - 2) >> 2;
    const int col0 = cgroup * CPT;
    // Combined scale table sc[kb][t] = xs[tok0 + t, kb] * ws[n0 / 128, kb], built by the 512 promotion threads while
    // the TMA and MMA warps already run ahead: consecutive threads read consecutive kb of one token (coalesced), four
    // independent loads in flight per thread.
    {
      const int total = nkb * TOK, ptid = threadIdx.x - 64;
      const float* wsrow = p.ws + (int64_t)(n0 >> 7) * nkb;
#pragma unroll 4
      for (int i = ptid; i < total; i += 512) {
        const int kb = i % nkb, t = i / nkb;
        const int tok = tok0 + t;
        sc[kb * SC_PITCH + t] = tok < p.M ? __ldg(p.xs + (int64_t)tok * nkb + kb) * __ldg(wsrow + kb) : 0.f;
      }
      asm volatile("bar.sync 1, 512;" ::: "memory");
    }
    float acc[CPT];
#pragma unroll
    for (int i = 0; i < CPT; ++i) acc[i] = 0.f;
    bool ok = true;
#pragma unroll 1
    for (int kb = 0; kb < nkb; ++kb) {
      const int b = kb % NBUF;
      ok = mbar_wait(acc_full + 8 * b, (kb / NBUF) & 1, abort_flag, p.status, ST_ACCFULL);
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int h = 0; h < CPT / 32; ++h) {
        uint32_t r0[32];
        tmem_ld32(tmem + ((uint32_t)(quad * 32) << 16) + b * TOK + col0 + h * 32, r0);
        tmem_ld_wait();
        if (h == CPT / 32 - 1) {
          // the buffer may be overwritten while the FMAs run
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(acc_empty + 8 * b);
        }
        const float4* s4 = reinterpret_cast<const float4*>(sc + kb * SC_PITCH + col0 + h * 32);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float4 v = s4[i];
          acc[h * 32 + 4 * i + 0] = fmaf(__uint_as_float(r0[4 * i + 0]), v.x, acc[h * 32 + 4 * i + 0]);
          acc[h * 32 + 4 * i + 1] = fmaf(__uint_as_float(r0[4 * i + 1]), v.y, acc[h * 32 + 4 * i + 1]);
          acc[h * 32 + 4 * i + 2] = fmaf(__uint_as_float(r0[4 * i + 2]), v.z, acc[h * 32 + 4 * i + 2]);
          acc[h * 32 + 4 * i + 3] = fmaf(__uint_as_float(r0[4 * i + 3]), v.w, acc[h * 32 + 4 * i + 3]);
        }
      }
    }
    if (ok) {
      const int n = n0 + quad * 32 + lane;
      if (n < p.N) {
        uint16_t* outp = reinterpret_cast<uint16_t*>(p.out);
#pragma unroll
        for (int i = 0; i < CPT; ++i) {
          const int tok = tok0 + col0 + i;
          if (tok < p.M)
            outp[(int64_t)tok * p.ldo + n] = p.out_bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(acc[i]))
                                                        : __half_as_ushort(__float2half_rn(acc[i]));
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

// ------------------------------------------------------------------------------------------------
// CTA-pair variant: two CTAs of a cluster own two neighbouring weight strips (256 rows) and ONE token tile of 128.
// tcgen05.mma cta_group::2 multiplies the pair's 256 x 128 tile in one instruction: each CTA contributes its own
// 128 weight rows as A and its own half (64 tokens) of the activation tile as B, and receives its 128 rows of the
// result in its own tensor memory.  A CTA therefore loads 16 KB of W + 8 KB of X per K block instead of 16 + 16:
// a quarter less operand traffic from L2 per flop.
// Status: parity-tested, opt-in (b2q_set_force_kernel(6)).  Measured on B200 at [4096 x 17408 x 5120]: 667 TFLOP/s
// against 1.21 PFLOP/s for the single-CTA kernel: with one accumulator per K block, every block's hand-back now
// crosses between the two SMs (remote arrivals on the leader's barrier, commit to both CTAs) and the four
// accumulator buffers cover that longer round trip even less than they cover the local one.  The pairing itself
// (cluster launch, pair allocation of tensor memory, 2-CTA loads and MMA) is what a plain GEMM without per-block
// promotion would reuse.
// Only completion signals cross between the CTAs (no multicast load): both CTAs' TMA loads count their bytes on the
// leader's `full` barrier, the leader's tcgen05.commit releases the stage and publishes the accumulator in both CTAs,
// and the promotion warps of both CTAs hand the accumulator back on the leader's `acc_empty` barrier.
namespace w8a8 {
constexpr int PAIR_STAGE = 16384 + 8192;     // per CTA: 128 rows of W + 64 tokens of X, one K block
constexpr int PAIR_S = 5;
constexpr int PAIR_PITCH = 128 + 4;
constexpr int pair_smem_bytes(int nkb) { return PAIR_S * PAIR_STAGE + nkb * PAIR_PITCH * 4 + 1024 + 256; }
}  // namespace w8a8

__global__ void __launch_bounds__(w8a8::THREADS, 1)
umma_w8a8_pair_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x, const W8A8Params p) {
  using namespace w8a8;
  constexpr int TOK = 128, NBUF = 4, S = PAIR_S, SC_PITCH = PAIR_PITCH;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  const int nkb = p.K >> 7;
  const uint32_t sc_off = S * PAIR_STAGE;
  float* sc = reinterpret_cast<float*>(gen + sc_off);
  const uint32_t bar = base + sc_off + nkb * SC_PITCH * 4;
  const uint32_t full = bar, empty = bar + 8 * S, acc_full = bar + 16 * S, acc_empty = acc_full + 8 * NBUF;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen + (acc_empty + 8 * NBUF - base));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + (acc_empty + 8 * NBUF + 8 - base));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();           // 0 = leader (issues the MMAs), 1 = peer
  // CTA pairs are formed along x: blockIdx.x = 2 * token tile + rank, blockIdx.y = pair of strips, so that neighbouring
  // clusters share their weight strips (as neighbouring CTAs do in the single-CTA kernel)
  const int tok0 = (int)(blockIdx.x >> 1) * TOK, n0 = (int)(2 * blockIdx.y + rank) * 128;

  if (threadIdx.x == 0) {
    for (int i = 0; i < S; ++i) { mbar_init(full + 8 * i, 1); mbar_init(empty + 8 * i, 1); }
    for (int i = 0; i < NBUF; ++i) { mbar_init(acc_full + 8 * i, 1); mbar_init(acc_empty + 8 * i, 32); }   // 16 warps x 2 CTAs
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512); tmem_relinquish_pair(); }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();              // both CTAs' barriers exist before anything is signalled across
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    // ---- producer (both CTAs): own W rows + own half of the token tile; bytes counted on the leader's barrier ----
    if (lane == 0) {
      tma_prefetch_desc(&tm_w);
      tma_prefetch_desc(&tm_x);
      for (int kb = 0; kb < nkb; ++kb) {
        const int s = kb % S;
        if (kb >= S && !mbar_wait(empty + 8 * s, ((kb / S) - 1) & 1, abort_flag, p.status, ST_EMPTY)) break;
        const uint32_t lead_full = map_to_cta(full + 8 * s, 0);
        if (rank == 0) mbar_expect_tx(full + 8 * s, 2 * PAIR_STAGE);
        tma_load_2d_pair(base + s * PAIR_STAGE, &tm_w, kb * 128, n0, lead_full);
        tma_load_2d_pair(base + s * PAIR_STAGE + 16384, &tm_x, kb * 128, tok0 + (int)rank * 64, lead_full);
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer: the leader's one thread drives both CTAs' tensor cores ----
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = instr_desc(0u, 0u, 256, TOK);
      for (int kb = 0; kb < nkb; ++kb) {
        const int s = kb % S, b = kb % NBUF;
        if (!mbar_wait(full + 8 * s, (kb / S) & 1, abort_flag, p.status, ST_FULL)) break;
        if (kb >= NBUF && !mbar_wait(acc_empty + 8 * b, ((kb / NBUF) - 1) & 1, abort_flag, p.status, ST_ACCEMPTY)) break;
        tc_fence_after();
        const uint64_t da = smem_desc_sw128(base + s * PAIR_STAGE);
        const uint64_t db = smem_desc_sw128(base + s * PAIR_STAGE + 16384);
        const uint32_t d = tmem + b * TOK;
        mma_f8_pair(d, da, db, idesc, 0u);
        mma_f8_pair(d, da + 2, db + 2, idesc, 1u);
        mma_f8_pair(d, da + 4, db + 4, idesc, 1u);
        mma_f8_pair(d, da + 6, db + 6, idesc, 1u);
        tc_commit_pair(empty + 8 * s, 3);
        tc_commit_pair(acc_full + 8 * b, 3);
      }
    }
  } else {
    // ---- promotion + epilogue, as in the single-CTA kernel, on this CTA's 128 rows ----
    const int quad = warp & 3, cgroup = (warp - 2) >> 2;
    const int col0 = cgroup * 32;
    {
      const int total = nkb * TOK, ptid = threadIdx.x - 64;
      const float* wsrow = p.ws + (int64_t)(n0 >> 7) * nkb;
#pragma unroll 4
      for (int i = ptid; i < total; i += 512) {
        const int kb = i % nkb, t = i / nkb;
        const int tok = tok0 + t;
        sc[kb * SC_PITCH + t] = tok < p.M ? __ldg(p.xs + (int64_t)tok * nkb + kb) * __ldg(wsrow + kb) : 0.f;
      }
      asm volatile("bar.sync 1, 512;" ::: "memory");
    }
    float acc[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) acc[i] = 0.f;
    bool ok = true;
#pragma unroll 1
    for (int kb = 0; kb < nkb; ++kb) {
      const int b = kb % NBUF;
      ok = mbar_wait(acc_full + 8 * b, (kb / NBUF) & 1, abort_flag, p.status, ST_ACCFULL);
      if (!ok) break;
      tc_fence_after();
      uint32_t r0[32];
      tmem_ld32(tmem + ((uint32_t)(quad * 32) << 16) + b * TOK + col0, r0);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(acc_empty + 8 * b, 0));   // always on the leader's barrier
      const float4* s4 = reinterpret_cast<const float4*>(sc + kb * SC_PITCH + col0);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float4 v = s4[i];
        acc[4 * i + 0] = fmaf(__uint_as_float(r0[4 * i + 0]), v.x, acc[4 * i + 0]);
        acc[4 * i + 1] = fmaf(__uint_as_float(r0[4 * i + 1]), v.y, acc[4 * i + 1]);
        acc[4 * i + 2] = fmaf(__uint_as_float(r0[4 * i + 2]), v.z, acc[4 * i + 2]);
        acc[4 * i + 3] = fmaf(__uint_as_float(r0[4 * i + 3]), v.w, acc[4 * i + 3]);
      }
    }
    if (ok) {
      const int n = n0 + quad * 32 + lane;
      if (n < p.N) {
        uint16_t* outp = reinterpret_cast<uint16_t*>(p.out);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int tok = tok0 + col0 + i;
          if (tok < p.M)
            outp[(int64_t)tok * p.ldo + n] = p.out_bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(acc[i]))
                                                        : __half_as_ushort(__float2half_rn(acc[i]));
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();              // neither CTA leaves (or frees tensor memory) while its partner may still signal it
  if (warp == 1) { tc_fence_after(); tmem_dealloc_pair(tmem, 512); }
}

static int launch_w8a8_pair(const UmmaW8A8Args& a, const W8A8Params& p, cudaStream_t st) {
  using namespace w8a8;
  CUtensorMap tw, tx;
  int rc = make_tmap_2d(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.w, a.N, a.K, (uint64_t)a.K, 128, 128, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  rc = make_tmap_2d(&tx, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.xq, a.M, a.K, (uint64_t)a.K, 64, 128, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  const int smem = pair_smem_bytes(a.K / 128);
  static thread_local int configured[16] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 16 || configured[dev] < smem) {
    if (cudaFuncSetAttribute(umma_w8a8_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return B2Q_ERR_CUDA;
    if (dev < 16) configured[dev] = smem;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * ((a.M + 127) / 128), ((a.N + 127) / 128) / 2, 1);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, umma_w8a8_pair_kernel, tw, tx, p) != cudaSuccess) return B2Q_ERR_CUDA;
  note_launch("umma_w8a8_pair");
  return launch_status();
}

template <int TOK>
static int launch_w8a8(const UmmaW8A8Args& a, const W8A8Params& p, cudaStream_t st) {
  using namespace w8a8;
  using C = Cfg<TOK>;
  CUtensorMap tw, tx;
  int rc = make_tmap_2d(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.w, a.N, a.K, (uint64_t)a.K, 128, 128, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  rc = make_tmap_2d(&tx, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.xq, a.M, a.K, (uint64_t)a.K, TOK, 128, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  const int smem = C::smem_bytes(a.K / 128);
  static thread_local int configured[16] = {0};      // largest dynamic shared-memory size set so far, per device
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 16 || configured[dev] < smem) {
    if (cudaFuncSetAttribute(umma_w8a8_kernel<TOK>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return B2Q_ERR_CUDA;
    if (dev < 16) configured[dev] = smem;
  }
  dim3 grid((a.M + TOK - 1) / TOK, (a.N + 127) / 128, 1);
  umma_w8a8_kernel<TOK><<<grid, THREADS, smem, st>>>(tw, tx, p);
  note_launch("umma_w8a8");
  return launch_status();
}

int umma_w8a8_block(const UmmaW8A8Args& a, cudaStream_t st) {
  using namespace w8a8;
  if ((a.K % 128) != 0 || a.K / 128 > MAX_KB) return B2Q_ERR_SHAPE;
  if (!tensor_map_encoder()) return B2Q_ERR_CUDA;
  W8A8Params p{};
  p.xs = a.xs; p.ws = a.ws; p.out = a.out; p.ldo = a.ldo; p.out_bf16 = a.bf16 ? 1 : 0;
  p.M = a.M; p.N = a.N; p.K = a.K;
  void* sym = nullptr;
  if (cudaGetSymbolAddress(&sym, g_w8a8_status) != cudaSuccess) return B2Q_ERR_CUDA;
  p.status = reinterpret_cast<int*>(sym);
  const int nkb = a.K / 128;
  if (Cfg<128>::smem_bytes(nkb) > 232448 - 1024) return B2Q_ERR_LIMIT;
  // the CTA-pair kernel needs whole pairs of strips and its scale table beside five stages of shared memory
  const int strips = (a.N + 127) / 128;
  if (tls().force_kernel == 6 && (strips % 2) == 0 && (a.N % 128) == 0 && pair_smem_bytes(a.K / 128) <= 232448 - 1024)
    return launch_w8a8_pair(a, p, st);
  return launch_w8a8<128>(a, p, st);
}

int w8a8_reset_state() {
  void* p = nullptr;
  if (cudaGetSymbolAddress(&p, g_w8a8_status) != cudaSuccess) return B2Q_ERR_CUDA;
  return cuda_status(cudaMemset(p, 0, sizeof(int)));
}
int w8a8_read_status(int* out) {
  return cuda_status(cudaMemcpyFromSymbol(out, g_w8a8_status, sizeof(int)));
}

}  // namespace b2q
