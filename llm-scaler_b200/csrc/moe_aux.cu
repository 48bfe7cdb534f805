// MoE routing / permutation / activation / combine kernels and the dynamic
// 1x128 activation quantiser.  All are HBM- or latency-bound integer / elementwise
// work; none uses tensor cores.
#include "common.cuh"
#include <cuda_fp8.h>
#include <math.h>

namespace b2q {

// ---------------------------------------------------------------------------
// softmax -> top-k -> renormalise.  One warp per token; lane l owns experts
// l, l+32, ... so loads are coalesced.  Selection order and tie rule follow
// MoE_TopK_V2_Kernel (csrc/xpu/esimd_kernels/moe_ops.h:106-219): k rounds of
// "global maximum, lowest index among bit-equal maxima, then mark as taken".
// ---------------------------------------------------------------------------
template <int PER_LANE>
__global__ void moe_topk_kernel(const void* __restrict__ logits, int ldt, int64_t T, int E, int top_k, int renorm,
                                void* __restrict__ weights, int wdt, int32_t* __restrict__ ids) {
  const int warps_per_block = blockDim.x >> 5;
  const int64_t tok = (int64_t)blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (tok >= T) return;
  float v[PER_LANE];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < PER_LANE; ++j) {
    const int e = lane + 32 * j;
    v[j] = e < E ? load_scalar(logits, tok * E + e, ldt) : -INFINITY;
    mx = fmaxf(mx, v[j]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < PER_LANE; ++j) {
    const int e = lane + 32 * j;
    v[j] = e < E ? expf(v[j] - mx) : 0.f;
    sum += v[j];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float inv = 1.0f / sum;
#pragma unroll
  for (int j = 0; j < PER_LANE; ++j) {
    const int e = lane + 32 * j;
    v[j] = e < E ? v[j] * inv : -2.f;
  }
  float tv = 0.f;   // lane r keeps the r-th selected probability
  int ti = 0;
  float tsum = 0.f;
  for (int r = 0; r < top_k; ++r) {
    float bv = -3.f;
    int bi = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < PER_LANE; ++j) {
      const int e = lane + 32 * j;
      if (v[j] > bv) { bv = v[j]; bi = e; }   // ascending e: first hit is the lowest index
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if ((bi & 31) == lane) {
#pragma unroll
      for (int j = 0; j < PER_LANE; ++j)
        if (lane + 32 * j == bi) v[j] = -1.f;
    }
    if (lane == r) { tv = bv; ti = bi; }
    tsum += bv;
  }
  if (lane < top_k) {
    if (renorm) tv *= (1.0f / tsum);
    store_scalar(weights, tok * top_k + lane, wdt, tv);
    ids[tok * top_k + lane] = ti;
  }
}

int moe_topk(const void* logits, int ldt, int64_t T, int E, int top_k, int renorm, void* weights, int wdt,
             int32_t* ids, cudaStream_t st) {
  const int wpb = 8;
  const int grid = (int)((T + wpb - 1) / wpb);
  if (grid == 0) return B2Q_OK;
#define B2Q_TOPK(P) moe_topk_kernel<P><<<grid, wpb * 32, 0, st>>>(logits, ldt, T, E, top_k, renorm, weights, wdt, ids)
  if (E <= 64) B2Q_TOPK(2);
  else if (E <= 128) B2Q_TOPK(4);
  else if (E <= 256) B2Q_TOPK(8);
  else if (E <= 512) B2Q_TOPK(16);
  else B2Q_TOPK(32);
#undef B2Q_TOPK
  note_launch("moe_topk");
  return launch_status();
}

// ---------------------------------------------------------------------------
// Stable counting sort of (token, slot) pairs by expert.  Three launches:
// per-chunk histogram, prefix over (expert, chunk), stable scatter.  Pair ids
// outside [0, E) are dropped (pair_to_perm = -1): that is how an expert map
// marks experts owned by another rank.
// ---------------------------------------------------------------------------
constexpr int ROUTE_CHUNK = 256;  // pairs per CTA (8 warps)

__global__ void route_hist_kernel(const int32_t* __restrict__ ids, int64_t n_pairs, int E, int32_t* __restrict__ counts) {
  extern __shared__ int32_t sh[];
  for (int i = threadIdx.x; i < E; i += blockDim.x) sh[i] = 0;
  __syncthreads();
  const int64_t i = (int64_t)blockIdx.x * ROUTE_CHUNK + threadIdx.x;
  if (i < n_pairs) {
    const int e = ids[i];
    if (e >= 0 && e < E) atomicAdd(&sh[e], 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) counts[(int64_t)blockIdx.x * E + e] = sh[e];
}

// counts[b][e] -> exclusive running sum over b (in place); expert_offsets[E+1]; rows_per_expert[E].
// One block of 1024 threads: 1024 / E threads share an expert's column of chunk counts, each summing one run of
// chunks, so the dependent chain is nchunks * E / 1024 loads long instead of nchunks.
__global__ void route_prefix_kernel(int32_t* __restrict__ counts, int nchunks, int E, int32_t* __restrict__ expert_offsets,
                                    int32_t* __restrict__ rows_per_expert) {
  __shared__ int32_t part[1024];     // [segment][expert]
  __shared__ int32_t tot[1024];
  __shared__ int32_t scan[1024];
  const int tid = threadIdx.x;
  const int segs = 1024 / E > 0 ? 1024 / E : 1;
  const int e = tid % E, seg = tid / E;
  const bool active = seg < segs;
  const int cps = (nchunks + segs - 1) / segs;
  const int b0 = seg * cps, b1 = min(nchunks, b0 + cps);
  int sum = 0;
  if (active) {
#pragma unroll 4
    for (int b = b0; b < b1; ++b) sum += counts[(int64_t)b * E + e];
    part[seg * E + e] = sum;
  }
  __syncthreads();
  if (active) {
    int run = 0;
    for (int s2 = 0; s2 < seg; ++s2) run += part[s2 * E + e];
#pragma unroll 4
    for (int b = b0; b < b1; ++b) {
      const int c = counts[(int64_t)b * E + e];
      counts[(int64_t)b * E + e] = run;
      run += c;
    }
  }
  int total = 0;
  if (tid < E)
    for (int s2 = 0; s2 < segs; ++s2) total += part[s2 * E + tid];
  tot[tid] = tid < E ? total : 0;
  __syncthreads();
  // Hillis-Steele inclusive scan over 1024 slots
  int val = tot[tid];
  scan[tid] = val;
  __syncthreads();
  for (int off = 1; off < 1024; off <<= 1) {
    const int add = tid >= off ? scan[tid - off] : 0;
    __syncthreads();
    val += add;
    scan[tid] = val;
    __syncthreads();
  }
  if (tid < E) {
    expert_offsets[tid] = val - tot[tid];
    if (rows_per_expert) rows_per_expert[tid] = tot[tid];
    if (tid == E - 1) expert_offsets[E] = val;
  }
}

__global__ void route_scatter_kernel(const int32_t* __restrict__ ids, int64_t n_pairs, int E,
                                     const int32_t* __restrict__ base, const int32_t* __restrict__ expert_offsets,
                                     int32_t* __restrict__ expert_tokens, int32_t* __restrict__ pair_to_perm) {
  extern __shared__ int32_t wc[];  // [8][E] per-warp counts
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < 8 * E; i += blockDim.x) wc[i] = 0;
  __syncthreads();
  const int64_t i = (int64_t)blockIdx.x * ROUTE_CHUNK + threadIdx.x;
  int e = -1;
  if (i < n_pairs) { e = ids[i]; if (e < 0 || e >= E) e = -1; }
  const unsigned peers = __match_any_sync(0xffffffffu, e);
  const int rank = __popc(peers & ((1u << lane) - 1u));
  if (e >= 0 && rank == 0) wc[warp * E + e] = __popc(peers);
  __syncthreads();
  if (i < n_pairs) {
    if (e >= 0) {
      int before = 0;
      for (int w2 = 0; w2 < warp; ++w2) before += wc[w2 * E + e];
      const int pos = expert_offsets[e] + base[(int64_t)blockIdx.x * E + e] + before + rank;
      expert_tokens[pos] = (int32_t)i;
      if (pair_to_perm) pair_to_perm[i] = pos;
    } else if (pair_to_perm) {
      pair_to_perm[i] = -1;
    }
  }
}

size_t moe_route_workspace_bytes(int64_t n_pairs, int E) {
  const int64_t nchunks = (n_pairs + ROUTE_CHUNK - 1) / ROUTE_CHUNK;
  return (size_t)(nchunks > 0 ? nchunks : 1) * (size_t)E * sizeof(int32_t);
}

int moe_route(const int32_t* ids, int64_t n_pairs, int E, int32_t* expert_offsets, int32_t* expert_tokens,
              int32_t* pair_to_perm, int32_t* rows_per_expert, void* workspace, cudaStream_t st) {
  const int nchunks = (int)((n_pairs + ROUTE_CHUNK - 1) / ROUTE_CHUNK);
  int32_t* counts = reinterpret_cast<int32_t*>(workspace);
  if (nchunks > 0) {
    route_hist_kernel<<<nchunks, ROUTE_CHUNK, E * sizeof(int32_t), st>>>(ids, n_pairs, E, counts);
    note_launch("route_hist");
  }
  route_prefix_kernel<<<1, 1024, 0, st>>>(counts, nchunks, E, expert_offsets, rows_per_expert);
  note_launch("route_prefix");
  if (nchunks > 0) {
    route_scatter_kernel<<<nchunks, ROUTE_CHUNK, 8 * E * sizeof(int32_t), st>>>(ids, n_pairs, E, counts, expert_offsets,
                                                                                 expert_tokens, pair_to_perm);
    note_launch("route_scatter");
  }
  return launch_status();
}

// ---------------------------------------------------------------------------
// Tile list for grouped GEMMs: for every expert with rows, ceil(rows/tile) entries
// (expert, first row within the expert).  n_tiles is written to tiles[0].x's
// neighbour: layout = int32 n_tiles, 3 pad ints, then int2 entries.
// ---------------------------------------------------------------------------
__global__ void moe_tiles_kernel(const int32_t* __restrict__ expert_offsets, int E, int tile, int32_t* __restrict__ ws) {
  __shared__ int32_t scan[1024];
  const int e = threadIdx.x;
  const int rows = e < E ? expert_offsets[e + 1] - expert_offsets[e] : 0;
  const int nt = (rows + tile - 1) / tile;
  int val = nt;
  scan[e] = val;
  __syncthreads();
  for (int off = 1; off < 1024; off <<= 1) {
    const int add = e >= off ? scan[e - off] : 0;
    __syncthreads();
    val += add;
    scan[e] = val;
    __syncthreads();
  }
  int2* list = reinterpret_cast<int2*>(ws + 4);
  const int start = val - nt;
  for (int i = 0; i < nt; ++i) list[start + i] = make_int2(e, i * tile);
  if (e == 1023) ws[0] = val;
}

int moe_build_tiles(const int32_t* expert_offsets, int E, int tile, int32_t* ws, cudaStream_t st) {
  moe_tiles_kernel<<<1, 1024, 0, st>>>(expert_offsets, E, tile, ws);
  note_launch("moe_tiles");
  return launch_status();
}

// ---------------------------------------------------------------------------
__global__ void gather_rows_kernel(const uint4* __restrict__ src, const int32_t* __restrict__ idx, int div,
                                   uint4* __restrict__ dst, int64_t rows, int64_t vec_per_row) {
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const int64_t s = idx ? (int64_t)(idx[r] / div) : r;
    for (int64_t c = threadIdx.x; c < vec_per_row; c += blockDim.x) dst[r * vec_per_row + c] = src[s * vec_per_row + c];
  }
}

int gather_rows(const void* src, const int32_t* idx, int div, void* dst, int64_t rows, int64_t cols, int elem_bytes,
                cudaStream_t st) {
  if (rows == 0) return B2Q_OK;
  const int64_t vec = cols * elem_bytes / 16;
  const int grid = (int)(rows < 148 * 32 ? rows : 148 * 32);
  gather_rows_kernel<<<grid, 128, 0, st>>>(reinterpret_cast<const uint4*>(src), idx, div, reinterpret_cast<uint4*>(dst),
                                           rows, vec);
  note_launch("gather_rows");
  return launch_status();
}

// ---------------------------------------------------------------------------
// out[r, j] = act(in[r, j]) * in[r, I + j] in fp32, one rounding.  GELU: the tanh form
// 0.5 g (1 + tanh(sqrt(2/pi) (g + 0.044715 g^3))) of csrc/xpu/esimd_kernels/moe_ops.h:678-723.
template <bool BF16, bool GELU>
__global__ void silu_mul_kernel(const uint4* __restrict__ in, uint4* __restrict__ out, int64_t rows, int64_t I8,
                                const int32_t* __restrict__ out_map, int64_t ld8) {
  using A = Act<BF16>;
  using T = typename A::T;
  const int64_t total = rows * I8;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / I8, c = idx % I8;
    const uint4 g = in[r * ld8 + c];
    const uint4 u = in[r * ld8 + I8 + c];
    const T* gp = reinterpret_cast<const T*>(&g);
    const T* up = reinterpret_cast<const T*>(&u);
    uint4 o;
    T* op = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gv = A::to_f(gp[j]);
      float s;
      if constexpr (GELU) s = 0.5f * gv * (1.0f + tanhf(0.7978845608f * (gv + 0.044715f * gv * gv * gv)));
      else s = gv / (1.0f + expf(-gv));
      op[j] = A::from_f(s * A::to_f(up[j]));
    }
    out[(out_map ? (int64_t)out_map[r] : r) * I8 + c] = o;
  }
}

int silu_mul(const void* in, void* out, int dtype, int64_t rows, int64_t I, const int32_t* out_map, cudaStream_t st,
             int64_t ld_in, bool gelu) {
  if (rows == 0) return B2Q_OK;
  const int64_t ld8 = (ld_in > 0 ? ld_in : 2 * I) / 8;       // source row pitch in 16-byte units
  const int64_t total = rows * (I / 8);
  int64_t g = (total + 255) / 256;
  if (g > 148 * 16) g = 148 * 16;
  auto ci = reinterpret_cast<const uint4*>(in);
  auto co = reinterpret_cast<uint4*>(out);
  if (dtype == B2Q_BF16) {
    if (gelu) silu_mul_kernel<true, true><<<(int)g, 256, 0, st>>>(ci, co, rows, I / 8, out_map, ld8);
    else silu_mul_kernel<true, false><<<(int)g, 256, 0, st>>>(ci, co, rows, I / 8, out_map, ld8);
  } else {
    if (gelu) silu_mul_kernel<false, true><<<(int)g, 256, 0, st>>>(ci, co, rows, I / 8, out_map, ld8);
    else silu_mul_kernel<false, false><<<(int)g, 256, 0, st>>>(ci, co, rows, I / 8, out_map, ld8);
  }
  note_launch(gelu ? "gelu_tanh_mul" : "silu_mul");
  return launch_status();
}

// ---------------------------------------------------------------------------
// Tail of the decode pipeline with a shared expert: out[t, :] = routed[t, :] + sigmoid(x[t, :] . gate_w) * shared[t, :],
// all in fp32 with one rounding.  One CTA per token; out may alias routed.
template <bool BF16>
__global__ void shared_gate_add_kernel(const uint4* __restrict__ x, const uint4* __restrict__ gate_w,
                                       const uint4* __restrict__ shared, const uint4* routed, uint4* out, int H8) {
  using A = Act<BF16>;
  using T = typename A::T;
  __shared__ float red[32];
  __shared__ float gate_sh;
  const int64_t t = blockIdx.x;
  float dot = 0.f;
  for (int c = threadIdx.x; c < H8; c += blockDim.x) {
    const uint4 xv = x[t * H8 + c], gv = gate_w[c];
    const T* xp = reinterpret_cast<const T*>(&xv);
    const T* gp = reinterpret_cast<const T*>(&gv);
#pragma unroll
    for (int j = 0; j < 8; ++j) dot += A::to_f(xp[j]) * A::to_f(gp[j]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = dot;
  __syncthreads();
  if (threadIdx.x == 0) {
    float a = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) a += red[i];
    gate_sh = 1.0f / (1.0f + expf(-a));
  }
  __syncthreads();
  const float gate = gate_sh;
  for (int c = threadIdx.x; c < H8; c += blockDim.x) {
    const uint4 sv = shared[t * H8 + c], rv = routed[t * H8 + c];
    const T* sp = reinterpret_cast<const T*>(&sv);
    const T* rp = reinterpret_cast<const T*>(&rv);
    uint4 o;
    T* op = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int j = 0; j < 8; ++j) op[j] = A::from_f(A::to_f(rp[j]) + gate * A::to_f(sp[j]));
    out[t * H8 + c] = o;
  }
}

int shared_gate_add(const void* x, const void* gate_w, const void* shared, const void* routed, void* out, int dtype,
                    int64_t T, int64_t H, cudaStream_t st) {
  if (T == 0) return B2Q_OK;
  auto u = [](const void* p) { return reinterpret_cast<const uint4*>(p); };
  if (dtype == B2Q_BF16)
    shared_gate_add_kernel<true><<<(unsigned)T, 256, 0, st>>>(u(x), u(gate_w), u(shared), u(routed), reinterpret_cast<uint4*>(out), (int)(H / 8));
  else
    shared_gate_add_kernel<false><<<(unsigned)T, 256, 0, st>>>(u(x), u(gate_w), u(shared), u(routed), reinterpret_cast<uint4*>(out), (int)(H / 8));
  note_launch("shared_gate_add");
  return launch_status();
}

// ---------------------------------------------------------------------------
// out[t, :] = sum_s w[t, s] * y[row(t, s), :], slots added in order s = 0..k-1 in fp32.
template <bool BF16>
__global__ void moe_combine_kernel(const uint4* __restrict__ y, const void* __restrict__ w, int wdt,
                                   const int32_t* __restrict__ perm, uint4* __restrict__ out, int64_t T, int top_k,
                                   int64_t H8, int w_by_row) {
  using A = Act<BF16>;
  using Ty = typename A::T;
  const int64_t total = T * H8;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = idx / H8, c = idx % H8;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int s = 0; s < top_k; ++s) {
      const int64_t pair = t * top_k + s;
      const int64_t row = perm ? (int64_t)perm[pair] : pair;
      if (row < 0) continue;
      const float wt = w ? load_scalar(w, w_by_row ? row : pair, wdt) : 1.0f;
      const uint4 v = y[row * H8 + c];
      const Ty* vp = reinterpret_cast<const Ty*>(&v);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += wt * A::to_f(vp[j]);
    }
    uint4 o;
    Ty* op = reinterpret_cast<Ty*>(&o);
#pragma unroll
    for (int j = 0; j < 8; ++j) op[j] = A::from_f(acc[j]);
    out[idx] = o;
  }
}

int moe_combine(const void* y, const void* w, int wdt, const int32_t* perm, void* out, int dtype, int64_t T, int top_k,
                int64_t H, int w_by_row, cudaStream_t st) {
  if (T == 0) return B2Q_OK;
  const int64_t total = T * (H / 8);
  int64_t g = (total + 255) / 256;
  if (g > 148 * 16) g = 148 * 16;
  if (dtype == B2Q_BF16)
    moe_combine_kernel<true><<<(int)g, 256, 0, st>>>(reinterpret_cast<const uint4*>(y), w, wdt, perm,
                                                     reinterpret_cast<uint4*>(out), T, top_k, H / 8, w_by_row);
  else
    moe_combine_kernel<false><<<(int)g, 256, 0, st>>>(reinterpret_cast<const uint4*>(y), w, wdt, perm,
                                                      reinterpret_cast<uint4*>(out), T, top_k, H / 8, w_by_row);
  note_launch("moe_combine");
  return launch_status();
}

// ---------------------------------------------------------------------------
// Dynamic e4m3 quantisation of activations, one warp per (row, 128 columns).
// scale = max(amax, 1e-12) / 448 ; q = e4m3_rn(x / scale) with true division,
// the recipe of tests/test_fp8_blockscale_gemm.py:13-28 applied to a 1x128 tile.
template <bool BF16>
__global__ void act_quant_1x128_kernel(const void* __restrict__ x, int64_t ldx, uint8_t* __restrict__ xq,
                                       float* __restrict__ xs, int64_t M, int64_t K) {
  using A = Act<BF16>;
  using T = typename A::T;
  const int64_t kb_n = K >> 7;
  const int64_t wid = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= M * kb_n) return;
  const int64_t m = wid / kb_n, kb = wid % kb_n;
  const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const T*>(x) + m * ldx + kb * 128 + lane * 4);
  const T* rp = reinterpret_cast<const T*>(&raw);
  float v[4];
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) { v[j] = A::to_f(rp[j]); amax = fmaxf(amax, fabsf(v[j])); }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float s = __fdiv_rn(fmaxf(amax, 1e-12f), 448.0f);
  uint32_t pk = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t b = __nv_cvt_float_to_fp8(__fdiv_rn(v[j], s), __NV_SATFINITE, __NV_E4M3);
    pk |= b << (8 * j);
  }
  *reinterpret_cast<uint32_t*>(xq + m * K + kb * 128 + lane * 4) = pk;
  if (lane == 0) xs[m * kb_n + kb] = s;
}

int act_quant_1x128(const void* x, int dtype, int64_t ldx, void* xq, float* xs, int64_t M, int64_t K, cudaStream_t st) {
  const int64_t warps = M * (K >> 7);
  if (warps == 0) return B2Q_OK;
  const int grid = (int)((warps + 7) / 8);
  if (dtype == B2Q_BF16)
    act_quant_1x128_kernel<true><<<grid, 256, 0, st>>>(x, ldx, reinterpret_cast<uint8_t*>(xq), xs, M, K);
  else
    act_quant_1x128_kernel<false><<<grid, 256, 0, st>>>(x, ldx, reinterpret_cast<uint8_t*>(xq), xs, M, K);
  note_launch("act_quant_1x128");
  return launch_status();
}

}  // namespace b2q

namespace b2q {

// ---------------------------------------------------------------------------
// Activation pre-pass for fp8-weight GEMMs with bf16 activations: rewrites every token row as
// fp16 times a per-token power of two, x16[m, k] = fp16(x[m, k] * 2^e_m) with 2^e_m chosen so
// that the row maximum lands in [2^14, 2^15).  A bf16 value has 8 significant bits, fp16 holds 11
// and reaches down to 2^-24, so every element within 2^-31 of its row maximum converts exactly;
// smaller ones keep an absolute error below rowmax * 2^-40.  inv_scale[m] = 2^-e_m (exact).
// The point: e4m3 / e5m2 weights convert to fp16 with one instruction per pair, to bf16 with four.
__global__ void act_to_scaled_f16_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx, __half* __restrict__ x16,
                                         float* __restrict__ inv_scale, int K) {
  __shared__ float red[32];
  __shared__ float sc_sh;
  const int64_t m = blockIdx.x;
  const __nv_bfloat16* row = x + m * ldx;
  float amax = 0.f;
  for (int k = threadIdx.x * 8; k < K; k += blockDim.x * 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(row + k);
    const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&v);
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(__bfloat162float(e[j])));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
    float a = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) a = fmaxf(a, red[i]);
    float sc = 1.f;
    if (a > 0.f && a < INFINITY) {
      const int ex = (int)((__float_as_uint(a) >> 23) & 0xFF) - 127;      // floor(log2 a) for normal a
      int sh = 14 - ex;
      sh = sh > 126 ? 126 : (sh < -126 ? -126 : sh);
      sc = __uint_as_float((uint32_t)(sh + 127) << 23);
    }
    sc_sh = sc;
    inv_scale[m] = 1.0f / sc;
  }
  __syncthreads();
  const float sc = sc_sh;
  for (int k = threadIdx.x * 8; k < K; k += blockDim.x * 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(row + k);
    const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&v);
    uint4 o;
    __half* oh = reinterpret_cast<__half*>(&o);
#pragma unroll
    for (int j = 0; j < 8; ++j) oh[j] = __float2half_rn(__bfloat162float(e[j]) * sc);
    *reinterpret_cast<uint4*>(x16 + m * (int64_t)K + k) = o;
  }
}

int act_to_scaled_f16(const void* x, int64_t ldx, void* x16, float* inv_scale, int64_t M, int K, cudaStream_t st) {
  if (M == 0) return B2Q_OK;
  int threads = (K / 8 + 31) / 32 * 32;
  threads = threads > 512 ? 512 : (threads < 32 ? 32 : threads);
  act_to_scaled_f16_kernel<<<(unsigned)M, threads, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(x), ldx,
                                                            reinterpret_cast<__half*>(x16), inv_scale, K);
  note_launch("act_to_scaled_f16");
  return launch_status();
}

}  // namespace b2q

// ---------------------------------------------------------------------------
// Routing without a caller-provided workspace.
//
// b2q_moe_route() needs a small scratch table (per-chunk expert histograms) that the caller has to
// allocate.  Some callers cannot: code that runs while a CUDA stream is being captured (cudaMalloc is
// illegal there), serving runtimes that plan all device memory up front and hand the kernels no
// allocator, and plain C hosts that have no pooled allocator and do not want a cudaMalloc/cudaFree
// pair on the decode path.  For them the same three kernels run on a table that lives in the
// library image itself.  The table is a fixed-size device array, so the problem size is capped, every
// GPU that loads the library carries the array until the process exits, and all calls share it.
// ---------------------------------------------------------------------------
namespace b2q {

constexpr int64_t ROUTE_STATIC_MAX_PAIRS = 65536;   // token * top_k pairs
constexpr int ROUTE_STATIC_MAX_EXPERTS = 256;
constexpr int64_t ROUTE_STATIC_WORDS = (ROUTE_STATIC_MAX_PAIRS / ROUTE_CHUNK) * ROUTE_STATIC_MAX_EXPERTS;  // 65536 int32 = 256 KB

static __device__ __align__(256) int32_t g_route_scratch[ROUTE_STATIC_WORDS];

// In host code `g_route_scratch` is only a handle for the runtime, not something a kernel can
// dereference; the device address has to be asked for, per device, with that device current.
static int route_scratch_address(int32_t** out) {
  static int32_t* cached[64] = {nullptr};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return B2Q_ERR_CUDA;
  int32_t* p = __atomic_load_n(&cached[dev], __ATOMIC_ACQUIRE);
  if (!p) {
    void* sym = nullptr;
    if (cudaGetSymbolAddress(&sym, g_route_scratch) != cudaSuccess || !sym) return B2Q_ERR_CUDA;
    p = reinterpret_cast<int32_t*>(sym);
    __atomic_store_n(&cached[dev], p, __ATOMIC_RELEASE);   // racing first calls store the same value
  }
  *out = p;
  return B2Q_OK;
}

int moe_route_static(const int32_t* ids, int64_t n_pairs, int E, int32_t* expert_offsets, int32_t* expert_tokens,
                     int32_t* pair_to_perm, int32_t* rows_per_expert, cudaStream_t st) {
  if (n_pairs > ROUTE_STATIC_MAX_PAIRS || E > ROUTE_STATIC_MAX_EXPERTS) return B2Q_ERR_LIMIT;
  int32_t* scratch = nullptr;
  const int rc = route_scratch_address(&scratch);
  if (rc) return rc;
  // Nothing in the table has to start at zero: the histogram kernel overwrites every (chunk, expert)
  // slot that the two later kernels read for this problem size.
  return moe_route(ids, n_pairs, E, expert_offsets, expert_tokens, pair_to_perm, rows_per_expert, scratch, st);
}

}  // namespace b2q

extern "C" B2Q_API int b2q_moe_route_static(const int32_t* ids, int64_t n_pairs, int E, int32_t* expert_offsets,
                                            int32_t* expert_tokens, int32_t* pair_to_perm, int32_t* rows_per_expert,
                                            void* stream) {
  if (!ids || !expert_offsets || !expert_tokens) return B2Q_ERR_NULL;
  if (n_pairs < 0 || E <= 0) return B2Q_ERR_SHAPE;
  return b2q::moe_route_static(ids, n_pairs, E, expert_offsets, expert_tokens, pair_to_perm, rows_per_expert,
                               (cudaStream_t)stream);
}

namespace b2q {

// ---------------------------------------------------------------------------
// General activation pre-pass in front of the tcgen05 GEMM: optional row gather, per-token
// power-of-two scaling into fp16 (see act_to_scaled_f16_kernel for why that is exact in practice)
// and an optional permutation inside every group of eight k so that the INT4 transform can emit
// its nibble pairs in the order the bit tricks produce them instead of re-sorting them:
//   perm 0: identity      perm 1: (0,4,1,5,2,6,3,7)  nibble i at bits 4i (GGML / N-major, plain K-major)
//                         perm 2: (0,2,4,6,1,3,5,7)  marlin-shuffled words
// dst row r = f(src row (idx ? idx[r] / div : r)); fp16 input keeps scale 1.
// GATED: the source row holds 2K values, gate then up, and the row fed to the GEMM is silu(gate) * up, computed in
// fp32 and rounded to the source type first, exactly as the separate silu_mul_kernel writes it.
template <bool IN_BF16, bool GATED>
__global__ void act_prep_kernel(const void* __restrict__ x, int64_t ldx, const int32_t* __restrict__ idx, int div,
                                __half* __restrict__ x16, float* __restrict__ inv_scale, int K, int perm, int release_early,
                                const int32_t* __restrict__ n_valid) {
  using A = Act<IN_BF16>;
  using T = typename A::T;
  __shared__ float red[32];
  __shared__ float sc_sh;
  // The GEMM that follows may start streaming its weights as soon as this kernel lets it.  With static
  // weights that is at once; otherwise only after everything before this kernel has completed, because the
  // kernel before might be the one that writes those weights.
  if (release_early) grid_dep_release();
  grid_dep_wait();
  if (!release_early) grid_dep_release();
  const int64_t r = blockIdx.x;
  // the launch covers the caller's upper bound of rows; the number actually routed here is only known on the device
  if (n_valid && r >= *n_valid) return;
  const int64_t srow = idx ? (int64_t)(idx[r] / div) : r;
  const uint16_t* row = reinterpret_cast<const uint16_t*>(x) + srow * ldx;
  // eight consecutive source values of the row as floats that are exactly representable in the source type
  auto load8 = [&](int k, float* f) {
    const uint4 v = *reinterpret_cast<const uint4*>(row + k);
    const T* e = reinterpret_cast<const T*>(&v);
    if constexpr (GATED) {
      const uint4 u = *reinterpret_cast<const uint4*>(row + K + k);
      const T* ue = reinterpret_cast<const T*>(&u);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float gv = A::to_f(e[j]);
        const float sl = gv / (1.0f + expf(-gv));
        f[j] = A::to_f(A::from_f(sl * A::to_f(ue[j])));
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = A::to_f(e[j]);
    }
  };
  const bool one_pass = K <= (int)blockDim.x * 8;      // every thread owns at most one group of eight: keep it
  float f[8];
  const int k0 = threadIdx.x * 8;
  if (one_pass && k0 < K) load8(k0, f);
  float sc = 1.f;
  if constexpr (IN_BF16) {
    float amax = 0.f;
    if (one_pass) {
      if (k0 < K) {
#pragma unroll
        for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(f[j]));
      }
    } else {
      for (int k = k0; k < K; k += blockDim.x * 8) {
        load8(k, f);
#pragma unroll
        for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(f[j]));
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    if (threadIdx.x == 0) {
      float a = 0.f;
      for (int i = 0; i < (int)(blockDim.x >> 5); ++i) a = fmaxf(a, red[i]);
      float s = 1.f;
      if (a > 0.f && a < INFINITY) {
        const int ex = (int)((__float_as_uint(a) >> 23) & 0xFF) - 127;
        int sh = 14 - ex;
        sh = sh > 126 ? 126 : (sh < -126 ? -126 : sh);
        s = __uint_as_float((uint32_t)(sh + 127) << 23);
      }
      sc_sh = s;
      inv_scale[r] = 1.0f / s;
    }
    __syncthreads();
    sc = sc_sh;
  } else {
    if (threadIdx.x == 0) inv_scale[r] = 1.0f;
  }
  for (int k = k0; k < K; k += blockDim.x * 8) {
    if (!one_pass) load8(k, f);
    __half h[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) h[j] = __float2half_rn(f[j] * sc);       // fp16 source: sc = 1, the value is exact
    uint4 o;
    __half* oh = reinterpret_cast<__half*>(&o);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      // position j of the stored group holds source element src(j)
      const int src = perm == 1 ? ((j & 1) * 4 + (j >> 1)) : (perm == 2 ? ((j & 3) * 2 + (j >> 2)) : j);
      oh[j] = h[src];
    }
    *reinterpret_cast<uint4*>(x16 + r * (int64_t)K + k) = o;
  }
}

// The same pre-pass with one WARP per row, for rows of at most MAXI * 256 values (K a multiple of 256): the lane keeps
// its MAXI 16-byte pieces in registers between the maximum and the conversion, all loads are issued before the first
// use, and the reduction is five shuffles.  Rows of a few KB were paying mostly for the block-wide barriers.
template <bool IN_BF16, bool GATED, int MAXI>
__global__ void __launch_bounds__(256) act_prep_warp_kernel(const void* __restrict__ x, int64_t ldx, const int32_t* __restrict__ idx,
                                                            int div, __half* __restrict__ x16, float* __restrict__ inv_scale,
                                                            int64_t rows, int K, int perm, int release_early,
                                                            const int32_t* __restrict__ n_valid) {
  using A = Act<IN_BF16>;
  using T = typename A::T;
  if (release_early) grid_dep_release();
  grid_dep_wait();
  if (!release_early) grid_dep_release();
  const int lane = threadIdx.x & 31;
  const int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= rows || (n_valid && r >= *n_valid)) return;
  const int64_t srow = idx ? (int64_t)(idx[r] / div) : r;
  const uint16_t* row = reinterpret_cast<const uint16_t*>(x) + srow * ldx;
  const int iters = K >> 8;
  uint4 raw[MAXI], up[GATED ? MAXI : 1];
#pragma unroll
  for (int i = 0; i < MAXI; ++i)
    if (i < iters) {
      raw[i] = *reinterpret_cast<const uint4*>(row + (i * 32 + lane) * 8);
      if constexpr (GATED) up[i] = *reinterpret_cast<const uint4*>(row + K + (i * 32 + lane) * 8);
    }
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < MAXI; ++i)
    if (i < iters) {
      T* e = reinterpret_cast<T*>(&raw[i]);
      if constexpr (GATED) {
        const T* ue = reinterpret_cast<const T*>(&up[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float gv = A::to_f(e[j]);
          const float sl = gv / (1.0f + expf(-gv));
          e[j] = A::from_f(sl * A::to_f(ue[j]));               // the activated value, rounded as silu_mul stores it
        }
      }
      if constexpr (IN_BF16) {
#pragma unroll
        for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(A::to_f(e[j])));
      }
    }
  float sc = 1.f;
  if constexpr (IN_BF16) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (amax > 0.f && amax < INFINITY) {
      const int ex = (int)((__float_as_uint(amax) >> 23) & 0xFF) - 127;
      int sh = 14 - ex;
      sh = sh > 126 ? 126 : (sh < -126 ? -126 : sh);
      sc = __uint_as_float((uint32_t)(sh + 127) << 23);
    }
  }
  if (lane == 0) inv_scale[r] = 1.0f / sc;
#pragma unroll
  for (int i = 0; i < MAXI; ++i)
    if (i < iters) {
      const T* e = reinterpret_cast<const T*>(&raw[i]);
      __half h[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) h[j] = __float2half_rn(A::to_f(e[j]) * sc);
      uint4 o;
      __half* oh = reinterpret_cast<__half*>(&o);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int src = perm == 1 ? ((j & 1) * 4 + (j >> 1)) : (perm == 2 ? ((j & 3) * 2 + (j >> 2)) : j);
        oh[j] = h[src];
      }
      *reinterpret_cast<uint4*>(x16 + r * (int64_t)K + (i * 32 + lane) * 8) = o;
    }
}

template <bool IN_BF16, bool GATED>
static cudaError_t act_prep_warp_launch(const void* x, int64_t ldx, const int32_t* idx, int div, void* x16, float* inv_scale,
                                        int64_t rows, int K, int perm, int mode, cudaStream_t st, const int32_t* n_valid) {
  const dim3 grid((unsigned)((rows + 7) / 8)), block(256);
  const int iters = K >> 8;
  auto go = [&](auto kern) {
    return launch_overlapped(kern, grid, block, 0, st, mode > 0, x, ldx, idx, div > 0 ? div : 1,
                             reinterpret_cast<__half*>(x16), inv_scale, rows, K, perm, mode == 2 ? 1 : 0, n_valid);
  };
  if (iters <= 4) return go(act_prep_warp_kernel<IN_BF16, GATED, 4>);
  if (iters <= 8) return go(act_prep_warp_kernel<IN_BF16, GATED, 8>);
  return go(act_prep_warp_kernel<IN_BF16, GATED, GATED ? 8 : 16>);
}

int act_prep(const void* x, bool in_bf16, bool gated, int64_t ldx, const int32_t* idx, int div, void* x16,
             float* inv_scale, int64_t rows, int K, int perm, cudaStream_t st, const int32_t* n_valid) {
  if (rows == 0) return B2Q_OK;
  // many short rows (the grouped GEMMs' pre-pass): one warp per row
  if (rows >= 1024 && (K & 255) == 0 && K <= (gated ? 2048 : 4096)) {
    const int mode = tls().overlap_mode;
    cudaError_t e;
    if (in_bf16) e = gated ? act_prep_warp_launch<true, true>(x, ldx, idx, div, x16, inv_scale, rows, K, perm, mode, st, n_valid)
                           : act_prep_warp_launch<true, false>(x, ldx, idx, div, x16, inv_scale, rows, K, perm, mode, st, n_valid);
    else         e = gated ? act_prep_warp_launch<false, true>(x, ldx, idx, div, x16, inv_scale, rows, K, perm, mode, st, n_valid)
                           : act_prep_warp_launch<false, false>(x, ldx, idx, div, x16, inv_scale, rows, K, perm, mode, st, n_valid);
    note_launch("act_prep");
    return e == cudaSuccess ? launch_status() : B2Q_ERR_CUDA;
  }
  int threads = (K / 8 + 31) / 32 * 32;
  threads = threads > 512 ? 512 : (threads < 32 ? 32 : threads);
  const int mode = tls().overlap_mode;
  auto go = [&](auto kern) {
    return launch_overlapped(kern, dim3((unsigned)rows), dim3(threads), 0, st, mode > 0, x, ldx, idx,
                             div > 0 ? div : 1, reinterpret_cast<__half*>(x16), inv_scale, K, perm, mode == 2 ? 1 : 0, n_valid);
  };
  cudaError_t e;
  if (in_bf16) e = gated ? go(act_prep_kernel<true, true>) : go(act_prep_kernel<true, false>);
  else         e = gated ? go(act_prep_kernel<false, true>) : go(act_prep_kernel<false, false>);
  note_launch("act_prep");
  return e == cudaSuccess ? launch_status() : B2Q_ERR_CUDA;
}

// ---------------------------------------------------------------------------
// Activation pre-pass of the FP8-weight decode GEMM: every row is scaled by a power of two so that its
// largest element lands in [128, 256) and then written as a sum of e4m3 terms,
//     x * 2^e = t0 + t1 / 16 (+ t2 / 256),
// t0 = rn(x * 2^e), t1 = rn(16 * remainder), ...  Each term keeps four more significant bits, so two terms
// reproduce a bf16 value and three an fp16 value exactly (elements more than 2^14 below the row maximum lose
// their last bits; their share of a dot product is below fp32 rounding).  Term j of token r is row j * Mp + r.
template <bool IN_BF16>
__global__ void act_split_fp8_kernel(const void* __restrict__ x, int64_t ldx, uint8_t* __restrict__ xq,
                                     float* __restrict__ inv_scale, int Mp, int K, int release_early) {
  __shared__ float red[32];
  __shared__ float sc_sh;
  if (release_early) grid_dep_release();
  grid_dep_wait();
  if (!release_early) grid_dep_release();
  const int64_t r = blockIdx.x;
  const uint16_t* row = reinterpret_cast<const uint16_t*>(x) + r * ldx;
  auto to_f = [](uint16_t h) -> float {
    if constexpr (IN_BF16) return __uint_as_float((uint32_t)h << 16);
    else return __half2float(__ushort_as_half(h));
  };
  float amax = 0.f;
  for (int k = threadIdx.x * 8; k < K; k += blockDim.x * 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(row + k);
    const uint16_t* e = reinterpret_cast<const uint16_t*>(&v);
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(to_f(e[j])));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
    float a = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) a = fmaxf(a, red[i]);
    float s = 1.f;
    if (a > 0.f && a < INFINITY) {
      int ex = (int)((__float_as_uint(a) >> 23) & 0xFF) - 127;
      if (ex < -126) ex = -126;                     // fp32-subnormal maximum (fp16 / bf16 inputs never get here)
      int sh = 7 - ex;
      sh = sh > 126 ? 126 : (sh < -126 ? -126 : sh);
      s = __uint_as_float((uint32_t)(sh + 127) << 23);
    }
    sc_sh = s;
    inv_scale[r] = 1.0f / s;
  }
  __syncthreads();
  const float sc = sc_sh;
  constexpr int NT = IN_BF16 ? 2 : 3;
  for (int k = threadIdx.x * 8; k < K; k += blockDim.x * 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(row + k);
    const uint16_t* e = reinterpret_cast<const uint16_t*>(&v);
    uint8_t t[NT][8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float rem = to_f(e[j]) * sc;
#pragma unroll
      for (int q = 0; q < NT; ++q) {
        const uint8_t b = (uint8_t)__nv_cvt_float_to_fp8(rem, __NV_SATFINITE, __NV_E4M3);
        t[q][j] = b;
        rem = (rem - fp8_to_float(b, false)) * 16.f;
      }
    }
#pragma unroll
    for (int q = 0; q < NT; ++q)
      *reinterpret_cast<uint2*>(xq + ((int64_t)q * Mp + r) * K + k) = *reinterpret_cast<const uint2*>(t[q]);
  }
}

int act_split_fp8(const void* x, bool in_bf16, int64_t ldx, void* xq, float* inv_scale, int64_t M, int K, cudaStream_t st) {
  if (M == 0) return B2Q_OK;
  int threads = (K / 8 + 31) / 32 * 32;
  threads = threads > 512 ? 512 : (threads < 32 ? 32 : threads);
  const int mode = tls().overlap_mode;
  const int mp = (int)((M + 7) / 8 * 8);
  cudaError_t e;
  if (in_bf16)
    e = launch_overlapped(act_split_fp8_kernel<true>, dim3((unsigned)M), dim3(threads), 0, st, mode > 0, x, ldx,
                          reinterpret_cast<uint8_t*>(xq), inv_scale, mp, K, mode == 2 ? 1 : 0);
  else
    e = launch_overlapped(act_split_fp8_kernel<false>, dim3((unsigned)M), dim3(threads), 0, st, mode > 0, x, ldx,
                          reinterpret_cast<uint8_t*>(xq), inv_scale, mp, K, mode == 2 ? 1 : 0);
  note_launch("act_split_fp8");
  return e == cudaSuccess ? launch_status() : B2Q_ERR_CUDA;
}

// ---------------------------------------------------------------------------
// Activation pre-pass of the INT4 decode GEMM on the int8 MMA: every row is scaled by a power of two so that its
// largest element lands in [32, 64) and written as three signed-byte terms,
//     x * 2^e = t0 + t1 / 128 + t2 / 16384      (t0 = rint(x 2^e), t1 = rint(128 * remainder), ...),
// 20 bits below the row maximum in all.  Inside every group of eight k the bytes are stored in the order
// (0, 2, 4, 6, 1, 3, 5, 7), the order in which the weight transform's two masks deliver a word's nibbles.
// Term j of token r is row j * Mp + r.  xsum[g][r] = sum over group g of the value token r's three terms stand for; the
// GEMM subtracts 8 x that to undo the nibble offset.
template <bool IN_BF16>
__global__ void act_split_i8_kernel(const void* __restrict__ x, int64_t ldx, int8_t* __restrict__ xq,
                                    float* __restrict__ inv_scale, float* __restrict__ xsum, int Mp, int K, int release_early) {
  __shared__ float red[32];
  __shared__ float sc_sh;
  if (release_early) grid_dep_release();
  grid_dep_wait();
  if (!release_early) grid_dep_release();
  const int64_t r = blockIdx.x;
  const uint16_t* row = reinterpret_cast<const uint16_t*>(x) + r * ldx;
  auto to_f = [](uint16_t h) -> float {
    if constexpr (IN_BF16) return __uint_as_float((uint32_t)h << 16);
    else return __half2float(__ushort_as_half(h));
  };
  float amax = 0.f;
  for (int k = threadIdx.x * 8; k < K; k += blockDim.x * 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(row + k);
    const uint16_t* e = reinterpret_cast<const uint16_t*>(&v);
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(to_f(e[j])));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
    float a = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) a = fmaxf(a, red[i]);
    float s = 1.f;
    if (a > 0.f && a < INFINITY) {
      int ex = (int)((__float_as_uint(a) >> 23) & 0xFF) - 127;
      if (ex < -126) ex = -126;
      int sh = 5 - ex;
      sh = sh > 126 ? 126 : (sh < -126 ? -126 : sh);
      s = __uint_as_float((uint32_t)(sh + 127) << 23);
    }
    sc_sh = s;
    inv_scale[r] = 1.0f / s;
  }
  __syncthreads();
  const float sc = sc_sh;
  // blockDim.x * 8 is a multiple of 256, so the 16 lanes of a half warp always cover exactly one group of 128 k
  for (int k0 = 0; k0 < K; k0 += blockDim.x * 8) {
    const int k = k0 + threadIdx.x * 8;
    float part = 0.f;
    if (k < K) {
      const uint4 v = *reinterpret_cast<const uint4*>(row + k);
      const uint16_t* e = reinterpret_cast<const uint16_t*>(&v);
      int8_t t[3][8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int src = (j & 3) * 2 + (j >> 2);            // stored position j holds source element src
        float rem = to_f(e[src]) * sc;
        const float full = rem;
        float rep = 0.f, w = 1.f;
#pragma unroll
        for (int q = 0; q < 3; ++q) {
          float ti = rintf(rem);
          ti = fminf(fmaxf(ti, -127.f), 127.f);
          t[q][j] = (int8_t)(int)ti;
          rep += ti * w;
          rem = (rem - ti) * 128.f;
          w *= 0.0078125f;
        }
        (void)full;
        part += rep;
      }
#pragma unroll
      for (int q = 0; q < 3; ++q)
        *reinterpret_cast<uint2*>(xq + ((int64_t)q * Mp + r) * K + k) = *reinterpret_cast<const uint2*>(t[q]);
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    if ((threadIdx.x & 15) == 0 && k < K) xsum[(int64_t)(k >> 7) * Mp + r] = part;
  }
}

int act_split_i8(const void* x, bool in_bf16, int64_t ldx, void* xq, float* inv_scale, float* xsum, int64_t M, int K,
                 cudaStream_t st) {
  if (M == 0) return B2Q_OK;
  int threads = (K / 8 + 31) / 32 * 32;
  threads = threads > 512 ? 512 : (threads < 32 ? 32 : threads);
  const int mode = tls().overlap_mode;
  const int mp = (int)((M + 7) / 8 * 8);
  cudaError_t e;
  if (in_bf16)
    e = launch_overlapped(act_split_i8_kernel<true>, dim3((unsigned)M), dim3(threads), 0, st, mode > 0, x, ldx,
                          reinterpret_cast<int8_t*>(xq), inv_scale, xsum, mp, K, mode == 2 ? 1 : 0);
  else
    e = launch_overlapped(act_split_i8_kernel<false>, dim3((unsigned)M), dim3(threads), 0, st, mode > 0, x, ldx,
                          reinterpret_cast<int8_t*>(xq), inv_scale, xsum, mp, K, mode == 2 ? 1 : 0);
  note_launch("act_split_i8");
  return e == cudaSuccess ? launch_status() : B2Q_ERR_CUDA;
}

// ---------------------------------------------------------------------------
// Residual add + RMSNorm in front of a decode GEMV (the first half of the reference's fused
// esimd_resadd_norm_gemv_* kernels, csrc/xpu/esimd_kernels/resadd_norm_gemv_int4.h and norm_gemv_fused.h):
//   s = hidden + residual (fp32);  residual <- s;  normed = s * rsqrt(mean(s^2) + eps) * weight  -> normed_out.
// The norm is taken of the fp32 sum, not of its 16-bit rounding, as the reference's step-by-step check does
// (tests/test_resadd_norm_gemv_int4.py:41-59).  One block per row; the GEMV's own pre-pass follows and overlaps
// through programmatic dependent launch.
// Generalised for the two further members of the family: `scalar` multiplies the sum before anything else
// (esimd_scaled_resadd_norm_gemv_fp8_pert, csrc/xpu/esimd_kernels/scaled_resadd_norm_gemv_fp8.h:70-95); hidden == nullptr
// skips the add and leaves the residual untouched, and a second weight writes a second normalised row from the same
// 1/rms (esimd_norm_gemv_norm_fp16, csrc/xpu/esimd_kernels/norm_gemv_norm_fp16.h:56-98).
template <bool BF16>
__global__ void resadd_rmsnorm_kernel(const void* __restrict__ hidden, void* __restrict__ residual, const void* __restrict__ weight,
                                      void* __restrict__ normed, const void* __restrict__ weight2, void* __restrict__ normed2,
                                      int K, float eps, float scalar) {
  using T = typename Act<BF16>::T;
  __shared__ float red[32];
  __shared__ float inv_sh;
  grid_dep_wait();
  grid_dep_release();
  const int64_t r = blockIdx.x;
  const T* h = hidden ? reinterpret_cast<const T*>(hidden) + r * K : nullptr;
  T* res = reinterpret_cast<T*>(residual) + r * K;
  const T* w = reinterpret_cast<const T*>(weight);
  const T* w2 = reinterpret_cast<const T*>(weight2);
  T* out = reinterpret_cast<T*>(normed) + r * K;
  T* out2 = normed2 ? reinterpret_cast<T*>(normed2) + r * K : nullptr;
  auto load8 = [&](int k, float* v) {
    const uint4 rv = *reinterpret_cast<const uint4*>(res + k);
    const T* re = reinterpret_cast<const T*>(&rv);
    if (h) {
      const uint4 hv = *reinterpret_cast<const uint4*>(h + k);
      const T* he = reinterpret_cast<const T*>(&hv);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = (Act<BF16>::to_f(he[j]) + Act<BF16>::to_f(re[j])) * scalar;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = Act<BF16>::to_f(re[j]);
    }
  };
  float ss = 0.f;
  for (int k = threadIdx.x * 8; k < K; k += blockDim.x * 8) {
    float v[8];
    load8(k, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) ss = fmaf(v[j], v[j], ss);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) t += red[i];
    inv_sh = rsqrtf(t / (float)K + eps);
  }
  __syncthreads();
  const float inv = inv_sh;
  // second pass over the same (cache-resident) inputs: only now is the residual overwritten
  for (int k = threadIdx.x * 8; k < K; k += blockDim.x * 8) {
    float v[8];
    load8(k, v);
    const uint4 wv = *reinterpret_cast<const uint4*>(w + k);
    const T* we = reinterpret_cast<const T*>(&wv);
    uint4 so, no;
    T* se = reinterpret_cast<T*>(&so);
    T* ne = reinterpret_cast<T*>(&no);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      se[j] = Act<BF16>::from_f(v[j]);
      ne[j] = Act<BF16>::from_f(v[j] * inv * Act<BF16>::to_f(we[j]));
    }
    if (h) *reinterpret_cast<uint4*>(res + k) = so;
    *reinterpret_cast<uint4*>(out + k) = no;
    if (out2) {
      const uint4 w2v = *reinterpret_cast<const uint4*>(w2 + k);
      const T* w2e = reinterpret_cast<const T*>(&w2v);
#pragma unroll
      for (int j = 0; j < 8; ++j) ne[j] = Act<BF16>::from_f(v[j] * inv * Act<BF16>::to_f(w2e[j]));
      *reinterpret_cast<uint4*>(out2 + k) = no;
    }
  }
}

int resadd_rmsnorm(const void* hidden, void* residual, const void* weight, void* normed, const void* weight2, void* normed2,
                   bool bf16, int64_t M, int K, float eps, float scalar, cudaStream_t st) {
  if (M == 0) return B2Q_OK;
  int threads = (K / 8 + 31) / 32 * 32;
  threads = threads > 1024 ? 1024 : (threads < 32 ? 32 : threads);
  const bool overlap = tls().overlap_mode > 0;
  cudaError_t e;
  if (bf16) e = launch_overlapped(resadd_rmsnorm_kernel<true>, dim3((unsigned)M), dim3(threads), 0, st, overlap, hidden, residual, weight, normed, weight2, normed2, K, eps, scalar);
  else e = launch_overlapped(resadd_rmsnorm_kernel<false>, dim3((unsigned)M), dim3(threads), 0, st, overlap, hidden, residual, weight, normed, weight2, normed2, K, eps, scalar);
  note_launch("resadd_rmsnorm");
  return e == cudaSuccess ? launch_status() : B2Q_ERR_CUDA;
}

// ---------------------------------------------------------------------------
// Residual add + RMSNorm and the FP8 decode GEMV's activation pre-pass in ONE launch (the reference fuses the norm
// into the GEMV kernel itself: csrc/xpu/esimd_kernels/norm_gemv_fused.h, scaled_resadd_norm_gemv_fp8.h:70-95).
// Per row:  v = (hidden + residual) * scalar;  residual <- v;  n = v * rsqrt(mean(v^2) + eps) * weight, rounded to
// the activation type and stored to normed_out exactly as resadd_rmsnorm_kernel stores it; then the row of ROUNDED
// values is scaled by a power of two and split into e4m3 terms exactly as act_split_fp8_kernel splits it.  Every
// thread reads back only what it wrote itself, so the three sweeps over the row need no grid-wide ordering.
template <bool BF16>
__global__ void resadd_norm_split_fp8_kernel(const void* __restrict__ hidden, void* __restrict__ residual,
                                             const void* __restrict__ weight, void* __restrict__ normed, float eps, float scalar,
                                             uint8_t* __restrict__ xq, float* __restrict__ inv_scale, int Mp, int K, int release_early) {
  using T = typename Act<BF16>::T;
  __shared__ float red[32];
  __shared__ float bc_sh;
  if (release_early) grid_dep_release();
  grid_dep_wait();
  if (!release_early) grid_dep_release();
  const int64_t r = blockIdx.x;
  const T* h = reinterpret_cast<const T*>(hidden) + r * K;
  T* res = reinterpret_cast<T*>(residual) + r * K;
  const T* w = reinterpret_cast<const T*>(weight);
  T* out = reinterpret_cast<T*>(normed) + r * K;
  auto load8 = [&](int k, float* v) {
    const uint4 rv = *reinterpret_cast<const uint4*>(res + k);
    const uint4 hv = *reinterpret_cast<const uint4*>(h + k);
    const T* re = reinterpret_cast<const T*>(&rv);
    const T* he = reinterpret_cast<const T*>(&hv);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = (Act<BF16>::to_f(he[j]) + Act<BF16>::to_f(re[j])) * scalar;
  };
  auto block_reduce = [&](float v, bool is_max) -> float {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float u = __shfl_xor_sync(0xffffffffu, v, o);
      v = is_max ? fmaxf(v, u) : v + u;
    }
    __syncthreads();                                    // red[] may still be read from the previous reduction
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = is_max ? 0.f : 0.f;
      for (int i = 0; i < (int)(blockDim.x >> 5); ++i) t = is_max ? fmaxf(t, red[i]) : t + red[i];
      bc_sh = t;
    }
    __syncthreads();
    return bc_sh;
  };
  float ss = 0.f;
  for (int k = threadIdx.x * 8; k < K; k += blockDim.x * 8) {
    float v[8];
    load8(k, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) ss = fmaf(v[j], v[j], ss);
  }
  const float inv = rsqrtf(block_reduce(ss, false) / (float)K + eps);
  float amax = 0.f;
  for (int k = threadIdx.x * 8; k < K; k += blockDim.x * 8) {
    float v[8];
    load8(k, v);
    const uint4 wv = *reinterpret_cast<const uint4*>(w + k);
    const T* we = reinterpret_cast<const T*>(&wv);
    uint4 so, no;
    T* se = reinterpret_cast<T*>(&so);
    T* ne = reinterpret_cast<T*>(&no);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      se[j] = Act<BF16>::from_f(v[j]);
      ne[j] = Act<BF16>::from_f(v[j] * inv * Act<BF16>::to_f(we[j]));
      amax = fmaxf(amax, fabsf(Act<BF16>::to_f(ne[j])));
    }
    *reinterpret_cast<uint4*>(res + k) = so;
    *reinterpret_cast<uint4*>(out + k) = no;
  }
  const float a = block_reduce(amax, true);
  float sc = 1.f;
  if (a > 0.f && a < INFINITY) {
    int ex = (int)((__float_as_uint(a) >> 23) & 0xFF) - 127;
    if (ex < -126) ex = -126;
    int sh = 7 - ex;
    sh = sh > 126 ? 126 : (sh < -126 ? -126 : sh);
    sc = __uint_as_float((uint32_t)(sh + 127) << 23);
  }
  if (threadIdx.x == 0) inv_scale[r] = 1.0f / sc;
  constexpr int NT = BF16 ? 2 : 3;
  for (int k = threadIdx.x * 8; k < K; k += blockDim.x * 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(out + k);          // this thread's own stores of the sweep above
    const T* e = reinterpret_cast<const T*>(&v);
    uint8_t t[NT][8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float rem = Act<BF16>::to_f(e[j]) * sc;
#pragma unroll
      for (int q = 0; q < NT; ++q) {
        const uint8_t b = (uint8_t)__nv_cvt_float_to_fp8(rem, __NV_SATFINITE, __NV_E4M3);
        t[q][j] = b;
        rem = (rem - fp8_to_float(b, false)) * 16.f;
      }
    }
#pragma unroll
    for (int q = 0; q < NT; ++q)
      *reinterpret_cast<uint2*>(xq + ((int64_t)q * Mp + r) * K + k) = *reinterpret_cast<const uint2*>(t[q]);
  }
}

int resadd_norm_split_fp8(const void* hidden, void* residual, const void* weight, void* normed, bool bf16, float eps, float scalar,
                          void* xq, float* inv_scale, int64_t M, int K, cudaStream_t st) {
  if (M == 0) return B2Q_OK;
  int threads = (K / 8 + 31) / 32 * 32;
  threads = threads > 512 ? 512 : (threads < 32 ? 32 : threads);
  const int mode = tls().overlap_mode;
  const int mp = (int)((M + 7) / 8 * 8);
  cudaError_t e;
  if (bf16)
    e = launch_overlapped(resadd_norm_split_fp8_kernel<true>, dim3((unsigned)M), dim3(threads), 0, st, mode > 0, hidden, residual, weight,
                          normed, eps, scalar, reinterpret_cast<uint8_t*>(xq), inv_scale, mp, K, mode == 2 ? 1 : 0);
  else
    e = launch_overlapped(resadd_norm_split_fp8_kernel<false>, dim3((unsigned)M), dim3(threads), 0, st, mode > 0, hidden, residual, weight,
                          normed, eps, scalar, reinterpret_cast<uint8_t*>(xq), inv_scale, mp, K, mode == 2 ? 1 : 0);
  note_launch("resadd_norm_split_fp8");
  return e == cudaSuccess ? launch_status() : B2Q_ERR_CUDA;
}

// ---------------------------------------------------------------------------
// Gated RMSNorm in front of a decode GEMV (first half of the reference's esimd_norm_gemv_* kernels,
// csrc/xpu/esimd_kernels/norm_gemv_fused.h, norm_gemv_int4.h):  per row of x [rows, V]
//   out = x * rsqrt(mean(x^2) + eps) * weight * silu(z),   all in fp32, one rounding to the activation type
// (the check of tests/test_fp8_blockscale_fusions.py:81-100).  One warp per row.
template <bool BF16>
__global__ void gated_rmsnorm_kernel(const void* __restrict__ x, const void* __restrict__ z, const void* __restrict__ weight,
                                     void* __restrict__ out, int rows, int V, float eps) {
  using T = typename Act<BF16>::T;
  grid_dep_wait();
  grid_dep_release();
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const T* xr = reinterpret_cast<const T*>(x) + (int64_t)row * V;
  const T* zr = reinterpret_cast<const T*>(z) + (int64_t)row * V;
  const T* w = reinterpret_cast<const T*>(weight);
  T* o = reinterpret_cast<T*>(out) + (int64_t)row * V;
  float ss = 0.f;
  for (int k = lane; k < V; k += 32) { const float v = Act<BF16>::to_f(xr[k]); ss = fmaf(v, v, ss); }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
  const float inv = rsqrtf(ss / (float)V + eps);
  for (int k = lane; k < V; k += 32) {
    const float g = Act<BF16>::to_f(zr[k]);
    const float silu = g / (1.f + __expf(-g));
    o[k] = Act<BF16>::from_f(Act<BF16>::to_f(xr[k]) * inv * Act<BF16>::to_f(w[k]) * silu);
  }
}

int gated_rmsnorm(const void* x, const void* z, const void* weight, void* out, bool bf16, int rows, int V, float eps, cudaStream_t st) {
  if (rows == 0) return B2Q_OK;
  const int wpb = 4;
  const bool overlap = tls().overlap_mode > 0;
  const dim3 grid((rows + wpb - 1) / wpb), block(wpb * 32);
  cudaError_t e;
  if (bf16) e = launch_overlapped(gated_rmsnorm_kernel<true>, grid, block, 0, st, overlap, x, z, weight, out, rows, V, eps);
  else e = launch_overlapped(gated_rmsnorm_kernel<false>, grid, block, 0, st, overlap, x, z, weight, out, rows, V, eps);
  note_launch("gated_rmsnorm");
  return e == cudaSuccess ? launch_status() : B2Q_ERR_CUDA;
}

}  // namespace b2q
