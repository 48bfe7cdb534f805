// Decode-shaped weight-only linear (1 <= M <= 64 per pass): an HBM-streaming
// kernel.  Weights are the only large operand; each warp streams its own
// 128-byte-wide column slab of a ROWS-row strip of W through a private
// cp.async ring in shared memory (16-byte coalesced copies, no CTA barrier in
// the main loop), dequantises in registers and feeds mma.sync m16n8k16 with
// the weight rows as the MMA's M dimension and the tokens as its N dimension.
// The four warps of a CTA split K and reduce once through shared memory.
//
// Role of this kernel relative to the reference: esimd_gemv_int4 /
// esimd_gemm_int4_pgrp (csrc/xpu/esimd_kernels/int4_GEMV.h:165-251,
// int4_GEMM.h:81-270), esimd_gemv_fp8_pern/pert (fp8_GEMV_v2.h:46-337) and
// esimd_gemm_fp8_blockscale (fp8_GEMM_blockscale.h:64-137).
#pragma once
#include "common.cuh"

namespace b2q {

enum { WF_INT4 = 0, WF_E4M3 = 1, WF_E5M2 = 2 };
enum { SM_GROUP = 0, SM_POST = 1, SM_BLOCK = 2 };  // POST = per-channel or per-tensor

struct SmallMParams {
  const void* x; int64_t ldx;           // [M, K] act dtype
  const uint8_t* w; int64_t w_row_bytes;
  const void* scale; int scale_dtype;
  int64_t s_stride_n, s_stride_g;       // int4 group scale strides / channel stride (0 = per tensor)
  void* out; int64_t ldo;
  int M, N, K;
  uint32_t xor_mask;                    // 0x88888888 for two's-complement nibbles
  // grouped (MoE) extension: when tiles != nullptr blockIdx.y indexes a device-built
  // tile list {int32 n_tiles, 3 pad, int2 (expert, first row in expert)...}
  const int32_t* tiles;
  const int32_t* expert_offsets;        // [E+1] rows of x/out per expert (sorted rows)
  const int32_t* row_map; int row_div;  // optional gather of input rows
  const int32_t* out_map;               // optional scatter of output rows
  int64_t w_expert_bytes, s_expert_elems;
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint4 ldg128(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

template <bool BF16>
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  if constexpr (BF16) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  } else {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
}

// Two nibbles (bits 0-3 and 16-19 of v) -> packed 16-bit floats holding (q - 8) exactly.
template <bool BF16> __device__ __forceinline__ uint32_t nib2_to_act(uint32_t v) {
  if constexpr (BF16) {
    uint32_t r = (v & 0x000F000Fu) | 0x43004300u;           // bf16(128 + q)
    __nv_bfloat162 h = *reinterpret_cast<__nv_bfloat162*>(&r);
    const uint32_t c = 0x43084308u;                          // bf16(136)
    h = __hsub2(h, *reinterpret_cast<const __nv_bfloat162*>(&c));
    return *reinterpret_cast<uint32_t*>(&h);
  } else {
    uint32_t r = (v & 0x000F000Fu) | 0x64006400u;           // fp16(1024 + q)
    __half2 h = *reinterpret_cast<__half2*>(&r);
    const uint32_t c = 0x64086408u;                          // fp16(1032)
    h = __hsub2(h, *reinterpret_cast<const __half2*>(&c));
    return *reinterpret_cast<uint32_t*>(&h);
  }
}

// Two fp8 bytes (low 16 bits of v) -> packed 16-bit floats.  For bf16 the result
// carries an exact factor 2^-112 (undone on the fp32 accumulator).
template <bool BF16, bool E5M2> __device__ __forceinline__ uint32_t fp8x2_to_act(uint32_t v) {
  uint32_t h;
  const unsigned short lo = (unsigned short)(v & 0xFFFFu);
  if constexpr (E5M2) asm("cvt.rn.f16x2.e5m2x2 %0, %1;\n" : "=r"(h) : "h"(lo));
  else asm("cvt.rn.f16x2.e4m3x2 %0, %1;\n" : "=r"(h) : "h"(lo));
  if constexpr (BF16) h = ((h >> 3) & 0x0FFF0FFFu) | (h & 0x80008000u);
  return h;
}

template <int RT> struct SmallMStages { static constexpr int value = RT == 1 ? 8 : (RT == 2 ? 6 : 4); };

template <int WF, int SMODE, bool BF16, int RT, int NT>
__global__ void __launch_bounds__(128) smallm_kernel(const SmallMParams p) {
  using A = Act<BF16>;
  using T = typename A::T;
  constexpr int ROWS = RT * 16;
  constexpr int STAGES = SmallMStages<RT>::value;
  constexpr int STAGE_BYTES = ROWS * 128;
  constexpr bool INT4 = (WF == WF_INT4);
  constexpr int KSLAB = INT4 ? 256 : 128;
  constexpr float UNBIAS = (!INT4 && BF16) ? 5192296858534827628530496329220096.0f : 1.0f;  // 2^112

  extern __shared__ __align__(128) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;

  // ---- problem slice (dense: one problem; grouped: one expert per blockIdx.z) ----
  int M = p.M, xrow0 = 0;
  const uint8_t* wbase = p.w;
  int64_t sbase = 0;
  int tok0 = blockIdx.y * (NT * 8);
  // The next kernel of the stream may start at once; this one waits for earlier kernels only before it first reads
  // something they may have written: the tile list (grouped launches, here) or the activations (dense launches, after
  // the first weight stages are already in flight).  Both are no-ops for a plain launch.
  grid_dep_release();
  if (p.tiles) {
    grid_dep_wait();
    if ((int)blockIdx.y >= p.tiles[0]) return;
    const int2 td = reinterpret_cast<const int2*>(p.tiles + 4)[blockIdx.y];
    const int e = td.x;
    tok0 = td.y;
    xrow0 = p.expert_offsets[e];
    M = p.expert_offsets[e + 1] - xrow0;
    wbase += (int64_t)e * p.w_expert_bytes;
    sbase = (int64_t)e * p.s_expert_elems;
  }
  if (tok0 >= M) return;
  const int row0 = blockIdx.x * ROWS;
  const int N = p.N, K = p.K;
  const int nslab = (K + KSLAB - 1) / KSLAB;
  const int n_my = (nslab > warp) ? (nslab - warp + 3) / 4 : 0;
  const uint32_t ring = (uint32_t)__cvta_generic_to_shared(smem) + warp * (STAGES * STAGE_BYTES);

  auto issue = [&](int it) {
    const int slab = warp + 4 * it;
    const uint32_t sb = ring + (it % STAGES) * STAGE_BYTES;
    const int c = lane & 7;
    const int64_t kbyte = (int64_t)slab * 128 + c * 16;
    const int nbytes = (kbyte < p.w_row_bytes) ? 16 : 0;
#pragma unroll
    for (int i = 0; i < ROWS / 4; ++i) {
      const int r = i * 4 + (lane >> 3);
      int row = row0 + r; row = row < N ? row : N - 1;
      const uint8_t* src = wbase + (int64_t)row * p.w_row_bytes + (nbytes ? kbyte : 0);
      cp_async16(sb + r * 128 + ((c ^ ((r & 1) << 2)) << 4), src, nbytes);
    }
  };

  // ---- token rows of this thread (B operand: token = tile*8 + g) ----
  const T* xptr[NT];
  bool xok[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int tok = tok0 + nt * 8 + g;
    xok[nt] = tok < M;
    int64_t r = xrow0 + (xok[nt] ? tok : 0);
    if (p.row_map) r = p.row_map[r] / p.row_div;
    xptr[nt] = reinterpret_cast<const T*>(p.x) + r * p.ldx;
  }

  float acc[RT][NT][4];
#pragma unroll
  for (int a = 0; a < RT; ++a)
#pragma unroll
    for (int b = 0; b < NT; ++b)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[a][b][c] = 0.f;

#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) { if (s < n_my) issue(s); cp_async_commit(); }
  if (!p.tiles) grid_dep_wait();

  for (int it = 0; it < n_my; ++it) {
    cp_async_wait<STAGES - 2>();
    __syncwarp();
    if (it + STAGES - 1 < n_my) issue(it + STAGES - 1);
    cp_async_commit();
    const int slab = warp + 4 * it;
    const uint32_t sb = ring + (it % STAGES) * STAGE_BYTES;

    if constexpr (INT4) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int kg = slab * 2 + h;
        const int k0 = slab * 256 + h * 128 + t * 32;
        if (kg * 128 < K) {
          // group scales: requested here as raw bits, decoded only where they are used (after the MMAs of this half
          // slab): decoding at the load would make the warp wait for DRAM right here, once per half slab
          uint32_t scr[RT][2];
#pragma unroll
          for (int mt = 0; mt < RT; ++mt)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
              int row = row0 + mt * 16 + g + hh * 8; row = row < N ? row : N - 1;
              scr[mt][hh] = load_scalar_raw(p.scale, sbase + (int64_t)row * p.s_stride_n + (int64_t)kg * p.s_stride_g, p.scale_dtype);
            }
          // activation fragments of the whole half slab in flight at once (few token tiles only: registers)
          constexpr bool XPRE = NT <= 2;
          uint4 xpre[XPRE ? 4 : 1][XPRE ? NT : 1];
          if constexpr (XPRE) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
              for (int nt = 0; nt < NT; ++nt) {
                xpre[i][nt] = make_uint4(0, 0, 0, 0);
                if (xok[nt]) xpre[i][nt] = ldg128(xptr[nt] + k0 + i * 8);
              }
          }
          float tmp[RT][NT][4];
#pragma unroll
          for (int a = 0; a < RT; ++a)
#pragma unroll
            for (int b = 0; b < NT; ++b)
#pragma unroll
              for (int c = 0; c < 4; ++c) tmp[a][b][c] = 0.f;
          uint4 wv[RT][2];
#pragma unroll
          for (int mt = 0; mt < RT; ++mt)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
              const int r = mt * 16 + g + hh * 8;
              wv[mt][hh] = lds128(sb + r * 128 + (((h * 4 + t) ^ ((r & 1) << 2)) << 4));
            }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint32_t bfr[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
              uint4 xv = make_uint4(0, 0, 0, 0);
              if constexpr (XPRE) xv = xpre[i][nt];
              else if (xok[nt]) xv = ldg128(xptr[nt] + k0 + i * 8);
              bfr[nt][0] = __byte_perm(xv.x, xv.z, 0x5410);  // (x0, x4)
              bfr[nt][1] = __byte_perm(xv.x, xv.z, 0x7632);  // (x1, x5)
              bfr[nt][2] = __byte_perm(xv.y, xv.w, 0x5410);  // (x2, x6)
              bfr[nt][3] = __byte_perm(xv.y, xv.w, 0x7632);  // (x3, x7)
            }
#pragma unroll
            for (int mt = 0; mt < RT; ++mt) {
              const uint32_t w0 = (i == 0 ? wv[mt][0].x : i == 1 ? wv[mt][0].y : i == 2 ? wv[mt][0].z : wv[mt][0].w) ^ p.xor_mask;
              const uint32_t w1 = (i == 0 ? wv[mt][1].x : i == 1 ? wv[mt][1].y : i == 2 ? wv[mt][1].z : wv[mt][1].w) ^ p.xor_mask;
              const uint32_t p0a = nib2_to_act<BF16>(w0), p1a = nib2_to_act<BF16>(w0 >> 4);
              const uint32_t p2a = nib2_to_act<BF16>(w0 >> 8), p3a = nib2_to_act<BF16>(w0 >> 12);
              const uint32_t p0b = nib2_to_act<BF16>(w1), p1b = nib2_to_act<BF16>(w1 >> 4);
              const uint32_t p2b = nib2_to_act<BF16>(w1 >> 8), p3b = nib2_to_act<BF16>(w1 >> 12);
#pragma unroll
              for (int nt = 0; nt < NT; ++nt) {
                mma16816<BF16>(tmp[mt][nt], p0a, p0b, p1a, p1b, bfr[nt][0], bfr[nt][1]);
                mma16816<BF16>(tmp[mt][nt], p2a, p2b, p3a, p3b, bfr[nt][2], bfr[nt][3]);
              }
            }
          }
#pragma unroll
          for (int mt = 0; mt < RT; ++mt)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
              const float s0 = scalar_from_raw(scr[mt][0], p.scale_dtype), s1 = scalar_from_raw(scr[mt][1], p.scale_dtype);
              acc[mt][nt][0] += s0 * tmp[mt][nt][0];
              acc[mt][nt][1] += s0 * tmp[mt][nt][1];
              acc[mt][nt][2] += s1 * tmp[mt][nt][2];
              acc[mt][nt][3] += s1 * tmp[mt][nt][3];
            }
        }
      }
    } else {
      constexpr bool E5 = (WF == WF_E5M2);
      float tmp[RT][NT][4];
      if constexpr (SMODE == SM_BLOCK) {
#pragma unroll
        for (int a = 0; a < RT; ++a)
#pragma unroll
          for (int b = 0; b < NT; ++b)
#pragma unroll
            for (int c = 0; c < 4; ++c) tmp[a][b][c] = 0.f;
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int k0 = slab * 128 + h * 64 + t * 16;
        const bool kok = k0 < K;
        uint32_t bfr[NT][8];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          uint4 xa = make_uint4(0, 0, 0, 0), xb = make_uint4(0, 0, 0, 0);
          if (xok[nt] && kok) { xa = ldg128(xptr[nt] + k0); xb = ldg128(xptr[nt] + k0 + 8); }
          bfr[nt][0] = xa.x; bfr[nt][1] = xa.y; bfr[nt][2] = xa.z; bfr[nt][3] = xa.w;
          bfr[nt][4] = xb.x; bfr[nt][5] = xb.y; bfr[nt][6] = xb.z; bfr[nt][7] = xb.w;
        }
#pragma unroll
        for (int mt = 0; mt < RT; ++mt) {
          const int r = mt * 16 + g;
          const uint4 wa = lds128(sb + r * 128 + (((h * 4 + t) ^ ((r & 1) << 2)) << 4));
          const uint4 wb = lds128(sb + (r + 8) * 128 + (((h * 4 + t) ^ ((r & 1) << 2)) << 4));
          const uint32_t wwa[4] = {wa.x, wa.y, wa.z, wa.w};
          const uint32_t wwb[4] = {wb.x, wb.y, wb.z, wb.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t a0 = fp8x2_to_act<BF16, E5>(wwa[i]), a2 = fp8x2_to_act<BF16, E5>(wwa[i] >> 16);
            const uint32_t a1 = fp8x2_to_act<BF16, E5>(wwb[i]), a3 = fp8x2_to_act<BF16, E5>(wwb[i] >> 16);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
              if constexpr (SMODE == SM_BLOCK) mma16816<BF16>(tmp[mt][nt], a0, a1, a2, a3, bfr[nt][2 * i], bfr[nt][2 * i + 1]);
              else mma16816<BF16>(acc[mt][nt], a0, a1, a2, a3, bfr[nt][2 * i], bfr[nt][2 * i + 1]);
            }
          }
        }
      }
      if constexpr (SMODE == SM_BLOCK) {
        // One 128-wide K block per slab; all ROWS rows of the strip share an N block
        // when ROWS divides 128 (it does: 16/32/64).
        const int nb = row0 >> 7;
        const int kblocks = (K + 127) >> 7;
        const float ws = reinterpret_cast<const float*>(p.scale)[sbase + (int64_t)nb * kblocks + slab] * UNBIAS;
#pragma unroll
        for (int mt = 0; mt < RT; ++mt)
#pragma unroll
          for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[mt][nt][c] += ws * tmp[mt][nt][c];
      }
    }
    __syncwarp();
  }
  cp_async_wait<0>();
  __syncthreads();

  // ---- cross-warp (split-K) reduction through shared memory, then store ----
  float* red = reinterpret_cast<float*>(smem);
  constexpr int TOKS = NT * 8;
  // layout red[warp][tok][row] (row fastest)
#pragma unroll
  for (int mt = 0; mt < RT; ++mt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int row = mt * 16 + g + (c >> 1) * 8;
        const int tok = nt * 8 + t * 2 + (c & 1);
        red[(warp * TOKS + tok) * ROWS + row] = acc[mt][nt][c];
      }
  __syncthreads();
  for (int idx = threadIdx.x; idx < TOKS * ROWS; idx += 128) {
    const int tok = idx / ROWS, row = idx % ROWS;
    const int n = row0 + row, m = tok0 + tok;
    if (n < N && m < M) {
      float v = red[idx] + red[TOKS * ROWS + idx] + red[2 * TOKS * ROWS + idx] + red[3 * TOKS * ROWS + idx];
      if constexpr (SMODE == SM_POST) {
        v *= UNBIAS;
        v *= load_scalar(p.scale, sbase + (int64_t)n * p.s_stride_n, p.scale_dtype);
      }
      int64_t orow = xrow0 + m;
      if (p.out_map) orow = p.out_map[orow];
      reinterpret_cast<T*>(p.out)[orow * p.ldo + n] = A::from_f(v);
    }
  }
}

template <int WF, int SMODE, bool BF16, int RT, int NT>
inline int smallm_launch_one(const SmallMParams& p, int m_max, int n_tiles_cap, cudaStream_t st) {
  constexpr int ROWS = RT * 16;
  constexpr int STAGES = SmallMStages<RT>::value;
  constexpr int pipe = 4 * STAGES * ROWS * 128;
  constexpr int red = 4 * NT * 8 * ROWS * 4;
  constexpr int smem = pipe > red ? pipe : red;
  auto kern = smallm_kernel<WF, SMODE, BF16, RT, NT>;
  static thread_local bool configured[16] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 16 && !configured[dev]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return B2Q_ERR_CUDA;
    configured[dev] = true;
  } else if (dev >= 16) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return B2Q_ERR_CUDA;
  }
  dim3 grid((p.N + ROWS - 1) / ROWS, p.tiles ? n_tiles_cap : (m_max + NT * 8 - 1) / (NT * 8), 1);
  // overlap with the previous kernel only when the caller has declared the weights static (overlap mode 2): this
  // kernel has no pre-pass of its own in front of it that would order it behind whatever wrote them
  // (and only for weights of more than 2^25 elements: launches this short measured 6 % slower overlapped, their CTAs all
  // reading the same activation rows at once)
  const bool overlap = tls().overlap_mode == 2 && !p.tiles && (int64_t)p.N * p.K > ((int64_t)1 << 25);
  if (launch_overlapped(kern, grid, dim3(128), (size_t)smem, st, overlap, p) != cudaSuccess) return B2Q_ERR_CUDA;
  note_launch("smallm");
  return launch_status();
}

// Picks the strip height (RT) from N so that the grid covers the 148 SMs a few
// times over, and the token tiling (NT) from the largest M of any problem.
template <int WF, int SMODE, bool BF16>
inline int smallm_dispatch(const SmallMParams& p, int m_max, int n_tiles_cap, cudaStream_t st) {
  // grouped mode: m_max is the token-tile height the tile list was built for (8/16/32/64)
  int nt = m_max <= 8 ? 1 : (m_max <= 16 ? 2 : (m_max <= 32 ? 4 : 8));
  const int64_t strips16 = ((int64_t)p.N + 15) / 16 * (p.tiles ? n_tiles_cap : 1);
  // Conversion ALU work, not bytes in flight, limits this kernel, so resident warps matter more
  // than strip height: 16-row strips give 3 CTAs (12 warps) per SM, 32-row strips 2 CTAs.
  int rt = (nt >= 4 && strips16 >= 2 * 444) ? 2 : 1;
  if (SMODE == SM_BLOCK && (p.N % 16) != 0) rt = 1;
#define B2Q_SM_CASE(R, T_) if (rt == R && nt == T_) return smallm_launch_one<WF, SMODE, BF16, R, T_>(p, m_max, n_tiles_cap, st);
  B2Q_SM_CASE(1, 1) B2Q_SM_CASE(1, 2) B2Q_SM_CASE(1, 4) B2Q_SM_CASE(1, 8)
  B2Q_SM_CASE(2, 1) B2Q_SM_CASE(2, 2) B2Q_SM_CASE(2, 4) B2Q_SM_CASE(2, 8)
  B2Q_SM_CASE(4, 1) B2Q_SM_CASE(4, 2) B2Q_SM_CASE(4, 4)
#undef B2Q_SM_CASE
  return B2Q_ERR_UNSUPPORTED;
}

// one translation unit per weight format keeps nvcc compile times parallel
int smallm_int4(const SmallMParams& p, bool bf16, int m_max, int n_tiles_cap, cudaStream_t st);
int smallm_fp8_bf16(const SmallMParams& p, int fmt, int smode, int m_max, int n_tiles_cap, cudaStream_t st);
int smallm_fp8_f16(const SmallMParams& p, int fmt, int smode, int m_max, int n_tiles_cap, cudaStream_t st);

}  // namespace b2q
