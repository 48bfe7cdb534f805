// Dequantisation kernels: the bit-exactness gate for every weight format the
// linear kernels consume.  HBM-bound elementwise work: one thread produces
// eight consecutive k of one row and stores them with a single 16-byte (or
// 32-byte for fp32) write.
#include <cuda_fp8.h>
#include "common.cuh"

namespace b2q {

// out[n, k] = round((q - 8) * s) with q taken from the layout-specific nibble.
// The fp32 product of an integer in [-8, 7] and a 16-bit scale is exact, so the
// single rounding to out_dtype matches ((q - 8).float() * s.float()).to(dtype).
__global__ void dequant_int4_kernel(const uint32_t* __restrict__ w, int layout, const void* __restrict__ scale,
                                    int scale_dtype, void* __restrict__ out, int out_dtype, int64_t N, int64_t K,
                                    int group) {
  const int64_t K8 = K >> 3;
  const int64_t total = N * K8;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    int64_t n, k8;
    const bool kmajor = (layout == B2Q_W4_KMAJOR || layout == B2Q_W4_KMAJOR_MARLIN);
    if (kmajor) { k8 = idx / N; n = idx % N; }   // coalesced reads along n
    else { n = idx / K8; k8 = idx % K8; }
    const uint32_t word = kmajor ? w[k8 * N + n] : w[n * K8 + k8];
    const int64_t kg = (k8 * 8) / group;
    const float s = kmajor ? load_scalar(scale, kg * N + n, scale_dtype)
                           : load_scalar(scale, n * (K / group) + kg, scale_dtype);
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int slot = nibble_slot(j, layout == B2Q_W4_KMAJOR_MARLIN);
      int q = (int)((word >> (4 * slot)) & 0xFu);
      if (layout == B2Q_W4_NMAJOR_S4) q = (q >= 8 ? q - 16 : q);
      else q -= 8;
      v[j] = (float)q * s;
    }
    const int64_t o = n * K + k8 * 8;
    if (out_dtype == B2Q_F32) {
      float4* po = reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + o);
      po[0] = make_float4(v[0], v[1], v[2], v[3]);
      po[1] = make_float4(v[4], v[5], v[6], v[7]);
    } else {
      uint32_t pk[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (out_dtype == B2Q_BF16) {
          __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
          pk[j] = *reinterpret_cast<uint32_t*>(&h);
        } else {
          __half2 h = __floats2half2_rn(v[2 * j], v[2 * j + 1]);
          pk[j] = *reinterpret_cast<uint32_t*>(&h);
        }
      }
      *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(out) + o) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
    }
  }
}

__global__ void dequant_fp8_kernel(const uint8_t* __restrict__ w, int fmt, const void* __restrict__ scale,
                                   int scale_dtype, int scale_mode, void* __restrict__ out, int out_dtype,
                                   int64_t N, int64_t K) {
  const int64_t K8 = K >> 3;
  const int64_t total = N * K8;
  const int64_t kblocks = (K + 127) >> 7;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t n = idx / K8, k8 = idx % K8;
    const uint2 raw = *reinterpret_cast<const uint2*>(w + n * K + k8 * 8);
    float s;
    if (scale_mode == B2Q_SCALE_CHANNEL) s = load_scalar(scale, n, scale_dtype);
    else if (scale_mode == B2Q_SCALE_TENSOR) s = load_scalar(scale, 0, scale_dtype);
    else s = load_scalar(scale, (n >> 7) * kblocks + ((k8 * 8) >> 7), scale_dtype);
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t b = ((j < 4 ? raw.x : raw.y) >> (8 * (j & 3))) & 0xFFu;
      v[j] = fp8_to_float(b, fmt == B2Q_E5M2) * s;
    }
    const int64_t o = n * K + k8 * 8;
    if (out_dtype == B2Q_F32) {
      float4* po = reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + o);
      po[0] = make_float4(v[0], v[1], v[2], v[3]);
      po[1] = make_float4(v[4], v[5], v[6], v[7]);
    } else {
      uint32_t pk[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (out_dtype == B2Q_BF16) {
          __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
          pk[j] = *reinterpret_cast<uint32_t*>(&h);
        } else {
          __half2 h = __floats2half2_rn(v[2 * j], v[2 * j + 1]);
          pk[j] = *reinterpret_cast<uint32_t*>(&h);
        }
      }
      *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(out) + o) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
    }
  }
}

static inline int grid_for(int64_t work, int block) {
  int64_t g = (work + block - 1) / block;
  const int64_t cap = 148 * 16;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

int dequant_int4(const void* w, int layout, const void* scale, int scale_dtype, void* out, int out_dtype,
                 int64_t N, int64_t K, int group, cudaStream_t st) {
  dequant_int4_kernel<<<grid_for(N * (K / 8), 256), 256, 0, st>>>(
      reinterpret_cast<const uint32_t*>(w), layout, scale, scale_dtype, out, out_dtype, N, K, group);
  note_launch("dequant_int4");
  return launch_status();
}

int dequant_fp8(const void* w, int fmt, const void* scale, int scale_dtype, int scale_mode, void* out,
                int out_dtype, int64_t N, int64_t K, cudaStream_t st) {
  dequant_fp8_kernel<<<grid_for(N * (K / 8), 256), 256, 0, st>>>(
      reinterpret_cast<const uint8_t*>(w), fmt, scale, scale_dtype, scale_mode, out, out_dtype, N, K);
  note_launch("dequant_fp8");
  return launch_status();
}

// ---------------------------------------------------------------------------
// GGML Q4_0 quantiser, group 128: the load-time step that produces the INT4 path's inputs.
// Restates csrc/xpu/q4_0_quant.sycl:29-125 operation by operation so that the bytes agree:
//   signed maximum of the group (the positive one wins a tie of magnitudes), d = max / -8 in fp32,
//   id = 1 / d in fp32 (0 when d == 0), scale = fp16(d), q = clamp(int(x * id + 8.5), 0, 15) with the
//   product and the sum rounded separately and the conversion truncating, nibble i of a word at bits 4i.
// One warp per (row, group): a lane owns four consecutive elements.
template <bool IN_BF16>
__global__ void quantize_q4_0_kernel(const void* __restrict__ x, int64_t ldx, uint32_t* __restrict__ qweight,
                                     __half* __restrict__ scale, int64_t M, int K) {
  const int lane = threadIdx.x & 31;
  const int64_t unit = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int groups = K >> 7;
  if (unit >= M * groups) return;
  const int64_t row = unit / groups;
  const int g = (int)(unit - row * groups);
  const uint16_t* src = reinterpret_cast<const uint16_t*>(x) + row * ldx + (int64_t)g * 128 + lane * 4;
  const uint2 raw = *reinterpret_cast<const uint2*>(src);
  const uint16_t h[4] = {(uint16_t)(raw.x & 0xFFFF), (uint16_t)(raw.x >> 16), (uint16_t)(raw.y & 0xFFFF), (uint16_t)(raw.y >> 16)};
  float v[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] = IN_BF16 ? __uint_as_float((uint32_t)h[i] << 16) : __half2float(__ushort_as_half(h[i]));
  float max_pos = fmaxf(fmaxf(v[0], v[1]), fmaxf(v[2], v[3]));
  float neg_max = fmaxf(fmaxf(-v[0], -v[1]), fmaxf(-v[2], -v[3]));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    max_pos = fmaxf(max_pos, __shfl_xor_sync(0xffffffffu, max_pos, o));
    neg_max = fmaxf(neg_max, __shfl_xor_sync(0xffffffffu, neg_max, o));
  }
  const float max_signed = max_pos >= neg_max ? max_pos : -neg_max;
  const float d = __fdiv_rn(max_signed, -8.0f);
  const float id = d != 0.0f ? __frcp_rn(d) : 0.0f;
  uint32_t nib = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int q = (int)__fadd_rn(__fmul_rn(v[i], id), 8.5f);      // two roundings, then truncation
    q = q < 0 ? 0 : (q > 15 ? 15 : q);
    nib |= (uint32_t)q << (4 * i);
  }
  const uint32_t other = __shfl_down_sync(0xffffffffu, nib, 1);
  if ((lane & 1) == 0) qweight[row * (int64_t)(K >> 3) + g * 16 + (lane >> 1)] = nib | (other << 16);
  if (lane == 0) scale[row * groups + g] = __float2half_rn(d);
}

int quantize_q4_0(const void* x, bool in_bf16, int64_t ldx, void* qweight, void* scale, int64_t M, int64_t K, cudaStream_t st) {
  const int64_t units = M * (K / 128);
  if (units == 0) return B2Q_OK;
  const int wpb = 8;
  const unsigned grid = (unsigned)((units + wpb - 1) / wpb);
  if (in_bf16)
    quantize_q4_0_kernel<true><<<grid, wpb * 32, 0, st>>>(x, ldx, reinterpret_cast<uint32_t*>(qweight),
                                                          reinterpret_cast<__half*>(scale), M, (int)K);
  else
    quantize_q4_0_kernel<false><<<grid, wpb * 32, 0, st>>>(x, ldx, reinterpret_cast<uint32_t*>(qweight),
                                                           reinterpret_cast<__half*>(scale), M, (int)K);
  note_launch("quantize_q4_0");
  return launch_status();
}

// ---------------------------------------------------------------------------
// FP8 (e4m3) weight quantisers, the load-time step that produces the FP8 GEMMs' inputs:
//   scale = max(amax, 1e-12) / 448 in fp32 over the scale's domain (a 128 x 128 block, an output row, the tensor),
//   q = e4m3(w / scale): an IEEE fp32 division, then one round-to-nearest-even conversion
// (tests/test_fp8_blockscale_gemm.py:13-28 for the block form).  Ragged edge blocks take their maximum over the
// elements that exist.  Source types: bf16, fp16, fp32.
__device__ __forceinline__ float load_src(const void* w, int64_t i, int dt) { return load_scalar(w, i, dt); }

__device__ __forceinline__ float block_max(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float a = 0.f;
  for (int i = 0; i < (int)(blockDim.x >> 5); ++i) a = fmaxf(a, red[i]);
  __syncthreads();
  return a;
}

__device__ __forceinline__ uint8_t to_e4m3(float v, float s) {
  return (uint8_t)__nv_cvt_float_to_fp8(__fdiv_rn(v, s), __NV_SATFINITE, __NV_E4M3);
}

// one CTA of 256 threads per 128 x 128 block; thread t owns column t % 128 of rows t / 128, t / 128 + 2, ...
__global__ void quantize_fp8_block_kernel(const void* __restrict__ w, int dt, int64_t ldw, uint8_t* __restrict__ wq,
                                          float* __restrict__ scale, int64_t N, int64_t K) {
  __shared__ float red[8];
  const int64_t kb = blockIdx.x, nb = blockIdx.y;
  const int c = threadIdx.x & 127, r0 = threadIdx.x >> 7;
  const int64_t k = kb * 128 + c;
  float amax = 0.f;
  if (k < K)
    for (int r = r0; r < 128; r += 2) {
      const int64_t n = nb * 128 + r;
      if (n < N) amax = fmaxf(amax, fabsf(load_src(w, n * ldw + k, dt)));
    }
  amax = block_max(amax, red);
  const float s = __fdiv_rn(fmaxf(amax, 1e-12f), 448.0f);
  if (threadIdx.x == 0) scale[nb * gridDim.x + kb] = s;
  if (k < K)
    for (int r = r0; r < 128; r += 2) {
      const int64_t n = nb * 128 + r;
      if (n < N) wq[n * K + k] = to_e4m3(load_src(w, n * ldw + k, dt), s);
    }
}

// one CTA per output row
__global__ void quantize_fp8_channel_kernel(const void* __restrict__ w, int dt, int64_t ldw, uint8_t* __restrict__ wq,
                                            float* __restrict__ scale, int64_t K) {
  __shared__ float red[32];
  const int64_t n = blockIdx.x;
  float amax = 0.f;
  for (int64_t k = threadIdx.x; k < K; k += blockDim.x) amax = fmaxf(amax, fabsf(load_src(w, n * ldw + k, dt)));
  amax = block_max(amax, red);
  const float s = __fdiv_rn(fmaxf(amax, 1e-12f), 448.0f);
  if (threadIdx.x == 0) scale[n] = s;
  for (int64_t k = threadIdx.x; k < K; k += blockDim.x) wq[n * K + k] = to_e4m3(load_src(w, n * ldw + k, dt), s);
}

// per tensor: the maximum is gathered in scale[0] as the bit pattern of a non-negative float (which orders like an
// unsigned integer), the elements are quantised against it, and a last one-thread launch turns it into the scale
__global__ void quantize_fp8_tensor_max_kernel(const void* __restrict__ w, int dt, int64_t ldw, float* scale, int64_t N,
                                               int64_t K) {
  __shared__ float red[32];
  float amax = 0.f;
  const int64_t total = N * K;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x)
    amax = fmaxf(amax, fabsf(load_src(w, (i / K) * ldw + (i % K), dt)));
  amax = block_max(amax, red);
  if (threadIdx.x == 0) atomicMax(reinterpret_cast<unsigned int*>(scale), __float_as_uint(amax));
}

__global__ void quantize_fp8_tensor_kernel(const void* __restrict__ w, int dt, int64_t ldw, uint8_t* __restrict__ wq,
                                           const float* scale, int64_t N, int64_t K) {
  const float s = __fdiv_rn(fmaxf(scale[0], 1e-12f), 448.0f);
  const int64_t total = N * K;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x)
    wq[i] = to_e4m3(load_src(w, (i / K) * ldw + (i % K), dt), s);
}

__global__ void quantize_fp8_tensor_finish_kernel(float* scale) { scale[0] = __fdiv_rn(fmaxf(scale[0], 1e-12f), 448.0f); }

int quantize_fp8(const void* w, int dt, int64_t ldw, void* wq, float* scale, int scale_mode, int64_t N, int64_t K,
                 cudaStream_t st) {
  if (N == 0 || K == 0) return B2Q_OK;
  uint8_t* q = reinterpret_cast<uint8_t*>(wq);
  if (scale_mode == B2Q_SCALE_BLOCK128) {
    const dim3 grid((unsigned)((K + 127) / 128), (unsigned)((N + 127) / 128));
    quantize_fp8_block_kernel<<<grid, 256, 0, st>>>(w, dt, ldw, q, scale, N, K);
    note_launch("quantize_fp8_block");
  } else if (scale_mode == B2Q_SCALE_CHANNEL) {
    quantize_fp8_channel_kernel<<<(unsigned)N, 256, 0, st>>>(w, dt, ldw, q, scale, K);
    note_launch("quantize_fp8_channel");
  } else {
    if (cudaMemsetAsync(scale, 0, sizeof(float), st) != cudaSuccess) return B2Q_ERR_CUDA;
    const int64_t total = N * K;
    int64_t g = (total + 1023) / 1024;
    g = g > 148 * 8 ? 148 * 8 : g;
    quantize_fp8_tensor_max_kernel<<<(unsigned)g, 256, 0, st>>>(w, dt, ldw, scale, N, K);
    quantize_fp8_tensor_kernel<<<(unsigned)g, 256, 0, st>>>(w, dt, ldw, q, scale, N, K);
    quantize_fp8_tensor_finish_kernel<<<1, 1, 0, st>>>(scale);
    note_launch("quantize_fp8_tensor");
  }
  return launch_status();
}

}  // namespace b2q
