// Dequantisation kernels: the bit-exactness gate for every weight format the
// linear kernels consume.  HBM-bound elementwise work: one thread produces
// eight consecutive k of one row and stores them with a single 16-byte (or
// 32-byte for fp32) write.
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

}  // namespace b2q
