// Shared host/device helpers for libb2q (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stddef.h>
#include "../../include/b2q.h"

namespace b2q {

// ---- per-thread bookkeeping exported through the C ABI --------------------
struct ThreadState {
  uint64_t launches = 0;
  const char* last_kernel = "none";
  int force_kernel = 0;
  int overlap_mode = 1;      // programmatic dependent launch: 0 off, 1 on, 2 on + weights declared static
};
ThreadState& tls();

inline void note_launch(const char* name, int n = 1) {
  ThreadState& t = tls();
  t.launches += (uint64_t)n;
  t.last_kernel = name;
}

inline int cuda_status(cudaError_t e) { return e == cudaSuccess ? B2Q_OK : B2Q_ERR_CUDA; }
inline int launch_status() { return cuda_status(cudaGetLastError()); }

// ---- programmatic dependent launch ---------------------------------------------------------------
// A kernel launched through launch_overlapped may begin while the kernel before it on the stream is
// still running; it must execute grid_dep_wait() before it touches anything an earlier kernel may have
// written (and before it writes anything an earlier kernel may still read).  grid_dep_release() lets
// the next kernel on the stream begin.  Both are no-ops for a plain launch.
__device__ __forceinline__ void grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dep_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_overlapped(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool overlap,
                                     Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = overlap ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline int dtype_bytes(int dt) { return dt == B2Q_F32 ? 4 : 2; }
inline bool is16(int dt) { return dt == B2Q_BF16 || dt == B2Q_F16; }

// ---- device: scalar conversions ------------------------------------------
template <bool BF16> struct Act;
template <> struct Act<true> {
  using T = __nv_bfloat16;
  static __device__ __forceinline__ float to_f(T v) { return __bfloat162float(v); }
  static __device__ __forceinline__ T from_f(float v) { return __float2bfloat16_rn(v); }
};
template <> struct Act<false> {
  using T = __half;
  static __device__ __forceinline__ float to_f(T v) { return __half2float(v); }
  static __device__ __forceinline__ T from_f(float v) { return __float2half_rn(v); }
};

__device__ __forceinline__ float load_scalar(const void* p, int64_t i, int dt) {
  if (dt == B2Q_F32) return reinterpret_cast<const float*>(p)[i];
  if (dt == B2Q_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(reinterpret_cast<const __half*>(p)[i]);
}
// The same load split in two: the raw bits now, the fp32 value where it is needed.  A scale fetched from DRAM well
// ahead of its use must stay raw in between, or the warp waits for it at the load.
__device__ __forceinline__ uint32_t load_scalar_raw(const void* p, int64_t i, int dt) {
  if (dt == B2Q_F32) return __ldg(reinterpret_cast<const uint32_t*>(p) + i);
  return (uint32_t)__ldg(reinterpret_cast<const unsigned short*>(p) + i);
}
__device__ __forceinline__ float scalar_from_raw(uint32_t raw, int dt) {
  if (dt == B2Q_F32) return __uint_as_float(raw);
  if (dt == B2Q_BF16) return __uint_as_float(raw << 16);
  return __half2float(__ushort_as_half((unsigned short)raw));
}
__device__ __forceinline__ void store_scalar(void* p, int64_t i, int dt, float v) {
  if (dt == B2Q_F32) reinterpret_cast<float*>(p)[i] = v;
  else if (dt == B2Q_BF16) reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
  else reinterpret_cast<__half*>(p)[i] = __float2half_rn(v);
}

// Exact decode of one fp8 byte to fp32 (e4m3fn: no inf, 0x7f/0xff = NaN; e5m2: IEEE-like).
__device__ __forceinline__ float fp8_to_float(uint32_t b, bool e5m2) {
  if (e5m2) {
    __half_raw h; h.x = (unsigned short)(b << 8);
    return __half2float(__half(h));
  }
  const uint32_t s = (b & 0x80u) << 24;
  const uint32_t e = (b >> 3) & 0xFu;
  const uint32_t m = b & 7u;
  float v;
  if (e == 0) v = (float)m * 0.001953125f;              // m * 2^-9 (subnormal)
  else if (e == 15 && m == 7) v = __int_as_float(0x7fc00000);
  else v = __int_as_float(((e + 120u) << 23) | (m << 20));
  return __int_as_float(__float_as_int(v) | s);
}

// nibble position (bit offset / 4) of k-within-word j for the given INT4 layout
__device__ __forceinline__ int nibble_slot(int j, bool marlin) {
  // marlin shuffle stores old nibble [0,4,1,5,2,6,3,7][p] at position p, so
  // k-within-word j lives at position {0,2,4,6,1,3,5,7}[j].
  return marlin ? ((j & 3) * 2 + (j >> 2)) : j;
}

}  // namespace b2q
