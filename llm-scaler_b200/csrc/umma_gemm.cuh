// Host-side interface of the tcgen05 (UMMA) weight-only GEMM family.
#pragma once
#include "common.cuh"

namespace b2q {

// Common tail of the argument blocks: optional grouped (MoE) mode.
struct UmmaGroupArgs {
  const int32_t* expert_offsets = nullptr;  // [E+1]; nullptr = dense
  int E = 0;
  const int32_t* row_map = nullptr; int row_div = 1;
  const int32_t* out_map = nullptr;
  int act = B2Q_ACT_NONE;
  const int32_t* tiles = nullptr;           // device tile list {n, pad3, int2...}
  int tile_cap = 0;
  int64_t s_expert_elems = 0;
  // scratch for the balanced decode mode (partial sums of strips cut between CTAs), umma_balanced_ws_bytes(M)
  // bytes; without it every strip is one CTA's job
  void* sk_ws = nullptr; size_t sk_ws_bytes = 0;
  // the activation pre-pass of the same call was launched directly before this GEMM: everything older on the
  // stream is then known to be complete, so the weight stream may start before the pre-pass has finished
  bool after_prep = false;
};

struct UmmaW4Args : UmmaGroupArgs {
  const void* x; int64_t ldx; bool bf16;      // bf16: element type of x (the MMA input type)
  bool out_bf16; const float* tok_scale;      // output type; optional per-token multiplier
  bool magic;                                 // x is the pre-pass output (fp16, scaled, pair-permuted)
  const void* w; int layout;
  const void* scale; int scale_dtype; int64_t s_stride_n, s_stride_g;
  void* out; int64_t ldo;
  int M, N, K;
  const struct PeerEpilogue* peer = nullptr;   // decode tiles: deliver the output to the owner ranks' reduction slots
};

struct UmmaW8Args : UmmaGroupArgs {
  const void* x; int64_t ldx; bool bf16;      // bf16: element type of x (the MMA input type)
  bool out_bf16; const float* tok_scale;      // output type; optional per-token multiplier
  const void* w; int fmt;
  const void* scale; int scale_dtype; int scale_mode;
  void* out; int64_t ldo;
  int M, N, K;
};

struct UmmaW8A8Args {
  const void* xq; const float* xs; const void* w; const float* ws;
  void* out; bool bf16; int64_t ldo;
  int M, N, K;
};

// FP8-weight decode GEMM on the 8-bit MMA: the activations arrive split into e4m3 terms (act_split_fp8).
struct UmmaW8DirectArgs {
  const void* xq; const float* inv_scale; int terms;      // [umma_w8_direct_rows, K] e4m3, [M], 2 (bf16) or 3 (fp16)
  const void* w; int fmt;
  const void* scale; int scale_dtype; int scale_mode;     // per channel or per tensor
  void* out; int64_t ldo; bool out_bf16;
  int M, N, K;
  void* partials; size_t partial_bytes;                   // umma_w8_direct_partial_bytes(M), or null: strips are not cut
};
int umma_w8_direct_rows(int64_t M, bool bf16);
size_t umma_w8_direct_partial_bytes(int64_t M);
int umma_w8_direct_linear(const UmmaW8DirectArgs& a, cudaStream_t st);

// INT4 decode GEMM on the int8 MMA: the activations arrive split into three int8 terms (act_split_i8).
struct UmmaW4I8Args {
  const void* xq; const float* inv_scale; const float* xsum;   // [umma_w4_i8_rows, K] s8 (k permuted in eights), [M], [K/128][Mp]
  const void* w; uint32_t xor_mask;                            // N-major nibbles; 0x88888888 for two's-complement storage
  const void* scale; int scale_dtype; int64_t s_stride_n, s_stride_g;
  void* out; int64_t ldo; bool out_bf16;
  int M, N, K;
  void* partials; size_t partial_bytes;                        // umma_w4_i8_partial_bytes(), or null: strips are not cut
};
int umma_w4_i8_rows(int64_t M);
bool umma_w4_i8_preferred(int64_t M, int64_t N, int64_t K);
size_t umma_w4_i8_partial_bytes();
int umma_w4_i8_linear(const UmmaW4I8Args& a, cudaStream_t st);

bool umma_w4_supported(const UmmaW4Args& a);
int umma_w4_token_tile(const UmmaW4Args& a);
int umma_w4_linear(const UmmaW4Args& a, cudaStream_t st);

bool umma_w8_supported(const UmmaW8Args& a);
int umma_w8_token_tile(const UmmaW8Args& a);
int umma_w8_linear(const UmmaW8Args& a, cudaStream_t st);

int umma_w8a8_block(const UmmaW8A8Args& a, cudaStream_t st);

size_t umma_balanced_ws_bytes(int64_t M);

// First device-side wait timeout recorded since the library was loaded (0 = none).  Synchronises.
int umma_read_status(int* out);
// Clears the status word of the tcgen05 weight-only kernels; launches the bounded-wait self-test (see the kernel).
int umma_reset_status();
int umma_selftest_bounded_wait(int code, int* gave_up_dev, cudaStream_t st);

}  // namespace b2q

namespace b2q {
struct PeerEpilogue;
int peer_epilogue(void* comm, int64_t M, int64_t N, PeerEpilogue* out);
}
