// placeholder until the tcgen05 kernels land
#include "umma_gemm.cuh"
namespace b2q {
bool umma_w4_supported(const UmmaW4Args&) { return false; }
int umma_w4_token_tile(const UmmaW4Args&) { return 64; }
int umma_w4_linear(const UmmaW4Args&, cudaStream_t) { return B2Q_ERR_UNSUPPORTED; }
bool umma_w8_supported(const UmmaW8Args&) { return false; }
int umma_w8_token_tile(const UmmaW8Args&) { return 64; }
int umma_w8_linear(const UmmaW8Args&, cudaStream_t) { return B2Q_ERR_UNSUPPORTED; }
int umma_w8a8_block(const UmmaW8A8Args&, cudaStream_t) { return B2Q_ERR_UNSUPPORTED; }
}  // namespace b2q
