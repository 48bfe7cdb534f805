// FP8 instantiations of the decode streaming kernel, bf16 activations.
#include "smallm.cuh"
namespace b2q {
int smallm_fp8_bf16(const SmallMParams& p, int fmt, int smode, int m_max, int n_tiles_cap, cudaStream_t st) {
  if (smode == SM_BLOCK) {
    if (fmt != B2Q_E4M3) return B2Q_ERR_UNSUPPORTED;
    return smallm_dispatch<WF_E4M3, SM_BLOCK, true>(p, m_max, n_tiles_cap, st);
  }
  return fmt == B2Q_E4M3 ? smallm_dispatch<WF_E4M3, SM_POST, true>(p, m_max, n_tiles_cap, st)
                         : smallm_dispatch<WF_E5M2, SM_POST, true>(p, m_max, n_tiles_cap, st);
}
}  // namespace b2q
