// INT4 (g=128) instantiations of the decode streaming kernel.
#include "smallm.cuh"
namespace b2q {
int smallm_int4(const SmallMParams& p, bool bf16, int m_max, int n_tiles_cap, cudaStream_t st) {
  return bf16 ? smallm_dispatch<WF_INT4, SM_GROUP, true>(p, m_max, n_tiles_cap, st)
              : smallm_dispatch<WF_INT4, SM_GROUP, false>(p, m_max, n_tiles_cap, st);
}
}  // namespace b2q
