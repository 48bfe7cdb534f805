// Buffer layout and flag protocol shared by the peer-memory reduction kernel (peer_reduce.cu) and the GEMM epilogue
// that performs the reduction's first step itself (umma_gemm.cu).
#pragma once
#include "common.cuh"

namespace b2q {

constexpr int PR_MAX_WORLD = 8;
constexpr int PR_MAX_BLOCKS = 512;        // column blocks of 128 per flag row: N / W (two steps) or N (one step) <= 65536
constexpr int PR_CB = 128;                // columns per block
constexpr int PR_CTRL_BYTES = 4096 + 2 * PR_MAX_WORLD * PR_MAX_BLOCKS * 4;

// control area at the start of every rank's buffer
struct PeerCtrl {
  uint32_t epoch;        // calls completed by this rank
  uint32_t done;         // CTAs of the current call that have finished (last one advances epoch)
  int32_t status;        // first expired wait (0 = none)
  uint32_t pad[1021];
  uint32_t flag1[PR_MAX_WORLD][PR_MAX_BLOCKS];   // [source rank][block]: partial block has landed (value = epoch)
  uint32_t flag2[PR_MAX_WORLD][PR_MAX_BLOCKS];   // [owner rank][block]: reduced block has landed
};
static_assert(sizeof(PeerCtrl) == PR_CTRL_BYTES, "control area layout");

enum { PST_FLAG1 = 201, PST_FLAG2 = 202 };

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}


// What a GEMM needs in order to deliver its output tile straight into the slots of the owner ranks (step 1 of the
// two-step reduction) instead of into local memory: a strip of 128 output columns belongs to one owner rank and one
// block.  The one-step form is not fed this way: there the strip would go to every rank with 2-byte peer stores from
// inside the GEMM, which measured slower on two GPUs than the GEMM followed by the reduction kernel.
struct PeerEpilogue {
  uint8_t* bufs[PR_MAX_WORLD];     // every rank's buffer as addressed from this rank
  int world, rank, slice, M;       // slice = N / world (a multiple of 128 for this path), M = rows of the tile
  size_t slot_off, slot_bytes;
};

}  // namespace b2q
