// Token exchange of an expert-parallel MoE layer over the GPUs of one box: rows travel to the rank that owns their
// expert and the results travel back, by plain peer stores, with every count kept on the device.
//
// The reference splits the experts contiguously over the ranks (vllm/patches/vllm_for_multi_arc.patch:3356-3365) and
// has no exchange kernel of its own: it emulates the all-to-all with an all-gather and a reduce-scatter of the whole
// batch (:1559-1563).  A library all-to-all needs the row counts on the host before it can be issued, i.e. a
// device-to-host read and a stalled stream twice per layer.  Here nothing leaves the device:
//
//   dispatch  rank r holds its (token, slot) pairs sorted by destination rank (a counting sort by b2q_moe_route with
//             the ranks as "experts": order[], offsets[W + 1]).  One kernel copies row order[p] / top_k of x into slot r
//             of the destination's receive area, at the pair's position inside its destination segment, together with
//             the expert's index on that rank; positions of the slot that stay empty get the index -1.  The last CTA
//             to finish writes the segment's length and its offset in r's send order next to the flags and raises
//             flag_d[r] on every rank.
//   compute   the owner waits for the W flags (one warp, bounded) and runs the grouped GEMMs over the whole receive
//             area [W x cap rows]: the counting sort drops the -1 entries, so only the filled rows are gathered, and
//             the kernels learn the row count from the sort's last offset, on the device.
//   return    one kernel copies result row (s, i), i < count_in[s], into position src_off[s] + i of rank s's return
//             area, i.e. into the source's send order; the last CTA raises flag_r on every rank.  The source waits for
//             its W flags and combines as on one GPU.
//
// cap = the largest number of pairs one rank can send (its tokens x top_k): a slot can take all of them, so nothing
// is ever dropped and no count has to be known before the copy.  Flags carry a pass number (epoch) that the last
// wait of a pass advances, so nothing is cleared between passes.  A rank can only begin pass k + 1 after every
// owner has returned its rows of pass k, which those owners do after they have finished reading their receive
// areas: the areas need no double buffering.  Every wait is bounded and reports through a status word; nothing
// faults or spins without end.
#include <new>
#include <string.h>
#include "common.cuh"
#include "peer_reduce.cuh"      // ld_acquire_sys / st_release_sys

namespace b2q {

constexpr int EP_MAX_WORLD = 8;
constexpr int EP_CTRL_BYTES = 4096;
enum { EST_DISPATCH = 301, EST_RETURN = 302 };

struct EpCtrl {
  uint32_t epoch;                    // passes completed by this rank
  uint32_t done_d, done_r;           // CTAs of the running dispatch / return kernel that have finished
  int32_t status;                    // first expired wait (0 = none)
  uint32_t flag_d[EP_MAX_WORLD];     // [source]: its rows for this rank have landed (value = pass number)
  uint32_t flag_r[EP_MAX_WORLD];     // [owner]: its results for this rank have landed
  int32_t count_in[EP_MAX_WORLD];    // [source]: rows it sent here in this pass
  int32_t src_off[EP_MAX_WORLD];     // [source]: where those rows sit in the source's send order
};
static_assert(sizeof(EpCtrl) <= EP_CTRL_BYTES, "control area layout");

struct EpComm {
  int rank, world, device;
  bool emulated;
  int64_t cap, H;
  size_t bytes, ids_off, rows_off, ret_off;
  uint8_t* local;
  uint8_t* peers[EP_MAX_WORLD];
  bool opened[EP_MAX_WORLD];
};

struct EpParams {
  uint8_t* bufs[EP_MAX_WORLD];
  int rank, world, top_k;
  int64_t cap, H, n_pairs;
  size_t ids_off, rows_off, ret_off;
  const uint16_t* x; int64_t ldx;           // dispatch: source rows ; return: the owner's results [W * cap, H]
  const int32_t* order; const int32_t* dest_offsets; const int32_t* local_ids;
};

// The CTA's stores are done (barrier), made visible box-wide (one fence), and counted; the last CTA of the kernel
// returns true to exactly one thread, which then publishes.
__device__ __forceinline__ bool last_cta_done(uint32_t* counter) {
  __syncthreads();
  if (threadIdx.x != 0) return false;
  __threadfence_system();
  const uint32_t old = atomicAdd(counter, 1u);
  if (old != gridDim.x - 1) return false;
  *counter = 0;
  __threadfence_system();
  return true;
}

__device__ __forceinline__ void copy_row(uint8_t* dst, const uint16_t* src, int64_t H, int lane) {
  const uint4* s = reinterpret_cast<const uint4*>(src);
  uint4* d = reinterpret_cast<uint4*>(dst);
  for (int64_t v = lane; v < (H >> 3); v += 32) d[v] = s[v];
}

// grid: any; 256 threads = 8 warps, one row per warp at a time
__global__ void __launch_bounds__(256) ep_dispatch_kernel(const EpParams p) {
  __shared__ int32_t off[EP_MAX_WORLD + 1];
  EpCtrl* ctrl = reinterpret_cast<EpCtrl*>(p.bufs[p.rank]);
  const uint32_t epoch = ctrl->epoch + 1;
  const int W = p.world, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x <= W) off[threadIdx.x] = p.dest_offsets[threadIdx.x];
  __syncthreads();
  const int64_t nwarps = (int64_t)gridDim.x * 8, w0 = (int64_t)blockIdx.x * 8 + warp;
  for (int64_t q = w0; q < p.n_pairs; q += nwarps) {
    int j = 0;
    while (j + 1 < W && q >= off[j + 1]) ++j;
    const int64_t i = q - off[j];
    const int pair = p.order[q];
    uint8_t* base = p.bufs[j];
    copy_row(base + p.rows_off + ((size_t)p.rank * p.cap + i) * p.H * 2, p.x + (int64_t)(pair / p.top_k) * p.ldx, p.H, lane);
    if (lane == 0) reinterpret_cast<int32_t*>(base + p.ids_off)[(size_t)p.rank * p.cap + i] = p.local_ids[q];
  }
  // the rest of this rank's slot on every destination is empty
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x, t0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (int64_t q = t0; q < (int64_t)W * p.cap; q += nthreads) {
    const int j = (int)(q / p.cap);
    const int64_t i = q - (int64_t)j * p.cap;
    if (i >= off[j + 1] - off[j]) reinterpret_cast<int32_t*>(p.bufs[j] + p.ids_off)[(size_t)p.rank * p.cap + i] = -1;
  }
  if (last_cta_done(&ctrl->done_d)) {
    for (int j = 0; j < W; ++j) {
      EpCtrl* c = reinterpret_cast<EpCtrl*>(p.bufs[j]);
      c->count_in[p.rank] = off[j + 1] - off[j];
      c->src_off[p.rank] = off[j];
    }
    __threadfence_system();
    for (int j = 0; j < W; ++j) st_release_sys(&reinterpret_cast<EpCtrl*>(p.bufs[j])->flag_d[p.rank], epoch);
  }
}

__global__ void __launch_bounds__(256) ep_return_kernel(const EpParams p) {
  EpCtrl* ctrl = reinterpret_cast<EpCtrl*>(p.bufs[p.rank]);
  const uint32_t epoch = ctrl->epoch + 1;
  const int W = p.world, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t nwarps = (int64_t)gridDim.x * 8, w0 = (int64_t)blockIdx.x * 8 + warp;
  for (int64_t q = w0; q < (int64_t)W * p.cap; q += nwarps) {
    const int s = (int)(q / p.cap);
    const int64_t i = q - (int64_t)s * p.cap;
    if (i >= ctrl->count_in[s]) continue;
    copy_row(p.bufs[s] + p.ret_off + ((size_t)ctrl->src_off[s] + i) * p.H * 2, p.x + q * p.ldx, p.H, lane);
  }
  if (last_cta_done(&ctrl->done_r))
    for (int j = 0; j < W; ++j) st_release_sys(&reinterpret_cast<EpCtrl*>(p.bufs[j])->flag_r[p.rank], epoch);
}

// One warp: lane s waits for rank s's flag of this pass.  phase 0: the dispatch flags; phase 1: the return flags,
// after which the pass is over and the pass number advances (also when a wait ran out: the next pass starts clean).
__global__ void ep_wait_kernel(uint8_t* local, int world, int phase, long long limit_ticks) {
  EpCtrl* ctrl = reinterpret_cast<EpCtrl*>(local);
  const uint32_t epoch = ctrl->epoch + 1;
  const int lane = threadIdx.x;
  if (lane < world) {
    const uint32_t* flag = phase == 0 ? &ctrl->flag_d[lane] : &ctrl->flag_r[lane];
    const long long t0 = clock64();
    while ((int32_t)(ld_acquire_sys(flag) - epoch) < 0) {
      if (clock64() - t0 > limit_ticks) {
        atomicCAS(&ctrl->status, 0, phase == 0 ? EST_DISPATCH : EST_RETURN);
        break;
      }
    }
  }
  __syncwarp();
  if (phase == 1 && lane == 0) {
    __threadfence();
    ctrl->epoch = epoch;
  }
}

}  // namespace b2q

using namespace b2q;

extern "C" {

int b2q_ep_create(int rank, int world, int64_t cap_rows, int64_t H, void** comm_out, void* ipc_handle_out) {
  if (!comm_out) return B2Q_ERR_NULL;
  if (world < 1 || world > EP_MAX_WORLD || rank < 0 || rank >= world) return B2Q_ERR_SHAPE;
  if (cap_rows <= 0 || H <= 0 || (H % 8) != 0) return B2Q_ERR_SHAPE;
  if (cap_rows > (1 << 20) || (int64_t)world * cap_rows > INT32_MAX) return B2Q_ERR_LIMIT;
  EpComm* c = new (std::nothrow) EpComm();
  if (!c) return B2Q_ERR_CUDA;
  c->rank = rank; c->world = world; c->emulated = false; c->cap = cap_rows; c->H = H;
  if (cudaGetDevice(&c->device) != cudaSuccess) { delete c; return B2Q_ERR_CUDA; }
  auto up = [](size_t v) { return (v + 255) / 256 * 256; };
  c->ids_off = EP_CTRL_BYTES;
  c->rows_off = c->ids_off + up((size_t)world * cap_rows * 4);
  c->ret_off = c->rows_off + up((size_t)world * cap_rows * H * 2);
  c->bytes = c->ret_off + up((size_t)cap_rows * H * 2);
  void* p = nullptr;
  if (cudaMalloc(&p, c->bytes) != cudaSuccess) { delete c; return B2Q_ERR_CUDA; }
  if (cudaMemset(p, 0, EP_CTRL_BYTES) != cudaSuccess) { cudaFree(p); delete c; return B2Q_ERR_CUDA; }
  c->local = reinterpret_cast<uint8_t*>(p);
  for (int i = 0; i < EP_MAX_WORLD; ++i) { c->peers[i] = nullptr; c->opened[i] = false; }
  c->peers[rank] = c->local;
  if (ipc_handle_out) {
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) { cudaFree(p); delete c; return B2Q_ERR_CUDA; }
    memcpy(ipc_handle_out, &h, sizeof(h));
  }
  *comm_out = c;
  return B2Q_OK;
}

int b2q_ep_connect(void* comm, const void* all_handles) {
  EpComm* c = reinterpret_cast<EpComm*>(comm);
  if (!c || !all_handles) return B2Q_ERR_NULL;
  const uint8_t* hs = reinterpret_cast<const uint8_t*>(all_handles);
  for (int r = 0; r < c->world; ++r) {
    if (r == c->rank) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, hs + (size_t)r * sizeof(h), sizeof(h));
    void* p = nullptr;
    if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) return B2Q_ERR_CUDA;
    c->peers[r] = reinterpret_cast<uint8_t*>(p);
    c->opened[r] = true;
  }
  return B2Q_OK;
}

int b2q_ep_connect_local(void** comms, int world) {
  if (!comms) return B2Q_ERR_NULL;
  for (int a = 0; a < world; ++a) {
    EpComm* ca = reinterpret_cast<EpComm*>(comms[a]);
    if (!ca || ca->world != world || ca->rank != a) return B2Q_ERR_SHAPE;
    for (int b = 0; b < world; ++b) {
      EpComm* cb = reinterpret_cast<EpComm*>(comms[b]);
      if (!cb || cb->device != ca->device || cb->cap != ca->cap || cb->H != ca->H) return B2Q_ERR_SHAPE;
      ca->peers[b] = cb->local;
    }
    ca->emulated = true;
  }
  return B2Q_OK;
}

int b2q_ep_destroy(void* comm) {
  EpComm* c = reinterpret_cast<EpComm*>(comm);
  if (!c) return B2Q_ERR_NULL;
  cudaDeviceSynchronize();
  for (int r = 0; r < c->world; ++r)
    if (c->opened[r]) cudaIpcCloseMemHandle(c->peers[r]);
  cudaFree(c->local);
  delete c;
  return B2Q_OK;
}

int b2q_ep_status(void* comm, int* out) {
  EpComm* c = reinterpret_cast<EpComm*>(comm);
  if (!c || !out) return B2Q_ERR_NULL;
  return cuda_status(cudaMemcpy(out, &reinterpret_cast<EpCtrl*>(c->local)->status, sizeof(int), cudaMemcpyDeviceToHost));
}

int b2q_ep_buffers(void* comm, void** recv_rows, void** recv_ids, void** ret_rows) {
  EpComm* c = reinterpret_cast<EpComm*>(comm);
  if (!c) return B2Q_ERR_NULL;
  if (recv_rows) *recv_rows = c->local + c->rows_off;
  if (recv_ids) *recv_ids = c->local + c->ids_off;
  if (ret_rows) *ret_rows = c->local + c->ret_off;
  return B2Q_OK;
}

static int ep_params(EpComm* c, EpParams& p) {
  for (int r = 0; r < c->world; ++r) {
    if (!c->peers[r]) return B2Q_ERR_NULL;       // not connected
    p.bufs[r] = c->peers[r];
  }
  p.rank = c->rank; p.world = c->world; p.cap = c->cap; p.H = c->H;
  p.ids_off = c->ids_off; p.rows_off = c->rows_off; p.ret_off = c->ret_off;
  return B2Q_OK;
}

int b2q_ep_dispatch(void* comm, const void* x, int dtype, int64_t ldx, const int32_t* order, int top_k,
                    const int32_t* dest_offsets, const int32_t* local_ids, int64_t n_pairs, void* stream) {
  EpComm* c = reinterpret_cast<EpComm*>(comm);
  if (!c || !x || !order || !dest_offsets || !local_ids) return B2Q_ERR_NULL;
  if (!is16(dtype)) return B2Q_ERR_DTYPE;
  if (n_pairs < 0 || n_pairs > c->cap || top_k <= 0 || ldx < c->H) return B2Q_ERR_SHAPE;
  if (!aligned16(x) || ((ldx * 2) & 15)) return B2Q_ERR_ALIGN;
  EpParams p{};
  int rc = ep_params(c, p);
  if (rc) return rc;
  p.top_k = top_k; p.n_pairs = n_pairs; p.x = reinterpret_cast<const uint16_t*>(x); p.ldx = ldx;
  p.order = order; p.dest_offsets = dest_offsets; p.local_ids = local_ids;
  const int64_t want = (n_pairs + 7) / 8;
  const unsigned grid = (unsigned)(want < 1 ? 1 : (want > 1184 ? 1184 : want));      // 8 CTAs per SM at most: rows in flight, not CTAs, move the bytes
  ep_dispatch_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(p);
  note_launch("ep_dispatch");
  return launch_status();
}

int b2q_ep_return(void* comm, const void* y, int dtype, int64_t ldy, void* stream) {
  EpComm* c = reinterpret_cast<EpComm*>(comm);
  if (!c || !y) return B2Q_ERR_NULL;
  if (!is16(dtype)) return B2Q_ERR_DTYPE;
  if (ldy < c->H) return B2Q_ERR_SHAPE;
  if (!aligned16(y) || ((ldy * 2) & 15)) return B2Q_ERR_ALIGN;
  EpParams p{};
  int rc = ep_params(c, p);
  if (rc) return rc;
  p.x = reinterpret_cast<const uint16_t*>(y); p.ldx = ldy;
  const int64_t want = ((int64_t)c->world * c->cap + 7) / 8;
  const unsigned grid = (unsigned)(want < 1 ? 1 : (want > 1184 ? 1184 : want));
  ep_return_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(p);
  note_launch("ep_return");
  return launch_status();
}

int b2q_ep_wait(void* comm, int phase, double wait_limit_ms, void* stream) {
  EpComm* c = reinterpret_cast<EpComm*>(comm);
  if (!c) return B2Q_ERR_NULL;
  if (phase != 0 && phase != 1) return B2Q_ERR_SHAPE;
  const double ms = wait_limit_ms > 0 ? wait_limit_ms : 2000.0;
  ep_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(c->local, c->world, phase, (long long)(ms * 1.9e6));
  note_launch("ep_wait");
  return launch_status();
}

}  // extern "C"
