// Sum of row-parallel partial results over the GPUs of one box, written for the decode shapes of the path
// (M <= 64 tokens, a [M, N] tile of 16-bit values per rank): the step that follows o_proj and down in a
// tensor-parallel decoder layer (vllm/patches/vllm_for_multi_arc.patch:10185, :10199, :8006-8010, where the
// reference calls the framework's all-reduce).
//
// Every rank owns a buffer that all ranks of the box can address (cudaMalloc + CUDA IPC between the processes of
// one box).  The sum runs over plain peer stores and loads; no multicast, no library collective.  Two forms:
//
// two steps (reduce-scatter, then broadcast; the traffic per rank does not grow with W):
//   1. rank r writes columns [j * N/W, (j + 1) * N/W) of its partial tile into slot r of rank j's buffer, for every
//      j, then raises flag1[r][block] on rank j                       (the GEMM epilogue can do this step itself)
//   2. rank j waits for the W flags of a column block, adds the W slots in rank order in fp32 (every rank therefore
//      computes bit-identical sums), rounds once, writes the block into the result area of EVERY rank, raises
//      flag2[j][block] there, and waits for the W flags of its own result.
// one step (decode-sized tiles, where the time is latency, not bytes: one trip over NVLink instead of two):
//   1. rank r writes its WHOLE partial tile into slot r of every rank's buffer and raises flag1[r][block] there
//   2. every rank waits for the W flags of a column block and adds the W slots in rank order in fp32 into its own
//      result area: all ranks add the same values in the same order, so the results are bit-identical here too.
//   Nothing tells a writer that its slot has been read, so the slots exist twice and calls alternate between the
//   sets: a rank can only be two calls ahead of a peer after that peer has raised its flags for the call in
//   between, i.e. after the peer's kernel of the call before that one has finished.
// A column block is 128 columns wide and belongs to one CTA; CTA b of rank j depends only on CTA b (or the GEMM
// CTAs that own those columns) of the other ranks, never on another CTA of its own GPU.
// Flags carry an epoch that the buffer's owner advances once per call, so nothing is cleared between calls.
// Every wait is bounded: when the limit runs out the CTA records a code in the buffer's status word and returns;
// the host reads it with b2q_comm_status.  Nothing faults or spins without bound.
#include <new>
#include <string.h>
#include "common.cuh"
#include "peer_reduce.cuh"

namespace b2q {

struct PeerComm {
  int rank, world, device;
  bool emulated;              // all ranks live in this process on one device (tests)
  bool oneshot;               // one-step form: full-width slots, two slot sets
  size_t bytes, slot_bytes, out_bytes;
  uint8_t* local;
  uint8_t* peers[PR_MAX_WORLD];
  bool opened[PR_MAX_WORLD];
  int64_t max_rows, max_cols;
  uint64_t calls;             // host-side count: picks the result area (two alternate)
};

struct PeerRankArgs {
  const void* in; int64_t ldi;         // this rank's partial tile (nullptr: step 1 was done by the producer)
  uint8_t* bufs[PR_MAX_WORLD];         // every rank's buffer as addressed from this rank
  int rank;
};
struct PeerReduceParams {
  PeerRankArgs r[PR_MAX_WORLD];        // r[0] only, except in the one-device emulation
  int world, M, N, slice, nblocks, bf16, out_sel, oneshot;
  size_t slot_off, slot_bytes, out_off, out_bytes;
  long long limit_ticks;
};

// Waits until *flag has reached `epoch` (flags only grow).  Returns false when the limit ran out.
__device__ __forceinline__ bool wait_flag(const uint32_t* flag, uint32_t epoch, long long limit, PeerCtrl* ctrl, int code) {
  if ((int32_t)(ld_acquire_sys(flag) - epoch) >= 0) return true;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i)          // the flag lives in this GPU's own memory (peers write it): polling is a local load
      if ((int32_t)(ld_acquire_sys(flag) - epoch) >= 0) return true;
    if (clock64() - t0 > limit) {
      atomicCAS(&ctrl->status, 0, code);
      return false;
    }
  }
}

template <bool BF16> __device__ __forceinline__ void add8(float (&acc)[8], const uint4& v) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if constexpr (BF16) {
      acc[2 * i] += __uint_as_float(w[i] << 16);
      acc[2 * i + 1] += __uint_as_float(w[i] & 0xFFFF0000u);
    } else {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      acc[2 * i] += f.x; acc[2 * i + 1] += f.y;
    }
  }
}
template <bool BF16> __device__ __forceinline__ uint4 pack8(const float (&acc)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if constexpr (BF16) {
      __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    } else {
      __half2 h = __floats2half2_rn(acc[2 * i], acc[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// grid (nblocks, ranks on this device); 256 threads.  Block b of rank `me` handles columns [b * 128, b * 128 + cw)
// of every rank's slice in step 1 and of its own slice in step 2.
template <bool BF16>
__global__ void __launch_bounds__(256) peer_reduce_kernel(const PeerReduceParams p) {
  const PeerRankArgs& ra = p.r[blockIdx.y];
  const int me = ra.rank, W = p.world, b = blockIdx.x;
  PeerCtrl* ctrl = reinterpret_cast<PeerCtrl*>(ra.bufs[me]);
  const uint32_t epoch = ctrl->epoch + 1;      // stable for the whole call: only the last CTA to finish advances it
  const int c0 = b * PR_CB;
  const int cw = min(PR_CB, (p.oneshot ? p.N : p.slice) - c0);      // columns of this block (multiple of 8)
  const int vpr = cw >> 3;                      // 16-byte vectors per row
  const int nvec = p.M * vpr;
  // slot layout: [source rank][block][row][128 columns]; result layout: [row][N]
  const size_t blk_off = (size_t)b * p.M * PR_CB * 2;
  bool ok = true;

  if (ra.in) {
    // ---- step 1: this rank's partial columns to their owners ----
    for (int jj = 0; jj < W; ++jj) {
      const int j = (me + 1 + jj) % W;            // start with the neighbour: spreads the links
      uint8_t* dst = ra.bufs[j] + p.slot_off + (size_t)me * p.slot_bytes + blk_off;
      const uint16_t* src = reinterpret_cast<const uint16_t*>(ra.in) + (p.oneshot ? 0 : (size_t)j * p.slice) + c0;
      for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
        const int m = v / vpr, c8 = v - m * vpr;
        const uint4 val = *reinterpret_cast<const uint4*>(src + (size_t)m * ra.ldi + c8 * 8);
        *reinterpret_cast<uint4*>(dst + ((size_t)m * PR_CB + c8 * 8) * 2) = val;
      }
    }
    // one system-scope release per flag covers the whole CTA's stores: the barrier orders them before it
    __syncthreads();
    if (threadIdx.x < W) {
      __threadfence_system();
      st_release_sys(&reinterpret_cast<PeerCtrl*>(ra.bufs[threadIdx.x])->flag1[me][b], epoch);
    }
  }

  // ---- step 2: wait for the W partial blocks, add them in rank order, publish the sum to every rank ----
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < W && !wait_flag(&ctrl->flag1[threadIdx.x][b], epoch, p.limit_ticks, ctrl, PST_FLAG1)) s_ok = 0;
  __syncthreads();
  ok = s_ok != 0;
  if (ok) {
    const uint8_t* slots = ra.bufs[me] + p.slot_off + blk_off;
    const size_t out_base = p.out_off + (size_t)p.out_sel * p.out_bytes;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      const int m = v / vpr, c8 = v - m * vpr;
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int r = 0; r < W; ++r)
        add8<BF16>(acc, __ldcg(reinterpret_cast<const uint4*>(slots + (size_t)r * p.slot_bytes + ((size_t)m * PR_CB + c8 * 8) * 2)));   // past L1: peers wrote it
      const uint4 o = pack8<BF16>(acc);
      if (p.oneshot) {
        *reinterpret_cast<uint4*>(ra.bufs[me] + out_base + ((size_t)m * p.N + c0 + c8 * 8) * 2) = o;
        continue;
      }
      const size_t off = out_base + ((size_t)m * p.N + (size_t)me * p.slice + c0 + c8 * 8) * 2;
      for (int jj = 0; jj < W; ++jj) {
        const int j = (me + jj) % W;
        *reinterpret_cast<uint4*>(ra.bufs[j] + off) = o;
      }
    }
    __syncthreads();
    if (!p.oneshot && threadIdx.x < W) {
      __threadfence_system();
      st_release_sys(&reinterpret_cast<PeerCtrl*>(ra.bufs[threadIdx.x])->flag2[me][b], epoch);
    }
    // ---- step 3: the same block of every other owner has landed here ----
    if (!p.oneshot && threadIdx.x < W && !wait_flag(&ctrl->flag2[threadIdx.x][b], epoch, p.limit_ticks, ctrl, PST_FLAG2)) s_ok = 0;
    __syncthreads();
  }
  // the last CTA of this rank to finish closes the call (also after an expired wait: the next call starts clean)
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t n = atomicAdd(&ctrl->done, 1u);
    if (n == gridDim.x - 1) {
      ctrl->done = 0;
      __threadfence();
      ctrl->epoch = epoch;
    }
  }
}

// buffer: control area | slot sets (one, or two in the one-step form) of W slots | two result areas
static size_t layout_bytes(int world, bool oneshot, int64_t max_rows, int64_t max_cols, size_t* slot_bytes, size_t* out_bytes) {
  const int64_t width = oneshot ? max_cols : max_cols / world;
  const int64_t nblocks = (width + PR_CB - 1) / PR_CB;
  *slot_bytes = (size_t)nblocks * (size_t)max_rows * PR_CB * 2;
  *out_bytes = ((size_t)max_rows * (size_t)max_cols * 2 + 255) / 256 * 256;
  return (size_t)PR_CTRL_BYTES + (oneshot ? 2 : 1) * (size_t)world * *slot_bytes + 2 * *out_bytes;
}
static size_t out_offset(const PeerComm* c) { return (size_t)PR_CTRL_BYTES + (c->oneshot ? 2 : 1) * (size_t)c->world * c->slot_bytes; }

}  // namespace b2q

using namespace b2q;

extern "C" {

int b2q_comm_create_mode(int rank, int world, int64_t max_rows, int64_t max_cols, int mode, void** comm_out, void* ipc_handle_out) {
  if (!comm_out) return B2Q_ERR_NULL;
  if (world < 1 || world > PR_MAX_WORLD || rank < 0 || rank >= world) return B2Q_ERR_SHAPE;
  if (max_rows <= 0 || max_cols <= 0 || (max_cols % (world * 8)) != 0) return B2Q_ERR_SHAPE;
  if (mode < B2Q_COMM_AUTO || mode > B2Q_COMM_TWO_STEPS) return B2Q_ERR_SHAPE;
  // one step while every rank's whole tile to every peer is still a few microseconds of NVLink time (8 MiB out per
  // rank at most): decode tiles on any number of ranks of a box
  const bool oneshot = mode == B2Q_COMM_ONE_STEP ||
                       (mode == B2Q_COMM_AUTO && (int64_t)(world - 1) * max_rows * max_cols * 2 <= ((int64_t)8 << 20));
  if (((oneshot ? max_cols : max_cols / world) + PR_CB - 1) / PR_CB > PR_MAX_BLOCKS || max_rows > 4096) return B2Q_ERR_LIMIT;
  PeerComm* c = new (std::nothrow) PeerComm();
  if (!c) return B2Q_ERR_CUDA;
  c->rank = rank; c->world = world; c->emulated = false; c->oneshot = oneshot; c->calls = 0;
  c->max_rows = max_rows; c->max_cols = max_cols;
  if (cudaGetDevice(&c->device) != cudaSuccess) { delete c; return B2Q_ERR_CUDA; }
  c->bytes = layout_bytes(world, oneshot, max_rows, max_cols, &c->slot_bytes, &c->out_bytes);
  void* p = nullptr;
  if (cudaMalloc(&p, c->bytes) != cudaSuccess) { delete c; return B2Q_ERR_CUDA; }
  if (cudaMemset(p, 0, c->bytes) != cudaSuccess) { cudaFree(p); delete c; return B2Q_ERR_CUDA; }
  c->local = reinterpret_cast<uint8_t*>(p);
  for (int i = 0; i < PR_MAX_WORLD; ++i) { c->peers[i] = nullptr; c->opened[i] = false; }
  c->peers[rank] = c->local;
  if (ipc_handle_out) {
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) { cudaFree(p); delete c; return B2Q_ERR_CUDA; }
    memcpy(ipc_handle_out, &h, sizeof(h));
  }
  *comm_out = c;
  return B2Q_OK;
}

int b2q_comm_create(int rank, int world, int64_t max_rows, int64_t max_cols, void** comm_out, void* ipc_handle_out) {
  return b2q_comm_create_mode(rank, world, max_rows, max_cols, B2Q_COMM_AUTO, comm_out, ipc_handle_out);
}

int b2q_comm_connect(void* comm, const void* all_handles) {
  PeerComm* c = reinterpret_cast<PeerComm*>(comm);
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

int b2q_comm_connect_local(void** comms, int world) {
  if (!comms) return B2Q_ERR_NULL;
  for (int a = 0; a < world; ++a) {
    PeerComm* ca = reinterpret_cast<PeerComm*>(comms[a]);
    if (!ca || ca->world != world || ca->rank != a) return B2Q_ERR_SHAPE;
    for (int b = 0; b < world; ++b) {
      PeerComm* cb = reinterpret_cast<PeerComm*>(comms[b]);
      if (!cb || cb->device != ca->device || cb->oneshot != ca->oneshot) return B2Q_ERR_SHAPE;
      ca->peers[b] = cb->local;
    }
    ca->emulated = true;
  }
  return B2Q_OK;
}

int b2q_comm_destroy(void* comm) {
  PeerComm* c = reinterpret_cast<PeerComm*>(comm);
  if (!c) return B2Q_ERR_NULL;
  cudaDeviceSynchronize();
  for (int r = 0; r < c->world; ++r)
    if (c->opened[r]) cudaIpcCloseMemHandle(c->peers[r]);
  cudaFree(c->local);
  delete c;
  return B2Q_OK;
}

int b2q_comm_result_ptr(void* comm, int which, void** out) {
  PeerComm* c = reinterpret_cast<PeerComm*>(comm);
  if (!c || !out) return B2Q_ERR_NULL;
  if (which < 0 || which > 1) return B2Q_ERR_SHAPE;
  *out = c->local + out_offset(c) + (size_t)which * c->out_bytes;
  return B2Q_OK;
}

int b2q_comm_status(void* comm, int* out) {
  PeerComm* c = reinterpret_cast<PeerComm*>(comm);
  if (!c || !out) return B2Q_ERR_NULL;
  return cuda_status(cudaMemcpy(out, &reinterpret_cast<PeerCtrl*>(c->local)->status, sizeof(int), cudaMemcpyDeviceToHost));
}

int b2q_comm_status_reset(void* comm) {
  PeerComm* c = reinterpret_cast<PeerComm*>(comm);
  if (!c) return B2Q_ERR_NULL;
  if (cudaDeviceSynchronize() != cudaSuccess) return B2Q_ERR_CUDA;
  PeerCtrl* ctrl = reinterpret_cast<PeerCtrl*>(c->local);
  if (cudaMemset(&ctrl->status, 0, sizeof(int)) != cudaSuccess) return B2Q_ERR_CUDA;
  return cuda_status(cudaMemset(&ctrl->done, 0, sizeof(uint32_t)));
}

static int fill_params(PeerComm* c, PeerReduceParams& p, int slot, const void* in, int64_t ldi, int64_t M, int64_t N, int dtype,
                       double limit_ms) {
  if (!is16(dtype)) return B2Q_ERR_DTYPE;
  if (M <= 0 || N <= 0 || M > c->max_rows || N > c->max_cols || (N % (c->world * 8)) != 0) return B2Q_ERR_SHAPE;
  if (in && (ldi < N || !aligned16(in) || ((ldi * 2) & 15))) return B2Q_ERR_ALIGN;
  p.r[slot].in = in; p.r[slot].ldi = ldi; p.r[slot].rank = c->rank;
  for (int r = 0; r < c->world; ++r) {
    if (!c->peers[r]) return B2Q_ERR_NULL;       // not connected
    p.r[slot].bufs[r] = c->peers[r];
  }
  p.world = c->world; p.M = (int)M; p.N = (int)N; p.slice = (int)(N / c->world); p.oneshot = c->oneshot ? 1 : 0;
  p.nblocks = ((c->oneshot ? p.N : p.slice) + PR_CB - 1) / PR_CB; p.bf16 = dtype == B2Q_BF16;
  p.slot_off = PR_CTRL_BYTES + (c->oneshot ? (size_t)(c->calls & 1) * c->world * c->slot_bytes : 0); p.slot_bytes = c->slot_bytes;
  p.out_off = out_offset(c); p.out_bytes = c->out_bytes;
  p.limit_ticks = (long long)(limit_ms * 1.9e6);
  return B2Q_OK;
}

}  // extern "C"

namespace b2q {
// Description of this communicator for a GEMM epilogue that performs step 1 itself (see PeerEpilogue).
int peer_epilogue(void* comm, int64_t M, int64_t N, PeerEpilogue* out) {
  PeerComm* c = reinterpret_cast<PeerComm*>(comm);
  if (!c || !out) return B2Q_ERR_NULL;
  if (c->emulated || c->oneshot) return B2Q_ERR_UNSUPPORTED;
  if (M <= 0 || M > c->max_rows || N > c->max_cols || (N % (c->world * 128)) != 0) return B2Q_ERR_SHAPE;
  for (int r = 0; r < c->world; ++r) {
    if (!c->peers[r]) return B2Q_ERR_NULL;
    out->bufs[r] = c->peers[r];
  }
  out->world = c->world; out->rank = c->rank; out->slice = (int)(N / c->world); out->M = (int)M;
  out->slot_off = PR_CTRL_BYTES; out->slot_bytes = c->slot_bytes;
  return B2Q_OK;
}
}  // namespace b2q

extern "C" {

int b2q_allreduce_sum(void* comm, const void* in, int dtype, int64_t ldi, int64_t M, int64_t N, double wait_limit_ms,
                      void** out, void* stream) {
  PeerComm* c = reinterpret_cast<PeerComm*>(comm);
  if (!c || !out) return B2Q_ERR_NULL;
  if (c->emulated) return B2Q_ERR_UNSUPPORTED;      // ranks that share a device run through b2q_allreduce_sum_emulated
  PeerReduceParams p{};
  int rc = fill_params(c, p, 0, in, ldi, M, N, dtype, wait_limit_ms > 0 ? wait_limit_ms : 2000.0);
  if (rc) return rc;
  p.out_sel = (int)(c->calls & 1);
  c->calls++;
  dim3 grid(p.nblocks, 1, 1);
  // A plain launch, on purpose: let the kernels behind this one begin early (programmatic stream serialization) and
  // the next GEMM's CTAs sit on the SMs polling their barriers while these 32 to 64 CTAs, whose time is all latency,
  // do the exchange: the tensor-parallel decoder layer measured 3 % slower on two GPUs that way.
  if (p.bf16) peer_reduce_kernel<true><<<grid, 256, 0, (cudaStream_t)stream>>>(p);
  else peer_reduce_kernel<false><<<grid, 256, 0, (cudaStream_t)stream>>>(p);
  note_launch("peer_reduce");
  *out = c->local + p.out_off + (size_t)p.out_sel * p.out_bytes;
  return launch_status();
}

int b2q_allreduce_sum_emulated(void** comms, int world, int n_present, const void* const* ins, int dtype, int64_t ldi,
                               int64_t M, int64_t N, double wait_limit_ms, void** outs, void* stream) {
  if (!comms || !ins || !outs) return B2Q_ERR_NULL;
  if (world < 1 || world > PR_MAX_WORLD || n_present < 1 || n_present > world) return B2Q_ERR_SHAPE;
  PeerReduceParams p{};
  for (int r = 0; r < n_present; ++r) {
    PeerComm* c = reinterpret_cast<PeerComm*>(comms[r]);
    if (!c || !c->emulated || c->world != world) return B2Q_ERR_SHAPE;
    int rc = fill_params(c, p, r, ins[r], ldi, M, N, dtype, wait_limit_ms > 0 ? wait_limit_ms : 2000.0);
    if (rc) return rc;
  }
  PeerComm* c0 = reinterpret_cast<PeerComm*>(comms[0]);
  p.out_sel = (int)(c0->calls & 1);
  for (int r = 0; r < n_present; ++r) {
    PeerComm* c = reinterpret_cast<PeerComm*>(comms[r]);
    c->calls++;
    outs[r] = c->local + p.out_off + (size_t)p.out_sel * p.out_bytes;
  }
  // the CTAs of different ranks wait for one another inside this one launch: they must all be resident
  dim3 grid(p.nblocks, n_present, 1);
  int dev = 0, sms = 0, per_sm = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (p.bf16) cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, peer_reduce_kernel<true>, 256, 0);
  else cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, peer_reduce_kernel<false>, 256, 0);
  if ((int)(grid.x * grid.y) > sms * per_sm) return B2Q_ERR_LIMIT;
  void* args[] = {(void*)&p};
  cudaError_t e = p.bf16 ? cudaLaunchCooperativeKernel((void*)peer_reduce_kernel<true>, grid, dim3(256), args, 0, (cudaStream_t)stream)
                         : cudaLaunchCooperativeKernel((void*)peer_reduce_kernel<false>, grid, dim3(256), args, 0, (cudaStream_t)stream);
  note_launch("peer_reduce");
  return cuda_status(e);
}

}  // extern "C"
