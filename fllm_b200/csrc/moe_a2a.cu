// Expert-parallel all-to-all over peer memory (NVLink P2P stores and system-scope atomics): the
// token rows a rank owns travel only to the ranks that hold their routed experts, and the expert
// outputs travel back to the owner. Four small kernels around the existing align / gather / grouped
// GEMM chain:
//
//   ep_dispatch   (token owner)  for every (token, slot): claim a row in the expert owner's receive
//                                buffer with one system-scope atomic, store the row and its tag there;
//                                the last CTA publishes "rank s is done" on every peer
//   ep_ingest     (expert owner) wait for every source's flag (bounded), read the row count, emit the
//                                expert id of every received row (-1 past the count) for moe_align
//   ep_return     (expert owner) store each computed row into its owner's combine buffer at
//                                (token, slot), reset the receive counter, publish "rank d returned"
//   ep_wait       (token owner)  wait for every expert owner's flag; moe_combine then forms the
//                                weighted sum locally
//
// Flags carry the call number (monotonic; every rank makes the same calls in the same order), so nothing
// is reset between calls except the row counter, which its owner clears before it publishes the return
// flag: no sender can claim a row of the next call earlier. The call number lives in device memory
// (`call_ctr`, local to the rank): the dispatch kernel uses counter + 1 and its last CTA stores that
// value back, the three kernels after it read the stored value. A captured graph therefore replays
// with the right number without the host. (A host-passed number is still accepted when no counter is given.)
// Every wait is poll-bounded and reports FLLM_ERR_PEER_TIMEOUT through the status word.
//
// The reference does this on the host (rust/engine/src/parallel/decoder_shard.rs:442-446 dispatch,
// :478-480, :506-508 combine).
#include <algorithm>

#include "fllm_ops.h"
#include "ptx.cuh"
#include "tma_host.h"

namespace fllm {

constexpr uint32_t kEpWaitPolls = 1u << 22;

struct EpPeers {
  __nv_bfloat16* recv_x[kMaxEp];      // [cap][hidden] on each rank
  int4* recv_meta[kMaxEp];            // [cap] {src_rank, src_entry, expert, 0}
  uint32_t* ctrl[kMaxEp];             // [0] row counter, [8..16) dispatch flags, [16..24) return flags, [24] done CTAs
  __nv_bfloat16* comb_y[kMaxEp];      // [max_entries][hidden] on each rank
  int ranks, my_rank, cap, hidden, experts_per_rank;
};

__global__ void __launch_bounds__(256)
ep_dispatch_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const int* __restrict__ ids, int entries, int k,
                   const EpPeers p, uint32_t epoch, uint32_t* __restrict__ call_ctr, int* __restrict__ status) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = p.hidden / 8;
  // read before this CTA reports itself done: the store below happens after every CTA did
  if (call_ctr) epoch = *reinterpret_cast<volatile uint32_t*>(call_ctr) + 1;
  for (int i = blockIdx.x * 8 + warp; i < entries; i += gridDim.x * 8) {
    const int e = ids[i];
    const int dst = e / p.experts_per_rank;
    if (e < 0 || dst >= p.ranks) continue;
    uint32_t slot = 0;
    if (lane == 0) slot = atomicAdd_system(p.ctrl[dst], 1u);
    slot = __shfl_sync(0xffffffffu, slot, 0);
    if (slot >= (uint32_t)p.cap) {                     // receive buffer too small for this routing
      if (lane == 0 && status) atomicCAS(status, FLLM_OK, FLLM_ERR_PEER_TIMEOUT);
      continue;
    }
    const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(i / k) * ldx);
    uint4* dstp = reinterpret_cast<uint4*>(p.recv_x[dst] + (size_t)slot * p.hidden);
    for (int v = lane; v < nvec; v += 32) dstp[v] = src[v];
    if (lane == 0) p.recv_meta[dst][slot] = make_int4(p.my_rank, i, e, 0);
  }
  // publish once every CTA's stores are out
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t* done = p.ctrl[p.my_rank] + 24;
    if (atomicAdd(done, 1u) == gridDim.x - 1) {
      *done = 0;
      if (call_ctr) *call_ctr = epoch;
      __threadfence_system();
      for (int d = 0; d < p.ranks; ++d) st_release_sys(p.ctrl[d] + 8 + p.my_rank, epoch);
    }
  }
}

// One CTA. ids_out[cap]: expert id of each received row, -1 for unused rows.
__global__ void __launch_bounds__(1024)
ep_ingest_kernel(const EpPeers p, uint32_t epoch, const uint32_t* __restrict__ call_ctr, int* __restrict__ ids_out,
                 int* __restrict__ count_out, int* __restrict__ status) {
  __shared__ int ok;
  if (call_ctr) epoch = *call_ctr;
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  if (threadIdx.x < p.ranks) {
    if (!wait_flag_ge(p.ctrl[p.my_rank] + 8 + threadIdx.x, epoch, kEpWaitPolls)) {
      ok = 0;
      if (status) atomicCAS(status, FLLM_OK, FLLM_ERR_PEER_TIMEOUT);
    }
  }
  __syncthreads();
  const int n = ok ? min((int)ld_acquire_sys(p.ctrl[p.my_rank]), p.cap) : 0;
  if (threadIdx.x == 0) *count_out = n;
  for (int i = threadIdx.x; i < p.cap; i += blockDim.x) ids_out[i] = i < n ? p.recv_meta[p.my_rank][i].z : -1;
}

// y: expert outputs in permuted order; row_of[slot]: permuted row of received row `slot`.
__global__ void __launch_bounds__(256)
ep_return_kernel(const __nv_bfloat16* __restrict__ y, long long ldy, const int* __restrict__ row_of,
                 const int* __restrict__ count, const EpPeers p, uint32_t epoch, const uint32_t* __restrict__ call_ctr) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = p.hidden / 8;
  const int n = *count;
  if (call_ctr) epoch = *call_ctr;
  for (int s = blockIdx.x * 8 + warp; s < n; s += gridDim.x * 8) {
    const int4 m = p.recv_meta[p.my_rank][s];
    const int row = row_of[s];
    if (row < 0 || m.x < 0 || m.x >= p.ranks) continue;
    const uint4* src = reinterpret_cast<const uint4*>(y + (size_t)row * ldy);
    uint4* dst = reinterpret_cast<uint4*>(p.comb_y[m.x] + (size_t)m.y * p.hidden);
    for (int v = lane; v < nvec; v += 32) dst[v] = src[v];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t* done = p.ctrl[p.my_rank] + 24;
    if (atomicAdd(done, 1u) == gridDim.x - 1) {
      *done = 0;
      *p.ctrl[p.my_rank] = 0;                           // rows of the next call start at 0 again
      __threadfence_system();
      for (int d = 0; d < p.ranks; ++d) st_release_sys(p.ctrl[d] + 16 + p.my_rank, epoch);
    }
  }
}

__global__ void ep_wait_kernel(const EpPeers p, uint32_t epoch, const uint32_t* __restrict__ call_ctr, int* __restrict__ status) {
  if (call_ctr) epoch = *call_ctr;
  if (threadIdx.x < p.ranks) {
    if (!wait_flag_ge(p.ctrl[p.my_rank] + 16 + threadIdx.x, epoch, kEpWaitPolls) && status)
      atomicCAS(status, FLLM_OK, FLLM_ERR_PEER_TIMEOUT);
  }
}

static EpPeers to_peers(const EpArgs& a) {
  if (a.ranks < 1 || a.ranks > kMaxEp) throw std::runtime_error("expert-parallel all-to-all: 1..8 ranks");
  if (a.hidden % 8) throw std::runtime_error("expert-parallel all-to-all: hidden must be a multiple of 8");
  EpPeers p{};
  for (int i = 0; i < a.ranks; ++i) {
    p.recv_x[i] = reinterpret_cast<__nv_bfloat16*>(a.recv_x[i]);
    p.recv_meta[i] = reinterpret_cast<int4*>(a.recv_meta[i]);
    p.ctrl[i] = reinterpret_cast<uint32_t*>(a.ctrl[i]);
    p.comb_y[i] = reinterpret_cast<__nv_bfloat16*>(a.comb_y[i]);
  }
  p.ranks = a.ranks; p.my_rank = a.my_rank; p.cap = a.cap; p.hidden = a.hidden; p.experts_per_rank = a.experts_per_rank;
  return p;
}

void ep_dispatch(const EpArgs& a, const void* x, long long ldx, const int* ids, int tokens, int k, unsigned epoch,
                 unsigned* call_ctr, int* status, cudaStream_t s) {
  const EpPeers p = to_peers(a);
  const int entries = tokens * k;
  const int blocks = std::max(1, std::min((entries + 7) / 8, 2 * sm_count()));
  ep_dispatch_kernel<<<blocks, 256, 0, s>>>((const __nv_bfloat16*)x, ldx, ids, entries, k, p, epoch, call_ctr, status);
  cuda_check(cudaGetLastError(), "ep_dispatch_kernel");
}

void ep_ingest(const EpArgs& a, unsigned epoch, const unsigned* call_ctr, int* ids_out, int* count_out, int* status,
               cudaStream_t s) {
  ep_ingest_kernel<<<1, 1024, 0, s>>>(to_peers(a), epoch, call_ctr, ids_out, count_out, status);
  cuda_check(cudaGetLastError(), "ep_ingest_kernel");
}

void ep_return(const EpArgs& a, const void* y, long long ldy, const int* row_of, const int* count, unsigned epoch,
               const unsigned* call_ctr, cudaStream_t s) {
  const EpPeers p = to_peers(a);
  const int blocks = std::max(1, std::min((a.cap + 7) / 8, 2 * sm_count()));
  ep_return_kernel<<<blocks, 256, 0, s>>>((const __nv_bfloat16*)y, ldy, row_of, count, p, epoch, call_ctr);
  cuda_check(cudaGetLastError(), "ep_return_kernel");
}

void ep_wait_returns(const EpArgs& a, unsigned epoch, const unsigned* call_ctr, int* status, cudaStream_t s) {
  ep_wait_kernel<<<1, 32, 0, s>>>(to_peers(a), epoch, call_ctr, status);
  cuda_check(cudaGetLastError(), "ep_wait_kernel");
}

}  // namespace fllm
