// Expert-parallel exchange over peer memory (NVLink), without a collective library call.
//
// Every rank owns a receive buffer for routed rows, a buffer for returned results and two small
// flag arrays; all of them are mapped into every other rank's address space (CUDA IPC, set up
// by the host layer).  A rank's kernels write rows straight into the destination's buffer with
// plain stores over NVLink, make them visible system-wide (__threadfence_system) and then bump
// a counter in the destination's flag array; the destination's next kernel in stream order is a
// one-CTA wait on those counters.  Counters only grow (each step adds the same, known amount),
// so nothing is reset and a step can be replayed from a CUDA graph.  Waits are bounded (~2 s):
// when one runs out, a status word is set and the kernel returns.
//
// No reference counterpart: the reference runs on one GPU (grouped_payload_sidecar.py:867-868).
// No multicast and no TMA are involved: stores and atomics to mapped peer memory only.
#include <string.h>

#include "common.cuh"

namespace tris {

constexpr int kEpSignalCtas = 296;  // CTAs of the packing and returning kernels: every one of them signals every peer once

__device__ __forceinline__ int ep_owner_of(int e, int base, int extra) {
  const int big = extra * (base + 1);
  return e < big ? e / (base + 1) : extra + (e - big) / max(base, 1);
}

__device__ __forceinline__ int32_t ld_acquire_sys(const int32_t* p) {
  int32_t v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// After this CTA's stores to peer memory: make them visible, then add 1 to counter `slot` of
// every peer's flag array (threads 0..world-1, one peer each).
__device__ __forceinline__ void ep_signal_peers(int32_t* const* peer_flags, int world, int slot) {
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < world) atomicAdd_system(peer_flags[threadIdx.x] + slot, 1);
}

// Dispatch.  Grouped rows are sorted by expert, hence by owner rank.  Slot (d, off) of the send
// layout is row off of the rows owned by rank d; it is written to rank d's receive buffer at
// slot (my_rank, off): two backbone outputs of rank_gu halves each and, behind them, the expert
// id as an int32 (unused slots: -1).  combine_index[flat] = d * capacity + off.
// Two phases, so that a capacity far above the rows in use (the never-dropping world * tokens * top_k)
// costs one 4-byte store per slot and nothing else: (1) one thread per slot writes the id word and the
// combine index; (2) thread groups copy the rows in use, one group per row.
__global__ void __launch_bounds__(128) ep_dispatch_peer_kernel(
    const __half* __restrict__ hidden_gate, const __half* __restrict__ hidden_up, int rank_gu,
    const int32_t* __restrict__ selected, const int32_t* __restrict__ perm, const int32_t* __restrict__ tok,
    int num_rows, int num_experts, int world, int my_rank, int capacity, __half* const* __restrict__ peer_recv,
    int row_stride, int32_t* __restrict__ combine_index, int32_t* __restrict__ overflow,
    int32_t* const* __restrict__ peer_flags) {
  __shared__ int32_t s_first[65];  // first grouped row owned by each rank (world <= 64), then num_rows
  pdl_wait();  // the route and the backbone outputs come from the kernels before this one
  pdl_launch_dependents();
  const int base = num_experts / world, extra = num_experts % world;
  if (threadIdx.x < world) {  // rows are sorted by owner: binary search for each owner's first row
    const int d = threadIdx.x;
    int lo = 0, hi = num_rows;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (ep_owner_of(selected[perm[mid]], base, extra) < d) lo = mid + 1;
      else hi = mid;
    }
    s_first[d] = lo;
  }
  if (threadIdx.x == 0) s_first[world] = num_rows;
  __syncthreads();
  const int total = world * capacity;
  for (int pos = blockIdx.x * blockDim.x + threadIdx.x; pos < total; pos += gridDim.x * blockDim.x) {
    const int d = pos / capacity, off = pos - d * capacity;
    const int row = s_first[d] + off, row_end = s_first[d + 1];
    const bool used = row < row_end;
    const int flat = used ? perm[row] : 0;
    __half* slot = peer_recv[d] + (static_cast<size_t>(my_rank) * capacity + off) * row_stride;
    *reinterpret_cast<int32_t*>(slot + 2 * rank_gu) = used ? selected[flat] : -1;
    if (used) combine_index[flat] = pos;
    if (off == capacity - 1 && row + 1 < row_end) *overflow = 1;  // more rows for this rank than slots
  }
  // rows: 2 * rank_gu / 8 16-byte vectors each, `lanes` threads per row.  Rows beyond an owner's capacity are
  // dropped and their combine index says so (every flat entry is written by exactly one thread of this
  // launch, so the caller need not initialise the array).
  const int vecs = rank_gu >> 3, per_row = 2 * vecs;
  const int lanes = min(per_row, static_cast<int>(blockDim.x));
  const int groups = blockDim.x / lanes;
  const int grp = threadIdx.x / lanes, l = threadIdx.x - grp * lanes;
  if (grp < groups) {
    for (int row = blockIdx.x * groups + grp; row < num_rows; row += gridDim.x * groups) {
      int d = 0;
      while (d + 1 < world && row >= s_first[d + 1]) ++d;
      const int off = row - s_first[d];
      if (off >= capacity) {
        if (l == 0) combine_index[perm[row]] = -1;
        continue;
      }
      const int t = tok[row];
      const uint4* g = reinterpret_cast<const uint4*>(hidden_gate + static_cast<size_t>(t) * rank_gu);
      const uint4* u = reinterpret_cast<const uint4*>(hidden_up + static_cast<size_t>(t) * rank_gu);
      uint4* dst = reinterpret_cast<uint4*>(peer_recv[d] + (static_cast<size_t>(my_rank) * capacity + off) * row_stride);
      for (int i = l; i < per_row; i += lanes) dst[i] = (i < vecs) ? g[i] : u[i - vecs];
    }
  }
  ep_signal_peers(peer_flags, world, my_rank);
}

// Return.  results [world * capacity, hidden] holds, in received-slot order, the output rows of
// the rows this rank processed; block s goes back to rank s, into block my_rank of its result
// buffer.  Rows whose received id is negative (padding) are skipped: every thread looks at one slot
// of a batch, the slots in use are listed in shared memory and the warps copy those, one row each.
__global__ void __launch_bounds__(256) ep_return_peer_kernel(
    const __half* __restrict__ results, const __half* __restrict__ recv_rows, int row_stride, int rank_gu,
    int hidden, int world, int my_rank, int capacity, __half* const* __restrict__ peer_back,
    int32_t* const* __restrict__ peer_flags) {
  __shared__ int32_t s_live[256];
  __shared__ int s_count;
  pdl_wait();
  pdl_launch_dependents();
  const int vecs = hidden >> 3;
  const int total = world * capacity;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  // slot of (batch, thread, CTA): consecutive threads of a CTA are gridDim.x slots apart, so the slots in
  // use (the first few of every peer's block) spread over all CTAs
  for (int first = 0; first < total; first += gridDim.x * blockDim.x) {
    if (threadIdx.x == 0) s_count = 0;
    __syncthreads();
    const int pos = first + threadIdx.x * gridDim.x + blockIdx.x;
    if (pos < total) {
      const int32_t id = *reinterpret_cast<const int32_t*>(recv_rows + static_cast<size_t>(pos) * row_stride + 2 * rank_gu);
      if (id >= 0) s_live[atomicAdd(&s_count, 1)] = pos;
    }
    __syncthreads();
    const int n = s_count;
    for (int j = warp; j < n; j += warps) {
      const int p = s_live[j];
      const int s = p / capacity, off = p - s * capacity;
      const uint4* src = reinterpret_cast<const uint4*>(results + static_cast<size_t>(p) * hidden);
      uint4* dst = reinterpret_cast<uint4*>(peer_back[s] + (static_cast<size_t>(my_rank) * capacity + off) * hidden);
      for (int i = lane; i < vecs; i += 32) dst[i] = src[i];
    }
    __syncthreads();  // the list is rebuilt by the next batch
  }
  ep_signal_peers(peer_flags, world, my_rank);
}

// One CTA: waits until every peer's counter has reached (*step + 1) * increment, then advances
// *step.  Gives up after ~2 s and records TRIS_ERR_TIMEOUT.
__global__ void ep_wait_kernel(const int32_t* flags, int32_t* step, int increment, int world, int32_t* status) {
  __shared__ int s_timeout;
  pdl_wait();  // *step was advanced by an earlier wait kernel of this stream
  if (threadIdx.x == 0) s_timeout = 0;
  __syncthreads();
  const int32_t target = (*step + 1) * increment;
  if (threadIdx.x < world) {
    const unsigned long long t0 = global_timer_ns();
    while (ld_acquire_sys(flags + threadIdx.x) - target < 0) {  // counters wrap like the target does
      if (global_timer_ns() - t0 > 2000000000ull) {
        s_timeout = 1;
        break;
      }
      __nanosleep(64);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    *step += 1;
    if (s_timeout && status) atomicExch(status, TRIS_ERR_TIMEOUT);
  }
}

}  // namespace tris

using namespace tris;

extern "C" int tris_ep_signal_increment(void) { return kEpSignalCtas; }

extern "C" int tris_ep_enable_peer_access(int32_t peer_device) {
  int dev = 0;
  TRIS_CUDA(cudaGetDevice(&dev));
  if (peer_device == dev) return TRIS_OK;
  int can = 0;
  TRIS_CUDA(cudaDeviceCanAccessPeer(&can, dev, peer_device));
  TRIS_REQUIRE(can != 0, TRIS_ERR_UNSUPPORTED, "device %d cannot access device %d (no NVLink / P2P path)", dev, peer_device);
  const cudaError_t err = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (err == cudaErrorPeerAccessAlreadyEnabled) {
    cudaGetLastError();  // clear the sticky "already enabled"
    return TRIS_OK;
  }
  return check_cuda(err, "cudaDeviceEnablePeerAccess");
}

// Maps memory another process exported with cudaIpcGetMemHandle into the current device's
// context (the device whose kernels will use it), enabling peer access to the exporting device
// as needed.  *base_out is the exporter's allocation base.
extern "C" int tris_ep_open_peer_memory(const void* ipc_handle_64, void** base_out) {
  TRIS_REQUIRE(ipc_handle_64 && base_out, TRIS_ERR_INVALID_ARG, "tris_ep_open_peer_memory: null pointer");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  cudaIpcMemHandle_t handle;
  memcpy(&handle, ipc_handle_64, sizeof(handle));
  return check_cuda(cudaIpcOpenMemHandle(base_out, handle, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
}

extern "C" int tris_ep_close_peer_memory(void* base) {
  TRIS_REQUIRE(base != nullptr, TRIS_ERR_INVALID_ARG, "tris_ep_close_peer_memory: null pointer");
  return check_cuda(cudaIpcCloseMemHandle(base), "cudaIpcCloseMemHandle");
}

extern "C" int tris_ep_dispatch_peer(const void* hidden_gate_f16, const void* hidden_up_f16, int32_t rank_gu,
                                     const int32_t* selected_experts, const int32_t* perm,
                                     const int32_t* grouped_token_indices, int32_t num_rows, int32_t num_experts,
                                     int32_t world, int32_t my_rank, int32_t capacity, void* const* peer_recv_rows_dev,
                                     int32_t row_stride, int32_t* combine_index, int32_t* overflow_dev,
                                     int32_t* const* peer_flags_dev, void* stream) {
  TRIS_REQUIRE(hidden_gate_f16 && hidden_up_f16 && selected_experts && perm && grouped_token_indices &&
                   peer_recv_rows_dev && combine_index && overflow_dev && peer_flags_dev,
               TRIS_ERR_INVALID_ARG, "tris_ep_dispatch_peer: null pointer");
  TRIS_REQUIRE(rank_gu > 0 && (rank_gu & 7) == 0, TRIS_ERR_UNSUPPORTED, "tris_ep_dispatch_peer: rank must be a multiple of 8");
  TRIS_REQUIRE(row_stride >= 2 * rank_gu + 8 && (row_stride & 7) == 0, TRIS_ERR_INVALID_ARG,
               "tris_ep_dispatch_peer: row_stride %d must be a multiple of 8 and >= 2*rank + 8", row_stride);
  TRIS_REQUIRE(num_rows >= 0 && num_experts > 0 && world >= 1 && world <= 64 && my_rank >= 0 && my_rank < world &&
                   capacity > 0,
               TRIS_ERR_INVALID_ARG, "tris_ep_dispatch_peer: bad sizes rows=%d world=%d rank=%d capacity=%d", num_rows,
               world, my_rank, capacity);
  return check_cuda(
      launch_kernel(ep_dispatch_peer_kernel, dim3(kEpSignalCtas), dim3(128), 0, static_cast<cudaStream_t>(stream),
                    programmatic_launch_default(), 1, static_cast<const __half*>(hidden_gate_f16),
                    static_cast<const __half*>(hidden_up_f16), rank_gu, selected_experts, perm, grouped_token_indices, num_rows,
                    num_experts, world, my_rank, capacity, reinterpret_cast<__half* const*>(peer_recv_rows_dev), row_stride,
                    combine_index, overflow_dev, peer_flags_dev),
      "ep_dispatch_peer_kernel launch");
}

extern "C" int tris_ep_return_peer(const void* results_f16, const void* recv_rows_f16, int32_t row_stride,
                                   int32_t rank_gu, int32_t hidden_size, int32_t world, int32_t my_rank,
                                   int32_t capacity, void* const* peer_back_dev, int32_t* const* peer_flags_dev,
                                   void* stream) {
  TRIS_REQUIRE(results_f16 && recv_rows_f16 && peer_back_dev && peer_flags_dev, TRIS_ERR_INVALID_ARG,
               "tris_ep_return_peer: null pointer");
  TRIS_REQUIRE(hidden_size > 0 && (hidden_size & 7) == 0 && row_stride >= 2 * rank_gu + 8, TRIS_ERR_INVALID_ARG,
               "tris_ep_return_peer: bad sizes hidden=%d stride=%d rank=%d", hidden_size, row_stride, rank_gu);
  TRIS_REQUIRE(world >= 1 && world <= 64 && my_rank >= 0 && my_rank < world && capacity > 0, TRIS_ERR_INVALID_ARG,
               "tris_ep_return_peer: bad sizes world=%d rank=%d capacity=%d", world, my_rank, capacity);
  return check_cuda(
      launch_kernel(ep_return_peer_kernel, dim3(kEpSignalCtas), dim3(256), 0, static_cast<cudaStream_t>(stream),
                    programmatic_launch_default(), 1, static_cast<const __half*>(results_f16),
                    static_cast<const __half*>(recv_rows_f16), row_stride, rank_gu, hidden_size, world, my_rank, capacity,
                    reinterpret_cast<__half* const*>(peer_back_dev), peer_flags_dev),
      "ep_return_peer_kernel launch");
}

extern "C" int tris_ep_wait(const int32_t* flags_dev, int32_t* step_dev, int32_t world, int32_t* status_dev,
                            void* stream) {
  TRIS_REQUIRE(flags_dev && step_dev, TRIS_ERR_INVALID_ARG, "tris_ep_wait: null pointer");
  TRIS_REQUIRE(world >= 1 && world <= 64, TRIS_ERR_INVALID_ARG, "tris_ep_wait: world=%d", world);
  return check_cuda(launch_kernel(ep_wait_kernel, dim3(1), dim3(64), 0, static_cast<cudaStream_t>(stream),
                                  programmatic_launch_default(), 1, flags_dev, step_dev, kEpSignalCtas, world, status_dev),
                    "ep_wait_kernel launch");
}
