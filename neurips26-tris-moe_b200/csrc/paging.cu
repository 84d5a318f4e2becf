// Streaming loader: gathers the payload blocks of the experts a batch routes to from pinned
// host memory into device staging slots.  The copy is a kernel that reads the (device-mapped)
// host buffers directly, so the set of active experts never has to travel to the host: the
// launch is enqueued on a side stream right after the route kernel and ordered with events.
#include <algorithm>

#include "common.cuh"

namespace tris {

struct PageArgs {
  TrisPageJob jobs[TRIS_MAX_PAGE_JOBS];
  int32_t num_jobs;
  const int32_t* expert_ids;
  const int32_t* num_segments_dev;
  int32_t num_segments;
  int32_t num_experts;
  int32_t* slot_table;
};

// grid (chunks, segment bound, jobs); 256 threads, 16 bytes per thread per step
__global__ void __launch_bounds__(256) page_experts_kernel(const __grid_constant__ PageArgs args) {
  const int seg = blockIdx.y;
  const int nseg = args.num_segments_dev ? min(*args.num_segments_dev, args.num_segments) : args.num_segments;
  if (seg >= nseg) return;
  const int e = args.expert_ids[seg];
  if (e < 0 || e >= args.num_experts) return;
  if (blockIdx.x == 0 && blockIdx.z == 0 && threadIdx.x == 0) args.slot_table[e] = seg;
  const TrisPageJob& job = args.jobs[blockIdx.z];
  const long long vecs = job.bytes_per_expert >> 4;
  const uint4* src = reinterpret_cast<const uint4*>(static_cast<const char*>(job.host_src) + e * job.bytes_per_expert);
  uint4* dst = reinterpret_cast<uint4*>(static_cast<char*>(job.dst) + seg * job.bytes_per_expert);
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  // eight independent 16-byte reads in flight per thread: host reads cross PCIe/C2C, whose latency
  // (microseconds) has to be covered by bytes in flight
  for (; i + 7 * stride < vecs; i += 8 * stride) {
    uint4 v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = __ldcs(src + i + j * stride);
#pragma unroll
    for (int j = 0; j < 8; ++j) dst[i + j * stride] = v[j];
  }
  for (; i < vecs; i += stride) dst[i] = __ldcs(src + i);
}

}  // namespace tris

using namespace tris;

extern "C" int tris_page_experts(const TrisPageJob* jobs, int32_t num_jobs, const int32_t* expert_ids,
                                 const int32_t* num_segments_dev, int32_t num_segments, int32_t num_experts,
                                 int32_t* slot_table, void* stream) {
  TRIS_REQUIRE(jobs && expert_ids && slot_table, TRIS_ERR_INVALID_ARG, "tris_page_experts: null pointer");
  TRIS_REQUIRE(num_jobs >= 1 && num_jobs <= TRIS_MAX_PAGE_JOBS, TRIS_ERR_INVALID_ARG,
               "tris_page_experts: %d jobs (1..%d supported)", num_jobs, TRIS_MAX_PAGE_JOBS);
  TRIS_REQUIRE(num_segments >= 0 && num_experts > 0, TRIS_ERR_INVALID_ARG, "tris_page_experts: bad sizes");
  if (num_segments == 0) return TRIS_OK;
  PageArgs args{};
  long long max_bytes = 0;
  for (int j = 0; j < num_jobs; ++j) {
    TRIS_REQUIRE(jobs[j].host_src && jobs[j].dst && jobs[j].bytes_per_expert > 0 && (jobs[j].bytes_per_expert & 15) == 0,
                 TRIS_ERR_INVALID_ARG, "tris_page_experts: job %d needs pointers and a block size that is a multiple of 16", j);
    TRIS_REQUIRE(((reinterpret_cast<uintptr_t>(jobs[j].host_src) | reinterpret_cast<uintptr_t>(jobs[j].dst)) & 15) == 0,
                 TRIS_ERR_INVALID_ARG, "tris_page_experts: job %d buffers must be 16-byte aligned", j);
    args.jobs[j] = jobs[j];
    // the kernel dereferences the host buffer: translate to its device alias (same address under UVA)
    void* dev_alias = nullptr;
    TRIS_CUDA(cudaHostGetDevicePointer(&dev_alias, const_cast<void*>(jobs[j].host_src), 0));
    args.jobs[j].host_src = dev_alias;
    max_bytes = std::max<long long>(max_bytes, jobs[j].bytes_per_expert);
  }
  args.num_jobs = num_jobs;
  args.expert_ids = expert_ids;
  args.num_segments_dev = num_segments_dev;
  args.num_segments = num_segments;
  args.num_experts = num_experts;
  args.slot_table = slot_table;
  // Experts that get no slot (more live segments than num_segments) must not keep a stale entry:
  // the grouped kernels treat -1 as "not paged in", store nothing and report TRIS_ERR_WORKSPACE.
  TRIS_CUDA(cudaMemsetAsync(slot_table, 0xFF, sizeof(int32_t) * static_cast<size_t>(num_experts), static_cast<cudaStream_t>(stream)));
  const int chunks = static_cast<int>(std::min<long long>(16, std::max<long long>(1, max_bytes / (256 * 16 * 8))));
  page_experts_kernel<<<dim3(chunks, num_segments, num_jobs), 256, 0, static_cast<cudaStream_t>(stream)>>>(args);
  return check_cuda(cudaGetLastError(), "page_experts_kernel launch");
}
