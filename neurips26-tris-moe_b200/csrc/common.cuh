// Shared helpers for the trismoe_b200 kernels: status plumbing, PTX wrappers.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/trismoe_b200.h"

static_assert(sizeof(TrisProjView) == 224, "TrisProjView layout is part of the ABI");
static_assert(sizeof(TrisPacked4View) == 112, "TrisPacked4View layout changed: update the ctypes mirror");
static_assert(sizeof(TrisRouteView) == 80, "TrisRouteView layout is part of the ABI");

namespace tris {

// ---- host-side error plumbing ---------------------------------------------------------
void set_last_error(const char* fmt, ...);
int fail(int status, const char* fmt, ...);
int check_cuda(cudaError_t err, const char* what);

#define TRIS_REQUIRE(cond, status, ...)            \
  do {                                             \
    if (!(cond)) return ::tris::fail((status), __VA_ARGS__); \
  } while (0)

#define TRIS_CUDA(call)                                              \
  do {                                                               \
    int _st = ::tris::check_cuda((call), #call);                     \
    if (_st != TRIS_OK) return _st;                                  \
  } while (0)

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Position (in halves) of column j of a 32-column group in "lane order" (TRIS_OUT_F16_LANE_ORDER,
// TRIS_ROUTE_HIDDEN_LANE_ORDER): lane t of a warp finds its eight columns t+8, t+24, t, t+16, t+12,
// t+28, t+4, t+20 in 16 consecutive bytes.
__host__ __device__ inline int lane_order_pos(int j) {
  const int t = j & 3, q = (j >> 2) & 3, h = (j >> 4) & 1;
  const int slot = (0x2031 >> (4 * q)) & 3;  // q = 0, 1, 2, 3 -> 1, 3, 0, 2
  return 8 * t + 2 * slot + h;
}
// Column position of output m in the layout `out_mode` names (TRIS_OUT_F16_*).
__host__ __device__ inline int out_mode_pos(int m, int out_mode) {
  if (out_mode == TRIS_OUT_F16_PAIR_INTERLEAVED) return (m & ~31) | ((m & 15) << 1) | ((m >> 4) & 1);
  if (out_mode == TRIS_OUT_F16_LANE_ORDER) return (m & ~31) | lane_order_pos(m & 31);
  return m;
}

// One matrix of the shared skinny GEMM (skinny_gemm.cu): out[n, m] = x[n, :] . a[m, :].
struct SkinnyProblem {
  const __half* a;   // [m, k]
  void* out;         // [n, m], layout TRIS_OUT_*
  int32_t m;
  int32_t out_mode;
};
int launch_shared_hidden(const SkinnyProblem* probs, int num_problems, const __half* x, const int32_t* row_gather,
                         int n, int k, cudaStream_t stream, bool pdl = false, const int32_t* n_dev = nullptr);

// tcgen05 / TMEM version of the same product (tc_gemm.cu), for row counts that make it a
// dense contraction.
bool tc_gemm_applicable(int n, int k, const __half* x, const SkinnyProblem* probs, int num_problems);
int launch_tc_gemm(const SkinnyProblem* probs, int num_problems, const __half* x, const int32_t* row_gather, int n,
                   int k, cudaStream_t stream, bool pdl, const int32_t* n_dev, int32_t* status);

// Launch with optional programmatic dependent launch (the kernel may start while its
// predecessor in the stream drains; it must execute griddepcontrol.wait before touching
// anything the predecessor writes) and an optional cluster size along z.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 bool pdl, int cluster_z, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (pdl) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster_z > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = 1;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = cluster_z;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Whether the stand-alone entry points launch with programmatic dependent launch
// (tris_set_programmatic_launch).
bool programmatic_launch_default();

// Options of the launches the fused layer path makes.
struct LaunchOpts {
  bool pdl = false;                  // programmatic dependent launch
  bool weights_before_wait = false;  // the route was complete before the predecessor kernel started
};
int grouped_forward_impl(const TrisProjView* proj, const TrisRouteView* route, const void* hidden_f16, void* out_f16,
                         cudaStream_t stream, LaunchOpts opts);
int grouped_pair_forward_impl(const TrisProjView* proj_a, const TrisProjView* proj_b, const TrisRouteView* route,
                              const void* hidden_a_f16, const void* hidden_b_f16, void* out_a_f16, void* out_b_f16,
                              int fuse_silu_mul, cudaStream_t stream, LaunchOpts opts);
// Tile-record path (grouped_tiled.cu).  mode: 0 single projection, 1 gate/up pair, 2 pair with SiLU * mul.
bool proj_has_tile_records(const TrisProjView& v);
int launch_grouped_tiled(const TrisProjView* proj_a, const TrisProjView* proj_b, const TrisRouteView* route,
                         const void* hidden_a, const void* hidden_b, void* out_a, void* out_b, int mode, int max_rows,
                         cudaStream_t stream, LaunchOpts opts);
// Rows per segment (the launch's estimate, route_rows_hint) above which the grouped entry points
// leave the decode-regime kernels for the tcgen05 kernel (tris_set_grouped_tc_min_rows).
int grouped_tc_min_rows();
int route_rows_hint(const TrisRouteView* route);
int launch_tiled_dump(const TrisProjView* proj, int32_t* dense_out, void* weights_out, cudaStream_t stream);
int combine_routed_impl(const void* down_out_f16, const int32_t* row_of_flat, const float* routing_weights,
                        int num_tokens, int top_k, int hidden_size, void* final_f16, cudaStream_t stream, bool pdl);
int launch_router_route(const float* logits, int num_tokens, int num_experts, int top_k, int norm, int m_tile,
                        int32_t* selected, float* weights, int32_t* perm, int32_t* tok, int32_t* slot,
                        int32_t* row_of_flat, int32_t* expert_ids, int32_t* segment_offsets, int32_t* problem_offsets,
                        int32_t* counts, cudaStream_t stream, int32_t* scratch = nullptr, size_t scratch_bytes = 0);

// ---- device helpers -------------------------------------------------------------------
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}

__device__ __forceinline__ uint32_t h2_as_u32(__half2 v) { return *reinterpret_cast<uint32_t*>(&v); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t v) { return *reinterpret_cast<__half2*>(&v); }

// D(16x8, f32) += A(16x16, f16, row) * B(16x8, f16, col)
__device__ __forceinline__ void mma_m16n8k16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                             uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Programmatic dependent launch: wait for the producer grid's memory to be visible /
// let the dependent grid start its prologue.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

}  // namespace tris

// ---- TMA bulk copies and mbarriers -------------------------------------------------------
namespace tris {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
// Makes mbarrier initialisation visible to the async proxy.
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
// Orders earlier generic-proxy accesses to shared memory before later async-proxy (TMA) writes.
// ---- cp.async (per-thread asynchronous copies, completion by commit groups) ---------------
__device__ __forceinline__ void cp_async_16(void* dst_smem, const void* src, bool valid) {
  // src-size 0 zero-fills the destination without reading the source
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst_smem)), "l"(src), "r"(valid ? 16 : 0)
               : "memory");
}
__device__ __forceinline__ void cp_async_16(void* dst_smem, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_4(void* dst_smem, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Barrier `id` (1..15; 0 is __syncthreads) for `nthreads` threads, a multiple of 32.
__device__ __forceinline__ void named_barrier_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Untiled TMA copy global -> shared; both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst_smem)),
               "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Waits for the phase with the given parity, giving up after ~1 s.  Returns false on
// time-out (the caller records TRIS_ERR_TIMEOUT and leaves; it never spins forever).
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_timer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (global_timer_ns() - t0 > 1000000000ull) return false;
  }
}

}  // namespace tris
