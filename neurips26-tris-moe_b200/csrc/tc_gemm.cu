// Backbone projection on the 5th-generation tensor cores (tcgen05 + TMEM), used when there
// are enough activation rows for a dense contraction (prefill, or the down backbone over
// all routed rows of a decode batch): out[n, m] = sum_k x[n, k] * A[m, k].
//
// One CTA computes a 128-output x NTILE-row tile over its share of K.  Operands are staged
// in shared memory in the K-major no-swizzle ("interleaved") core-matrix layout: 8 rows x
// 16 bytes per core matrix, all rows of one 8-column K chunk contiguous, so
//   byte offset(row, k) = (k / 8) * ROWS * 16 + row * 16 + (k % 8) * 2,
// stride between 8-row groups (SBO) = 128 B, stride between K chunks (LBO) = ROWS * 16 B.
// A single thread issues tcgen05.mma (M = 128, N = NTILE, K = 16 per instruction) into a
// TMEM accumulator; completion is tracked with tcgen05.commit on mbarriers, two shared-memory
// stages deep, so the loads of chunk i+1 overlap the MMAs of chunk i.  The split-K partial
// tiles of a thread-block cluster are reduced through distributed shared memory.
// Every mbarrier wait is bounded; a time-out frees the TMEM allocation and reports
// TRIS_ERR_TIMEOUT through the status word.
#include <cooperative_groups.h>
#include <cuda.h>  // CUtensorMap and its enums; cuTensorMapEncodeTiled itself comes from the driver entry point

#include <algorithm>
#include <atomic>

#include "umma.cuh"

namespace cg = cooperative_groups;

namespace tris {

struct TcGemmArgs {
  SkinnyProblem prob[3];
  int32_t num_problems;
  const __half* x;
  const int32_t* row_gather;
  const int32_t* n_dev;
  int32_t* status;
  int32_t n;
  int32_t k;
  int32_t k_per_cta;  // multiple of kTcKChunk
};

constexpr int kTcStages = 4;

template <int NTILE>
struct alignas(128) TcSmem {
  uint8_t a[kTcStages][kTcM * kTcKChunk * 2];
  uint8_t b[kTcStages][NTILE * kTcKChunk * 2];
  uint64_t mbar[kTcStages];
  uint32_t tmem_base;
  int32_t timed_out;
};

// Accumulator -> fp32 partial tile in shared memory -> (cluster reduction over the K split) ->
// outputs.  `part` is the CTA's shared memory from its start (the stage buffers are free by now).
template <int NTILE>
__device__ __forceinline__ void tc_gemm_epilogue(const TcGemmArgs& args, const SkinnyProblem& pb, float* part,
                                                 uint32_t tmem, bool failed, int nchunks, int m0, int n0, int n_live,
                                                 cg::cluster_group& cluster) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // accumulator -> fp32 partial tile in shared memory, [NTILE][128] (stage buffers are free now)
  if (!failed && nchunks > 0) {
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
#pragma unroll 1
    for (int c0 = 0; c0 < NTILE; c0 += 16) {
      float v[16];
      tmem_ld_16(tmem + lane_base + c0, v);
#pragma unroll
      for (int j = 0; j < 16; ++j) part[(c0 + j) * kTcM + warp * 32 + lane] = v[j];
    }
  } else {
    for (int i = threadIdx.x; i < NTILE * kTcM; i += kTcThreads) part[i] = 0.f;
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, NTILE);
  if (failed && threadIdx.x == 0 && args.status) atomicExch(args.status, TRIS_ERR_TIMEOUT);

  cluster.sync();
  {
    // every CTA of the cluster reduces and stores its own slice of the tile; the remote
    // reads of one element are independent, so they are all in flight together
    const unsigned nblk = cluster.num_blocks(), rank = cluster.block_rank();
    constexpr int kVec = NTILE * kTcM / 4;
    const int per = (kVec + nblk - 1) / nblk;
    const int v_end = min(kVec, static_cast<int>((rank + 1) * per));
    const float4* parts[8];
#pragma unroll
    for (unsigned r = 0; r < 8; ++r)
      parts[r] = reinterpret_cast<const float4*>(cluster.map_shared_rank(part, r < nblk ? r : 0));
    for (int i4 = rank * per + threadIdx.x; i4 < v_end; i4 += kTcThreads) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      float4 v[8];
#pragma unroll
      for (unsigned r = 0; r < 8; ++r) v[r] = (r < nblk) ? parts[r][i4] : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (unsigned r = 0; r < 8; ++r) { acc.x += v[r].x; acc.y += v[r].y; acc.z += v[r].z; acc.w += v[r].w; }
      const int n = n0 + (4 * i4) / kTcM, mbase = m0 + (4 * i4) % kTcM;
      if (n >= n_live) continue;
      const float vals[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int m = mbase + u;
        if (m >= pb.m) continue;
        if (pb.out_mode == TRIS_OUT_F32) {
          static_cast<float*>(pb.out)[static_cast<size_t>(n) * pb.m + m] = vals[u];
        } else {
          const int mm = out_mode_pos(m, pb.out_mode);
          static_cast<__half*>(pb.out)[static_cast<size_t>(n) * pb.m + mm] = __float2half_rn(vals[u]);
        }
      }
    }
  }
  cluster.sync();  // keep every CTA's shared memory alive until its peers have read it
}

// grid (m tiles over all problems, ceil(n / NTILE), ksplit); cluster (1, 1, ksplit).
// After the MMAs the stage buffers are reused as the fp32 partial tile [NTILE][128].
template <int NTILE>
__global__ void __launch_bounds__(kTcThreads) umma_gemm_kernel(const __grid_constant__ TcGemmArgs args) {
  extern __shared__ uint4 smem_raw[];
  auto& sm = *reinterpret_cast<TcSmem<NTILE>*>(smem_raw);
  cg::cluster_group cluster = cg::this_cluster();
  const int warp = threadIdx.x >> 5;

  int tile = blockIdx.x, pi = 0;
  while (pi + 1 < args.num_problems && tile >= (args.prob[pi].m + kTcM - 1) / kTcM) {
    tile -= (args.prob[pi].m + kTcM - 1) / kTcM;
    ++pi;
  }
  const SkinnyProblem& pb = args.prob[pi];
  const int m0 = tile * kTcM;
  const int n0 = blockIdx.y * NTILE;
  const int K = args.k;
  const int kbeg = blockIdx.z * args.k_per_cta;
  const int kend = min(K, kbeg + args.k_per_cta);
  const int nchunks = max(0, (kend - kbeg + kTcKChunk - 1) / kTcKChunk);

  if (threadIdx.x == 0) {
#pragma unroll
    for (int i = 0; i < kTcStages; ++i) mbar_init(&sm.mbar[i], 1);
    fence_mbar_init();
    sm.timed_out = 0;
  }
  if (warp == 0) tmem_alloc(&sm.tmem_base, NTILE);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem = sm.tmem_base;

  pdl_wait();  // x, row_gather and n_dev come from earlier kernels
  pdl_launch_dependents();
  const int n_live = args.n_dev ? min(args.n, *args.n_dev) : args.n;
  const uint32_t idesc = umma_idesc_f16(kTcM, NTILE);

  // Every thread copies the same (row, 16-byte column) pieces of every K chunk: work out their
  // source rows and shared-memory offsets once, so that a chunk costs one add and one cp.async
  // per piece (address arithmetic per piece per chunk used to dominate this kernel).
  constexpr int kAPieces = kTcM * 8 / kTcThreads, kBPieces = NTILE * 8 / kTcThreads;
  static_assert(kTcM * 8 % kTcThreads == 0 && NTILE * 8 % kTcThreads == 0, "pieces per thread");
  const __half* a_src[kAPieces];
  const __half* b_src[kBPieces];
  uint32_t a_off[kAPieces], b_off[kBPieces];
  uint32_t a_live = 0u, b_live = 0u;
  auto piece = [](int idx, int rows, int& row, int& c) {
    // a warp covers 8 rows x 4 chunks: 64 contiguous source bytes per row, and every 8
    // consecutive lanes write 128 contiguous shared-memory bytes
    const int r_lo = idx & 7, c_lo = (idx >> 3) & 3, rest = idx >> 5;
    c = ((rest & 1) << 2) | c_lo;
    row = ((rest >> 1) << 3) | r_lo;
    (void)rows;
  };
#pragma unroll
  for (int it = 0; it < kAPieces; ++it) {
    int row, c;
    piece(threadIdx.x + it * kTcThreads, kTcM, row, c);
    const int m = m0 + row;
    a_off[it] = static_cast<uint32_t>((c * kTcM + row) * 16);
    a_src[it] = pb.a;
    if (m < pb.m) {
      a_src[it] = pb.a + static_cast<size_t>(m) * K + kbeg + 8 * c;
      a_live |= 1u << it;
    }
  }
#pragma unroll
  for (int it = 0; it < kBPieces; ++it) {
    int row, c;
    piece(threadIdx.x + it * kTcThreads, NTILE, row, c);
    const int n = n0 + row;
    b_off[it] = static_cast<uint32_t>((c * NTILE + row) * 16);
    b_src[it] = args.x;
    if (n < n_live) {
      const int src = args.row_gather ? args.row_gather[n] : n;
      b_src[it] = args.x + static_cast<size_t>(src) * K + kbeg + 8 * c;
      b_live |= 1u << it;
    }
  }
  auto issue_chunk = [&](int i) {
    const int s = i % kTcStages;
    const int koff = i * kTcKChunk;  // halves from the start of this CTA's K range
#pragma unroll
    for (int it = 0; it < kAPieces; ++it) {
      const bool live = (a_live >> it) & 1u;
      cp_async_16(sm.a[s] + a_off[it], live ? a_src[it] + koff : a_src[it], live);
    }
#pragma unroll
    for (int it = 0; it < kBPieces; ++it) {
      const bool live = (b_live >> it) & 1u;
      cp_async_16(sm.b[s] + b_off[it], live ? b_src[it] + koff : b_src[it], live);
    }
  };

  // Software pipeline over the K chunks: copies run kTcStages-1 chunks ahead of the MMAs.
  uint32_t phase_bits = 0u;  // bit s = parity to wait for on mbar[s]
  bool ok = true;
#pragma unroll
  for (int i = 0; i < kTcStages - 1; ++i) {
    if (i < nchunks) issue_chunk(i);
    cp_async_commit();
  }
  for (int i = 0; i < nchunks; ++i) {
    const int s = i % kTcStages;
    cp_async_wait<kTcStages - 2>();  // this thread's copies of chunk i have landed
    fence_proxy_async();             // ... and are visible to the tensor core's reads
    __syncthreads();
    if (threadIdx.x == 0) {
      tcgen05_fence_after();
      const uint32_t a_addr = smem_u32(sm.a[s]), b_addr = smem_u32(sm.b[s]);
#pragma unroll
      for (int j = 0; j < kTcKChunk / 16; ++j) {
        const uint64_t da = umma_smem_desc(a_addr + j * 2 * kTcM * 16, kTcM * 16, 128);
        const uint64_t db = umma_smem_desc(b_addr + j * 2 * NTILE * 16, NTILE * 16, 128);
        umma_f16_ss(tmem, da, db, idesc, (i > 0 || j > 0) ? 1u : 0u);
      }
      umma_commit(&sm.mbar[s]);
    }
    // refill the stage that chunk i-1 used, once its MMAs have drained
    const int nxt = i + kTcStages - 1;
    if (nxt < nchunks) {
      if (i >= 1) {
        const int ps = (i - 1) % kTcStages;
        if (!mbar_wait_bounded(&sm.mbar[ps], (phase_bits >> ps) & 1u)) ok = false;
        phase_bits ^= 1u << ps;
      }
      issue_chunk(nxt);
    }
    cp_async_commit();
  }
  // drain: chunks up to nchunks - kTcStages - 1 were waited for when their stage was refilled
  for (int c = max(0, nchunks - kTcStages); c < nchunks; ++c) {
    const int s = c % kTcStages;
    if (!mbar_wait_bounded(&sm.mbar[s], (phase_bits >> s) & 1u)) ok = false;
    phase_bits ^= 1u << s;
  }
  if (!ok) sm.timed_out = 1;
  tcgen05_fence_after();
  __syncthreads();
  const bool failed = sm.timed_out != 0;

  tc_gemm_epilogue<NTILE>(args, pb, reinterpret_cast<float*>(smem_raw), tmem, failed, nchunks, m0, n0, n_live, cluster);
}

// ---- TMA-fed variant ------------------------------------------------------------------------
// Same tile, same operand layout, but a K chunk of an operand arrives with ONE tensor copy: the
// row-major matrix [rows, K] is described to the TMA unit as a 3-D tensor (8 halves, rows, K/8)
// with byte strides (2, 2K, 16), and a box of (8, ROWS, 8) lands in shared memory as
// [K chunk][row][16 bytes] - exactly the K-major no-swizzle core-matrix layout the MMA reads.
// Rows past the matrix read as zeros.  One thread issues the copies (a full/empty mbarrier pair
// per stage), one thread the MMAs; all four warps run the epilogue.  Used when the activation
// rows are not gathered (row_gather == nullptr).
struct TcTmaMaps {
  CUtensorMap a[3];
  CUtensorMap x;
};

template <int NTILE>
struct alignas(128) TcTmaSmem {
  uint8_t a[kTcStages][kTcM * kTcKChunk * 2];
  uint8_t b[kTcStages][NTILE * kTcKChunk * 2];
  uint64_t full[kTcStages];
  uint64_t empty[kTcStages];
  uint64_t done;
  uint32_t tmem_base;
  int32_t timed_out;
};

__device__ __forceinline__ void tma_load_3d(void* dst_smem, const CUtensorMap* map, int c0, int c1, int c2, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(smem_u32(dst_smem)), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar))
      : "memory");
}

template <int NTILE>
__global__ void __launch_bounds__(kTcThreads) umma_gemm_tma_kernel(const __grid_constant__ TcGemmArgs args,
                                                                   const __grid_constant__ TcTmaMaps maps) {
  extern __shared__ uint4 smem_raw[];
  auto& sm = *reinterpret_cast<TcTmaSmem<NTILE>*>(smem_raw);
  cg::cluster_group cluster = cg::this_cluster();
  const int warp = threadIdx.x >> 5;

  int tile = blockIdx.x, pi = 0;
  while (pi + 1 < args.num_problems && tile >= (args.prob[pi].m + kTcM - 1) / kTcM) {
    tile -= (args.prob[pi].m + kTcM - 1) / kTcM;
    ++pi;
  }
  const SkinnyProblem& pb = args.prob[pi];
  const int m0 = tile * kTcM;
  const int n0 = blockIdx.y * NTILE;
  const int K = args.k;
  const int kbeg = blockIdx.z * args.k_per_cta;
  const int kend = min(K, kbeg + args.k_per_cta);
  const int nchunks = max(0, (kend - kbeg + kTcKChunk - 1) / kTcKChunk);

  if (threadIdx.x == 0) {
#pragma unroll
    for (int i = 0; i < kTcStages; ++i) {
      mbar_init(&sm.full[i], 1);
      mbar_init(&sm.empty[i], 1);
    }
    mbar_init(&sm.done, 1);
    fence_mbar_init();
    sm.timed_out = 0;
  }
  if (warp == 0) tmem_alloc(&sm.tmem_base, NTILE);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem = sm.tmem_base;

  pdl_wait();  // x and n_dev come from earlier kernels
  pdl_launch_dependents();
  const int n_live = args.n_dev ? min(args.n, *args.n_dev) : args.n;

  if (threadIdx.x == 0) {
    // producer: one tensor copy per operand per K chunk, kTcStages chunks in flight
    constexpr uint32_t kBytes = (kTcM + NTILE) * kTcKChunk * 2;
    for (int i = 0; i < nchunks; ++i) {
      const int s = i % kTcStages;
      if (i >= kTcStages && !mbar_wait_bounded(&sm.empty[s], ((i / kTcStages) - 1) & 1)) {
        sm.timed_out = 1;
        break;
      }
      mbar_arrive_expect_tx(&sm.full[s], kBytes);
      const int kc = (kbeg + i * kTcKChunk) >> 3;
      tma_load_3d(sm.a[s], &maps.a[pi], 0, m0, kc, &sm.full[s]);
      tma_load_3d(sm.b[s], &maps.x, 0, n0, kc, &sm.full[s]);
    }
  } else if (threadIdx.x == 32) {
    // consumer: four K=16 MMAs per chunk; the commit frees the stage for the producer
    const uint32_t idesc = umma_idesc_f16(kTcM, NTILE);
    bool ok = true;
    for (int i = 0; i < nchunks && ok; ++i) {
      const int s = i % kTcStages;
      ok = mbar_wait_bounded(&sm.full[s], (i / kTcStages) & 1);
      if (!ok) break;
      tcgen05_fence_after();
      const uint32_t a_addr = smem_u32(sm.a[s]), b_addr = smem_u32(sm.b[s]);
#pragma unroll
      for (int j = 0; j < kTcKChunk / 16; ++j) {
        const uint64_t da = umma_smem_desc(a_addr + j * 2 * kTcM * 16, kTcM * 16, 128);
        const uint64_t db = umma_smem_desc(b_addr + j * 2 * NTILE * 16, NTILE * 16, 128);
        umma_f16_ss(tmem, da, db, idesc, (i > 0 || j > 0) ? 1u : 0u);
      }
      umma_commit(&sm.empty[s]);
    }
    if (!ok) sm.timed_out = 1;
    umma_commit(&sm.done);  // arrives once every MMA issued so far has completed
  }
  __syncwarp();
  if (!mbar_wait_bounded(&sm.done, 0)) sm.timed_out = 1;
  tcgen05_fence_after();
  __syncthreads();
  const bool failed = sm.timed_out != 0;
  tc_gemm_epilogue<NTILE>(args, pb, reinterpret_cast<float*>(smem_raw), tmem, failed, nchunks, m0, n0, n_live, cluster);
}

template <int NTILE>
static int launch_umma(const TcGemmArgs& args, int mtiles, int ksplit, cudaStream_t stream, bool pdl) {
  const size_t smem = std::max(sizeof(TcSmem<NTILE>), static_cast<size_t>(NTILE) * kTcM * 4 + 128);
  static bool configured[64] = {};
  int dev = 0;
  TRIS_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    TRIS_CUDA(cudaFuncSetAttribute(umma_gemm_kernel<NTILE>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  return check_cuda(launch_kernel(umma_gemm_kernel<NTILE>, dim3(mtiles, ceil_div(args.n, NTILE), ksplit),
                                  dim3(kTcThreads), smem, stream, pdl, ksplit, args),
                    "umma_gemm_kernel launch");
}

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link against libcuda).
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled_fn() {
  static std::atomic<void*> cached{nullptr};
  static std::atomic<bool> tried{false};
  if (!tried.load(std::memory_order_acquire)) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      fn = nullptr;
    cudaGetLastError();
    cached.store(fn, std::memory_order_release);
    tried.store(true, std::memory_order_release);
  }
  return reinterpret_cast<EncodeTiledFn>(cached.load(std::memory_order_acquire));
}

// Describes the row-major fp16 matrix [rows, k] as (8 halves, rows, k/8) with a box of
// (8, box_rows, 8): one copy = one 64-column chunk of box_rows rows in core-matrix order.
static bool encode_operand_map(CUtensorMap* map, const void* base, int rows, int k, int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr || rows <= 0) return false;
  const cuuint64_t dims[3] = {8, static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(k / 8)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(k) * 2, 16};  // bytes, dimensions 1 and 2
  const cuuint32_t box[3] = {8, static_cast<cuuint32_t>(box_rows), 8};
  const cuuint32_t estr[3] = {1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int NTILE>
static int launch_umma_tma(const TcGemmArgs& args, const TcTmaMaps& maps, int mtiles, int ksplit, cudaStream_t stream,
                           bool pdl) {
  const size_t smem = std::max(sizeof(TcTmaSmem<NTILE>), static_cast<size_t>(NTILE) * kTcM * 4 + 128);
  static bool configured[64] = {};
  int dev = 0;
  TRIS_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    TRIS_CUDA(cudaFuncSetAttribute(umma_gemm_tma_kernel<NTILE>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  return check_cuda(launch_kernel(umma_gemm_tma_kernel<NTILE>, dim3(mtiles, ceil_div(args.n, NTILE), ksplit),
                                  dim3(kTcThreads), smem, stream, pdl, ksplit, args, maps),
                    "umma_gemm_tma_kernel launch");
}

// True when the tensor-core path applies: enough rows for a dense contraction, K a multiple
// of the 64-column chunk, 16-byte aligned rows.
bool tc_gemm_applicable(int n, int k, const __half* x, const SkinnyProblem* probs, int num_problems) {
  if (n < 64 || (k % kTcKChunk) != 0 || (reinterpret_cast<uintptr_t>(x) & 15u)) return false;
  for (int i = 0; i < num_problems; ++i)
    if (reinterpret_cast<uintptr_t>(probs[i].a) & 15u) return false;
  return true;
}

int launch_tc_gemm(const SkinnyProblem* probs, int num_problems, const __half* x, const int32_t* row_gather, int n,
                   int k, cudaStream_t stream, bool pdl, const int32_t* n_dev, int32_t* status) {
  TcGemmArgs args{};
  int mtiles = 0;
  for (int i = 0; i < num_problems; ++i) {
    args.prob[i] = probs[i];
    mtiles += ceil_div(probs[i].m, kTcM);
  }
  args.num_problems = num_problems;
  args.x = x;
  args.row_gather = row_gather;
  args.n_dev = n_dev;
  args.status = status;
  args.n = n;
  args.k = k;
  const int ntile = n <= 2048 ? 64 : 128;
  const int ntiles = ceil_div(n, ntile);
  int ksplit = 1;
  // split K over the cluster until the GPU is full or a CTA would get fewer than two 64-column chunks: a CTA's
  // time is its chain of chunk loads and MMAs, so shorter chains win (measured at 128 and 1024 rows: 85.7 us
  // per layer with a floor of two chunks, 86.8 with four; a cluster of 16 is slower again)
  while (ksplit < 8 && mtiles * ntiles * ksplit < 148 && k / (ksplit * 2) >= 2 * kTcKChunk) ksplit *= 2;
  args.k_per_cta = ceil_div(ceil_div(k, ksplit), kTcKChunk) * kTcKChunk;
  if (row_gather == nullptr) {  // operands by tensor copies
    TcTmaMaps maps;
    bool ok = encode_operand_map(&maps.x, x, n, k, ntile);
    for (int i = 0; i < 3 && ok; ++i) {
      const SkinnyProblem& pr = probs[i < num_problems ? i : 0];
      ok = encode_operand_map(&maps.a[i], pr.a, pr.m, k, kTcM);
    }
    if (ok) {
      if (ntile == 64) return launch_umma_tma<64>(args, maps, mtiles, ksplit, stream, pdl);
      return launch_umma_tma<128>(args, maps, mtiles, ksplit, stream, pdl);
    }
  }
  if (ntile == 64) return launch_umma<64>(args, mtiles, ksplit, stream, pdl);
  return launch_umma<128>(args, mtiles, ksplit, stream, pdl);
}

}  // namespace tris
