// tcgen05 (5th-generation tensor core) and TMEM primitives shared by the tensor-core kernels:
// shared-memory and instruction descriptors, MMA issue and commit, TMEM allocation and loads,
// and the cp.async staging of a row-major fp16 tile into the K-major no-swizzle core-matrix
// layout (8 rows x 16 bytes per core matrix; byte offset(row, k) =
// (k/8) * ROWS * 16 + row * 16 + (k%8) * 2; SBO = 128 B between 8-row groups, LBO = ROWS * 16 B
// between 8-column K chunks).
#pragma once
#include "common.cuh"

namespace tris {

constexpr int kTcThreads = 128;
constexpr int kTcM = 128;   // outputs per tile = TMEM lanes
constexpr int kTcKChunk = 64;

__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  // start address [0,14) (>>4), leading byte offset [16,30) (>>4), stride byte offset [32,46) (>>4),
  // descriptor version 1 at [46,48), layout type 0 (no swizzle) at [61,64)
  return static_cast<uint64_t>((smem_addr >> 4) & 0x3FFFu) | (static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16) |
         (static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46);
}

// kind::f16 instruction descriptor: fp16 A and B, both K-major, fp32 accumulate, M x N.
__device__ __forceinline__ uint32_t umma_idesc_f16(int m, int n) {
  return (1u << 4) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

__device__ __forceinline__ void umma_f16_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// 32 lanes x 16 consecutive 32-bit columns of the accumulator: thread t of the warp gets lane
// (taddr.lane + t), registers = columns.
__device__ __forceinline__ void tmem_ld_16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Starts the asynchronous copy of a ROWS x 64 fp16 tile (row-major source, 128 B per row) into
// the core-matrix layout.  row_ptr(r) returns the source row (already offset to the chunk's
// first column) or nullptr for a row that must read as zeros.
// Only the first `valid_chunks` 8-column groups of the 64 columns exist in the source; the
// rest read as zeros.
template <int ROWS, typename RowPtr>
__device__ __forceinline__ void stage_operand_async(uint8_t* dst, const __half* fallback, RowPtr row_ptr,
                                                    int valid_chunks = 8) {
  constexpr int kVecs = ROWS * 8;
  for (int idx = threadIdx.x; idx < kVecs; idx += blockDim.x) {
    // a warp covers 8 rows x 4 chunks: 64 contiguous source bytes per row, and every 8
    // consecutive lanes write 128 contiguous shared-memory bytes
    const int r_lo = idx & 7, c_lo = (idx >> 3) & 3, rest = idx >> 5;
    const int c = ((rest & 1) << 2) | c_lo, row = ((rest >> 1) << 3) | r_lo;
    const __half* src = row_ptr(row);
    const bool valid = src != nullptr && c < valid_chunks;
    cp_async_16(dst + (c * ROWS + row) * 16, valid ? src + 8 * c : fallback, valid);
  }
}


}  // namespace tris
