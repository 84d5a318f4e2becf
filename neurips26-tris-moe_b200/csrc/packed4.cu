// 4-bit packed backbone -> fp16, once at load time.
//
// Real TriS-MoE checkpoints store the shared input-side backbone as a GPTQ-style 4-bit matrix
// (PackedQuantMatrix4bit, qlinear_cuda.py:2668-2784): qweight [ceil(cols/8), rows] int32 holds
// the nibbles of input columns 8i..8i+7 of output row r (nibble j at bits 4j), qzeros
// [groups, ceil(rows/8)] int32 the zero points minus one packed the same way along the rows,
// scales [groups, rows] fp16, g_idx [cols] the group of each input column.  The fp16 matrix
// weight[r, c] = fp16((q - zero) * scale) is what PackedQuantMatrix4bit.dequantize
// (qlinear_cuda.py:2756-2784) hands to F.linear; it is built here bit for bit and then used
// by the fp16 backbone GEMMs.
#include "common.cuh"

namespace tris {

// one thread: 8 consecutive input columns of one output row -> one 16-byte store
__global__ void __launch_bounds__(256) packed4_dequantize_kernel(const int32_t* __restrict__ qweight,
                                                                 const int32_t* __restrict__ qzeros,
                                                                 const __half* __restrict__ scales,
                                                                 const int32_t* __restrict__ g_idx, int rows, int cols,
                                                                 int groups, __half* __restrict__ out) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;  // consecutive threads: consecutive rows (coalesced qweight)
  const int c8 = blockIdx.y;
  if (r >= rows) return;
  const uint32_t q = static_cast<uint32_t>(qweight[static_cast<size_t>(c8) * rows + r]);
  const int zwords = (rows + 7) >> 3;
  __align__(16) __half vals[8];
  int g_prev = -1;
  int zero = 0;
  __half scale = __ushort_as_half(0);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int c = 8 * c8 + j;
    vals[j] = __ushort_as_half(0);
    if (c >= cols) continue;
    int g = g_idx[c];
    g = min(max(g, 0), groups - 1);  // a corrupt group index must not read out of bounds
    if (g != g_prev) {
      g_prev = g;
      zero = static_cast<int>((static_cast<uint32_t>(qzeros[static_cast<size_t>(g) * zwords + (r >> 3)]) >> (4 * (r & 7))) & 0xFu) + 1;
      scale = scales[static_cast<size_t>(g) * rows + r];
    }
    const int diff = static_cast<int>((q >> (4 * j)) & 0xFu) - zero;  // exact in fp16
    vals[j] = __hmul(__int2half_rn(diff), scale);
  }
  __half* dst = out + static_cast<size_t>(r) * cols + 8 * c8;
  if ((cols & 7) == 0 && (reinterpret_cast<uintptr_t>(out) & 15u) == 0) {
    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(vals);
  } else {
    for (int j = 0; j < 8 && 8 * c8 + j < cols; ++j) dst[j] = vals[j];
  }
}

}  // namespace tris

using namespace tris;

extern "C" int tris_packed4_dequantize(const int32_t* qweight, const int32_t* qzeros, const void* scales_f16,
                                       const int32_t* g_idx, int32_t rows, int32_t cols, int32_t num_groups,
                                       void* weight_f16, void* stream) {
  TRIS_REQUIRE(qweight && qzeros && scales_f16 && g_idx && weight_f16, TRIS_ERR_INVALID_ARG,
               "tris_packed4_dequantize: null pointer");
  TRIS_REQUIRE(rows > 0 && cols > 0 && num_groups > 0, TRIS_ERR_INVALID_ARG,
               "tris_packed4_dequantize: bad sizes rows=%d cols=%d groups=%d", rows, cols, num_groups);
  const dim3 grid(ceil_div(rows, 256), ceil_div(cols, 8));
  TRIS_REQUIRE(grid.y <= 65535u, TRIS_ERR_UNSUPPORTED, "tris_packed4_dequantize: more than 524280 input columns");
  packed4_dequantize_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      qweight, qzeros, static_cast<const __half*>(scales_f16), g_idx, rows, cols, num_groups,
      static_cast<__half*>(weight_f16));
  return check_cuda(cudaGetLastError(), "packed4_dequantize_kernel launch");
}
