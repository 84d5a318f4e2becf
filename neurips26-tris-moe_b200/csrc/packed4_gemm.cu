// GEMMs that read GPTQ-style 4-bit matrices as they are stored (no fp16 copy in HBM):
//
//   * the null-space compensation of ns_mode == 2 experts, comp = (x . C2^T) . C1^T per routed
//     segment, with every expert's C2 / C1 inside one concatenated tensor
//     (run_grouped_ns_compensation_forward, qlinear_cuda.py:2024-2128; kernels
//     GroupedPacked4LinearOffset{Segment,Decode}{C2,C1}, TriSMoE_cuda_kernel.cu:1208-2144), and
//   * the shared backbone product hidden = x . shared_sv^T on the packed matrix
//     (_run_packed_4bit_linear_cuda, qlinear_cuda.py:1148-1168; Packed4LinearKernelTiledLop3[SplitK],
//     TriSMoE_cuda_kernel.cu:914-1104).
//
// Numerics: every weight is fp16((q - zero) * scale) with one rounding, bit for bit the matrix
// PackedQuantMatrix4bit.dequantize (qlinear_cuda.py:2756-2784) hands to F.linear in the reference's
// fallback; products accumulate in fp32 on the tensor cores and are rounded to fp16 once.
//
// Shape of the work: few activation rows (a decode batch, or the rows of one routed segment) against
// a matrix whose bytes dominate, so the matrix is the A operand of mma.m16n8k16 (16 outputs x 16
// inputs per instruction, 8 activation rows as the N side) and each nibble is expanded exactly once
// per pass, in registers.  A CTA owns 16 outputs of one problem; its 8 warps split every 256-column
// chunk of the contraction (32 columns each) and add their partial sums through shared memory.
#include "common.cuh"

namespace tris {

constexpr int kP4Threads = 256;
constexpr int kP4Warps = 8;
constexpr int kP4TileN = 16;              // outputs per CTA
constexpr int kP4SuperCols = 4096;        // contraction columns whose nibbles a CTA holds in shared memory at once
constexpr int kP4SuperWords = kP4SuperCols / 8;
constexpr int kP4RedStride = 20;          // floats per (warp, activation row) in the reduction buffer
constexpr int kP4MaxGroups = kP4SuperCols / 32 + 1;  // groups a super chunk can touch (group size >= 32)
// fp16 scales of 16 outputs + two zero words per group, rounded so that what follows stays 16-byte aligned
constexpr int kP4GroupBytes = (kP4MaxGroups * (kP4TileN * 2 + 8) + 15) & ~15;
static_assert((kP4SuperWords * kP4TileN * 4) % 16 == 0 && kP4GroupBytes % 16 == 0, "activation stages must start on 16 bytes");

// activation columns per staged chunk: about 32 KB per stage (64 KB at 128 rows), two stages
__host__ __device__ constexpr int p4_chunk_cols(int nt) { return nt == 1 ? 2048 : nt == 2 ? 1024 : nt == 4 ? 512 : 256; }
__host__ __device__ constexpr int p4_row_halfs(int nt) { return p4_chunk_cols(nt) + 8; }  // +16 bytes: rows on different banks
__host__ __device__ constexpr size_t p4_stage_bytes(int nt) { return static_cast<size_t>(8 * nt) * p4_row_halfs(nt) * 2; }
__host__ __device__ constexpr size_t p4_red_bytes(int nt) { return static_cast<size_t>(kP4Warps) * 8 * nt * kP4RedStride * 4; }
__host__ __device__ constexpr size_t p4_smem_bytes(int nt) {
  return kP4SuperWords * kP4TileN * 4 + kP4GroupBytes + (2 * p4_stage_bytes(nt) > p4_red_bytes(nt) ? 2 * p4_stage_bytes(nt) : p4_red_bytes(nt));
}

struct P4Args {
  TrisPacked4View w;
  const int32_t* expert_ids;
  const int32_t* segment_offsets;
  const int32_t* num_segments_dev;
  int num_segments;  // 0: one problem over all rows (expert 0)
  const int32_t* row_gather;
  const __half* x;
  int x_ld;
  int num_rows;
  __half* out;
  int out_ld;
  int out_mode;
  int accumulate;
  int x_aligned;  // rows of x start on 16-byte boundaries
  int w_aligned;  // rows of qweight start on 16-byte boundaries
};

__device__ __forceinline__ void cp_async16_zfill(void* dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(src_bytes) : "memory");
}
// byte t of `word` holds the nibbles of input columns 2t (low) and 2t+1 (high): returns
// half2(fp16((q_lo - zero) * scale), fp16((q_hi - zero) * scale)); zc = 1024 + zero as half2
__device__ __forceinline__ uint32_t p4_dequant_pair(uint32_t word, int t, __half2 zc, __half2 sc) {
  const uint32_t b = (word >> (8 * t)) & 0xFFu;
  const uint32_t v = ((b * 4097u) & 0x000F000Fu) | 0x64006400u;  // 1024 + q, exact in fp16
  return h2_as_u32(__hmul2(__hsub2(u32_as_h2(v), zc), sc));
}

template <int NT>
__global__ void __launch_bounds__(kP4Threads) packed4_gemm_kernel(const __grid_constant__ P4Args a) {
  constexpr int kRows = 8 * NT;
  constexpr int kChunk = p4_chunk_cols(NT);
  constexpr int kRowHalfs = p4_row_halfs(NT);
  extern __shared__ __align__(16) unsigned char p4_smem[];
  uint32_t* ws = reinterpret_cast<uint32_t*>(p4_smem);                                   // [kP4SuperWords][16] nibble words
  __half* gsc = reinterpret_cast<__half*>(p4_smem + kP4SuperWords * kP4TileN * 4);      // [kP4MaxGroups][16] scales
  uint32_t* gzw = reinterpret_cast<uint32_t*>(gsc + kP4MaxGroups * kP4TileN);            // [kP4MaxGroups][2] zero words
  __half* xs = reinterpret_cast<__half*>(p4_smem + kP4SuperWords * kP4TileN * 4 + kP4GroupBytes);  // [2][kRows][kRowHalfs]
  float* red = reinterpret_cast<float*>(xs);                                             // after the main loop

  pdl_wait();  // activations (and a device-built route) come from the kernels before this one
  int e = 0, row0 = 0, rows = a.num_rows;
  if (a.num_segments > 0) {
    const int seg = blockIdx.y;
    const int nseg = a.num_segments_dev ? min(*a.num_segments_dev, a.num_segments) : a.num_segments;
    if (seg >= nseg) return;
    e = a.expert_ids[seg];
    if (e < 0 || e >= a.w.num_experts) return;
    row0 = a.segment_offsets[seg];
    rows = min(a.segment_offsets[seg + 1], a.num_rows) - row0;
  }
  const int N = a.w.n_count ? a.w.n_count[e] : a.w.n;
  const int K = a.w.k_count ? a.w.k_count[e] : a.w.k;
  const int G = max(1, a.w.g_count ? a.w.g_count[e] : a.w.num_groups);
  const int n0 = blockIdx.x * kP4TileN;
  if (rows <= 0 || n0 >= N || row0 < 0) return;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int n_off = a.w.n_off ? a.w.n_off[e] : 0;
  const int g_off = a.w.g_off ? a.w.g_off[e] : 0;
  const int32_t* qw = a.w.qweight + static_cast<size_t>(a.w.kw_off ? a.w.kw_off[e] : 0) * a.w.q_ld + n_off;
  const int32_t* qz = a.w.qzeros + static_cast<size_t>(g_off) * a.w.z_ld + (a.w.z_off ? a.w.z_off[e] : 0);
  const __half* sc = static_cast<const __half*>(a.w.scales) + static_cast<size_t>(g_off) * a.w.s_ld + n_off;
  const int kwords = (K + 7) >> 3;
  const bool quad16 = a.w_aligned && ((n_off + n0) & 3) == 0;  // 16-byte copies of four outputs' words

  // stage activation rows [r0, r0 + kRows) x columns [k, k + kChunk) into stage `st`: 16-byte granules, zero past K / rows
  auto stage_x = [&](int st, int r0, int k_begin) {
    __half* base = xs + static_cast<size_t>(st) * kRows * kRowHalfs;
    for (int i = tid; i < kRows * (kChunk / 8); i += kP4Threads) {
      const int r = i / (kChunk / 8), c = i % (kChunk / 8);
      const int k = k_begin + 8 * c;
      const int valid = (r0 + r < rows) ? max(0, min(8, K - k)) : 0;
      __half* dst = base + r * kRowHalfs + 8 * c;
      if (k >= ((K + 31) & ~31)) continue;  // past the last 32-column block that holds a column: never read
      const int src_row = valid ? (a.row_gather ? a.row_gather[row0 + r0 + r] : row0 + r0 + r) : 0;
      const __half* src = a.x + static_cast<size_t>(src_row) * a.x_ld + k;
      if (a.x_aligned) {
        cp_async16_zfill(dst, valid ? src : a.x, 2 * valid);
      } else {
        for (int j = 0; j < 8; ++j) dst[j] = j < valid ? src[j] : __ushort_as_half(0);
      }
    }
  };

  for (int r0 = 0; r0 < rows; r0 += kRows) {
    float acc[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;

    for (int kk0 = 0; kk0 < K; kk0 += kP4SuperCols) {
      // every nibble this CTA needs for these columns, requested at once: [word row][16 outputs]
      const int nkw = min(kP4SuperWords, kwords - (kk0 >> 3));
      for (int i = tid; i < nkw * 4; i += kP4Threads) {
        const int kw = i >> 2, q = i & 3;
        const int32_t* row = qw + static_cast<size_t>((kk0 >> 3) + kw) * a.w.q_ld;
        uint32_t* dst = ws + kw * kP4TileN + 4 * q;
        if (quad16 && n0 + 4 * q + 3 < N) {
          cp_async16_zfill(dst, row + n0 + 4 * q, 16);
        } else {  // ragged edge or unaligned rows: word by word, outputs past N repeat the last one
#pragma unroll
          for (int j = 0; j < 4; ++j) cp_async_4(dst + j, row + min(n0 + 4 * q + j, N - 1));
        }
      }
      const int span = min(kP4SuperCols, K - kk0);
      // scales and zero points of the groups these columns fall into (outputs past N repeat the last one)
      const int gs = a.w.group_size > 0 ? a.w.group_size : (K + kP4SuperCols);
      const int grp0 = min(kk0 / gs, G - 1);
      const int ngrp = min((kk0 + span - 1) / gs, G - 1) - grp0 + 1;
      for (int i = tid; i < ngrp * (kP4TileN + 2); i += kP4Threads) {
        const int gi = i / (kP4TileN + 2), j = i % (kP4TileN + 2);
        if (j < kP4TileN) {
          gsc[gi * kP4TileN + j] = __ldg(sc + static_cast<size_t>(grp0 + gi) * a.w.s_ld + min(n0 + j, N - 1));
        } else {
          gzw[gi * 2 + (j - kP4TileN)] =
              static_cast<uint32_t>(__ldg(qz + static_cast<size_t>(grp0 + gi) * a.w.z_ld + (min(n0 + 8 * (j - kP4TileN), N - 1) >> 3)));
        }
      }
      const int nchunks = (span + kChunk - 1) / kChunk;
      stage_x(0, r0, kk0);
      cp_async_commit();
      for (int c = 0; c < nchunks; ++c) {
        if (c + 1 < nchunks) {
          stage_x((c + 1) & 1, r0, kk0 + (c + 1) * kChunk);
          cp_async_commit();
          cp_async_wait<1>();
        } else {
          cp_async_wait<0>();
        }
        __syncthreads();
        const __half* xb = xs + static_cast<size_t>(c & 1) * kRows * kRowHalfs;
        for (int blk = warp; blk < kChunk / 32; blk += kP4Warps) {
          const int kl = c * kChunk + 32 * blk;  // column inside this super chunk
          const int kc = kk0 + kl;
          if (kc >= K) break;
          const int gi = min(kc / gs, G - 1) - grp0;
          const uint32_t za = (gzw[gi * 2] >> (4 * g)) & 0xFu, zb = (gzw[gi * 2 + 1] >> (4 * g)) & 0xFu;
          const __half2 zca = __half2half2(__ushort_as_half(static_cast<unsigned short>(0x6400u + za + 1u)));
          const __half2 zcb = __half2half2(__ushort_as_half(static_cast<unsigned short>(0x6400u + zb + 1u)));
          const __half2 sca = __half2half2(gsc[gi * kP4TileN + g]);
          const __half2 scb = __half2half2(gsc[gi * kP4TileN + g + 8]);
          const uint32_t* wk = ws + (kl >> 3) * kP4TileN;
#pragma unroll
          for (int s = 0; s < 2; ++s) {
            const uint32_t a0 = p4_dequant_pair(wk[(2 * s) * kP4TileN + g], t, zca, sca);
            const uint32_t a1 = p4_dequant_pair(wk[(2 * s) * kP4TileN + g + 8], t, zcb, scb);
            const uint32_t a2 = p4_dequant_pair(wk[(2 * s + 1) * kP4TileN + g], t, zca, sca);
            const uint32_t a3 = p4_dequant_pair(wk[(2 * s + 1) * kP4TileN + g + 8], t, zcb, scb);
            const __half* xk = xb + g * kRowHalfs + 32 * blk + 16 * s + 2 * t;
#pragma unroll
            for (int i = 0; i < NT; ++i) {
              const uint32_t b0 = *reinterpret_cast<const uint32_t*>(xk + i * 8 * kRowHalfs);
              const uint32_t b1 = *reinterpret_cast<const uint32_t*>(xk + i * 8 * kRowHalfs + 8);
              mma_m16n8k16(acc[i], a0, a1, a2, a3, b0, b1);
            }
          }
        }
        __syncthreads();  // this stage (and, after the last chunk, the nibble tile) may be overwritten now
      }
    }

    // add the eight warps' partial sums: red[warp][activation row][output]
#pragma unroll
    for (int i = 0; i < NT; ++i) {
      float* base = red + (warp * kRows + 8 * i + 2 * t) * kP4RedStride;
      base[g] = acc[i][0];
      base[kP4RedStride + g] = acc[i][1];
      base[g + 8] = acc[i][2];
      base[kP4RedStride + g + 8] = acc[i][3];
    }
    __syncthreads();
    for (int i = tid; i < kRows * kP4TileN; i += kP4Threads) {
      const int r = i / kP4TileN, n = i % kP4TileN;
      if (r0 + r >= rows || n0 + n >= N) continue;
      float sum = 0.f;
#pragma unroll
      for (int w = 0; w < kP4Warps; ++w) sum += red[(w * kRows + r) * kP4RedStride + n];
      __half* dst = a.out + static_cast<size_t>(row0 + r0 + r) * a.out_ld + out_mode_pos(n0 + n, a.out_mode);
      __half v = __float2half_rn(sum);
      if (a.accumulate) v = __hadd(*dst, v);  // what out.add_(compensation) does in fp16
      *dst = v;
    }
    __syncthreads();
  }
  pdl_launch_dependents();
}

template <int NT>
static int launch_p4(const P4Args& args, dim3 grid, cudaStream_t stream) {
  constexpr size_t smem = p4_smem_bytes(NT);
  if (smem > 48 * 1024) {
    TRIS_CUDA(cudaFuncSetAttribute(packed4_gemm_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  }
  return check_cuda(launch_kernel(packed4_gemm_kernel<NT>, grid, dim3(kP4Threads), smem, stream, programmatic_launch_default(), 1, args),
                    "packed4_gemm_kernel launch");
}

}  // namespace tris

using namespace tris;

extern "C" int tris_packed4_grouped_forward(const TrisPacked4View* w, const TrisRouteView* route, const void* x_f16,
                                            int32_t x_ld, int32_t num_rows, void* out_f16, int32_t out_ld,
                                            int32_t out_mode, int32_t accumulate, void* stream) {
  TRIS_REQUIRE(w && x_f16 && out_f16, TRIS_ERR_INVALID_ARG, "tris_packed4_grouped_forward: null pointer");
  TRIS_REQUIRE(w->qweight && w->qzeros && w->scales, TRIS_ERR_INVALID_ARG, "tris_packed4_grouped_forward: null matrix pointer");
  TRIS_REQUIRE(w->n > 0 && w->k >= 0 && w->num_groups >= 0 && w->num_experts > 0 && w->q_ld > 0 && w->z_ld > 0 && w->s_ld > 0,
               TRIS_ERR_INVALID_ARG, "tris_packed4_grouped_forward: bad sizes n=%d k=%d groups=%d", w->n, w->k, w->num_groups);
  TRIS_REQUIRE(w->group_size <= 0 || w->group_size % 32 == 0 || w->num_groups <= 1, TRIS_ERR_UNSUPPORTED,
               "tris_packed4_grouped_forward: group size %d (a multiple of 32, or a single group, is supported)", w->group_size);
  TRIS_REQUIRE(out_mode == TRIS_OUT_F16 || out_mode == TRIS_OUT_F16_PAIR_INTERLEAVED || out_mode == TRIS_OUT_F16_LANE_ORDER,
               TRIS_ERR_INVALID_ARG, "tris_packed4_grouped_forward: out_mode %d", out_mode);
  TRIS_REQUIRE(out_mode == TRIS_OUT_F16 || w->n % 32 == 0, TRIS_ERR_INVALID_ARG,
               "tris_packed4_grouped_forward: permuted output layouts need n %% 32 == 0");
  TRIS_REQUIRE(x_ld >= w->k && out_ld >= w->n && num_rows >= 0, TRIS_ERR_INVALID_ARG,
               "tris_packed4_grouped_forward: row strides x_ld=%d out_ld=%d", x_ld, out_ld);
  if (num_rows == 0) return TRIS_OK;
  P4Args args{};
  args.w = *w;
  int hint = num_rows;
  if (route) {
    TRIS_REQUIRE(route->expert_ids && route->segment_offsets && route->num_segments >= 0, TRIS_ERR_INVALID_ARG,
                 "tris_packed4_grouped_forward: incomplete route");
    if (route->num_segments == 0) return TRIS_OK;
    args.expert_ids = route->expert_ids;
    args.segment_offsets = route->segment_offsets;
    args.num_segments_dev = route->num_segments_dev;
    args.num_segments = route->num_segments;
    args.row_gather = route->row_gather;
    if (route->max_rows_per_segment > 0) hint = std::min(hint, route->max_rows_per_segment);
  }
  args.x = static_cast<const __half*>(x_f16);
  args.x_ld = x_ld;
  args.num_rows = num_rows;
  args.out = static_cast<__half*>(out_f16);
  args.out_ld = out_ld;
  args.out_mode = out_mode;
  args.accumulate = accumulate ? 1 : 0;
  args.x_aligned = ((reinterpret_cast<uintptr_t>(x_f16) & 15u) == 0 && x_ld % 8 == 0) ? 1 : 0;
  args.w_aligned = ((reinterpret_cast<uintptr_t>(w->qweight) & 15u) == 0 && w->q_ld % 4 == 0) ? 1 : 0;
  const dim3 grid(ceil_div(w->n, kP4TileN), route ? route->num_segments : 1);
  TRIS_REQUIRE(grid.y <= 65535u, TRIS_ERR_UNSUPPORTED, "tris_packed4_grouped_forward: more than 65535 segments");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (hint <= 8) return launch_p4<1>(args, grid, s);
  if (hint <= 16) return launch_p4<2>(args, grid, s);
  if (hint <= 32) return launch_p4<4>(args, grid, s);
  if (hint <= 64) return launch_p4<8>(args, grid, s);
  return launch_p4<16>(args, grid, s);
}
