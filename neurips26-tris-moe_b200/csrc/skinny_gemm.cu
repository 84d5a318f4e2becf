// Input-side backbone projection: out[n, m] = sum_k x[n, k] * A[m, k] for a tall-skinny
// fp16 problem (A = shared_sv [rank, in], x = activation rows), fp32 accumulation.
//
// The K dimension is split over the CTAs of a thread-block cluster and over the 4 warps of
// each CTA; warps stream A and x straight from global memory as 128-bit loads into
// m16n8k16 fragments (the same 8 contiguous halves feed matching k slots of A and B, so no
// shared-memory transposition is needed).  Partial tiles are reduced through shared memory
// inside the CTA and through distributed shared memory across the cluster, so there are no
// atomics and the result does not depend on scheduling.
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace tris {

constexpr int kSkinnyThreads = 128;
constexpr int kMaxProblems = 3;

struct SkinnyArgs {
  SkinnyProblem prob[kMaxProblems];
  int32_t num_problems;
  const __half* x;            // [*, k]
  const int32_t* row_gather;  // optional [n]
  const int32_t* n_dev;       // optional device scalar: only the first *n_dev rows are live
  int32_t n;
  int32_t k;
  int32_t k_per_cta;          // multiple of 32
};

// grid (total m tiles over all problems, ceil(n / (NT*8)), ksplit); cluster (1, 1, ksplit)
template <int NT>
__global__ void __launch_bounds__(kSkinnyThreads) skinny_gemm_kernel(const __grid_constant__ SkinnyArgs args) {
  __shared__ float red[4][NT][32][4];
  cg::cluster_group cluster = cg::this_cluster();

  int tile = blockIdx.x, pi = 0;
  while (pi + 1 < args.num_problems && tile >= (args.prob[pi].m + 15) / 16) {
    tile -= (args.prob[pi].m + 15) / 16;
    ++pi;
  }
  const SkinnyProblem& pb = args.prob[pi];
  const int m0 = tile * 16;
  const int n0 = blockIdx.y * NT * 8;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int K = args.k;
  const int kbeg = blockIdx.z * args.k_per_cta;
  const int kend = min(K, kbeg + args.k_per_cta);

  const int ma = m0 + g, mb = m0 + g + 8;
  const __half* arow_a = pb.a + static_cast<size_t>(min(ma, pb.m - 1)) * K;
  const __half* arow_b = pb.a + static_cast<size_t>(min(mb, pb.m - 1)) * K;
  pdl_wait();  // x and row_gather may come from the preceding kernel
  pdl_launch_dependents();  // the next kernel may stage its weights while this one runs
  const int n_live = args.n_dev ? min(args.n, *args.n_dev) : args.n;
  const __half* xrow[NT];
  bool xvalid[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int n = n0 + nt * 8 + g;
    xvalid[nt] = n < n_live;
    const int src = xvalid[nt] ? (args.row_gather ? args.row_gather[n] : n) : 0;
    xrow[nt] = args.x + static_cast<size_t>(src) * K;
  }

  float acc[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[nt][c] = 0.f;

  const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll 2
  for (int k0 = kbeg + warp * 32; k0 < kend; k0 += 4 * 32) {
    const int kk = k0 + 8 * t;
    const bool kin = kk + 8 <= K;
    uint4 va = zero4, vb = zero4;
    if (kin && ma < pb.m) va = __ldg(reinterpret_cast<const uint4*>(arow_a + kk));
    if (kin && mb < pb.m) vb = __ldg(reinterpret_cast<const uint4*>(arow_b + kk));
    uint4 xv[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
      xv[nt] = (kin && xvalid[nt]) ? *reinterpret_cast<const uint4*>(xrow[nt] + kk) : zero4;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      mma_m16n8k16(acc[nt], va.x, vb.x, va.y, vb.y, xv[nt].x, xv[nt].y);
      mma_m16n8k16(acc[nt], va.z, vb.z, va.w, vb.w, xv[nt].z, xv[nt].w);
    }
  }

#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
    *reinterpret_cast<float4*>(&red[warp][nt][lane][0]) = make_float4(acc[nt][0], acc[nt][1], acc[nt][2], acc[nt][3]);
  __syncthreads();
  // each thread folds the 4 warps for a slice of the tile into red[0]
  for (int i = threadIdx.x; i < NT * 32 * 4; i += kSkinnyThreads) {
    float* base = &red[0][0][0][0];
    base[i] = base[i] + base[NT * 128 + i] + base[2 * NT * 128 + i] + base[3 * NT * 128 + i];
  }
  cluster.sync();
  if (cluster.block_rank() == 0) {
    const unsigned nblk = cluster.num_blocks();
    for (int i = threadIdx.x; i < NT * 32 * 4; i += kSkinnyThreads) {
      float v = (&red[0][0][0][0])[i];
      for (unsigned r = 1; r < nblk; ++r) v += cluster.map_shared_rank(&red[0][0][0][0], r)[i];
      const int c = i & 3, ln = (i >> 2) & 31, nt = i >> 7;
      const int n = n0 + nt * 8 + 2 * (ln & 3) + (c & 1);
      const int m = m0 + (ln >> 2) + 8 * (c >> 1);
      if (n < n_live && m < pb.m) {
        if (pb.out_mode == TRIS_OUT_F32) {
          static_cast<float*>(pb.out)[static_cast<size_t>(n) * pb.m + m] = v;
        } else {
          const int mm = out_mode_pos(m, pb.out_mode);
          static_cast<__half*>(pb.out)[static_cast<size_t>(n) * pb.m + mm] = __float2half_rn(v);
        }
      }
    }
  }
  cluster.sync();  // keep every CTA's shared memory alive until rank 0 has read it
}

template <int NT>
static int launch_skinny(const SkinnyArgs& args, int mtiles, int ksplit, cudaStream_t stream, bool pdl) {
  return check_cuda(launch_kernel(skinny_gemm_kernel<NT>, dim3(mtiles, ceil_div(args.n, NT * 8), ksplit),
                                  dim3(kSkinnyThreads), 0, stream, pdl, ksplit, args),
                    "skinny_gemm_kernel launch");
}

// Launches up to kMaxProblems matrices that share x.
int launch_shared_hidden(const SkinnyProblem* probs, int num_problems, const __half* x, const int32_t* row_gather,
                         int n, int k, cudaStream_t stream, bool pdl, const int32_t* n_dev) {
  TRIS_REQUIRE(num_problems >= 1 && num_problems <= kMaxProblems, TRIS_ERR_INVALID_ARG, "shared hidden: bad problem count");
  TRIS_REQUIRE(n >= 0 && k > 0, TRIS_ERR_INVALID_ARG, "shared hidden: bad sizes n=%d k=%d", n, k);
  TRIS_REQUIRE((k & 7) == 0, TRIS_ERR_UNSUPPORTED, "shared hidden: in_features=%d must be a multiple of 8", k);
  if (n == 0) return TRIS_OK;
  for (int i = 0; i < num_problems; ++i)
    TRIS_REQUIRE(probs[i].a && probs[i].out && probs[i].m > 0, TRIS_ERR_INVALID_ARG, "shared hidden: bad problem %d", i);
  // enough rows for a dense contraction: tcgen05 / TMEM tiles
  if (tc_gemm_applicable(n, k, x, probs, num_problems))
    return launch_tc_gemm(probs, num_problems, x, row_gather, n, k, stream, pdl, n_dev, nullptr);
  SkinnyArgs args{};
  int mtiles = 0;
  for (int i = 0; i < num_problems; ++i) {
    TRIS_REQUIRE(probs[i].a && probs[i].out && probs[i].m > 0, TRIS_ERR_INVALID_ARG, "shared hidden: bad problem %d", i);
    args.prob[i] = probs[i];
    mtiles += ceil_div(probs[i].m, 16);
  }
  args.num_problems = num_problems;
  args.x = x;
  args.row_gather = row_gather;
  args.n_dev = n_dev;
  args.n = n;
  args.k = k;
  const int nt = n <= 8 ? 1 : (n <= 16 ? 2 : (n <= 32 ? 4 : 8));
  const int row_chunks = ceil_div(n, nt * 8);
  // split K over a cluster until the grid covers the 148 SMs about twice, keeping at
  // least one 32-column step per warp
  int ksplit = 1;
  while (ksplit < 8 && mtiles * row_chunks * ksplit < 296 && k / (ksplit * 2) >= 128) ksplit *= 2;
  args.k_per_cta = ceil_div(ceil_div(k, ksplit), 32) * 32;
  switch (nt) {
    case 1: return launch_skinny<1>(args, mtiles, ksplit, stream, pdl);
    case 2: return launch_skinny<2>(args, mtiles, ksplit, stream, pdl);
    case 4: return launch_skinny<4>(args, mtiles, ksplit, stream, pdl);
    default: return launch_skinny<8>(args, mtiles, ksplit, stream, pdl);
  }
}

}  // namespace tris

using namespace tris;

extern "C" int tris_shared_hidden_forward(const void* x_f16, const int32_t* row_gather, int32_t num_rows,
                                          const int32_t* num_rows_dev, int32_t in_features,
                                          const void* shared_sv_f16, int32_t rank, void* out, int32_t out_mode,
                                          void* stream) {
  TRIS_REQUIRE(x_f16 && shared_sv_f16 && out, TRIS_ERR_INVALID_ARG, "tris_shared_hidden_forward: null pointer");
  TRIS_REQUIRE(rank > 0, TRIS_ERR_INVALID_ARG, "tris_shared_hidden_forward: rank=%d", rank);
  TRIS_REQUIRE(out_mode >= TRIS_OUT_F16 && out_mode <= TRIS_OUT_F16_LANE_ORDER, TRIS_ERR_INVALID_ARG,
               "tris_shared_hidden_forward: unknown out_mode %d", out_mode);
  TRIS_REQUIRE((out_mode != TRIS_OUT_F16_PAIR_INTERLEAVED && out_mode != TRIS_OUT_F16_LANE_ORDER) || rank % 32 == 0,
               TRIS_ERR_INVALID_ARG, "tris_shared_hidden_forward: the permuted layouts need rank % 32 == 0");
  SkinnyProblem pb{static_cast<const __half*>(shared_sv_f16), out, rank, out_mode};
  return launch_shared_hidden(&pb, 1, static_cast<const __half*>(x_f16), row_gather, num_rows, in_features,
                              static_cast<cudaStream_t>(stream), programmatic_launch_default(), num_rows_dev);
}

// Both input-side backbones and the router logits in one pass over x (what the layer entry
// point does internally): three matrices that share the activation rows.
extern "C" int tris_input_projections(const void* x_f16, int32_t num_rows, int32_t in_features,
                                      const void* shared_gate_f16, const void* shared_up_f16, int32_t rank,
                                      const void* router_weight_f16, int32_t num_experts, void* hidden_gate,
                                      void* hidden_up, int32_t hidden_out_mode, float* router_logits_f32,
                                      void* stream) {
  TRIS_REQUIRE(x_f16 && shared_gate_f16 && shared_up_f16 && hidden_gate && hidden_up, TRIS_ERR_INVALID_ARG,
               "tris_input_projections: null pointer");
  TRIS_REQUIRE(rank > 0 && num_rows >= 0 && in_features > 0, TRIS_ERR_INVALID_ARG,
               "tris_input_projections: bad sizes rows=%d in=%d rank=%d", num_rows, in_features, rank);
  TRIS_REQUIRE((router_weight_f16 == nullptr) == (router_logits_f32 == nullptr) && (!router_weight_f16 || num_experts > 0),
               TRIS_ERR_INVALID_ARG, "tris_input_projections: router weight and logits go together");
  TRIS_REQUIRE(hidden_out_mode == TRIS_OUT_F16 ||
                   ((hidden_out_mode == TRIS_OUT_F16_PAIR_INTERLEAVED || hidden_out_mode == TRIS_OUT_F16_LANE_ORDER) && rank % 32 == 0),
               TRIS_ERR_INVALID_ARG, "tris_input_projections: out_mode %d (the permuted layouts need rank %% 32 == 0)",
               hidden_out_mode);
  if (num_rows == 0) return TRIS_OK;
  SkinnyProblem probs[3] = {
      {static_cast<const __half*>(shared_gate_f16), hidden_gate, rank, hidden_out_mode},
      {static_cast<const __half*>(shared_up_f16), hidden_up, rank, hidden_out_mode},
      {static_cast<const __half*>(router_weight_f16), router_logits_f32, num_experts, TRIS_OUT_F32},
  };
  return launch_shared_hidden(probs, router_weight_f16 ? 3 : 2, static_cast<const __half*>(x_f16), nullptr, num_rows,
                              in_features, static_cast<cudaStream_t>(stream), programmatic_launch_default(), nullptr);
}
