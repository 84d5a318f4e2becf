// Router head (softmax + top-k), grouped route construction and the weighted combine.
//
// The route is built entirely on the device and written into arrays padded to the number
// of experts, so the launch sequence of a layer never waits on the host.
#include <algorithm>

#include "common.cuh"

namespace tris {

constexpr int kRouteThreads = 1024;
constexpr int kMaxExpertsPerLane = 8;  // experts <= 256

// Softmax + top-k of one token by one warp.  Ties go to the lower expert index.
__device__ __forceinline__ void topk_one_token(const float* __restrict__ row, int num_experts, int top_k, int norm,
                                               int32_t* __restrict__ selected, float* __restrict__ weights, int lane) {
  float v[kMaxExpertsPerLane];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < kMaxExpertsPerLane; ++i) {
    const int e = lane + 32 * i;
    v[i] = (e < num_experts) ? row[e] : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxExpertsPerLane; ++i) {
    const int e = lane + 32 * i;
    v[i] = (e < num_experts) ? expf(v[i] - mx) : -1.f;  // probabilities are >= 0; -1 marks "taken/absent"
    if (e < num_experts) sum += v[i];
  }
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
  const float inv = 1.f / sum;
  float picked_sum = 0.f;
  float my_w = 0.f;  // lane s keeps the weight of slot s (top_k <= 32)
  int my_e = 0;
  for (int s = 0; s < top_k; ++s) {
    float best = -1.f;
    int best_e = 0x7FFFFFFF;
#pragma unroll
    for (int i = 0; i < kMaxExpertsPerLane; ++i) {
      const int e = lane + 32 * i;
      if (v[i] > best) { best = v[i]; best_e = e; }  // ascending e inside a lane: first max wins
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xFFFFFFFFu, best, o);
      const int oe = __shfl_xor_sync(0xFFFFFFFFu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
    }
#pragma unroll
    for (int i = 0; i < kMaxExpertsPerLane; ++i)
      if (lane + 32 * i == best_e) v[i] = -1.f;
    const float p = best * inv;
    picked_sum += p;
    if (lane == s) { my_w = p; my_e = best_e; }
  }
  if (lane < top_k) {
    selected[lane] = my_e;
    weights[lane] = norm ? my_w / picked_sum : my_w;
  }
}

// One warp per token.
__global__ void router_topk_kernel(const float* __restrict__ logits, int num_tokens, int num_experts, int top_k,
                                   int norm, int32_t* __restrict__ selected, float* __restrict__ weights) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= num_tokens) return;
  pdl_wait();
  topk_one_token(logits + static_cast<size_t>(warp) * num_experts, num_experts, top_k, norm,
                 selected + static_cast<size_t>(warp) * top_k, weights + static_cast<size_t>(warp) * top_k, lane);
}

// The flat (token, slot) list of expert ids: entry f is base[f * stride] - offset (stride 1, offset 0 for
// a plain [T, k] array; an exchange buffer keeps the id of slot f behind that slot's activation row and
// numbers experts globally).
struct SelectedIds {
  const int32_t* base;
  int stride, offset;
  __device__ __forceinline__ int operator[](int f) const { return base[static_cast<size_t>(f) * stride] - offset; }
};

// One warp: per-expert row counts -> first grouped row of every expert (`start`) and the segment
// arrays of the active experts (padded to num_experts so that no size is read back).
__device__ __forceinline__ void route_scan_segments(const int32_t* count, int32_t* start, int num_experts, int m_tile,
                                                    int32_t* __restrict__ expert_ids, int32_t* __restrict__ segment_offsets,
                                                    int32_t* __restrict__ problem_offsets, int32_t* __restrict__ counts_out,
                                                    int lane) {
    // each lane owns a contiguous run of experts; warp scan of (segments, rows, tiles)
    const int epl = (num_experts + 31) / 32;
    const int e0 = lane * epl, e1 = min(num_experts, e0 + epl);
    int segs = 0, rows = 0, tiles = 0;
    for (int e = e0; e < e1; ++e) {
      const int c = count[e];
      if (c > 0) { ++segs; rows += c; tiles += (c + m_tile - 1) / m_tile; }
    }
    int psegs = segs, prows = rows, ptiles = tiles;
    for (int o = 1; o < 32; o <<= 1) {
      const int a = __shfl_up_sync(0xFFFFFFFFu, psegs, o);
      const int b = __shfl_up_sync(0xFFFFFFFFu, prows, o);
      const int c = __shfl_up_sync(0xFFFFFFFFu, ptiles, o);
      if (lane >= o) { psegs += a; prows += b; ptiles += c; }
    }
    const int nseg = __shfl_sync(0xFFFFFFFFu, psegs, 31);
    const int nrows = __shfl_sync(0xFFFFFFFFu, prows, 31);
    const int ntiles = __shfl_sync(0xFFFFFFFFu, ptiles, 31);
    int s = psegs - segs, r = prows - rows, t = ptiles - tiles;  // exclusive prefixes
    for (int e = e0; e < e1; ++e) {
      start[e] = r;
      const int c = count[e];
      if (c > 0) {
        expert_ids[s] = e;
        segment_offsets[s] = r;
        problem_offsets[s] = t;
        r += c;
        t += (c + m_tile - 1) / m_tile;
        ++s;
      }
    }
    for (int q = nseg + lane; q <= num_experts; q += 32) {
      segment_offsets[q] = nrows;
      problem_offsets[q] = ntiles;
      if (q < num_experts) expert_ids[q] = -1;
    }
    if (lane == 0) {
      counts_out[0] = nseg;
      counts_out[1] = ntiles;
    }
  }

// Single CTA.  Stable counting sort of the flat (token, slot) list by expert: every warp owns
// a contiguous chunk of the list, counts its experts, a scan over (expert, warp) turns the
// counts into write offsets, and a second pass places the elements in order.
// `sh` holds (34 * E) ints: count[E], start[E], per-warp counts/offsets [32][E].
__device__ __forceinline__ void build_route_body(
    int32_t* sh, const SelectedIds selected, int num_tokens, int top_k, int num_experts, int m_tile,
    int32_t* __restrict__ perm, int32_t* __restrict__ tok, int32_t* __restrict__ slot,
    int32_t* __restrict__ row_of_flat, int32_t* __restrict__ expert_ids, int32_t* __restrict__ segment_offsets,
    int32_t* __restrict__ problem_offsets, int32_t* __restrict__ counts_out) {
  constexpr int NW = kRouteThreads / 32;
  int32_t* count = sh;                      // [E]
  int32_t* start = sh + num_experts;        // [E] first grouped row of each expert
  int32_t* woff = sh + 2 * num_experts;     // [NW][E]
  const int R = num_tokens * top_k;
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int chunk = ((R + NW - 1) / NW + 31) & ~31;  // elements per warp, whole 32-element batches
  const int f0 = warp * chunk, f1 = min(R, f0 + chunk);
  for (int i = tid; i < NW * num_experts; i += kRouteThreads) woff[i] = 0;
  __syncthreads();
  for (int base = f0; base < f1; base += 32) {
    const int f = base + lane;
    int e = (f < f1) ? selected[f] : -1;
    if (e >= num_experts) e = -1;
    const unsigned peers = __match_any_sync(0xFFFFFFFFu, e);
    if (e >= 0 && lane == __ffs(peers) - 1) woff[warp * num_experts + e] += __popc(peers);
    __syncwarp();
  }
  __syncthreads();
  for (int e = tid; e < num_experts; e += kRouteThreads) {
    int total = 0;
    for (int w = 0; w < NW; ++w) total += woff[w * num_experts + e];
    count[e] = total;
  }
  __syncthreads();
  if (warp == 0)
    route_scan_segments(count, start, num_experts, m_tile, expert_ids, segment_offsets, problem_offsets, counts_out, lane);
  __syncthreads();
  for (int e = tid; e < num_experts; e += kRouteThreads) {  // counts -> write offsets per warp
    int run = start[e];
    for (int w = 0; w < NW; ++w) {
      const int c = woff[w * num_experts + e];
      woff[w * num_experts + e] = run;
      run += c;
    }
  }
  __syncthreads();
  for (int base = f0; base < f1; base += 32) {
    const int f = base + lane;
    int e = (f < f1) ? selected[f] : -1;
    if (e >= num_experts) e = -1;
    const unsigned peers = __match_any_sync(0xFFFFFFFFu, e);
    if (e >= 0) {
      const int pos = woff[warp * num_experts + e] + __popc(peers & ((1u << lane) - 1u));
      perm[pos] = f;
      const int tk = f / top_k;
      tok[pos] = tk;
      slot[pos] = f - tk * top_k;
      row_of_flat[f] = pos;
    } else if (f < f1) {
      row_of_flat[f] = -1;  // expert id out of range (padding rows of a fixed-capacity exchange)
    }
    __syncwarp();
    if (e >= 0 && lane == __ffs(peers) - 1) woff[warp * num_experts + e] += __popc(peers);
    __syncwarp();
  }
}

__global__ void __launch_bounds__(kRouteThreads) build_route_kernel(
    const SelectedIds selected, int num_tokens, int top_k, int num_experts, int m_tile,
    int32_t* __restrict__ perm, int32_t* __restrict__ tok, int32_t* __restrict__ slot,
    int32_t* __restrict__ row_of_flat, int32_t* __restrict__ expert_ids, int32_t* __restrict__ segment_offsets,
    int32_t* __restrict__ problem_offsets, int32_t* __restrict__ counts_out, int sel_cap) {
  extern __shared__ int32_t sh[];
  pdl_wait();
  pdl_launch_dependents();
  build_route_body(sh, selected, num_tokens, top_k, num_experts, m_tile, perm, tok, slot, row_of_flat, expert_ids,
                   segment_offsets, problem_offsets, counts_out);
}

// ---- the same route built by several CTAs (prefill-sized batches) -------------------------------------
// count: every CTA histograms its 2048-element chunk of the flat list; scan: one CTA turns the
// (chunk, expert) counts into write offsets and writes the segment arrays; place: every CTA places
// its chunk, warp by warp in list order, so rows of a segment stay in ascending (token, slot) order.
constexpr int kRouteParChunk = 2048;
constexpr int kRouteParThreads = 256;

__global__ void __launch_bounds__(kRouteParThreads) route_count_kernel(const SelectedIds selected, int num_rows,
                                                                       int num_experts, int32_t* __restrict__ counts_blk) {
  extern __shared__ int32_t sh[];  // [E]
  pdl_wait();
  pdl_launch_dependents();
  for (int e = threadIdx.x; e < num_experts; e += kRouteParThreads) sh[e] = 0;
  __syncthreads();
  const int f0 = blockIdx.x * kRouteParChunk, f1 = min(num_rows, f0 + kRouteParChunk);
  for (int f = f0 + threadIdx.x; f < f1; f += kRouteParThreads) {
    const int e = selected[f];
    if (e >= 0 && e < num_experts) atomicAdd(&sh[e], 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < num_experts; e += kRouteParThreads) counts_blk[blockIdx.x * num_experts + e] = sh[e];
}

__global__ void __launch_bounds__(kRouteThreads) route_scan_kernel(int32_t* __restrict__ counts_blk, int num_blocks, int num_experts,
                                                                   int m_tile, int32_t* __restrict__ expert_ids,
                                                                   int32_t* __restrict__ segment_offsets,
                                                                   int32_t* __restrict__ problem_offsets,
                                                                   int32_t* __restrict__ counts_out) {
  extern __shared__ int32_t sh[];  // count[E], start[E]
  int32_t* count = sh;
  int32_t* start = sh + num_experts;
  pdl_wait();
  pdl_launch_dependents();
  for (int e = threadIdx.x; e < num_experts; e += kRouteThreads) {
    int total = 0;
    for (int b = 0; b < num_blocks; ++b) total += counts_blk[b * num_experts + e];
    count[e] = total;
  }
  __syncthreads();
  if (threadIdx.x < 32)
    route_scan_segments(count, start, num_experts, m_tile, expert_ids, segment_offsets, problem_offsets, counts_out, threadIdx.x);
  __syncthreads();
  for (int e = threadIdx.x; e < num_experts; e += kRouteThreads) {  // counts -> first row of every (chunk, expert)
    int run = start[e];
    for (int b = 0; b < num_blocks; ++b) {
      const int c = counts_blk[b * num_experts + e];
      counts_blk[b * num_experts + e] = run;
      run += c;
    }
  }
}

__global__ void __launch_bounds__(kRouteParThreads) route_place_kernel(const SelectedIds selected, int num_rows, int top_k,
                                                                       int num_experts, const int32_t* __restrict__ start_blk,
                                                                       int32_t* __restrict__ perm, int32_t* __restrict__ tok,
                                                                       int32_t* __restrict__ slot, int32_t* __restrict__ row_of_flat) {
  constexpr int NW = kRouteParThreads / 32;
  extern __shared__ int32_t sh[];  // woff[NW][E]
  int32_t* woff = sh;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  pdl_wait();
  pdl_launch_dependents();
  for (int i = tid; i < NW * num_experts; i += kRouteParThreads) woff[i] = 0;
  __syncthreads();
  const int f0 = blockIdx.x * kRouteParChunk + warp * (kRouteParChunk / NW);
  const int f1 = min(num_rows, f0 + kRouteParChunk / NW);
  for (int base = f0; base < f1; base += 32) {
    const int f = base + lane;
    int e = (f < f1) ? selected[f] : -1;
    if (e >= num_experts) e = -1;
    const unsigned peers = __match_any_sync(0xFFFFFFFFu, e);
    if (e >= 0 && lane == __ffs(peers) - 1) woff[warp * num_experts + e] += __popc(peers);
    __syncwarp();
  }
  __syncthreads();
  for (int e = tid; e < num_experts; e += kRouteParThreads) {
    int run = start_blk[blockIdx.x * num_experts + e];
    for (int w = 0; w < NW; ++w) {
      const int c = woff[w * num_experts + e];
      woff[w * num_experts + e] = run;
      run += c;
    }
  }
  __syncthreads();
  for (int base = f0; base < f1; base += 32) {
    const int f = base + lane;
    int e = (f < f1) ? selected[f] : -1;
    if (e >= num_experts) e = -1;
    const unsigned peers = __match_any_sync(0xFFFFFFFFu, e);
    if (e >= 0) {
      const int pos = woff[warp * num_experts + e] + __popc(peers & ((1u << lane) - 1u));
      perm[pos] = f;
      const int tk = f / top_k;
      tok[pos] = tk;
      slot[pos] = f - tk * top_k;
      row_of_flat[f] = pos;
    } else if (f < f1) {
      row_of_flat[f] = -1;
    }
    __syncwarp();
    if (e >= 0 && lane == __ffs(peers) - 1) woff[warp * num_experts + e] += __popc(peers);
    __syncwarp();
  }
}

// Route of a prefill-sized batch with `scratch` (>= ceil(R / 2048) * E ints, caller-owned, free until
// the launch ends); launched after the kernel that wrote `selected`.
static int launch_route_parallel(const SelectedIds selected, int num_tokens, int top_k, int num_experts, int m_tile, int32_t* perm,
                                 int32_t* tok, int32_t* slot, int32_t* row_of_flat, int32_t* expert_ids,
                                 int32_t* segment_offsets, int32_t* problem_offsets, int32_t* counts, int32_t* scratch,
                                 cudaStream_t stream, bool first_pdl = true) {
  const int R = num_tokens * top_k;
  const int nb = ceil_div(R, kRouteParChunk);
  int st = check_cuda(launch_kernel(route_count_kernel, dim3(nb), dim3(kRouteParThreads), sizeof(int32_t) * num_experts, stream,
                                    first_pdl, 1, selected, R, num_experts, scratch),
                      "route_count_kernel launch");
  if (st != TRIS_OK) return st;
  st = check_cuda(launch_kernel(route_scan_kernel, dim3(1), dim3(kRouteThreads), 2 * sizeof(int32_t) * num_experts, stream,
                                /*pdl=*/true, 1, scratch, nb, num_experts, m_tile, expert_ids, segment_offsets, problem_offsets,
                                counts),
                  "route_scan_kernel launch");
  if (st != TRIS_OK) return st;
  return check_cuda(launch_kernel(route_place_kernel, dim3(nb), dim3(kRouteParThreads),
                                  sizeof(int32_t) * (kRouteParThreads / 32) * num_experts, stream, /*pdl=*/true, 1, selected, R,
                                  top_k, num_experts, static_cast<const int32_t*>(scratch), perm, tok, slot, row_of_flat),
                    "route_place_kernel launch");
}

// Router head and route in one single-CTA launch (decode-sized batches).
__global__ void __launch_bounds__(kRouteThreads) router_route_kernel(
    const float* __restrict__ logits, int num_tokens, int top_k, int num_experts, int norm, int m_tile,
    int32_t* selected, float* __restrict__ weights, int32_t* __restrict__ perm, int32_t* __restrict__ tok,
    int32_t* __restrict__ slot, int32_t* __restrict__ row_of_flat, int32_t* __restrict__ expert_ids,
    int32_t* __restrict__ segment_offsets, int32_t* __restrict__ problem_offsets, int32_t* __restrict__ counts_out,
    int sel_cap) {
  extern __shared__ int32_t sh[];
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int tk = warp; tk < num_tokens; tk += kRouteThreads / 32)
    topk_one_token(logits + static_cast<size_t>(tk) * num_experts, num_experts, top_k, norm,
                   selected + static_cast<size_t>(tk) * top_k, weights + static_cast<size_t>(tk) * top_k, lane);
  __syncthreads();  // selected[] written above is read back by every thread below
  pdl_launch_dependents();
  build_route_body(sh, SelectedIds{selected, 1, 0}, num_tokens, top_k, num_experts, m_tile, perm, tok, slot, row_of_flat,
                   expert_ids, segment_offsets, problem_offsets, counts_out);
}

// final[t, :] = sum_s w[t, s] * rows[row_of_flat[t*k+s], :]; one thread per 8 output halves.
__global__ void combine_routed_kernel(const __half* __restrict__ rows, const int32_t* __restrict__ row_of_flat,
                                      const float* __restrict__ weights, int num_tokens, int top_k, int hidden,
                                      __half* __restrict__ out) {
  const int vec_per_row = hidden >> 3;
  const long long id = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (id >= static_cast<long long>(num_tokens) * vec_per_row) return;
  const int t = static_cast<int>(id / vec_per_row), c = static_cast<int>(id % vec_per_row) * 8;
  pdl_wait();
  float acc[8];
#pragma unroll
  for (int u = 0; u < 8; ++u) acc[u] = 0.f;
  for (int s0 = 0; s0 < top_k; s0 += 8) {  // indices, then rows, 8 at a time: loads of a batch are independent
    int r[8];
    float w[8];
    uint4 v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const bool in = s0 + j < top_k;
      r[j] = in ? row_of_flat[t * top_k + s0 + j] : 0;
      w[j] = in ? weights[t * top_k + s0 + j] : 0.f;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j)
      v[j] = (s0 + j < top_k && r[j] >= 0)
                 ? *reinterpret_cast<const uint4*>(rows + static_cast<size_t>(r[j]) * hidden + c)
                 : make_uint4(0u, 0u, 0u, 0u);  // negative index = no row (contributes zero)
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const __half2* h2 = reinterpret_cast<const __half2*>(&v[j]);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float2 f = __half22float2(h2[u]);
        acc[2 * u] += w[j] * f.x;
        acc[2 * u + 1] += w[j] * f.y;
      }
    }
  }
  uint4 o;
  __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
  for (int u = 0; u < 4; ++u) oh[u] = __floats2half2_rn(acc[2 * u], acc[2 * u + 1]);
  *reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * hidden + c) = o;
}

static int route_smem_bytes(int num_experts, int rows, int* sel_cap) {
  (void)rows;
  *sel_cap = 0;
  return static_cast<int>((2 + kRouteThreads / 32) * num_experts * sizeof(int32_t));
}

// Router head + route for the fused layer path: one single-CTA launch for batches of up to
// 32 tokens (one warp per token), otherwise a token-parallel top-k launch followed by the
// single-CTA route kernel.
int launch_router_route(const float* logits, int num_tokens, int num_experts, int top_k, int norm, int m_tile,
                        int32_t* selected, float* weights, int32_t* perm, int32_t* tok, int32_t* slot,
                        int32_t* row_of_flat, int32_t* expert_ids, int32_t* segment_offsets, int32_t* problem_offsets,
                        int32_t* counts, cudaStream_t stream, int32_t* scratch, size_t scratch_bytes) {
  TRIS_REQUIRE(num_experts <= 32 * kMaxExpertsPerLane && top_k <= 32 && top_k <= num_experts, TRIS_ERR_UNSUPPORTED,
               "router: supports up to %d experts and top-32", 32 * kMaxExpertsPerLane);
  int sel_cap = 0;
  const int smem = route_smem_bytes(num_experts, num_tokens * top_k, &sel_cap);
  if (num_tokens <= kRouteThreads / 32) {
    router_route_kernel<<<1, kRouteThreads, smem, stream>>>(logits, num_tokens, top_k, num_experts, norm, m_tile,
                                                            selected, weights, perm, tok, slot, row_of_flat,
                                                            expert_ids, segment_offsets, problem_offsets, counts, sel_cap);
    return check_cuda(cudaGetLastError(), "router_route_kernel launch");
  }
  const int threads = 128;
  router_topk_kernel<<<ceil_div(num_tokens * 32, threads), threads, 0, stream>>>(logits, num_tokens, num_experts, top_k,
                                                                                 norm, selected, weights);
  int st = check_cuda(cudaGetLastError(), "router_topk_kernel launch");
  if (st != TRIS_OK) return st;
  const int rows = num_tokens * top_k;
  if (scratch && rows >= 4 * kRouteParChunk &&
      scratch_bytes >= sizeof(int32_t) * static_cast<size_t>(ceil_div(rows, kRouteParChunk)) * num_experts)
    return launch_route_parallel(SelectedIds{selected, 1, 0}, num_tokens, top_k, num_experts, m_tile, perm, tok, slot, row_of_flat,
                                 expert_ids, segment_offsets, problem_offsets, counts, scratch, stream);
  return check_cuda(launch_kernel(build_route_kernel, dim3(1), dim3(kRouteThreads), smem, stream, /*pdl=*/true, 1,
                                  SelectedIds{selected, 1, 0}, num_tokens, top_k, num_experts, m_tile, perm,
                                  tok, slot, row_of_flat, expert_ids, segment_offsets, problem_offsets, counts, sel_cap),
                    "build_route_kernel launch");
}

// Owner rank of an expert under the contiguous partition (sizes differ by at most one).
__device__ __forceinline__ int ep_owner(int e, int base, int extra) {
  const int big = extra * (base + 1);
  return e < big ? e / (base + 1) : extra + (e - big) / max(base, 1);
}

// grid = rows (one warp-sized group of 16-byte copies per row), 128 threads
__global__ void __launch_bounds__(128) ep_pack_rows_kernel(
    const __half* __restrict__ hidden_gate, const __half* __restrict__ hidden_up, int rank_gu,
    const int32_t* __restrict__ selected, const int32_t* __restrict__ perm, const int32_t* __restrict__ tok,
    int num_rows, int top_k, int num_experts, int world, int capacity, __half* __restrict__ send_rows,
    int send_row_stride, int32_t* __restrict__ send_ids, int32_t* __restrict__ combine_index,
    int32_t* __restrict__ overflow) {
  __shared__ int32_t s_first[64];  // first grouped row owned by each rank (world <= 64)
  const int base = num_experts / world, extra = num_experts % world;
  // rows are sorted by expert, so the first row of rank d is a lower bound: binary search
  if (threadIdx.x < world) {
    const int d = threadIdx.x;
    int lo = 0, hi = num_rows;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (ep_owner(selected[perm[mid]], base, extra) < d) lo = mid + 1;
      else hi = mid;
    }
    s_first[d] = lo;
  }
  __syncthreads();
  for (int pos = blockIdx.x; pos < world * capacity; pos += gridDim.x) {
    // slot pos = (owner d, offset): which grouped row, if any, lands here?
    const int d = pos / capacity, off = pos - d * capacity;
    const int row = s_first[d] + off;
    const int row_end = (d + 1 < world) ? s_first[d + 1] : num_rows;
    const bool used = row < row_end;
    if (threadIdx.x == 0) {
      const int32_t id = used ? selected[perm[row]] : -1;
      if (send_ids) send_ids[pos] = id;
      if (send_row_stride >= 2 * rank_gu + 8)
        *reinterpret_cast<int32_t*>(send_rows + static_cast<size_t>(pos) * send_row_stride + 2 * rank_gu) = id;
      if (used) combine_index[perm[row]] = pos;
      if (off == capacity - 1 && row + 1 < row_end) *overflow = 1;  // more rows for this rank than slots
    }
    if (!used) continue;
    const int t = tok[row];
    const uint4* g = reinterpret_cast<const uint4*>(hidden_gate + static_cast<size_t>(t) * rank_gu);
    const uint4* u = reinterpret_cast<const uint4*>(hidden_up + static_cast<size_t>(t) * rank_gu);
    uint4* dst = reinterpret_cast<uint4*>(send_rows + static_cast<size_t>(pos) * send_row_stride);
    const int vecs = rank_gu >> 3;
    for (int i = threadIdx.x; i < 2 * vecs; i += blockDim.x) dst[i] = (i < vecs) ? g[i] : u[i - vecs];
  }
  // rows beyond an owner's capacity are dropped: their combine index says so (every flat entry is
  // written by exactly one thread of this launch, so the caller need not initialise the array)
  for (int row = blockIdx.x * blockDim.x + threadIdx.x; row < num_rows; row += gridDim.x * blockDim.x) {
    int d = 0;
    while (d + 1 < world && row >= s_first[d + 1]) ++d;
    if (row - s_first[d] >= capacity) combine_index[perm[row]] = -1;
  }
}

}  // namespace tris

using namespace tris;

extern "C" int tris_ep_pack_rows(const void* hidden_gate_f16, const void* hidden_up_f16, int32_t rank_gu,
                                 const int32_t* selected_experts, const int32_t* perm,
                                 const int32_t* grouped_token_indices, int32_t num_rows, int32_t top_k,
                                 int32_t num_experts, int32_t world, int32_t capacity, void* send_rows_f16,
                                 int32_t send_row_stride, int32_t* send_ids, int32_t* combine_index,
                                 int32_t* overflow_dev, void* stream) {
  TRIS_REQUIRE(hidden_gate_f16 && hidden_up_f16 && selected_experts && perm && grouped_token_indices && send_rows_f16 &&
                   combine_index && overflow_dev,
               TRIS_ERR_INVALID_ARG, "tris_ep_pack_rows: null pointer");
  TRIS_REQUIRE(send_row_stride >= 2 * rank_gu && (send_row_stride & 7) == 0, TRIS_ERR_INVALID_ARG,
               "tris_ep_pack_rows: send_row_stride %d must be a multiple of 8 and >= 2*rank", send_row_stride);
  TRIS_REQUIRE(send_ids != nullptr || send_row_stride >= 2 * rank_gu + 8, TRIS_ERR_INVALID_ARG,
               "tris_ep_pack_rows: no place for the expert ids (send_ids NULL and no room behind the rows)");
  TRIS_REQUIRE(rank_gu > 0 && (rank_gu & 7) == 0, TRIS_ERR_UNSUPPORTED, "tris_ep_pack_rows: rank must be a multiple of 8");
  TRIS_REQUIRE(num_rows >= 0 && top_k > 0 && num_experts > 0 && world >= 1 && world <= 64 && capacity > 0,
               TRIS_ERR_INVALID_ARG, "tris_ep_pack_rows: bad sizes rows=%d world=%d capacity=%d", num_rows, world, capacity);
  const int slots = world * capacity;
  ep_pack_rows_kernel<<<std::min(slots, 4096), 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __half*>(hidden_gate_f16), static_cast<const __half*>(hidden_up_f16), rank_gu, selected_experts,
      perm, grouped_token_indices, num_rows, top_k, num_experts, world, capacity, static_cast<__half*>(send_rows_f16),
      send_row_stride, send_ids, combine_index, overflow_dev);
  return check_cuda(cudaGetLastError(), "ep_pack_rows_kernel launch");
}

extern "C" int tris_router_topk(const float* router_logits, int32_t num_tokens, int32_t num_experts, int32_t top_k,
                                int32_t norm_topk_prob, int32_t* selected_experts, float* routing_weights,
                                void* stream) {
  TRIS_REQUIRE(router_logits && selected_experts && routing_weights, TRIS_ERR_INVALID_ARG, "tris_router_topk: null pointer");
  TRIS_REQUIRE(num_tokens >= 0 && num_experts > 0 && top_k > 0 && top_k <= num_experts, TRIS_ERR_INVALID_ARG,
               "tris_router_topk: bad sizes T=%d E=%d k=%d", num_tokens, num_experts, top_k);
  TRIS_REQUIRE(num_experts <= 32 * kMaxExpertsPerLane && top_k <= 32, TRIS_ERR_UNSUPPORTED,
               "tris_router_topk: supports up to %d experts and top-32", 32 * kMaxExpertsPerLane);
  if (num_tokens == 0) return TRIS_OK;
  const int threads = 128;
  return check_cuda(launch_kernel(router_topk_kernel, dim3(ceil_div(num_tokens * 32, threads)), dim3(threads), 0,
                                  static_cast<cudaStream_t>(stream), programmatic_launch_default(), 1, router_logits,
                                  num_tokens, num_experts, top_k, norm_topk_prob, selected_experts, routing_weights),
                    "router_topk_kernel launch");
}

extern "C" int tris_build_grouped_route(const int32_t* selected_experts, int32_t num_tokens, int32_t top_k,
                                        int32_t num_experts, int32_t m_tile, int32_t* perm,
                                        int32_t* grouped_token_indices, int32_t* grouped_slots, int32_t* row_of_flat,
                                        int32_t* expert_ids, int32_t* segment_offsets, int32_t* problem_offsets,
                                        int32_t* counts, void* stream) {
  TRIS_REQUIRE(selected_experts && perm && grouped_token_indices && grouped_slots && row_of_flat && expert_ids &&
                   segment_offsets && problem_offsets && counts,
               TRIS_ERR_INVALID_ARG, "tris_build_grouped_route: null pointer");
  TRIS_REQUIRE(num_tokens >= 0 && top_k > 0 && num_experts > 0 && m_tile > 0, TRIS_ERR_INVALID_ARG,
               "tris_build_grouped_route: bad sizes T=%d k=%d E=%d m_tile=%d", num_tokens, top_k, num_experts, m_tile);
  return tris_build_grouped_route_ex(selected_experts, 1, 0, num_tokens, top_k, num_experts, m_tile, perm, grouped_token_indices,
                                     grouped_slots, row_of_flat, expert_ids, segment_offsets, problem_offsets, counts, nullptr, 0,
                                     stream);
}

extern "C" int tris_build_grouped_route_ex(const int32_t* selected_experts, int32_t selected_stride, int32_t id_offset,
                                           int32_t num_tokens, int32_t top_k, int32_t num_experts, int32_t m_tile,
                                           int32_t* perm, int32_t* grouped_token_indices, int32_t* grouped_slots,
                                           int32_t* row_of_flat, int32_t* expert_ids, int32_t* segment_offsets,
                                           int32_t* problem_offsets, int32_t* counts, int32_t* scratch,
                                           size_t scratch_bytes, void* stream) {
  TRIS_REQUIRE(selected_experts && perm && grouped_token_indices && grouped_slots && row_of_flat && expert_ids &&
                   segment_offsets && problem_offsets && counts,
               TRIS_ERR_INVALID_ARG, "tris_build_grouped_route: null pointer");
  TRIS_REQUIRE(num_tokens >= 0 && top_k > 0 && num_experts > 0 && m_tile > 0, TRIS_ERR_INVALID_ARG,
               "tris_build_grouped_route: bad sizes T=%d k=%d E=%d m_tile=%d", num_tokens, top_k, num_experts, m_tile);
  TRIS_REQUIRE(num_experts <= 320, TRIS_ERR_UNSUPPORTED, "tris_build_grouped_route: more than 320 experts");
  TRIS_REQUIRE(selected_stride >= 1, TRIS_ERR_INVALID_ARG, "tris_build_grouped_route: selected_stride %d", selected_stride);
  const SelectedIds ids{selected_experts, selected_stride, id_offset};
  const int rows = num_tokens * top_k;
  if (scratch && rows >= 4 * kRouteParChunk &&
      scratch_bytes >= sizeof(int32_t) * static_cast<size_t>(ceil_div(rows, kRouteParChunk)) * num_experts)
    return launch_route_parallel(ids, num_tokens, top_k, num_experts, m_tile, perm, grouped_token_indices,
                                 grouped_slots, row_of_flat, expert_ids, segment_offsets, problem_offsets, counts, scratch,
                                 static_cast<cudaStream_t>(stream), programmatic_launch_default());
  int sel_cap = 0;
  const int smem = route_smem_bytes(num_experts, rows, &sel_cap);
  return check_cuda(launch_kernel(build_route_kernel, dim3(1), dim3(kRouteThreads), smem, static_cast<cudaStream_t>(stream),
                                  programmatic_launch_default(), 1, ids, num_tokens, top_k, num_experts, m_tile,
                                  perm, grouped_token_indices, grouped_slots, row_of_flat, expert_ids, segment_offsets,
                                  problem_offsets, counts, sel_cap),
                    "build_route_kernel launch");
}

int tris::combine_routed_impl(const void* down_out_f16, const int32_t* row_of_flat, const float* routing_weights,
                              int num_tokens, int top_k, int hidden_size, void* final_f16, cudaStream_t stream,
                              bool pdl) {
  TRIS_REQUIRE(down_out_f16 && row_of_flat && routing_weights && final_f16, TRIS_ERR_INVALID_ARG, "tris_combine_routed: null pointer");
  TRIS_REQUIRE(num_tokens >= 0 && top_k > 0 && hidden_size > 0, TRIS_ERR_INVALID_ARG, "tris_combine_routed: bad sizes");
  TRIS_REQUIRE((hidden_size & 7) == 0, TRIS_ERR_UNSUPPORTED, "tris_combine_routed: hidden_size must be a multiple of 8");
  if (num_tokens == 0) return TRIS_OK;
  const long long total = static_cast<long long>(num_tokens) * (hidden_size / 8);
  const int threads = 256;
  return check_cuda(launch_kernel(combine_routed_kernel, dim3(static_cast<unsigned>((total + threads - 1) / threads)),
                                  dim3(threads), 0, stream, pdl, 1, static_cast<const __half*>(down_out_f16),
                                  row_of_flat, routing_weights, num_tokens, top_k, hidden_size,
                                  static_cast<__half*>(final_f16)),
                    "combine_routed_kernel launch");
}

extern "C" int tris_combine_routed(const void* down_out_f16, const int32_t* row_of_flat, const float* routing_weights,
                                   int32_t num_tokens, int32_t top_k, int32_t hidden_size, void* final_f16,
                                   void* stream) {
  return combine_routed_impl(down_out_f16, row_of_flat, routing_weights, num_tokens, top_k, hidden_size, final_f16,
                             static_cast<cudaStream_t>(stream), programmatic_launch_default());
}
