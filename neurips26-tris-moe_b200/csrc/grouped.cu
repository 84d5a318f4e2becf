// Grouped compact3 dequant-matmul kernels (decode / skinny regime), block-GR index build,
// and the two dump kernels used by the parity tests.
//
// One CTA = one (expert segment, output tile).  Per K chunk it stages the compressed
// planes (block-GR decode across the CTA's lanes, sign planes, scale tables) into shared
// memory, then every warp unpacks weights straight into m16n8k16 A fragments and
// multiplies them with the staged activation rows; no dequantized weight is written
// anywhere but registers.  fp32 accumulation.
#include <cooperative_groups.h>
#include <math.h>

#include <algorithm>

#include "compact3_tile.cuh"

namespace cg = cooperative_groups;

namespace tris {

// ---- block-GR sub-stream index -----------------------------------------------------------
__global__ void block_gr_build_index_kernel(TrisProjView v, uint32_t* index_out, int sub, int32_t* status) {
  const int nblk = proj_num_blocks(v);
  const long long total = static_cast<long long>(v.num_experts) * nblk;
  for (long long id = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; id < total;
       id += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int e = static_cast<int>(id / nblk), bi = static_cast<int>(id % nblk);
    const int32_t* off = v.q_gmap_gr_offsets + static_cast<size_t>(e) * (nblk + 1);
    const int begin = off[bi], end = off[bi + 1];
    const int meta = v.q_gmap_gr_meta[static_cast<size_t>(e) * nblk + bi];
    uint32_t* out = index_out + static_cast<size_t>(id) * sub;
    for (int j = 0; j < sub; ++j) out[j] = 0u;
    const int count = end - begin;
    const bool raw = (meta & TRIS_GR_META_RAW_FLAG) != 0;
    const int k = meta & TRIS_GR_META_K_MASK;
    const int one_count = meta >> TRIS_GR_META_ONE_COUNT_SHIFT;
    bool ok = begin >= 0 && count >= 0 && end <= v.gr_max_words && count <= TRIS_GR_BLOCK_WORDS;
    if (bi == 0 && begin != 0) ok = false;
    if (raw) {
      ok = ok && count == TRIS_GR_BLOCK_WORDS;
    } else {
      ok = ok && k <= TRIS_GR_MAX_K && one_count >= 0 && one_count <= TRIS_GR_BLOCK_WORDS * 32 &&
           (meta & ~(TRIS_GR_META_K_MASK | (0x1FFF << TRIS_GR_META_ONE_COUNT_SHIFT))) == 0 &&
           (one_count == 0 || count > 0);
    }
    if (!ok) {
      atomicExch(status, TRIS_ERR_CORRUPT);
      continue;
    }
    if (raw || one_count == 0) continue;
    const uint32_t* w =
        reinterpret_cast<const uint32_t*>(v.q_gmap_gr_words) + static_cast<size_t>(e) * v.gr_max_words + begin;
    const int per = (one_count + sub - 1) / sub;
    const int total_bits = count << 5;
    const uint32_t kmask = (1u << k) - 1u;
    int bitpos = 0, flatpos = 0;
    bool bad = false;
    for (int n = 0; n < one_count; ++n) {
      if (n % per == 0) out[n / per] = static_cast<uint32_t>(bitpos) | (static_cast<uint32_t>(flatpos) << 16);
      int q = 0;
      uint32_t bits = gr_peek32(w, count, bitpos);
      while (bits == 0u) {
        q += 32;
        bitpos += 32;
        if (bitpos >= total_bits) { bad = true; break; }
        bits = gr_peek32(w, count, bitpos);
      }
      if (bad) break;
      const int t = __ffs(bits) - 1;
      q += t;
      bitpos += t + 1;
      const uint32_t rem = gr_peek32(w, count, bitpos) & kmask;
      bitpos += k;
      flatpos += (q << k) | static_cast<int>(rem);
      if (bitpos > total_bits || flatpos >= TRIS_GR_BLOCK_WORDS * 32) { bad = true; break; }
      ++flatpos;
    }
    if (bad) atomicExch(status, TRIS_ERR_CORRUPT);
  }
}

// ---- packed-row group table ---------------------------------------------------------------
__global__ void build_row_groups_kernel(const int32_t* g_idx, int num_experts, int rank, int num_groups,
                                        int32_t* out, int32_t* status) {
  const int pr = (rank + 31) >> 5;
  const int total = num_experts * pr;
  for (int id = blockIdx.x * blockDim.x + threadIdx.x; id < total; id += gridDim.x * blockDim.x) {
    const int e = id / pr, p = id % pr;
    const int32_t* gi = g_idx + static_cast<size_t>(e) * rank;
    const int c0 = 32 * p, c1 = min(rank, c0 + 32);
    const int grp = gi[c0];
    bool ok = grp >= 0 && grp < num_groups;
    for (int c = c0 + 1; c < c1; ++c) ok = ok && gi[c] == grp;
    out[id] = ok ? grp : -1;
    if (!ok) atomicExch(status, TRIS_ERR_UNSUPPORTED);
  }
}

// ---- dump kernels -------------------------------------------------------------------------
__device__ __forceinline__ void init_barriers(uint64_t* mbar) { init_stage_barriers(mbar); }

// Second, equally bounded, wait for copies that may still be in flight before a CTA that
// saw a time-out leaves; then the status word is set.
template <typename Smem>
__device__ __forceinline__ void leave_after_timeout(Smem& sm, uint32_t par_w, uint32_t par_h, int32_t* status) {
  mbar_wait_bounded(&sm.mbar[0], par_w);
  mbar_wait_bounded(&sm.mbar[1], par_w);
  mbar_wait_bounded(&sm.mbar[2], par_h);
  if (threadIdx.x == 0 && status) atomicExch(status, TRIS_ERR_TIMEOUT);
}

// grid (ceil(O/128), ceil(pr/8), E); dense_out and weights_out may each be null
__global__ void __launch_bounds__(kThreads) compact3_dump_kernel(TrisProjView v, int32_t* dense_out,
                                                                  __half* weights_out, int32_t* status) {
  extern __shared__ uint4 smem_raw[];
  auto& sm = *reinterpret_cast<TileSmem<1, 1>*>(smem_raw);
  const int o0 = blockIdx.x * 128, p0 = blockIdx.y * KC;
  const int e = v.expert_slot ? v.expert_slot[blockIdx.z] : blockIdx.z;  // payload row block of the expert
  init_barriers(sm.mbar);
  stage_issue_weights<1, 1>(sm, &v, e, static_cast<int>(blockIdx.z), o0, p0);
  __syncthreads();
  uint32_t* dump = reinterpret_cast<uint32_t*>(sm.hrows);  // 4608 B >= 1024 words
  const bool ok = stage_finish_weights<1, 1>(sm, &v, e, static_cast<int>(blockIdx.z), o0, p0, 0u, 0u, dense_out ? dump : nullptr);
  if (__syncthreads_or(!ok)) {
    if (threadIdx.x == 0 && status) atomicExch(status, TRIS_ERR_TIMEOUT);
    return;
  }
  const int pr = proj_packed_rows(v);
  if (dense_out) {
    for (int i = threadIdx.x; i < kTileWords; i += kThreads) {
      const int p = i / 128, o = i % 128;
      if (p0 + p < pr && o0 + o < v.out_features)
        dense_out[(static_cast<size_t>(blockIdx.z) * pr + p0 + p) * v.out_features + o0 + o] =
            static_cast<int32_t>(dump[plane_index<1>(0, p, o)]);
    }
  }
  if (weights_out) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    RowScales rs[2];
    int rs_slot = -1;
    for (int p = 0; p < KC && p0 + p < pr; ++p) {
      uint32_t a[2][4];
      unpack_fragments<1, 1>(sm, 0, p, warp * 16, lane, rs, rs_slot, a);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int og = o0 + warp * 16 + g + 8 * h;
        if (og >= v.out_features) continue;
        __half* row = weights_out + (static_cast<size_t>(blockIdx.z) * v.out_features + og) * v.rank;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int ca = 32 * (p0 + p) + 4 * t + i, cb = ca + 16;
          if (ca < v.rank) row[ca] = __ushort_as_half(static_cast<unsigned short>(a[h][i] & 0xFFFFu));
          if (cb < v.rank) row[cb] = __ushort_as_half(static_cast<unsigned short>(a[h][i] >> 16));
        }
      }
    }
  }
}

// ---- grouped forward ----------------------------------------------------------------------


// ---- main loop of one 256-column chunk ------------------------------------------------------
// The warp's 16 outputs (lane (g, t): outputs g and g+8, column pairs 4t+i / 4t+i+16) against
// up to NT tiles of 8 activation rows; packed rows [p_lo, p_end) of the chunk.
template <int NPROJ, int NT>
__device__ __forceinline__ void main_chunk(const TileSmem<NPROJ, NT>& sm, int proj, int out_local, int lane,
                                           int nt_count, int p_lo, int p_end, float (&acc)[NT][4]) {
  constexpr int OW = Geom<NPROJ>::OW;
  const int g = lane >> 2, t = lane & 3;
  // Per-lane base addresses; inside the fully unrolled loop every access is base + constant.
  constexpr int NOB = Geom<NPROJ>::NOB;
  const int word0 = plane_index<NPROJ>(proj, 0, out_local + g);  // packed row p adds a constant
  const uint32_t* s1_base = sm.s1 + word0;
  const uint32_t* sel_base = sm.g + word0;
  const uint4* col_base = sm.coltab + proj * KC * 16 + t;
  const PackedRowInfo* pinfo = sm.ptab + proj * (KC + 1);
  const uint8_t* h_base = sm.hrows + (proj * NT * 8 + g) * kHiddenRowBytes + t * 16;
  const uint2* row_base = sm.rowtab + (proj * OW + out_local + g) * sm.row_stride;
  const int row_step = 8 * sm.row_stride;
  RowScales rs[2];
  int rs_slot = -1;
#pragma unroll
  for (int p = 0; p < KC; ++p) {
    if (p < p_lo || p >= p_end) continue;  // warp-uniform
    const PackedRowInfo info = pinfo[p];
    if (info.gslot != rs_slot) {  // groups span several packed rows
      rs_slot = info.gslot;
      rs[0] = broadcast_row_scales(row_base[rs_slot]);
      rs[1] = broadcast_row_scales(row_base[row_step + rs_slot]);
    }
    uint4 ct[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) ct[i] = col_base[p * 16 + i * 4];
    const bool any_salient = info.cw != 0u;
    uint32_t a[2][4];
    constexpr int kRowPair = NOB * 128;  // words between k blocks of the same output block
    const int poff = (p >> 1) * kRowPair + (p & 1) * 64;
    unpack_row(s1_base[poff], sel_base[poff], rs[0], ct, any_salient, t, a[0]);
    unpack_row(s1_base[poff + 8], sel_base[poff + 8], rs[1], ct, any_salient, t, a[1]);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      if (nt < nt_count) {
        const uint4 hv = *reinterpret_cast<const uint4*>(h_base + nt * 8 * kHiddenRowBytes + p * 64);
        mma_m16n8k16(acc[nt], a[0][0], a[1][0], a[0][1], a[1][1], hv.x, hv.y);
        mma_m16n8k16(acc[nt], a[0][2], a[1][2], a[0][3], a[1][3], hv.z, hv.w);
      }
    }
  }
}

// ---- epilogue of one row pass -----------------------------------------------------------------
// acc[nt] = {(out g, row 2t), (out g, row 2t+1), (out g+8, row 2t), (out g+8, row 2t+1)}.
// Output scale and bias, then for the gate/up pair SiLU(gate) * up: warps w (gate) and w+4
// (up) hold the two factors of the same 16 outputs.  They split the row tiles: tile nt is
// finished by projection (nt & 1), the other warp hands its values over through `xbuf`
// (4 * NT * 512 bytes of shared memory nobody else touches meanwhile).  With `pair_barrier`
// the buffer is free on entry and only the two warps meet, at a named barrier; otherwise the
// whole CTA synchronises before the buffer is written and before it is read.
template <int NPROJ, int NT, int EPI>
__device__ __forceinline__ void finish_rows(const GroupedArgs& args, float* xbuf, bool pair_barrier, int proj,
                                            int out_local, int warp, int lane, int expert, int o0, int r0, int rows,
                                            int nt_count, float (&acc)[NT][4]) {
  const int g = lane >> 2, t = lane & 3;
  const TrisProjView& v = args.proj[proj];
  float scale[2] = {1.f, 1.f}, bias[2] = {0.f, 0.f};
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int og = o0 + out_local + g + 8 * h;
    if (og < v.out_features) {
      if (v.output_scale) scale[h] = __half2float(reinterpret_cast<const __half*>(v.output_scale)[static_cast<size_t>(expert) * v.out_features + og]);
      if (v.bias) bias[h] = __half2float(reinterpret_cast<const __half*>(v.bias)[static_cast<size_t>(expert) * v.out_features + og]);
    }
  }
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[nt][c] = acc[nt][c] * scale[c >> 1] + bias[c >> 1];

  if (EPI == EPI_SILU_MUL) {
    if (!pair_barrier) __syncthreads();
    const int pw = warp & 3;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
      if (nt < nt_count && (nt & 1) != proj)
        *reinterpret_cast<float4*>(xbuf + ((pw * NT + nt) * 32 + lane) * 4) =
            make_float4(acc[nt][0], acc[nt][1], acc[nt][2], acc[nt][3]);
    if (pair_barrier) named_barrier_sync(1 + pw, 64);
    else __syncthreads();
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      if (nt >= nt_count || (nt & 1) != proj) continue;
      const float4 o = *reinterpret_cast<const float4*>(xbuf + ((pw * NT + nt) * 32 + lane) * 4);
      const float other[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float gv = proj == 0 ? acc[nt][c] : other[c];
        const float uv = proj == 0 ? other[c] : acc[nt][c];
        acc[nt][c] = __fdividef(gv, 1.f + __expf(-gv)) * uv;
      }
    }
  }
  {
    __half* outp = args.out[EPI == EPI_SILU_MUL ? 0 : proj];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      if (nt >= nt_count) break;
      if (EPI == EPI_SILU_MUL && (nt & 1) != proj) continue;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int n = nt * 8 + 2 * t + (c & 1);
        const int og = o0 + out_local + g + 8 * (c >> 1);
        if (n < rows && og < v.out_features) {
          const int orow = args.out_scatter ? args.out_scatter[r0 + n] : r0 + n;
          if (orow >= 0) outp[static_cast<size_t>(orow) * v.out_features + og] = __float2half_rn(acc[nt][c]);
        }
      }
    }
  }
}

// grid (ceil(O/OW), num_segments bound, ksplit); cluster (1, 1, ksplit).  With ksplit > 1 the
// CTAs of a cluster split every 256-column chunk between them and cluster rank 0 adds the
// partial tiles (read through distributed shared memory) before the epilogue: small batches
// have too few (expert, tile) units to fill the GPU otherwise.
template <int NPROJ, int NT, int EPI>
__global__ void __launch_bounds__(kThreads, (NT <= 4) ? 3 : 2) grouped_compact3_kernel(const __grid_constant__ GroupedArgs args) {
  constexpr int OW = Geom<NPROJ>::OW;
  extern __shared__ uint4 smem_raw[];
  auto& sm = *reinterpret_cast<TileSmem<NPROJ, NT>*>(smem_raw);
  cg::cluster_group cluster = cg::this_cluster();
  const int ksplit = args.ksplit > 1 ? args.ksplit : 1;
  const int p_lo = (KC / ksplit) * static_cast<int>(blockIdx.z), p_hi = p_lo + KC / ksplit;

  init_barriers(sm.mbar);
  // Activations come from the predecessor kernel; the route arrays too, unless the caller
  // says they are older, in which case the weight staging below overlaps the predecessor.
  bool waited = false;
  if (!args.weights_before_wait) {
    pdl_wait();
    pdl_launch_dependents();
    waited = true;
  }
  // seg < gridDim.y <= num_segments, the arrays' length: read them before the live count
  // is known, so that the four loads are in flight together
  const int seg = blockIdx.y;
  const int expert = args.expert_ids[seg];
  const int row_begin = args.segment_offsets[seg];
  const int row_end = min(args.segment_offsets[seg + 1], args.num_rows);
  const int nseg = args.num_segments_dev ? min(*args.num_segments_dev, args.num_segments) : args.num_segments;
  if (seg >= nseg) return;
  if (expert < 0 || expert >= args.proj[0].num_experts || row_end <= row_begin) return;
  // row block of the expert inside the payload tensors (a staging slot when they are paged in)
  const int e = args.proj[0].expert_slot ? args.proj[0].expert_slot[expert] : expert;
  // A paged payload whose expert was not brought in (more active experts than staging slots): the
  // slot table says -1.  Report it and store nothing rather than read another expert's bytes.
  if (e < 0 || (args.proj[0].gmap_slot && args.proj[0].gmap_slot[expert] < 0)) {
    if (threadIdx.x == 0 && args.status) atomicExch(args.status, TRIS_ERR_WORKSPACE);
    return;
  }

  const int o0 = blockIdx.x * OW;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int proj = (NPROJ == 2) ? (warp >> 2) : 0;
  const int out_local = (NPROJ == 2) ? (warp & 3) * 16 : warp * 16;
  const int pr = proj_packed_rows(args.proj[0]);
  const int num_chunks = (pr + KC - 1) / KC;
  const bool interleaved = args.hidden_interleaved != 0;

  int staged_chunk = -1;
  uint32_t par_w = 0u, par_h = 0u;
  bool dead = false;  // a bounded wait ran out: skip the work but keep meeting the cluster barriers
  for (int r0 = row_begin; r0 < row_end; r0 += NT * 8) {
    const int rows = min(NT * 8, row_end - r0);
    const int nt_count = (rows + 7) >> 3;
    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[nt][c] = 0.f;

    for (int kc = 0; kc < num_chunks; ++kc) {
      const int p0 = kc * KC;
      __syncthreads();  // previous consumers of the staging buffers are done
      if (dead) break;
      const bool need_w = staged_chunk != kc;
      auto row_src = [&](int n) { return args.row_gather ? args.row_gather[r0 + n] : (r0 + n); };
      if (need_w) stage_issue_weights<NPROJ, NT>(sm, args.proj, e, expert, o0, p0, p_lo, p_hi);
      if (waited) stage_issue_hidden<NPROJ, NT>(sm, args.hidden, args.proj, p0, rows, interleaved, args.hidden_stride, row_src);
      __syncthreads();
      bool ok = true;
      if (need_w) {
        ok = stage_finish_weights<NPROJ, NT>(sm, args.proj, e, expert, o0, p0, par_w, par_w, nullptr, p_lo, p_hi);
        par_w ^= 1u;
        staged_chunk = kc;
      }
      if (!waited) {  // first pass of a CTA that staged its weights ahead of the predecessor's end
        pdl_wait();
        pdl_launch_dependents();
        waited = true;
        stage_issue_hidden<NPROJ, NT>(sm, args.hidden, args.proj, p0, rows, interleaved, args.hidden_stride, row_src);
        __syncthreads();
      }
      ok = mbar_wait_bounded(&sm.mbar[2], par_h) && ok;
      par_h ^= 1u;
      if (__syncthreads_or(!ok)) {
        leave_after_timeout(sm, par_w ^ 1u, par_h ^ 1u, args.status);
        dead = true;
        break;
      }

      main_chunk<NPROJ, NT>(sm, proj, out_local, lane, nt_count, p_lo, min(p_hi, pr - p0), acc);
    }

    if (ksplit > 1) {
      // partial tiles of the cluster -> rank 0 (the activation rows are dead by now)
      __syncthreads();
      float4* part = reinterpret_cast<float4*>(sm.hrows);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
        part[(warp * NT + nt) * 32 + lane] = make_float4(acc[nt][0], acc[nt][1], acc[nt][2], acc[nt][3]);
      cluster.sync();
      if (cluster.block_rank() == 0) {
        for (int r = 1; r < ksplit; ++r) {
          const float4* remote = cluster.map_shared_rank(part, r);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            const float4 v = remote[(warp * NT + nt) * 32 + lane];
            acc[nt][0] += v.x; acc[nt][1] += v.y; acc[nt][2] += v.z; acc[nt][3] += v.w;
          }
        }
      }
      cluster.sync();  // peers keep their shared memory until rank 0 has read it
      if (cluster.block_rank() != 0) continue;  // next row pass (same trip count in every CTA)
    }
    if (dead) continue;
    {
      // Up to 4 tiles the SiLU exchange buffer is the staged bitmap data (dead since the select
      // plane was built); the 8-tile variant needs the activation rows' space and full barriers.
      constexpr bool kPairBarrier = NT <= 4;
      static_assert(!kPairBarrier || 4 * NT * 32 * 16 <= sizeof(sm.s2raw) + sizeof(sm.gmraw), "exchange buffer");
      float* xbuf = reinterpret_cast<float*>(kPairBarrier ? reinterpret_cast<void*>(sm.s2raw) : reinterpret_cast<void*>(sm.hrows));
      finish_rows<NPROJ, NT, EPI>(args, xbuf, kPairBarrier, proj, out_local, warp, lane, expert, o0, r0, rows, nt_count, acc);
    }
  }
}

// tensor-core path for prefill-sized segments (grouped_umma.cu)
bool grouped_umma_applicable(const GroupedArgs& args, int rows_hint);
int launch_grouped_umma(const GroupedArgs& args, int nproj, int epi, cudaStream_t stream, bool pdl);

// ---- host launchers -----------------------------------------------------------------------
static int validate_proj(const TrisProjView* v, const char* name, bool need_runtime) {
  TRIS_REQUIRE(v != nullptr, TRIS_ERR_INVALID_ARG, "%s: null projection view", name);
  TRIS_REQUIRE(v->num_experts > 0 && v->out_features > 0 && v->rank > 0 && v->num_groups > 0,
               TRIS_ERR_INVALID_ARG, "%s: non-positive dims E=%d O=%d r=%d G=%d", name, v->num_experts,
               v->out_features, v->rank, v->num_groups);
  TRIS_REQUIRE(v->qweight1 && v->c_map && v->col_pack3 && v->row_pack3, TRIS_ERR_INVALID_ARG,
               "%s: qweight1/c_map/col_pack3/row_pack3 must be set", name);
  TRIS_REQUIRE(v->sign2_rows >= 0 && (v->sign2_rows == 0 || (v->qweight2_sparse && v->qweight2_sparse_prefix)),
               TRIS_ERR_INVALID_ARG, "%s: qweight2_sparse needs its prefix", name);
  if (v->use_block_gr) {
    TRIS_REQUIRE(v->q_gmap_gr_words && v->q_gmap_gr_offsets && v->q_gmap_gr_meta && v->gr_max_words >= 0,
                 TRIS_ERR_INVALID_ARG, "%s: block-GR tensors missing", name);
    if (need_runtime) {
      TRIS_REQUIRE(v->gr_index != nullptr, TRIS_ERR_INVALID_ARG,
                   "%s: block-GR payload has no sub-stream index (call tris_block_gr_build_index)", name);
      const int s = v->gr_substreams;
      TRIS_REQUIRE(s >= 1 && s <= 32 && (s & (s - 1)) == 0, TRIS_ERR_INVALID_ARG,
                   "%s: gr_substreams=%d must be a power of two <= 32", name, s);
    }
  } else {
    TRIS_REQUIRE(v->gmap_sparse_rows == 0 || (v->q_gmap_sparse && v->q_gmap_sparse_prefix), TRIS_ERR_INVALID_ARG,
                 "%s: q_gmap_sparse needs its prefix", name);
  }
  TRIS_REQUIRE(!(v->gmap_slot && v->expert_slot), TRIS_ERR_INVALID_ARG,
               "%s: gmap_slot and expert_slot are mutually exclusive", name);
  if (need_runtime)
    TRIS_REQUIRE(v->packed_row_group != nullptr || v->num_groups == 1, TRIS_ERR_INVALID_ARG,
                 "%s: packed_row_group missing (call tris_build_row_groups)", name);
  return TRIS_OK;
}

template <int NPROJ, int NT, int EPI>
static int launch_grouped(const GroupedArgs& args, cudaStream_t stream, bool pdl) {
  const size_t smem = sizeof(TileSmem<NPROJ, NT>);
  auto kernel = grouped_compact3_kernel<NPROJ, NT, EPI>;
  static bool configured[64] = {};  // per instantiation, per device
  int dev = 0;
  TRIS_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    TRIS_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  const int ksplit = args.ksplit > 1 ? args.ksplit : 1;
  dim3 grid(ceil_div(args.proj[0].out_features, Geom<NPROJ>::OW), args.num_segments, ksplit);
  return check_cuda(launch_kernel(kernel, grid, dim3(kThreads), smem, stream, pdl, ksplit, args),
                    "grouped_compact3_kernel launch");
}

template <int NPROJ, int EPI>
static int dispatch_grouped(const GroupedArgs& args, int max_rows, cudaStream_t stream, bool pdl) {
  // one 256-column chunk and no K split: persistent CTAs that prefetch their next tile
  if (max_rows <= 8) return launch_grouped<NPROJ, 1, EPI>(args, stream, pdl);
  if (max_rows <= 16) return launch_grouped<NPROJ, 2, EPI>(args, stream, pdl);
  if (max_rows <= 32) return launch_grouped<NPROJ, 4, EPI>(args, stream, pdl);
  return launch_grouped<NPROJ, 8, EPI>(args, stream, pdl);
}

static int fill_route(GroupedArgs& a, const TrisRouteView* route) {
  TRIS_REQUIRE(route != nullptr && route->expert_ids && route->segment_offsets, TRIS_ERR_INVALID_ARG,
               "route: expert_ids/segment_offsets must be set");
  TRIS_REQUIRE(route->num_segments >= 0 && route->num_rows >= 0, TRIS_ERR_INVALID_ARG, "route: negative sizes");
  a.expert_ids = route->expert_ids;
  a.segment_offsets = route->segment_offsets;
  a.num_segments_dev = route->num_segments_dev;
  a.row_gather = route->row_gather;
  a.out_scatter = route->out_row_scatter;
  a.num_segments = route->num_segments;
  a.num_rows = route->num_rows;
  a.status = route->status_dev;
  a.hidden_interleaved = (route->flags & TRIS_ROUTE_HIDDEN_PAIR_INTERLEAVED) != 0;
  a.hidden_stride = route->hidden_row_stride;
  return TRIS_OK;
}

// CTAs per tile: small batches have few (segment, tile) units, so a cluster splits each
// unit's K range to put more SMs to work.
static int pick_ksplit(const TrisProjView* proj, const TrisRouteView* route, int out_per_cta) {
  // Measured on B200 at decode batch 1 (128 units): splitting K over 4 CTAs shortens the main
  // loop, but block-GR decode (a per-lane chain of ~12 codewords), the staging round trips and
  // the two cluster barriers do not shrink, and the layer got slower (54 vs 38 us).  The split
  // stays available for shapes with long K, where the main loop dominates.
  const int units = ceil_div(proj->out_features, out_per_cta) * std::max(1, route->num_segments);
  if (proj->rank >= 2048 && units <= 160) return 2;
  return 1;
}

// Rows per segment (the launch's estimate) up to which the tile-record kernel is used.  It multiplies
// 32 rows per pass and re-unpacks the weights for every pass; from ~64 rows per segment on, the
// plane-staging kernel (64 rows per pass) and, beyond grouped_tc_min_rows(), the tcgen05 kernel do
// less work per row.
static int tiled_max_rows() { return std::min(64, grouped_tc_min_rows()); }
// Above that, up to the tcgen05 threshold, the tile-record kernel that keeps a chunk's unpacked weights in
// registers across row passes takes single-chunk projections (rank <= 256).
static bool tiled_takes(const TrisProjView& v, int rows) {
  return rows <= tiled_max_rows() || (v.rank <= 256 && rows <= grouped_tc_min_rows());
}

// Rows per activation tile: sized for the typical segment (mean + 4 sigma of a balanced
// router), never above the caller's bound; longer segments take several passes.
static int rows_hint(const TrisRouteView* route) { return route_rows_hint(route); }
int route_rows_hint(const TrisRouteView* route) {
  const int bound = route->max_rows_per_segment > 0 ? route->max_rows_per_segment : route->num_rows;
  if (route->num_segments <= 0) return bound;
  const double mean = static_cast<double>(route->num_rows) / route->num_segments;
  const int typical = static_cast<int>(mean + 4.0 * sqrt(mean));
  return std::max(1, std::min(bound, typical));
}

}  // namespace tris

using namespace tris;

extern "C" size_t tris_block_gr_index_bytes(int32_t num_experts, int32_t packed_rows, int32_t out_features,
                                            int32_t substreams) {
  if (num_experts <= 0 || packed_rows <= 0 || out_features <= 0 || substreams <= 0) return 0;
  const size_t nblk = static_cast<size_t>((packed_rows + 1) / 2) * ((out_features + 63) / 64);
  return static_cast<size_t>(num_experts) * nblk * substreams * sizeof(uint32_t);
}

extern "C" int tris_block_gr_build_index(const TrisProjView* proj, uint32_t* gr_index_out, int32_t substreams,
                                         int32_t* status_dev, void* stream) {
  int st = validate_proj(proj, "tris_block_gr_build_index", false);
  if (st != TRIS_OK) return st;
  TRIS_REQUIRE(proj->use_block_gr, TRIS_ERR_INVALID_ARG, "tris_block_gr_build_index: payload is not block-GR");
  TRIS_REQUIRE(gr_index_out && status_dev, TRIS_ERR_INVALID_ARG, "tris_block_gr_build_index: null output");
  TRIS_REQUIRE(substreams >= 1 && substreams <= 32 && (substreams & (substreams - 1)) == 0, TRIS_ERR_INVALID_ARG,
               "tris_block_gr_build_index: substreams=%d must be a power of two <= 32", substreams);
  const int pr = (proj->rank + 31) / 32;
  const long long total = static_cast<long long>(proj->num_experts) * ((pr + 1) / 2) * ((proj->out_features + 63) / 64);
  const int threads = 128;
  const int blocks = static_cast<int>(std::min<long long>((total + threads - 1) / threads, 65535));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  TRIS_CUDA(cudaMemsetAsync(status_dev, 0, sizeof(int32_t), s));
  block_gr_build_index_kernel<<<blocks, threads, 0, s>>>(*proj, gr_index_out, substreams, status_dev);
  return check_cuda(cudaGetLastError(), "block_gr_build_index_kernel launch");
}

extern "C" int tris_build_row_groups(const int32_t* g_idx, int32_t num_experts, int32_t rank, int32_t num_groups,
                                     int32_t* packed_row_group_out, int32_t* status_dev, void* stream) {
  TRIS_REQUIRE(g_idx && packed_row_group_out && status_dev, TRIS_ERR_INVALID_ARG, "tris_build_row_groups: null pointer");
  TRIS_REQUIRE(num_experts > 0 && rank > 0 && num_groups > 0, TRIS_ERR_INVALID_ARG, "tris_build_row_groups: bad dims");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int total = num_experts * ((rank + 31) / 32);
  TRIS_CUDA(cudaMemsetAsync(status_dev, 0, sizeof(int32_t), s));
  build_row_groups_kernel<<<ceil_div(total, 128), 128, 0, s>>>(g_idx, num_experts, rank, num_groups,
                                                               packed_row_group_out, status_dev);
  return check_cuda(cudaGetLastError(), "build_row_groups_kernel launch");
}

extern "C" int tris_block_gr_decode(const TrisProjView* proj, int32_t* dense_out, void* stream) {
  int st = validate_proj(proj, "tris_block_gr_decode", true);
  if (st != TRIS_OK) return st;
  TRIS_REQUIRE(proj->use_block_gr && dense_out, TRIS_ERR_INVALID_ARG, "tris_block_gr_decode: needs a block-GR payload and an output");
  if (proj_has_tile_records(*proj)) return launch_tiled_dump(proj, dense_out, nullptr, static_cast<cudaStream_t>(stream));
  const int pr = (proj->rank + 31) / 32;
  dim3 grid(ceil_div(proj->out_features, 128), ceil_div(pr, KC), proj->num_experts);
  const size_t smem = sizeof(TileSmem<1, 1>);
  TRIS_CUDA(cudaFuncSetAttribute(compact3_dump_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  compact3_dump_kernel<<<grid, kThreads, smem, static_cast<cudaStream_t>(stream)>>>(*proj, dense_out, nullptr, nullptr);
  return check_cuda(cudaGetLastError(), "compact3_dump_kernel launch");
}

extern "C" int tris_compact3_dequantize(const TrisProjView* proj, void* weights_out_f16, void* stream) {
  int st = validate_proj(proj, "tris_compact3_dequantize", true);
  if (st != TRIS_OK) return st;
  TRIS_REQUIRE(weights_out_f16, TRIS_ERR_INVALID_ARG, "tris_compact3_dequantize: null output");
  if (proj_has_tile_records(*proj)) return launch_tiled_dump(proj, nullptr, weights_out_f16, static_cast<cudaStream_t>(stream));
  const int pr = (proj->rank + 31) / 32;
  dim3 grid(ceil_div(proj->out_features, 128), ceil_div(pr, KC), proj->num_experts);
  const size_t smem = sizeof(TileSmem<1, 1>);
  TRIS_CUDA(cudaFuncSetAttribute(compact3_dump_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  compact3_dump_kernel<<<grid, kThreads, smem, static_cast<cudaStream_t>(stream)>>>(
      *proj, nullptr, static_cast<__half*>(weights_out_f16), nullptr);
  return check_cuda(cudaGetLastError(), "compact3_dump_kernel launch");
}

// Tile-record form of the tcgen05 kernel: lane-order activation rows, single-chunk projections, segments
// above the tensor-core threshold.
static bool umma_records_applicable(const TrisProjView& v, const GroupedArgs& a, bool lane_order, int rows) {
  const int stride = a.hidden_stride > 0 ? a.hidden_stride : v.rank;
  return lane_order && rows > grouped_tc_min_rows() && v.rank % 32 == 0 && v.rank <= 256 && stride % 8 == 0 && stride >= v.rank;
}
static void fill_record_slots(GroupedArgs& a) {
  const int rec = std::max(a.proj[0].max_record_bytes, a.proj[1].max_record_bytes);
  a.rec_slot_bytes = ((rec + 15) & ~15) + 16;
  a.col_slot_bytes = std::max(a.proj[0].col_record_bytes, a.proj[1].col_record_bytes);
  a.hidden_lane_order = 1;
  a.ksplit = 1;
}

int tris::grouped_forward_impl(const TrisProjView* proj, const TrisRouteView* route, const void* hidden_f16,
                               void* out_f16, cudaStream_t stream, LaunchOpts opts) {
  int st = validate_proj(proj, "tris_grouped_forward", true);
  if (st != TRIS_OK) return st;
  TRIS_REQUIRE(hidden_f16 && out_f16, TRIS_ERR_INVALID_ARG, "tris_grouped_forward: null hidden/out");
  GroupedArgs a{};
  st = fill_route(a, route);
  if (st != TRIS_OK) return st;
  if (a.num_segments == 0 || a.num_rows == 0) return TRIS_OK;
  const bool lane_order = (route->flags & TRIS_ROUTE_HIDDEN_LANE_ORDER) != 0;
  TRIS_REQUIRE(!lane_order || (proj_has_tile_records(*proj) && !a.hidden_interleaved), TRIS_ERR_INVALID_ARG,
               "tris_grouped_forward: lane-order activations need a projection with tile records");
  const bool col_scaled = route->hidden_col_scale != nullptr;
  TRIS_REQUIRE(!col_scaled || (proj_has_tile_records(*proj) && !a.hidden_interleaved && !lane_order), TRIS_ERR_UNSUPPORTED,
               "tris_grouped_forward: hidden_col_scale needs tile records and row-major activations");
  if (proj_has_tile_records(*proj) && !a.hidden_interleaved && umma_records_applicable(*proj, a, lane_order, rows_hint(route))) {
    if (a.hidden_stride <= 0) a.hidden_stride = proj->rank;
    a.proj[0] = a.proj[1] = *proj;
    a.hidden[0] = a.hidden[1] = static_cast<const __half*>(hidden_f16);
    a.out[0] = a.out[1] = static_cast<__half*>(out_f16);
    a.weights_before_wait = opts.pdl && opts.weights_before_wait;
    fill_record_slots(a);
    return launch_grouped_umma(a, 1, EPI_STORE, stream, opts.pdl);
  }
  if (proj_has_tile_records(*proj) && !a.hidden_interleaved && (lane_order || col_scaled || tiled_takes(*proj, rows_hint(route))))
    return launch_grouped_tiled(proj, nullptr, route, hidden_f16, nullptr, out_f16, nullptr, 0, rows_hint(route), stream, opts);
  TRIS_REQUIRE(!a.hidden_interleaved || proj->rank % 32 == 0, TRIS_ERR_INVALID_ARG,
               "tris_grouped_forward: pair-interleaved activations need rank % 32 == 0");
  if (a.hidden_stride <= 0) a.hidden_stride = proj->rank;
  TRIS_REQUIRE(a.hidden_stride >= proj->rank, TRIS_ERR_INVALID_ARG, "tris_grouped_forward: hidden_row_stride < rank");
  TRIS_REQUIRE(!a.hidden_interleaved || (a.hidden_stride % 2 == 0 && reinterpret_cast<uintptr_t>(hidden_f16) % 4 == 0),
               TRIS_ERR_INVALID_ARG, "tris_grouped_forward: pair-interleaved activation rows must be 4-byte aligned");
  a.proj[0] = *proj;
  a.proj[1] = *proj;
  a.hidden[0] = a.hidden[1] = static_cast<const __half*>(hidden_f16);
  a.out[0] = a.out[1] = static_cast<__half*>(out_f16);
  a.weights_before_wait = opts.pdl && opts.weights_before_wait;
  a.ksplit = pick_ksplit(proj, route, 128);
  if (grouped_umma_applicable(a, rows_hint(route))) return launch_grouped_umma(a, 1, EPI_STORE, stream, opts.pdl);
  return dispatch_grouped<1, EPI_STORE>(a, rows_hint(route), stream, opts.pdl);
}

extern "C" int tris_grouped_hidden_layout(const TrisProjView* proj_a, const TrisProjView* proj_b, int32_t num_rows,
                                          int32_t num_segments, int32_t max_rows_per_segment) {
  if (proj_a == nullptr || proj_a->rank % 32 != 0) return TRIS_OUT_F16;
  TrisRouteView route{};
  route.num_rows = num_rows;
  route.num_segments = num_segments;
  route.max_rows_per_segment = max_rows_per_segment;
  const bool records = proj_has_tile_records(*proj_a) && (proj_b == nullptr || proj_has_tile_records(*proj_b));
  // single-chunk projections with records read lane order at every size (decode kernels, the register-cached
  // kernel, the tile-record form of the tcgen05 kernel); larger ranks only where the decode kernels take them
  return (records && (proj_a->rank <= 256 || tiled_takes(*proj_a, route_rows_hint(&route)))) ? TRIS_OUT_F16_LANE_ORDER
                                                                                             : TRIS_OUT_F16_PAIR_INTERLEAVED;
}

extern "C" int tris_grouped_forward(const TrisProjView* proj, const TrisRouteView* route, const void* hidden_f16,
                                    void* out_f16, void* stream) {
  LaunchOpts opts;
  opts.pdl = programmatic_launch_default();
  return grouped_forward_impl(proj, route, hidden_f16, out_f16, static_cast<cudaStream_t>(stream), opts);
}

int tris::grouped_pair_forward_impl(const TrisProjView* proj_a, const TrisProjView* proj_b,
                                    const TrisRouteView* route, const void* hidden_a_f16, const void* hidden_b_f16,
                                    void* out_a_f16, void* out_b_f16, int fuse_silu_mul, cudaStream_t stream,
                                    LaunchOpts opts) {
  int st = validate_proj(proj_a, "tris_grouped_pair_forward(a)", true);
  if (st != TRIS_OK) return st;
  st = validate_proj(proj_b, "tris_grouped_pair_forward(b)", true);
  if (st != TRIS_OK) return st;
  TRIS_REQUIRE(proj_a->num_experts == proj_b->num_experts && proj_a->out_features == proj_b->out_features &&
                   proj_a->rank == proj_b->rank && proj_a->num_groups == proj_b->num_groups,
               TRIS_ERR_UNSUPPORTED, "tris_grouped_pair_forward: the two projections must share E, O, r and G");
  TRIS_REQUIRE((proj_a->use_block_gr != 0) == (proj_b->use_block_gr != 0) &&
                   (!proj_a->use_block_gr || proj_a->gr_substreams == proj_b->gr_substreams),
               TRIS_ERR_UNSUPPORTED, "tris_grouped_pair_forward: the two projections must share the g_map format");
  TRIS_REQUIRE(hidden_a_f16 && hidden_b_f16 && out_a_f16 && (fuse_silu_mul || out_b_f16), TRIS_ERR_INVALID_ARG,
               "tris_grouped_pair_forward: null hidden/out");
  GroupedArgs a{};
  st = fill_route(a, route);
  if (st != TRIS_OK) return st;
  if (a.num_segments == 0 || a.num_rows == 0) return TRIS_OK;
  const bool lane_order = (route->flags & TRIS_ROUTE_HIDDEN_LANE_ORDER) != 0;
  const bool records = proj_has_tile_records(*proj_a) && proj_has_tile_records(*proj_b);
  TRIS_REQUIRE(!lane_order || (records && !a.hidden_interleaved), TRIS_ERR_INVALID_ARG,
               "tris_grouped_pair_forward: lane-order activations need projections with tile records");
  const bool col_scaled = route->hidden_col_scale != nullptr;
  TRIS_REQUIRE(!col_scaled || (records && !a.hidden_interleaved && !lane_order), TRIS_ERR_UNSUPPORTED,
               "tris_grouped_pair_forward: hidden_col_scale needs tile records and row-major activations");
  if (records && !a.hidden_interleaved && umma_records_applicable(*proj_a, a, lane_order, rows_hint(route))) {
    if (a.hidden_stride <= 0) a.hidden_stride = proj_a->rank;
    a.proj[0] = *proj_a;
    a.proj[1] = *proj_b;
    a.hidden[0] = static_cast<const __half*>(hidden_a_f16);
    a.hidden[1] = static_cast<const __half*>(hidden_b_f16);
    a.out[0] = static_cast<__half*>(out_a_f16);
    a.out[1] = static_cast<__half*>(out_b_f16);
    a.weights_before_wait = opts.pdl && opts.weights_before_wait;
    fill_record_slots(a);
    return launch_grouped_umma(a, 2, fuse_silu_mul ? EPI_SILU_MUL : EPI_STORE, stream, opts.pdl);
  }
  if (records && !a.hidden_interleaved && (lane_order || col_scaled || tiled_takes(*proj_a, rows_hint(route))))
    return launch_grouped_tiled(proj_a, proj_b, route, hidden_a_f16, hidden_b_f16, out_a_f16, out_b_f16, fuse_silu_mul ? 2 : 1,
                                rows_hint(route), stream, opts);
  TRIS_REQUIRE(!a.hidden_interleaved || proj_a->rank % 32 == 0, TRIS_ERR_INVALID_ARG,
               "tris_grouped_pair_forward: pair-interleaved activations need rank % 32 == 0");
  if (a.hidden_stride <= 0) a.hidden_stride = proj_a->rank;
  TRIS_REQUIRE(a.hidden_stride >= proj_a->rank, TRIS_ERR_INVALID_ARG, "tris_grouped_pair_forward: hidden_row_stride < rank");
  TRIS_REQUIRE(!a.hidden_interleaved || (a.hidden_stride % 2 == 0 && reinterpret_cast<uintptr_t>(hidden_a_f16) % 4 == 0 &&
                                         reinterpret_cast<uintptr_t>(hidden_b_f16) % 4 == 0),
               TRIS_ERR_INVALID_ARG, "tris_grouped_pair_forward: pair-interleaved activation rows must be 4-byte aligned");
  a.proj[0] = *proj_a;
  a.proj[1] = *proj_b;
  a.hidden[0] = static_cast<const __half*>(hidden_a_f16);
  a.hidden[1] = static_cast<const __half*>(hidden_b_f16);
  a.out[0] = static_cast<__half*>(out_a_f16);
  a.out[1] = static_cast<__half*>(out_b_f16);
  a.weights_before_wait = opts.pdl && opts.weights_before_wait;
  a.ksplit = pick_ksplit(proj_a, route, 64);
  const int max_rows = rows_hint(route);
  if (grouped_umma_applicable(a, max_rows))
    return launch_grouped_umma(a, 2, fuse_silu_mul ? EPI_SILU_MUL : EPI_STORE, stream, opts.pdl);
  if (fuse_silu_mul) return dispatch_grouped<2, EPI_SILU_MUL>(a, max_rows, stream, opts.pdl);
  return dispatch_grouped<2, EPI_STORE>(a, max_rows, stream, opts.pdl);
}

extern "C" int tris_grouped_pair_forward(const TrisProjView* proj_a, const TrisProjView* proj_b,
                                         const TrisRouteView* route, const void* hidden_a_f16,
                                         const void* hidden_b_f16, void* out_a_f16, void* out_b_f16,
                                         int32_t fuse_silu_mul, void* stream) {
  LaunchOpts opts;
  opts.pdl = programmatic_launch_default();
  return grouped_pair_forward_impl(proj_a, proj_b, route, hidden_a_f16, hidden_b_f16, out_a_f16, out_b_f16,
                                   fuse_silu_mul, static_cast<cudaStream_t>(stream), opts);
}

