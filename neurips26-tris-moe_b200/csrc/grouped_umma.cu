// Grouped compact3 dequant-matmul on the tcgen05 tensor cores, for segments with enough rows
// to be a dense contraction (prefill).  One CTA owns one (expert segment, 128-output tile):
//
//   1. the compressed tile of each projection is staged and decoded exactly as in the decode
//      kernel (TMA copies, block-GR decode, select plane), then unpacked ONCE into a shared-
//      memory A operand (fp16, K-major core-matrix layout) - 64 KB per projection for the
//      256-column chunk;
//   2. the segment's activation rows stream through in passes of NB rows: cp.async stages
//      them as the B operand, one thread issues tcgen05.mma (M = 128 outputs, N = NB rows,
//      K = 16 per instruction) into TMEM accumulators (gate and up side by side), and the
//      epilogue reads TMEM, applies SiLU*mul or scale/bias, and stores fp16.
//
// The K order of both operands is the pair-interleaved order of the activation rows (column
// j of a 32-column group at position 2*(j%16) + j/16): a lane's four column pairs are then
// eight consecutive K positions, i.e. one 16-byte core-matrix row, so the unpack writes its
// fragments with two 128-bit stores per packed row.  Needs rank % 32 == 0 and rank <= 256.
#include <algorithm>
#include <atomic>

#include "compact3_tile.cuh"
#include "tile_records.cuh"
#include "umma.cuh"

namespace tris {

template <int NPROJ>
struct UmmaGeom {
  static constexpr int NB = 128 / NPROJ;            // activation rows per pass
  static constexpr int kABytes = kTcM * 256 * 2;    // one projection's A operand
  static constexpr int kBBytes = NB * 256 * 2;      // one projection's B operand
  static constexpr int kUnionBytes =
      (NPROJ * kBBytes > static_cast<int>(sizeof(TileSmem<1, 1>))) ? NPROJ * kBBytes : static_cast<int>(sizeof(TileSmem<1, 1>));
  static constexpr int kSmemBytes = NPROJ * kABytes + kUnionBytes + 128;
};

__device__ __forceinline__ void mbar_inval(uint64_t* bar) {
  asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Phase 1 from tile records (REC): the 128-output tile is two 64-output records of the chunk plus the
// (expert, chunk) column record, fetched with three bulk copies; 8 warps decode the 8 Golomb-Rice blocks,
// then warp w unpacks record w / 4, outputs 16 * (w % 4) .. + 15: the non-salient fragments of a packed row
// are the lane's eight consecutive K positions of the lane-order activation layout, i.e. one 16-byte
// core-matrix row of the A operand; the salient columns are then written over their (zero) places.
// Staging area inside the region that later holds the B operand: [mbarrier 64][record 0][record 1][column
// record][two g_map planes].
template <int NPROJ>
__device__ __forceinline__ bool umma_unpack_from_records(const GroupedArgs& args, uint8_t* region, uint8_t* a_op, int expert,
                                                         int warp, int lane, uint32_t& parity) {
  using namespace tr;
  uint64_t* bar = reinterpret_cast<uint64_t*>(region);
  uint8_t* rec_base = region + 64;
  uint8_t* col = rec_base + 2 * args.rec_slot_bytes;
  uint32_t* gmap_base = reinterpret_cast<uint32_t*>(col + args.col_slot_bytes);
  const int tiles = tiles_per_expert(args.proj[0].out_features);
  const int tile0 = 2 * static_cast<int>(blockIdx.x);
  const int r = warp >> 2, og = warp & 3, g = lane >> 2, t = lane & 3;
  bool ok = true;
#pragma unroll 1
  for (int proj = 0; proj < NPROJ; ++proj) {
    const TrisProjView& v = args.proj[proj];
    __syncthreads();  // the staging area is free (previous projection unpacked)
    if (lane == 0 && warp < 2) {
      const bool valid = tile0 + warp < tiles;
      const uint2 d = valid ? load_desc(v, expert, tile0 + warp, 0) : make_uint2(0u, 0u);
      issue_record(v, expert, 0, d, rec_base + warp * args.rec_slot_bytes, warp == 0 ? col : nullptr, valid, bar);
    }
    reinterpret_cast<uint4*>(gmap_base)[threadIdx.x] = make_uint4(0u, 0u, 0u, 0u);  // both planes
    __syncthreads();
    ok = mbar_wait_bounded(bar, parity) && ok;
    parity ^= 1u;
    const bool tile_valid = tile0 + r < tiles;
    StagedTile st{rec_base + r * args.rec_slot_bytes, col, gmap_base + r * 512};
    if (ok && tile_valid) gr_decode_block(st.rec, og, const_cast<uint32_t*>(st.gmap), lane);
    if (__syncthreads_or(!ok)) {  // also publishes the decoded planes
      mbar_wait_bounded(bar, parity ^ 1u);  // copies that may still be in flight must not land in a dead CTA
      return false;
    }
    uint8_t* a_dst = a_op + proj * (kTcM * 256 * 2);
    const int out0 = r * kTileOut + og * 16 + g;  // this lane's outputs inside the 128-output tile: out0, out0 + 8
    const LaneShifts ls = lane_shifts(t);
    const ColHeader* ch = reinterpret_cast<const ColHeader*>(col);
    if (tile_valid) {
      int p = 0;
      for (int slot = 0; slot < ch->num_slots; ++slot) {
        const RowScalesNs rs = load_row_scales_ns(st, slot, og * 16, lane);
        const int p_end = min(static_cast<int>(ch->slot_end[slot]), kChunkRows);
        for (; p < p_end; ++p) {
          uint32_t a[2][4];
          unpack_fragments_ns(st, p, og * 16, lane, rs, ls, a);
#pragma unroll
          for (int h = 0; h < 2; ++h)
            *reinterpret_cast<uint4*>(a_dst + ((4 * p + t) * kTcM + out0 + 8 * h) * 16) = make_uint4(a[h][0], a[h][1], a[h][2], a[h][3]);
        }
      }
      __syncwarp();  // the salient halves below land in core-matrix rows other lanes of this warp wrote above
      const int sal_words = ch->sal_words;
      for (int q = 0; q < sal_words; ++q) {
        uint32_t a[2][4];
        unpack_fragments_sal(st, q, og * 16, lane, ls, a);
        const uint16_t* salcol = reinterpret_cast<const uint16_t*>(col + kColHdrBytes + kColTabBytes + q * kSalEntryBytes + 192);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int slot = lane_pair_col(t, i);
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const unsigned c = salcol[slot + 16 * half];  // column inside the chunk, 0xFFFF: unused slot
            if (c == 0xFFFFu) continue;
            const int pos = lane_order_pos(static_cast<int>(c & 31u));
            const int kchunk = 4 * static_cast<int>(c >> 5) + (pos >> 3);
#pragma unroll
            for (int h = 0; h < 2; ++h)
              *reinterpret_cast<uint16_t*>(a_dst + (kchunk * kTcM + out0 + 8 * h) * 16 + (pos & 7) * 2) =
                  static_cast<uint16_t>(half ? (a[h][i] >> 16) : (a[h][i] & 0xFFFFu));
          }
        }
      }
    } else {
      // outputs past the projection: a zero tile (their results are never stored, but keep the MMA finite)
      const int pr = (v.rank + 31) >> 5;
      for (int p = 0; p < pr && p < kChunkRows; ++p)
#pragma unroll
        for (int h = 0; h < 2; ++h)
          *reinterpret_cast<uint4*>(a_dst + ((4 * p + t) * kTcM + out0 + 8 * h) * 16) = make_uint4(0u, 0u, 0u, 0u);
    }
  }
  return ok;
}

// grid (ceil(O/128), num_segments bound); 256 threads
template <int NPROJ, int EPI, bool REC>
__global__ void __launch_bounds__(kThreads, 1) grouped_umma_kernel(const __grid_constant__ GroupedArgs args) {
  constexpr int NB = UmmaGeom<NPROJ>::NB;
  extern __shared__ uint4 smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(smem_raw);
  uint8_t* a_op = smem;                                          // [NPROJ][128 x 256 fp16]
  uint8_t* shared_region = smem + NPROJ * UmmaGeom<NPROJ>::kABytes;
  auto& stage = *reinterpret_cast<TileSmem<1, 1>*>(shared_region);  // phase 1
  uint8_t* b_op = shared_region;                                 // phase 2: [NPROJ][NB x 256 fp16]
  uint64_t* mma_bar = reinterpret_cast<uint64_t*>(shared_region + UmmaGeom<NPROJ>::kUnionBytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(mma_bar + 1);
  int32_t* flag = reinterpret_cast<int32_t*>(mma_bar + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint64_t* rec_bar = reinterpret_cast<uint64_t*>(shared_region);  // REC: record copies (two issuing lanes arrive)
  if (REC) {
    if (threadIdx.x == 0) mbar_init(rec_bar, 2);
  } else {
    init_stage_barriers(stage.mbar);
  }
  if (threadIdx.x == 0) {
    mbar_init(mma_bar, 1);
    fence_mbar_init();
    *flag = 0;
  }
  if (warp == 0) tmem_alloc(tmem_slot, NPROJ * NB);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem = *tmem_slot;

  bool waited = false;
  if (!args.weights_before_wait) {
    pdl_wait();
    pdl_launch_dependents();
    waited = true;
  }
  const int seg = blockIdx.y;
  const int nseg = args.num_segments_dev ? min(*args.num_segments_dev, args.num_segments) : args.num_segments;
  int expert = -1, row_begin = 0, row_end = 0;
  if (seg < nseg) {
    expert = args.expert_ids[seg];
    row_begin = args.segment_offsets[seg];
    row_end = min(args.segment_offsets[seg + 1], args.num_rows);
  }
  bool live = expert >= 0 && expert < args.proj[0].num_experts && row_end > row_begin;
  bool unpaged = false;  // a paged payload whose expert has no staging slot (the slot table says -1)
  if (live && ((args.proj[0].expert_slot && args.proj[0].expert_slot[expert] < 0) ||
               (args.proj[0].gmap_slot && args.proj[0].gmap_slot[expert] < 0))) {
    live = false;
    unpaged = true;
  }
  const int o0 = blockIdx.x * kTcM;
  const int rank = args.proj[0].rank;
  const int pr = proj_packed_rows(args.proj[0]);
  bool ok = true;

  if (live && REC) {
    uint32_t rec_parity = 0u;
    ok = umma_unpack_from_records<NPROJ>(args, shared_region, a_op, expert, warp, lane, rec_parity);
  } else if (live) {
    const int e = args.proj[0].expert_slot ? args.proj[0].expert_slot[expert] : expert;
    const int g = lane >> 2, t = lane & 3;
    // ---- phase 1: decode and unpack each projection's tile into its A operand --------------
#pragma unroll 1
    for (int proj = 0; proj < NPROJ; ++proj) {
      __syncthreads();
      stage_issue_weights<1, 1>(stage, &args.proj[proj], e, expert, o0, 0);
      __syncthreads();
      ok = stage_finish_weights<1, 1>(stage, &args.proj[proj], e, expert, o0, 0, static_cast<uint32_t>(proj & 1), static_cast<uint32_t>(proj & 1), nullptr) && ok;
      __syncthreads();
      uint8_t* a_dst = a_op + proj * UmmaGeom<NPROJ>::kABytes;
      RowScales rs[2];
      int rs_slot = -1;
      for (int p = 0; p < pr && p < KC; ++p) {
        uint32_t a[2][4];
        unpack_fragments<1, 1>(stage, 0, p, warp * 16, lane, rs, rs_slot, a);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int out = warp * 16 + g + 8 * h;
          *reinterpret_cast<uint4*>(a_dst + ((4 * p + t) * kTcM + out) * 16) = make_uint4(a[h][0], a[h][1], a[h][2], a[h][3]);
        }
      }
    }
  }
  if (!waited) {
    pdl_wait();
    pdl_launch_dependents();
  }
  // Every thread ran its own bounded waits in phase 1: make the verdict CTA-uniform before any
  // branch that contains barriers (this barrier also ends the life of the staging structure,
  // whose memory becomes the B operand).
  ok = !__syncthreads_or(!ok);
  if (threadIdx.x == 0) {
    if (REC) {
      mbar_inval(rec_bar);
    } else {
      mbar_inval(&stage.mbar[0]);
      mbar_inval(&stage.mbar[1]);
      mbar_inval(&stage.mbar[2]);
    }
  }
  __syncthreads();

  // ---- phase 2: stream the segment's rows through the tensor core ---------------------------
  if (live && ok) {
    const uint32_t idesc = umma_idesc_f16(kTcM, NB);
    const int ksteps = rank / 16;
    const int kchunks = rank / 64 + ((rank % 64) ? 1 : 0);
    uint32_t parity = 0u;
    const int quad = warp & 3, col_half = warp >> 2;
    const int og = o0 + quad * 32 + lane;
    float scale[NPROJ], bias[NPROJ];
#pragma unroll
    for (int proj = 0; proj < NPROJ; ++proj) {
      const TrisProjView& v = args.proj[proj];
      scale[proj] = 1.f;
      bias[proj] = 0.f;
      if (og < v.out_features) {
        if (v.output_scale) scale[proj] = __half2float(reinterpret_cast<const __half*>(v.output_scale)[static_cast<size_t>(expert) * v.out_features + og]);
        if (v.bias) bias[proj] = __half2float(reinterpret_cast<const __half*>(v.bias)[static_cast<size_t>(expert) * v.out_features + og]);
      }
    }
    for (int r0 = row_begin; r0 < row_end; r0 += NB) {
      const int rows = min(NB, row_end - r0);
#pragma unroll
      for (int proj = 0; proj < NPROJ; ++proj) {
        const __half* hid = args.hidden[proj];
        for (int cc = 0; cc < kchunks; ++cc) {
          stage_operand_async<NB>(b_op + proj * UmmaGeom<NPROJ>::kBBytes + cc * 8 * NB * 16, hid, [&](int n) -> const __half* {
            if (n >= rows) return nullptr;
            const int src = args.row_gather ? args.row_gather[r0 + n] : (r0 + n);
            return hid + static_cast<size_t>(src) * args.hidden_stride + 64 * cc;
          }, min(8, (rank - 64 * cc) / 8));
        }
      }
      cp_async_commit();
      cp_async_wait<0>();
      fence_proxy_async();  // A (first pass) and B stores -> visible to the tensor core
      __syncthreads();
      if (threadIdx.x == 0) {
        tcgen05_fence_after();
#pragma unroll
        for (int proj = 0; proj < NPROJ; ++proj) {
          const uint32_t a_addr = smem_u32(a_op + proj * UmmaGeom<NPROJ>::kABytes);
          const uint32_t b_addr = smem_u32(b_op + proj * UmmaGeom<NPROJ>::kBBytes);
          for (int j = 0; j < ksteps; ++j)
            umma_f16_ss(tmem + proj * NB, umma_smem_desc(a_addr + j * 2 * kTcM * 16, kTcM * 16, 128),
                        umma_smem_desc(b_addr + j * 2 * NB * 16, NB * 16, 128), idesc, j > 0 ? 1u : 0u);
        }
        umma_commit(mma_bar);
      }
      if (!mbar_wait_bounded(mma_bar, parity)) ok = false;
      tcgen05_fence_after();
      if (__syncthreads_or(!ok)) {
        // the MMAs may still be in flight: give them one more bounded wait before TMEM is released
        mbar_wait_bounded(mma_bar, parity);
        ok = false;
        break;
      }
      parity ^= 1u;

      // epilogue: this warp reads TMEM lanes [32*quad, +32) (outputs) and half of the row columns
      const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
      const TrisProjView& v0 = args.proj[0];
#pragma unroll 1
      for (int c0 = col_half * (NB / 2); c0 < (col_half + 1) * (NB / 2); c0 += 16) {
        if (c0 >= rows) break;
        float va[16], vb[16];
        tmem_ld_16(tmem + lane_base + c0, va);
        if (NPROJ == 2) tmem_ld_16(tmem + lane_base + NB + c0, vb);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int n = c0 + j;
          if (n >= rows || og >= v0.out_features) continue;
          const int orow = args.out_scatter ? args.out_scatter[r0 + n] : r0 + n;  // same address for the warp
          if (orow < 0) continue;
          const size_t oi = static_cast<size_t>(orow) * v0.out_features + og;
          const float x = va[j] * scale[0] + bias[0];
          if (EPI == EPI_SILU_MUL) {
            const float u = vb[j] * scale[NPROJ - 1] + bias[NPROJ - 1];
            args.out[0][oi] = __float2half_rn(__fdividef(x, 1.f + __expf(-x)) * u);
          } else {
            args.out[0][oi] = __float2half_rn(x);
            if (NPROJ == 2) args.out[1][oi] = __float2half_rn(vb[j] * scale[NPROJ - 1] + bias[NPROJ - 1]);
          }
        }
      }
      tcgen05_fence_before();
      __syncthreads();  // TMEM and the B operand are free for the next pass
    }
  }
  if (!ok) *flag = 1;
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, NPROJ * NB);
  if (*flag && threadIdx.x == 0 && args.status) atomicExch(args.status, TRIS_ERR_TIMEOUT);
  if (unpaged && threadIdx.x == 0 && args.status) atomicExch(args.status, TRIS_ERR_WORKSPACE);
}

template <int NPROJ, int EPI, bool REC>
static int launch_umma_grouped(const GroupedArgs& args, cudaStream_t stream, bool pdl) {
  auto kernel = grouped_umma_kernel<NPROJ, EPI, REC>;
  const size_t smem = UmmaGeom<NPROJ>::kSmemBytes;
  static bool configured[64] = {};
  int dev = 0;
  TRIS_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    TRIS_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  dim3 grid(ceil_div(args.proj[0].out_features, kTcM), args.num_segments);
  return check_cuda(launch_kernel(kernel, grid, dim3(kThreads), smem, stream, pdl, 1, args), "grouped_umma_kernel launch");
}

// Rows per segment above which the launchers pick this kernel.  Measured on B200 (OLMoE- and
// Mixtral-shaped layers, 256 to 4096 prefill tokens, up to ~1000 rows per expert): the register
// path (eight 8-row tiles per pass, two CTAs per SM, weights re-unpacked every pass) is faster
// throughout - 220 vs 298 us per layer at 512 tokens, 616 vs 661 at 2048 (OLMoE), 1872 vs 1935 at
// 4096 (Mixtral) - because this kernel holds a whole SM (192 KB of shared memory) while its
// decode-and-unpack phase runs on eight warps.  So the default sits above the measured range.
static std::atomic<int> g_tc_min_rows{2048};

int grouped_tc_min_rows() { return g_tc_min_rows.load(std::memory_order_relaxed); }

// Dense-contraction path: activations must be pair-interleaved, rank a multiple of 32 and at
// most one 256-column chunk.
bool grouped_umma_applicable(const GroupedArgs& args, int rows_hint) {
  const TrisProjView& v = args.proj[0];
  return rows_hint > g_tc_min_rows.load(std::memory_order_relaxed) && (args.hidden_interleaved || args.hidden_lane_order) &&
         (v.rank % 32) == 0 && v.rank <= 256 && args.ksplit <= 1 && (args.hidden_stride % 8) == 0;
}

int launch_grouped_umma(const GroupedArgs& args, int nproj, int epi, cudaStream_t stream, bool pdl) {
  if (args.hidden_lane_order) {  // tile records
    TRIS_REQUIRE(64 + 2 * static_cast<size_t>(args.rec_slot_bytes) + args.col_slot_bytes + 4096 <= static_cast<size_t>(UmmaGeom<1>::kUnionBytes),
                 TRIS_ERR_UNSUPPORTED, "grouped_umma_kernel: tile records of %d bytes do not fit the staging area", args.rec_slot_bytes);
    if (nproj == 1) return launch_umma_grouped<1, EPI_STORE, true>(args, stream, pdl);
    if (epi == EPI_SILU_MUL) return launch_umma_grouped<2, EPI_SILU_MUL, true>(args, stream, pdl);
    return launch_umma_grouped<2, EPI_STORE, true>(args, stream, pdl);
  }
  if (nproj == 1) return launch_umma_grouped<1, EPI_STORE, false>(args, stream, pdl);
  if (epi == EPI_SILU_MUL) return launch_umma_grouped<2, EPI_SILU_MUL, false>(args, stream, pdl);
  return launch_umma_grouped<2, EPI_STORE, false>(args, stream, pdl);
}

}  // namespace tris

extern "C" int tris_set_grouped_tc_min_rows(int32_t rows) {
  return tris::g_tc_min_rows.exchange(rows < 0 ? 0 : rows, std::memory_order_relaxed);
}
