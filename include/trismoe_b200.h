/*
 * trismoe_b200 — C ABI of the B200 (sm_100a) grouped-expert dequant-GEMM runtime for
 * TriS-MoE compact3 payloads.
 *
 * Every entry point takes plain pointers and sizes (device pointers unless the name ends
 * in `_host`), an explicit cudaStream_t passed as `void*`, and returns an int status
 * (TRIS_OK == 0).  The library owns no device memory: weights, activations, outputs,
 * workspaces and derived indexes are caller-owned buffers.  Nothing here falls back to
 * the CPU; a launch that cannot run returns a non-zero status and `tris_last_error()`
 * holds the reason for the calling thread.
 *
 * Reference interfaces these entry points stand in for are cited per declaration as
 * path:line inside the TriS-MoE source tree
 * (QL  = AutoGPTQ/auto_gptq/nn_modules/qlinear/qlinear_cuda.py,
 *  CPP = AutoGPTQ/autogptq_extension/TriSMoE/TriSMoE_cuda.cpp,
 *  CU  = AutoGPTQ/autogptq_extension/TriSMoE/TriSMoE_cuda_kernel.cu,
 *  SC  = AutoGPTQ/auto_gptq/modeling_tris_moe/grouped_payload_sidecar.py,
 *  MO  = AutoGPTQ/auto_gptq/modeling_tris_moe/modeling_olmoe.py,
 *  RW  = tools/rewrite_runtime_min_checkpoint.py).
 */
#ifndef TRISMOE_B200_H_
#define TRISMOE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Mirrors TRIS_COMPACT3_KERNEL_ABI_VERSION (CPP:1138-1139); the payload layout is ABI 2. */
#define TRIS_COMPACT3_KERNEL_ABI_VERSION 2
#define TRIS_B200_ABI_VERSION 4

enum {
  TRIS_OK = 0,
  TRIS_ERR_INVALID_ARG = 1,   /* null pointer, negative size, inconsistent dims            */
  TRIS_ERR_UNSUPPORTED = 2,   /* shape/layout this build does not cover                    */
  TRIS_ERR_CUDA = 3,          /* a CUDA runtime call or launch failed                      */
  TRIS_ERR_CORRUPT = 4,       /* payload failed validation (offsets, meta, prefixes)      */
  TRIS_ERR_WORKSPACE = 5,     /* caller workspace too small                               */
  TRIS_ERR_TIMEOUT = 6        /* a bounded device-side wait ran out (status word set)     */
};

/* Block Golomb-Rice constants (QL:486-494, CU:63-68). */
#define TRIS_GR_BLOCK_OUT 64
#define TRIS_GR_BLOCK_PACKED_ROWS 2
#define TRIS_GR_BLOCK_WORDS 128
#define TRIS_GR_META_K_MASK 0xF
#define TRIS_GR_META_RAW_FLAG 16
#define TRIS_GR_META_ONE_COUNT_SHIFT 8
#define TRIS_GR_MAX_K 7
/* Sub-streams per block recorded by tris_block_gr_build_index (power of two, <= 32). */
#define TRIS_GR_DEFAULT_SUBSTREAMS 32

/*
 * One E-stacked compact3 projection, i.e. the dict returned by
 * build_grouped_precomputed_payload (QL:1512-1636) with every tensor replaced by its
 * device pointer.  Shapes use O = out_features, r = rank (K), pr = ceil(r/32).
 */
typedef struct TrisProjView {
  int32_t num_experts;          /* E                                                       */
  int32_t out_features;         /* O                                                       */
  int32_t rank;                 /* r: columns of the per-expert factor                     */
  int32_t num_groups;           /* G: row_pack3 is [E, O, G]                               */
  int32_t sign2_rows;           /* rows of qweight2_sparse  (max over experts)             */
  int32_t gmap_sparse_rows;     /* rows of q_gmap_sparse (0 when absent)                   */
  int32_t gr_max_words;         /* words per expert in q_gmap_gr_words (0 when absent)     */
  int32_t use_block_gr;         /* compact3_use_block_gr                                   */
  const int32_t* qweight1;               /* [E, pr, O]      sign plane 1                   */
  const int32_t* qweight2_sparse;        /* [E, sign2_rows, O] sign plane 2, salient cols  */
  const int32_t* qweight2_sparse_prefix; /* [E, pr+1]                                      */
  const int32_t* q_gmap_sparse;          /* [E, gmap_sparse_rows, O] (streaming format)    */
  const int32_t* q_gmap_sparse_prefix;   /* [E, pr+1]                                      */
  const int32_t* q_gmap_gr_words;        /* [E, gr_max_words]                              */
  const int32_t* q_gmap_gr_offsets;      /* [E, nblk+1]                                    */
  const int32_t* q_gmap_gr_meta;         /* [E, nblk]                                      */
  const int32_t* c_map;                  /* [E, pr]  bit = salient column                  */
  const int32_t* g_idx;                  /* [E, r]   group of each column                  */
  const int64_t* col_pack3;              /* [E, r]   4 x fp16                              */
  const int64_t* row_pack3;              /* [E, O, G] 4 x fp16                             */
  const void* output_scale;              /* [E, O] fp16 or NULL (has_output_scale False)   */
  const void* bias;                      /* [E, O] fp16 or NULL                            */
  /* Derived at load time by tris_block_gr_build_index / tris_build_row_groups.           */
  const uint32_t* gr_index;              /* [E, nblk, gr_substreams] or NULL               */
  int32_t gr_substreams;
  const int32_t* packed_row_group;       /* [E, pr] group id of each 32-column word        */
  /* When non-NULL, expert e of this view reads q_gmap_sparse row block
     gmap_slot[e] of a staging buffer instead of row block e (SC:1104-1106). */
  const int32_t* gmap_slot;
  /* When non-NULL, every E-stacked tensor of this view (q_gmap_sparse included, unless
     gmap_slot overrides it) is a staging buffer in which expert e occupies row block
     expert_slot[e]: the layout tris_page_experts fills from pinned host memory. */
  const int32_t* expert_slot;
  /* Tile-major records built at load time by tris_tile_records_plan / _build (NULL when absent):
     per (expert, 64 outputs, 256 columns) one contiguous piece holding everything a CTA needs
     of that tile, so that it arrives with a single bulk copy, plus per (expert, 256 columns)
     a record of finished column-scale tables.  When present, the grouped entry points and the
     two dump entry points read the records instead of the tensors above. */
  const void* tile_records;
  const uint32_t* tile_desc;             /* [records + 1][2]: {offset / 16, bytes}                */
  const void* col_records;               /* [E, chunks] x col_record_bytes                        */
  int32_t col_record_bytes;
  int32_t max_record_bytes;              /* largest tile record of this projection                */
  int32_t max_sal_words;                 /* salient words per column record                       */
  int32_t reserved0;
} TrisProjView;

/*
 * Grouped route on the device (QL:1328-1338).  Arrays may be padded to E (+1): segment s
 * is live when s < *num_segments_dev (or s < num_segments when num_segments_dev is NULL).
 */
typedef struct TrisRouteView {
  const int32_t* expert_ids;        /* [>= num_segments] expert of each segment            */
  const int32_t* segment_offsets;   /* [>= num_segments+1] row range of each segment       */
  const int32_t* num_segments_dev;  /* optional device scalar (no host sync needed)        */
  int32_t num_segments;             /* upper bound used to size the grid                   */
  int32_t num_rows;                 /* R: routed rows                                      */
  int32_t max_rows_per_segment;     /* upper bound (<= tokens); 0 = num_rows               */
  const int32_t* row_gather;        /* optional [R]: source row of each grouped row        */
  int32_t* status_dev;              /* optional device int32: set to TRIS_ERR_TIMEOUT when a
                                       bounded wait inside a kernel ran out                */
  int32_t flags;                    /* TRIS_ROUTE_* bits                                   */
  int32_t hidden_row_stride;        /* halves between activation rows; 0 = the projection's rank */
  const int32_t* out_row_scatter;   /* optional [R]: output row of each grouped row (default: the
                                       grouped row itself); no reference counterpart - lets a
                                       caller get results back in its own row order without a
                                       second pass                                          */
  const void* hidden_col_scale;     /* optional fp16 [rank]: every activation row is multiplied by it,
                                       rounded to fp16, while it is staged - the input scale
                                       vector of an ordinary compact3 linear with ns_mode == 1
                                       (compact3_linear_forward, has_input_scale, CU:2176-2200).
                                       Row-major activations and a projection with tile records only */
} TrisRouteView;

/* Activation rows handed to the grouped kernels are "pair-interleaved": inside every group
   of 32 columns, column j sits at position 2*(j%16) + j/16 (what tris_shared_hidden_forward
   writes with out_mode = TRIS_OUT_F16_PAIR_INTERLEAVED).  Needs rank % 32 == 0. */
#define TRIS_ROUTE_HIDDEN_PAIR_INTERLEAVED 1
/* Activation rows in "lane order", the order the tile-record kernels consume: inside every group
   of 32 columns, column j sits at 8*(j%4) + 2*s + j/16 with s = 1, 3, 0, 2 for (j/4)%4 = 0..3
   (what tris_shared_hidden_forward writes with out_mode = TRIS_OUT_F16_LANE_ORDER).  Needs
   rank % 32 == 0 and a projection with tile records. */
#define TRIS_ROUTE_HIDDEN_LANE_ORDER 2

#define TRIS_OUT_F16 0
#define TRIS_OUT_F32 1
#define TRIS_OUT_F16_PAIR_INTERLEAVED 2
#define TRIS_OUT_F16_LANE_ORDER 3

/* ---- library / errors -------------------------------------------------------------- */

/* Replaces the import-time ABI check of the pybind11 module (QL:14-37, CPP:1138-1139). */
int tris_abi_version(void);
int tris_compact3_kernel_abi_version(void);
const char* tris_status_string(int status);
/* Message of the last non-zero status returned on this thread (TORCH_CHECK text in CU). */
const char* tris_last_error(void);

/*
 * Programmatic dependent launch for the stand-alone entry points (process-wide switch, off by
 * default; returns the previous value).  When on, every kernel these entry points launch may start
 * while its predecessor in the stream drains and waits (griddepcontrol.wait) before it touches what
 * the predecessor wrote - the launch gaps of a chain of small kernels (router, route, exchange,
 * grouped kernels, combine) overlap instead of adding up.  tris_moe_layer_forward always launches
 * this way.  No reference counterpart.
 */
int tris_set_programmatic_launch(int32_t enable);

/* ---- block Golomb-Rice ------------------------------------------------------------- */

/*
 * Host encoder of one dense packed g_map [pr, O] into the block-GR stream; same format as
 * QuantLinear._pack_block_gr_gmap_tensor (QL:3793-3859) / pack_block_gr_gmap_tensor
 * (RW:252-347).  `words_out` needs room for nblk*128 words; `*num_words` receives the
 * count actually written.
 */
int tris_block_gr_encode_host(const int32_t* dense_words, int32_t packed_rows, int32_t out_features,
                              int32_t force_raw, int32_t* words_out, int64_t words_capacity,
                              int32_t* offsets_out, int32_t* meta_out, int64_t* num_words);

/* The same with the Rice parameter searched in [k_min, k_max] only (k_min == k_max fixes it): the
   --blockgr-k / --blockgr-k-min / --blockgr-k-max options of the reference exporter
   (pack_block_gr_gmap_tensor(fixed_k, k_min, k_max), RW:252-347; bounds RW:227-250). */
int tris_block_gr_encode_host_k(const int32_t* dense_words, int32_t packed_rows, int32_t out_features,
                                int32_t force_raw, int32_t k_min, int32_t k_max, int32_t* words_out,
                                int64_t words_capacity, int32_t* offsets_out, int32_t* meta_out, int64_t* num_words);

/* Bytes of the derived sub-stream index for a projection. */
size_t tris_block_gr_index_bytes(int32_t num_experts, int32_t packed_rows, int32_t out_features,
                                 int32_t substreams);

/*
 * Validates offsets/meta of every block (monotone offsets, k <= 7, one_count <= 4096,
 * stream inside gr_max_words) and records, per block, where each of `substreams` equal
 * runs of ones starts (bit offset and flat position).  No reference counterpart: the
 * reference decodes each block on one thread (CU:426-479); this index lets a warp share
 * a block.  `status_dev` (device int32) receives 0 or TRIS_ERR_CORRUPT.
 */
int tris_block_gr_build_index(const TrisProjView* proj, uint32_t* gr_index_out, int32_t substreams,
                              int32_t* status_dev, void* stream);

/*
 * Expands the block-GR stream of every expert to the dense packed g_map [E, pr, O]
 * (what decode_block_gr_block, CU:426-479, leaves in shared memory; also the predecode of
 * compact3_tris_grouped_block_gr_predecode, CPP / CU:4683-4718, QL:1452-1509).
 * Runs the same device decoder as the grouped kernels.
 */
int tris_block_gr_decode(const TrisProjView* proj, int32_t* dense_out, void* stream);

/* ---- compact3 ---------------------------------------------------------------------- */

/* Per packed row group table + validation of g_idx (prepare_compact3_k64_groups, QL:364-407). */
int tris_build_row_groups(const int32_t* g_idx, int32_t num_experts, int32_t rank, int32_t num_groups,
                          int32_t* packed_row_group_out, int32_t* status_dev, void* stream);

/*
 * Dequantized weights [E, O, r] fp16 (QuantLinear._dequantize_compact3_matrix, QL:4200-4236;
 * device form load_compact3_weight_from_packs_gmap_word, CU:709-743), produced by the same
 * tile staging and register unpack code as the grouped kernels.
 */
int tris_compact3_dequantize(const TrisProjView* proj, void* weights_out_f16, void* stream);

/* ---- tile records ------------------------------------------------------------------ */

/*
 * Load-time repack of a block-GR projection into tile-major records (no reference counterpart:
 * the reference kernels gather each tile from the E-stacked planes on every launch,
 * CU:5382-5586).  Sequence: tris_tile_record_count -> allocate desc [count + 1][2] uint32 and a
 * device int64[4] -> tris_tile_records_plan (fills desc; info = {total record bytes, largest
 * record, salient words per column record, 0}) -> read info, allocate `total` bytes of records
 * and tris_col_record_bytes(proj, salient words) of column records (both 16-byte aligned) ->
 * tris_tile_records_build -> set the tile_* fields of the view.  The view passed in needs the
 * sub-stream index (32 sub-streams) and packed_row_group.  The records repeat, re-arranged, what
 * the E-stacked tensors hold; the byte total is DRAM traffic of the kernels, not algorithmic bytes.
 */
int64_t tris_tile_record_count(const TrisProjView* proj);
int64_t tris_col_record_bytes(const TrisProjView* proj, int32_t max_sal_words);
int tris_tile_records_plan(const TrisProjView* proj, uint32_t* desc_out, int64_t* info_out, void* stream);
int tris_tile_records_build(const TrisProjView* proj, const uint32_t* desc, void* records_out,
                            void* col_records_out, int32_t max_sal_words, void* stream);

/* ---- route ------------------------------------------------------------------------- */

/*
 * build_grouped_route (QL:1301-1378, CPP:741-793) without the host sync: all outputs are
 * device arrays padded to num_experts(+1).  selected_experts is [T, k] int32.  Rows of one
 * expert are ordered by ascending flat (token, slot) index.
 *   perm[R], grouped_token_indices[R], grouped_slots[R], row_of_flat[R] (inverse of perm; -1 for
 *   entries whose expert id is outside [0, E), which are left out of every segment),
 *   expert_ids[E] (unused tail = -1), segment_offsets[E+1] (tail = R),
 *   problem_offsets[E+1] (ceil(len/m_tile) prefix), counts[2] = {num_segments, total_problem_tiles}.
 */
int tris_build_grouped_route(const int32_t* selected_experts, int32_t num_tokens, int32_t top_k,
                             int32_t num_experts, int32_t m_tile, int32_t* perm,
                             int32_t* grouped_token_indices, int32_t* grouped_slots,
                             int32_t* row_of_flat, int32_t* expert_ids, int32_t* segment_offsets,
                             int32_t* problem_offsets, int32_t* counts, void* stream);

/*
 * The same route with two extensions.  (1) Entry f of the flat id list is read as
 * selected_experts[f * selected_stride] - id_offset (1 and 0 for a plain [T, k] array): the receiver
 * of an expert-parallel exchange finds the id of slot f behind that slot's activation row and
 * numbered globally, and routes in place.  (2) With `scratch` (caller-owned device memory, at least
 * ceil(num_tokens * top_k / 2048) * num_experts int32, free for the duration of the launches) and
 * >= 8192 routed rows the sort runs on several CTAs (count, scan, place) instead of one; results
 * are identical.  scratch == NULL keeps the single CTA.
 */
int tris_build_grouped_route_ex(const int32_t* selected_experts, int32_t selected_stride, int32_t id_offset,
                                int32_t num_tokens, int32_t top_k, int32_t num_experts, int32_t m_tile, int32_t* perm,
                                int32_t* grouped_token_indices, int32_t* grouped_slots, int32_t* row_of_flat,
                                int32_t* expert_ids, int32_t* segment_offsets, int32_t* problem_offsets,
                                int32_t* counts, int32_t* scratch, size_t scratch_bytes, void* stream);

/*
 * Router head of OlmoeSparseMoeBlock.forward (MO:1052-1058): softmax over fp32 logits
 * [T, E], top-k, optional renormalisation.  Outputs selected_experts [T,k] int32 and
 * routing_weights [T,k] fp32.
 */
int tris_router_topk(const float* router_logits, int32_t num_tokens, int32_t num_experts,
                     int32_t top_k, int32_t norm_topk_prob, int32_t* selected_experts,
                     float* routing_weights, void* stream);

/*
 * Expert-parallel dispatch packing (no reference counterpart: the reference is single-GPU).
 * Rows of the grouped order are sorted by expert, hence by owner rank (rank g of `world` owns
 * a contiguous range of experts, sizes differing by at most one).  For every grouped row the
 * kernel copies its two backbone outputs (hidden_gate[tok], hidden_up[tok], each `rank_gu`
 * halves) side by side into slot (owner, position among the rows for that owner) of
 * send_rows [world * capacity, send_row_stride] (send_row_stride halves per slot, a multiple of
 * 8, >= 2*rank_gu).  The row's expert id (unused slots: -1) is written as an int32 right behind
 * the two activation rows when send_row_stride >= 2*rank_gu + 8 (so that one exchange moves
 * rows and ids together), and into send_ids [world * capacity] when that is not NULL.
 * combine_index[flat] = the slot of the flat (token, slot) entry the row came from.
 * capacity >= rows sent to any one rank (tokens * top_k always suffices); a row beyond it is
 * dropped and *overflow_dev set to 1.
 */
int tris_ep_pack_rows(const void* hidden_gate_f16, const void* hidden_up_f16, int32_t rank_gu,
                      const int32_t* selected_experts, const int32_t* perm, const int32_t* grouped_token_indices,
                      int32_t num_rows, int32_t top_k, int32_t num_experts, int32_t world, int32_t capacity,
                      void* send_rows_f16, int32_t send_row_stride, int32_t* send_ids, int32_t* combine_index,
                      int32_t* overflow_dev, void* stream);

/*
 * Expert-parallel exchange over peer memory (no reference counterpart; no collective library
 * call).  Every rank owns a receive buffer [world * capacity, row_stride] fp16 for routed rows,
 * a result buffer [world * capacity, hidden] fp16 and two int32[world] counter arrays (zeroed
 * once), all mapped into every peer (CUDA IPC or the like; the caller sets that up and passes
 * device arrays of the world's pointers, its own included).
 *
 * tris_ep_dispatch_peer  = tris_ep_pack_rows writing slot (owner d, off) straight into rank d's
 *                          receive buffer at slot (my_rank, off), expert id behind the two
 *                          activation rows, then adding 1 per CTA to counter my_rank of every
 *                          peer's dispatch counters.
 * tris_ep_return_peer    sends block s of `results` (received-slot order; rows whose received id
 *                          is negative are skipped) to block my_rank of rank s's result buffer and
 *                          bumps every peer's return counters the same way.
 * tris_ep_wait           one CTA: waits until all `world` counters have reached
 *                          (*step_dev + 1) * tris_ep_signal_increment(), then increments
 *                          *step_dev (a device int32, zeroed once).  Gives up after ~2 s and
 *                          writes TRIS_ERR_TIMEOUT to *status_dev.  Counters only grow, so the
 *                          sequence can be replayed from a CUDA graph; every rank must run the
 *                          same number of steps.
 */
int tris_ep_signal_increment(void);
/* Lets kernels on the current device use memory of `peer_device` (cudaDeviceEnablePeerAccess;
   "already enabled" is success).  TRIS_ERR_UNSUPPORTED when the devices have no P2P path. */
int tris_ep_enable_peer_access(int32_t peer_device);
/* Maps an allocation another process exported (the 64 bytes of its cudaIpcMemHandle_t) into the
   current device's context; *base_out = the allocation's base address in this process.  One open
   per allocation and process; tris_ep_close_peer_memory unmaps it. */
int tris_ep_open_peer_memory(const void* ipc_handle_64, void** base_out);
int tris_ep_close_peer_memory(void* base);
int tris_ep_dispatch_peer(const void* hidden_gate_f16, const void* hidden_up_f16, int32_t rank_gu,
                          const int32_t* selected_experts, const int32_t* perm, const int32_t* grouped_token_indices,
                          int32_t num_rows, int32_t num_experts, int32_t world, int32_t my_rank, int32_t capacity,
                          void* const* peer_recv_rows_dev, int32_t row_stride, int32_t* combine_index,
                          int32_t* overflow_dev, int32_t* const* peer_flags_dev, void* stream);
int tris_ep_return_peer(const void* results_f16, const void* recv_rows_f16, int32_t row_stride, int32_t rank_gu,
                        int32_t hidden_size, int32_t world, int32_t my_rank, int32_t capacity,
                        void* const* peer_back_dev, int32_t* const* peer_flags_dev, void* stream);
int tris_ep_wait(const int32_t* flags_dev, int32_t* step_dev, int32_t world, int32_t* status_dev, void* stream);

/* ---- backbone ---------------------------------------------------------------------- */

/*
 * PackedQuantMatrix4bit.dequantize (QL:2756-2784): the shared backbone of real checkpoints is a
 * GPTQ-style 4-bit matrix - qweight [ceil(cols/8), rows] int32 (nibble j of word [i, r] = input
 * column 8i+j of output row r), qzeros [num_groups, ceil(rows/8)] int32 (zero points minus one,
 * packed along rows), scales [num_groups, rows] fp16, g_idx [cols] int32.  Writes
 * weight[r, c] = fp16((q - zero) * scale) as fp16 [rows, cols], bit for bit what the reference
 * hands to F.linear; run it once at load time and use the result as shared_sv.
 */
int tris_packed4_dequantize(const int32_t* qweight, const int32_t* qzeros, const void* scales_f16,
                            const int32_t* g_idx, int32_t rows, int32_t cols, int32_t num_groups,
                            void* weight_f16, void* stream);

/*
 * One or several GPTQ-style 4-bit matrices inside shared tensors, as the reference concatenates the
 * null-space matrices of a layer's experts (build_grouped_ns_compensation_payload, QL:1734-1882):
 * expert e's matrix has n outputs and k inputs and is found at
 *   qweight[(kw_off[e] + k/8) * q_ld + n_off[e] + n]           (nibble k%8 of the word)
 *   qzeros [(g_off[e] + group) * z_ld + z_off[e] + n/8]        (nibble n%8; zero point minus one)
 *   scales [(g_off[e] + group) * s_ld + n_off[e] + n]          fp16
 * with group = min(k / group_size, groups - 1) (group_size <= 0: one group).  Any of the offset /
 * count arrays may be NULL (offset 0, the common n / k / num_groups).  C2 of the reference payload:
 * n_off = ns_c2_rank_offsets, z_off = ns_c2_rank_word_offsets, n_count = ns_rank_per_expert,
 * k = infeatures.  C1: kw_off = ns_c1_rank_word_offsets, g_off = ns_c1_group_offsets, k_count =
 * ns_rank_per_expert, n = outfeatures.  A single PackedQuantMatrix4bit (QL:2637-2784) with uniform
 * groups is the case num_experts = 1 with every array NULL.
 */
typedef struct TrisPacked4View {
  const int32_t* qweight;
  const int32_t* qzeros;
  const void* scales;        /* fp16 */
  const int32_t* n_off;      /* [num_experts] or NULL */
  const int32_t* z_off;      /* [num_experts] or NULL */
  const int32_t* kw_off;     /* [num_experts] or NULL */
  const int32_t* g_off;      /* [num_experts] or NULL */
  const int32_t* n_count;    /* [num_experts] or NULL: outputs of each expert (<= n)  */
  const int32_t* k_count;    /* [num_experts] or NULL: inputs of each expert (<= k)   */
  const int32_t* g_count;    /* [num_experts] or NULL: groups of each expert          */
  int32_t q_ld, z_ld, s_ld;  /* elements per row of qweight / qzeros / scales         */
  int32_t n, k, num_groups, group_size, num_experts;
} TrisPacked4View;

/*
 * out[row, :] (+)= x[row, :] . dequant(W_e)^T for every routed segment (rows of segment s use the
 * matrix of expert_ids[s]); route == NULL: one problem, expert 0, all num_rows rows.  Replaces
 * grouped_ns_compensation_forward / run_grouped_ns_c1_forward (QL:2024-2128, 1963-2021;
 * GroupedPacked4LinearOffset{Segment,Decode}{C2,C1}, CU:1208-2144) - call it once with the C2 view
 * (out = hidden [R, max_ns_rank]) and once with the C1 view - and, with route == NULL, the packed
 * backbone product of _run_packed_4bit_linear_cuda (QL:1148-1168; Packed4LinearKernelTiledLop3,
 * CU:914-1104).  Weights are fp16((q - zero) * scale) bit for bit as PackedQuantMatrix4bit.dequantize
 * builds them, sums are fp32, results rounded to fp16 once.  accumulate != 0: out = fp16(out + result)
 * (what out.add_(compensation) does, QL:2620-2633).  route->row_gather, when set, names the source
 * row of x for every grouped row.  out_mode: TRIS_OUT_F16, _PAIR_INTERLEAVED or _LANE_ORDER.  Group
 * sizes must be multiples of 32 (or the matrix has one group).  Columns >= k_count[e] of x are never
 * read, outputs >= n_count[e] never written.
 */
int tris_packed4_grouped_forward(const TrisPacked4View* w, const TrisRouteView* route, const void* x_f16,
                                 int32_t x_ld, int32_t num_rows, void* out_f16, int32_t out_ld,
                                 int32_t out_mode, int32_t accumulate, void* stream);


/*
 * hidden = x . shared_sv^T (QuantLinear.compute_shared_hidden fp16 branch, QL:4454-4502):
 * x [N, in] fp16 (rows optionally gathered through row_gather), shared_sv [r, in] fp16,
 * out [N, r] in the layout named by out_mode (TRIS_OUT_*).  num_rows_dev (optional device
 * scalar, final before the launch is enqueued) limits the work to the first *num_rows_dev rows.
 */
int tris_shared_hidden_forward(const void* x_f16, const int32_t* row_gather, int32_t num_rows,
                               const int32_t* num_rows_dev, int32_t in_features,
                               const void* shared_sv_f16, int32_t rank, void* out, int32_t out_mode,
                               void* stream);

/*
 * The three products that share the block's input rows, in one launch: hidden_gate =
 * x * shared_gate^T, hidden_up = x * shared_up^T (each [num_rows, rank] fp16, TRIS_OUT_F16 or
 * TRIS_OUT_F16_PAIR_INTERLEAVED) and, when router_weight_f16 is given, router_logits =
 * x * router_weight^T as fp32 [num_rows, num_experts] (the router nn.Linear of MO:1052 and the
 * two compute_shared_hidden calls of MO:944-953, which the reference runs as three GEMMs).
 */
int tris_input_projections(const void* x_f16, int32_t num_rows, int32_t in_features, const void* shared_gate_f16,
                           const void* shared_up_f16, int32_t rank, const void* router_weight_f16,
                           int32_t num_experts, void* hidden_gate, void* hidden_up, int32_t hidden_out_mode,
                           float* router_logits_f32, void* stream);

/* ---- grouped expert kernels -------------------------------------------------------- */

/*
 * compact3_tris_precomputed_grouped_forward[_block_gr] (CPP:795-834, CPP:1018-1063; Python
 * run_grouped_structured_expert_forward, QL:2131-2335): out[R, O] fp16 = per-segment
 * dequant(U_e) . hidden rows.  hidden is [*, r] fp16; row i of the grouped order reads
 * hidden row route->row_gather[i] when row_gather is set, else row i.
 */
int tris_grouped_forward(const TrisProjView* proj, const TrisRouteView* route, const void* hidden_f16,
                         void* out_f16, void* stream);

/*
 * compact3_tris_precomputed_grouped_dual_forward[_block_gr] (CPP:1065-1136; Python
 * run_grouped_structured_expert_pair_forward, QL:2338-2634).  With fuse_silu_mul = 0 writes
 * out_a and out_b [R, O]; with fuse_silu_mul = 1 writes silu(a) * b to out_a only
 * (the act_fn(gate) * up of MO:1005) and ignores out_b.
 */
int tris_grouped_pair_forward(const TrisProjView* proj_a, const TrisProjView* proj_b,
                              const TrisRouteView* route, const void* hidden_a_f16,
                              const void* hidden_b_f16, void* out_a_f16, void* out_b_f16,
                              int32_t fuse_silu_mul, void* stream);

/*
 * The activation layout (TRIS_OUT_F16, TRIS_OUT_F16_PAIR_INTERLEAVED or TRIS_OUT_F16_LANE_ORDER) the
 * grouped entry points read fastest for these projections (proj_b may be NULL) and a route of
 * num_rows rows in num_segments segments of at most max_rows_per_segment rows: lane order for
 * projections with tile records in the decode regime, pair-interleaved otherwise, row-major for
 * ranks that are not a multiple of 32.  Ask the backbone GEMM for that out_mode and set the
 * matching TRIS_ROUTE_HIDDEN_* flag.  No reference counterpart (the reference kernels read
 * row-major activations only).
 */
int tris_grouped_hidden_layout(const TrisProjView* proj_a, const TrisProjView* proj_b, int32_t num_rows,
                               int32_t num_segments, int32_t max_rows_per_segment);

/*
 * final[T, H] fp16 = sum over slots of routing_weights[t, s] * down_out[row_of_flat[t*k+s]]
 * (the index_add_ of MO:1038-1043, as a deterministic gather in fp32).  A negative row index
 * contributes nothing.
 */
int tris_combine_routed(const void* down_out_f16, const int32_t* row_of_flat,
                        const float* routing_weights, int32_t num_tokens, int32_t top_k,
                        int32_t hidden_size, void* final_f16, void* stream);

/*
 * Rows per expert segment (the launch's upper estimate) above which the grouped entry points use
 * their tcgen05/TMEM kernel instead of the register kernel; returns the previous value.  The
 * default (2048) lies above the range in which the register kernel measured faster on B200; the
 * tests lower it to exercise the tensor-core kernel.  Process-wide; no reference counterpart
 * (the reference decides per call in run_grouped_structured_expert_forward, QL:2187-2229).
 */
int tris_set_grouped_tc_min_rows(int32_t rows);

/*
 * Upper limit on how many CTAs share the row passes of one (segment, output tile) unit in the
 * register-cached grouped kernel (segments of more than 64 rows); returns the previous value.  The
 * launcher splits only while there are fewer units than two CTAs per SM - few local experts with long
 * segments, as on an expert-parallel rank.  Default 4; 1 switches the split off.  Results do not depend
 * on it.  Process-wide; no reference counterpart.
 */
int tris_set_grouped_row_split_max(int32_t ctas);

/* ---- streaming ----------------------------------------------------------------------- */

/* One tensor to page: expert e's block of `bytes_per_expert` bytes (a multiple of 16) is
   copied from host_src + e * bytes_per_expert to dst + slot * bytes_per_expert. */
typedef struct TrisPageJob {
  const void* host_src;      /* pinned, device-accessible host memory, [E, bytes_per_expert]  */
  void* dst;                 /* device staging buffer, [slots, bytes_per_expert]              */
  int64_t bytes_per_expert;
} TrisPageJob;
#define TRIS_MAX_PAGE_JOBS 16

/*
 * Streaming loader step (GroupedQGmapCPUStagingManager.run_grouped / stage, SC:943-1136):
 * for every live segment s of the route, copies the blocks of expert expert_ids[s] of each
 * job from pinned host memory into slot s of the job's staging buffer and records
 * slot_table[expert] = s.  The copy is a kernel that reads host memory directly, driven by
 * the device-side route, so the host never learns which experts are active and nothing
 * synchronises; run it on a side stream and order it with events.  slot_table is [E] int32; every
 * entry is first reset to -1, so an expert beyond the num_segments slots (a batch that activates
 * more experts than the caller sized its staging buffers for) is left "not paged": the grouped
 * kernels then skip its segment and set the route's status word to TRIS_ERR_WORKSPACE instead of
 * reading another expert's bytes.  (The reference pages such a batch in chunks, SC:1047-1136; here
 * the caller sizes the buffers for the experts a batch can activate, or gets the error.)
 */
int tris_page_experts(const TrisPageJob* jobs, int32_t num_jobs, const int32_t* expert_ids,
                      const int32_t* num_segments_dev, int32_t num_segments, int32_t num_experts,
                      int32_t* slot_table, void* stream);

/* ---- whole MoE block --------------------------------------------------------------- */

typedef struct TrisMoeLayerView {
  int32_t hidden_size;        /* H                                                        */
  int32_t intermediate_size;  /* I                                                        */
  int32_t num_experts;        /* E                                                        */
  int32_t top_k;
  int32_t norm_topk_prob;
  const void* router_weight;  /* [E, H] fp16 or NULL when logits are passed in            */
  const void* shared_gate;    /* [r_gu, H] fp16 backbone of gate_proj                     */
  const void* shared_up;      /* [r_gu, H] fp16                                           */
  const void* shared_down;    /* [r_d, I] fp16                                            */
  TrisProjView gate;          /* O = I, r = r_gu                                          */
  TrisProjView up;
  TrisProjView down;          /* O = H, r = r_d                                           */
  /* Optional: the same backbones as 4-bit packed matrices (num_experts = 1, no offset arrays),
     read in place by tris_packed4_grouped_forward instead of the fp16 copies above, which may
     then be NULL (shared_sv_quant, QL:4703-4706).  gate and up switch together. */
  const TrisPacked4View* packed_gate;
  const TrisPacked4View* packed_up;
  const TrisPacked4View* packed_down;
} TrisMoeLayerView;

size_t tris_moe_layer_workspace_bytes(const TrisMoeLayerView* layer, int32_t num_tokens);

/*
 * Status word of the kernels a layer entry point launched: 0, or TRIS_ERR_TIMEOUT when a bounded
 * wait inside one of them ran out (that CTA skipped its stores, so the output rows it owned are
 * stale).  The word lives at byte 8 of the caller's workspace - zero the first 16 bytes of a
 * workspace once, when it is allocated - and is sticky: the kernels only ever set it, so one read
 * covers every call since the last clear.  Pass the workspace given to tris_moe_layer_forward, or
 * NULL for the built-in scratch of tris_moe_layer_forward_static on the current device.  Reads the
 * word back on `stream` and synchronises that stream; clear != 0 resets a non-zero word.  Stands in
 * for the C++ exception a failed TORCH_CHECK raises in the reference extension (CU:49-54).
 */
int tris_moe_layer_last_status(void* workspace, int32_t clear, void* stream, int32_t* status_out);

/*
 * OlmoeSparseMoeBlock.forward -> _forward_grouped (MO:1046-1105, MO:916-1044) as one
 * stream-ordered launch sequence with no host synchronisation: router (from router_logits
 * [T, E] fp32 when given, else x . router_weight^T), route, both input-side backbones,
 * grouped gate/up with SiLU*mul, down backbone, grouped down, weighted combine.
 * x, y: [T, H] fp16.  router_logits_out (optional) receives the fp32 logits.
 */
int tris_moe_layer_forward(const TrisMoeLayerView* layer, const void* x_f16,
                           const float* router_logits, int32_t num_tokens, void* y_f16,
                           float* router_logits_out, void* workspace, size_t workspace_bytes,
                           void* stream);

/*
 * Same computation as tris_moe_layer_forward for callers that cannot provide a workspace
 * because they are not allowed to allocate device memory: for example a serving process
 * whose memory pool claimed the whole GPU at start-up (a later cudaMalloc fails or
 * fragments the pool), a plugin running under a host framework that forbids driver
 * allocations on its worker threads, or a latency-critical loop where an allocation's
 * implicit device synchronisation is not acceptable.  This entry point has no counterpart
 * in the reference.
 *
 * The scratch lives in a file-scope device array of TRIS_STATIC_SCRATCH_BYTES inside the
 * library; every GPU that calls this function holds that much memory until the process
 * exits.  Batches whose scratch need (tris_moe_layer_workspace_bytes) exceeds it are rejected
 * with TRIS_ERR_WORKSPACE and a message naming both sizes.  The function calls no cudaMalloc,
 * cudaFree or other allocating routine.  The first call on each device looks up the array's
 * device address (cudaGetSymbolAddress, with that device current); make that first call
 * outside any stream capture.  All calls on a device share the one array, which keeps the
 * previous call's contents (the words that must start at zero are cleared on the stream
 * first): calls that can overlap on the GPU, e.g. on two streams, race and must be ordered by
 * the caller.  x, y, router_logits, router_logits_out as in tris_moe_layer_forward.
 */
#define TRIS_STATIC_SCRATCH_BYTES (8u << 20)
int tris_moe_layer_forward_static(const TrisMoeLayerView* layer, const void* x_f16,
                                  const float* router_logits, int32_t num_tokens, void* y_f16,
                                  float* router_logits_out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TRISMOE_B200_H_ */
