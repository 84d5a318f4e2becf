// Whole MoE block as one stream-ordered launch sequence (no host synchronisation):
//   router logits + both input-side backbones  (one skinny-GEMM launch sharing x)
//   softmax/top-k, grouped route
//   grouped gate/up with SiLU*mul epilogue
//   down backbone on the routed rows
//   grouped down
//   weighted combine back to token order
#include <algorithm>
#include <mutex>

#include "common.cuh"

namespace tris {
struct LayerWorkspace {
  float* logits;
  int32_t* selected;
  float* weights;
  int32_t* perm;
  int32_t* tok;
  int32_t* slot;
  int32_t* row_of_flat;
  int32_t* expert_ids;
  int32_t* segment_offsets;
  int32_t* problem_offsets;
  int32_t* counts;
  __half* hidden_gate;
  __half* hidden_up;
  __half* mlp;
  __half* hidden_down;
  __half* down_out;
  size_t bytes;
};

static LayerWorkspace carve(const TrisMoeLayerView* L, int T, char* base) {
  LayerWorkspace w{};
  size_t off = 0;
  auto take = [&](size_t bytes) {
    char* p = base ? base + off : nullptr;
    off += (bytes + 255) & ~static_cast<size_t>(255);
    return p;
  };
  const size_t R = static_cast<size_t>(T) * L->top_k;
  const size_t E = L->num_experts;
  w.counts = reinterpret_cast<int32_t*>(take(16));  // {segments, problem tiles, status, -}: first, so the status word is at a fixed offset
  w.logits = reinterpret_cast<float*>(take(sizeof(float) * T * E));
  w.selected = reinterpret_cast<int32_t*>(take(4 * R));
  w.weights = reinterpret_cast<float*>(take(4 * R));
  w.perm = reinterpret_cast<int32_t*>(take(4 * R));
  w.tok = reinterpret_cast<int32_t*>(take(4 * R));
  w.slot = reinterpret_cast<int32_t*>(take(4 * R));
  w.row_of_flat = reinterpret_cast<int32_t*>(take(4 * R));
  w.expert_ids = reinterpret_cast<int32_t*>(take(4 * E));
  w.segment_offsets = reinterpret_cast<int32_t*>(take(4 * (E + 1)));
  w.problem_offsets = reinterpret_cast<int32_t*>(take(4 * (E + 1)));
  w.hidden_gate = reinterpret_cast<__half*>(take(2 * static_cast<size_t>(T) * L->gate.rank));
  w.hidden_up = reinterpret_cast<__half*>(take(2 * static_cast<size_t>(T) * L->up.rank));
  w.mlp = reinterpret_cast<__half*>(take(2 * R * L->intermediate_size));
  w.hidden_down = reinterpret_cast<__half*>(take(2 * R * L->down.rank));
  w.down_out = reinterpret_cast<__half*>(take(2 * R * L->hidden_size));
  w.bytes = off;
  return w;
}

static int validate_layer(const TrisMoeLayerView* L) {
  TRIS_REQUIRE(L != nullptr, TRIS_ERR_INVALID_ARG, "moe layer: null view");
  TRIS_REQUIRE(L->hidden_size > 0 && L->intermediate_size > 0 && L->num_experts > 0 && L->top_k > 0 &&
                   L->top_k <= L->num_experts,
               TRIS_ERR_INVALID_ARG, "moe layer: bad dims H=%d I=%d E=%d k=%d", L->hidden_size, L->intermediate_size,
               L->num_experts, L->top_k);
  const bool packed_gu = L->packed_gate && L->packed_up;
  TRIS_REQUIRE((packed_gu || (L->shared_gate && L->shared_up)) && (L->packed_down || L->shared_down), TRIS_ERR_INVALID_ARG,
               "moe layer: backbone matrices missing");
  TRIS_REQUIRE(!packed_gu || (L->packed_gate->n == L->gate.rank && L->packed_up->n == L->up.rank &&
                              L->packed_gate->k == L->hidden_size && L->packed_up->k == L->hidden_size),
               TRIS_ERR_INVALID_ARG, "moe layer: packed gate/up backbones do not match rank / hidden size");
  TRIS_REQUIRE(!L->packed_down || (L->packed_down->n == L->down.rank && L->packed_down->k == L->intermediate_size),
               TRIS_ERR_INVALID_ARG, "moe layer: packed down backbone does not match rank / intermediate size");
  TRIS_REQUIRE(L->gate.out_features == L->intermediate_size && L->up.out_features == L->intermediate_size &&
                   L->down.out_features == L->hidden_size,
               TRIS_ERR_INVALID_ARG, "moe layer: projection out_features do not match H/I");
  TRIS_REQUIRE(L->gate.num_experts == L->num_experts && L->up.num_experts == L->num_experts &&
                   L->down.num_experts == L->num_experts,
               TRIS_ERR_INVALID_ARG, "moe layer: projection expert counts differ");
  return TRIS_OK;
}
}  // namespace tris

using namespace tris;

extern "C" size_t tris_moe_layer_workspace_bytes(const TrisMoeLayerView* layer, int32_t num_tokens) {
  if (layer == nullptr || num_tokens < 0 || validate_layer(layer) != TRIS_OK) return 0;
  return carve(layer, num_tokens, nullptr).bytes;
}

extern "C" int tris_moe_layer_forward(const TrisMoeLayerView* layer, const void* x_f16, const float* router_logits,
                                      int32_t num_tokens, void* y_f16, float* router_logits_out, void* workspace,
                                      size_t workspace_bytes, void* stream) {
  int st = validate_layer(layer);
  if (st != TRIS_OK) return st;
  TRIS_REQUIRE(x_f16 && y_f16, TRIS_ERR_INVALID_ARG, "tris_moe_layer_forward: null x/y");
  TRIS_REQUIRE(num_tokens >= 0, TRIS_ERR_INVALID_ARG, "tris_moe_layer_forward: negative token count");
  TRIS_REQUIRE(router_logits || layer->router_weight, TRIS_ERR_INVALID_ARG,
               "tris_moe_layer_forward: need router_logits or a router weight");
  if (num_tokens == 0) return TRIS_OK;
  const int T = num_tokens;
  TRIS_REQUIRE(workspace != nullptr, TRIS_ERR_WORKSPACE, "tris_moe_layer_forward: null workspace");
  LayerWorkspace w = carve(layer, T, static_cast<char*>(workspace));
  TRIS_REQUIRE(workspace_bytes >= w.bytes, TRIS_ERR_WORKSPACE, "tris_moe_layer_forward: workspace %zu < %zu bytes",
               workspace_bytes, w.bytes);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int R = T * layer->top_k;
  const __half* x = static_cast<const __half*>(x_f16);

  // Launch order.  With logits given, router + route run first, so that the grouped
  // gate/up kernel can stage its weights while the backbone GEMM is still running
  // (programmatic dependent launch); otherwise the logits come out of the backbone GEMM.
  // Activation layout between the backbone GEMMs and the grouped kernels: lane order for the
  // tile-record kernels, pair-interleaved for the plane-staging kernels, row-major for odd ranks.
  TrisRouteView route{};
  route.num_segments = std::min(layer->num_experts, R);
  route.num_rows = R;
  route.max_rows_per_segment = T;  // top-k experts of a token are distinct
  auto hidden_mode = [&](const TrisProjView& a, const TrisProjView& b) {
    return tris_grouped_hidden_layout(&a, &b, route.num_rows, route.num_segments, route.max_rows_per_segment);
  };
  auto route_flags = [](int mode) {
    return mode == TRIS_OUT_F16_LANE_ORDER ? TRIS_ROUTE_HIDDEN_LANE_ORDER
                                           : (mode == TRIS_OUT_F16_PAIR_INTERLEAVED ? TRIS_ROUTE_HIDDEN_PAIR_INTERLEAVED : 0);
  };
  const int gu_mode = hidden_mode(layer->gate, layer->up);
  const int down_mode = hidden_mode(layer->down, layer->down);
  SkinnyProblem probs[3];
  int np = 0;
  const bool packed_gu = layer->packed_gate && layer->packed_up;  // 4-bit backbones are read in place
  if (!packed_gu) {
    probs[np++] = {static_cast<const __half*>(layer->shared_gate), w.hidden_gate, layer->gate.rank, gu_mode};
    probs[np++] = {static_cast<const __half*>(layer->shared_up), w.hidden_up, layer->up.rank, gu_mode};
  }
  const bool logits_given = router_logits != nullptr;
  const float* logits = router_logits;
  if (logits_given) {
    if (router_logits_out && router_logits_out != router_logits)
      TRIS_CUDA(cudaMemcpyAsync(router_logits_out, router_logits, sizeof(float) * T * layer->num_experts,
                                cudaMemcpyDeviceToDevice, s));
  } else {
    float* dst = router_logits_out ? router_logits_out : w.logits;
    probs[np++] = {static_cast<const __half*>(layer->router_weight), dst, layer->num_experts, TRIS_OUT_F32};
    logits = dst;
  }
  auto route_launch = [&]() {
    return launch_router_route(logits, T, layer->num_experts, layer->top_k, layer->norm_topk_prob, 4, w.selected,
                               w.weights, w.perm, w.tok, w.slot, w.row_of_flat, w.expert_ids, w.segment_offsets,
                               w.problem_offsets, w.counts, s,
                               // nothing uses the grouped-down output buffer before the route exists: scratch of the
                               // multi-CTA route
                               reinterpret_cast<int32_t*>(w.down_out), 2 * static_cast<size_t>(R) * layer->hidden_size);
  };
  if (logits_given) {
    st = route_launch();
    if (st != TRIS_OK) return st;
  }
  if (np > 0) {
    st = launch_shared_hidden(probs, np, x, nullptr, T, layer->hidden_size, s, /*pdl=*/logits_given);
    if (st != TRIS_OK) return st;
  }
  if (packed_gu) {
    st = tris_packed4_grouped_forward(layer->packed_gate, nullptr, x, layer->hidden_size, T, w.hidden_gate, layer->gate.rank,
                                      gu_mode, 0, s);
    if (st != TRIS_OK) return st;
    st = tris_packed4_grouped_forward(layer->packed_up, nullptr, x, layer->hidden_size, T, w.hidden_up, layer->up.rank, gu_mode,
                                      0, s);
    if (st != TRIS_OK) return st;
  }
  if (!logits_given) {
    st = route_launch();
    if (st != TRIS_OK) return st;
  }

  route.expert_ids = w.expert_ids;
  route.segment_offsets = w.segment_offsets;
  route.num_segments_dev = w.counts;
  route.status_dev = w.counts + 2;

  // gate/up + SiLU*mul; rows read the per-token backbone outputs through tok[]
  route.row_gather = w.tok;
  route.flags = route_flags(gu_mode);
  LaunchOpts opts;
  opts.pdl = true;
  opts.weights_before_wait = logits_given;
  st = grouped_pair_forward_impl(&layer->gate, &layer->up, &route, w.hidden_gate, w.hidden_up, w.mlp, nullptr, 1, s, opts);
  if (st != TRIS_OK) return st;

  // down backbone on routed rows
  if (layer->packed_down) {
    st = tris_packed4_grouped_forward(layer->packed_down, nullptr, w.mlp, layer->intermediate_size, R, w.hidden_down,
                                      layer->down.rank, down_mode, 0, s);
  } else {
    SkinnyProblem down{static_cast<const __half*>(layer->shared_down), w.hidden_down, layer->down.rank, down_mode};
    st = launch_shared_hidden(&down, 1, w.mlp, nullptr, R, layer->intermediate_size, s, /*pdl=*/true);
  }
  if (st != TRIS_OK) return st;

  // grouped down: the route is older than the GEMM before it, so weights stage early
  route.row_gather = nullptr;
  route.flags = route_flags(down_mode);
  opts.weights_before_wait = true;
  st = grouped_forward_impl(&layer->down, &route, w.hidden_down, w.down_out, s, opts);
  if (st != TRIS_OK) return st;

  // combine
  return combine_routed_impl(w.down_out, w.row_of_flat, w.weights, T, layer->top_k, layer->hidden_size, y_f16, s, true);
}

// ---- variant that allocates nothing ----------------------------------------------------------
// Scratch for tris_moe_layer_forward_static.  Lives in every process image that loads the
// library, once per GPU that touches it, until the process exits.
static __device__ __align__(256) unsigned char g_layer_static_scratch[TRIS_STATIC_SCRATCH_BYTES];

namespace {
std::mutex g_static_scratch_mutex;
void* g_static_scratch_ptr[64] = {};  // device address of the array, per device ordinal
}  // namespace

extern "C" int tris_moe_layer_forward_static(const TrisMoeLayerView* layer, const void* x_f16,
                                             const float* router_logits, int32_t num_tokens, void* y_f16,
                                             float* router_logits_out, void* stream) {
  int st = validate_layer(layer);
  if (st != TRIS_OK) return st;
  TRIS_REQUIRE(num_tokens >= 0, TRIS_ERR_INVALID_ARG, "tris_moe_layer_forward_static: negative token count");
  if (num_tokens == 0) return TRIS_OK;
  LayerWorkspace probe = carve(layer, num_tokens, nullptr);
  TRIS_REQUIRE(probe.bytes <= TRIS_STATIC_SCRATCH_BYTES, TRIS_ERR_WORKSPACE,
               "tris_moe_layer_forward_static: %d tokens need %zu bytes of scratch, the built-in array holds %u; "
               "use tris_moe_layer_forward with a caller workspace",
               num_tokens, probe.bytes, static_cast<unsigned>(TRIS_STATIC_SCRATCH_BYTES));
  int dev = -1;
  TRIS_CUDA(cudaGetDevice(&dev));
  TRIS_REQUIRE(dev >= 0 && dev < 64, TRIS_ERR_UNSUPPORTED, "tris_moe_layer_forward_static: device ordinal %d", dev);
  void* scratch = nullptr;
  {
    // In host code the array's name is only a handle; the kernels need its device address,
    // which is looked up once per device with that device current.
    std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
    if (g_static_scratch_ptr[dev] == nullptr) {
      void* ptr = nullptr;
      TRIS_CUDA(cudaGetSymbolAddress(&ptr, g_layer_static_scratch));
      TRIS_REQUIRE(ptr != nullptr, TRIS_ERR_CUDA, "tris_moe_layer_forward_static: no device address for the scratch array");
      g_static_scratch_ptr[dev] = ptr;
    }
    scratch = g_static_scratch_ptr[dev];
  }
  // The array keeps whatever the previous call left.  Everything the launch sequence reads it
  // writes first, except the two count words, which are cleared here; the status word behind
  // them is sticky (it starts at zero with the array and only tris_moe_layer_last_status clears it).
  LayerWorkspace w = carve(layer, num_tokens, static_cast<char*>(scratch));
  TRIS_CUDA(cudaMemsetAsync(w.counts, 0, 8, static_cast<cudaStream_t>(stream)));
  return tris_moe_layer_forward(layer, x_f16, router_logits, num_tokens, y_f16, router_logits_out, scratch,
                                TRIS_STATIC_SCRATCH_BYTES, stream);
}

// Offset of the sticky status word inside a layer workspace (and inside the built-in scratch array).
static constexpr size_t kStatusWordOffset = 8;

extern "C" int tris_moe_layer_last_status(void* workspace, int32_t clear, void* stream, int32_t* status_out) {
  TRIS_REQUIRE(status_out != nullptr, TRIS_ERR_INVALID_ARG, "tris_moe_layer_last_status: null output");
  char* base = static_cast<char*>(workspace);
  if (base == nullptr) {  // the built-in scratch of tris_moe_layer_forward_static on the current device
    int dev = -1;
    TRIS_CUDA(cudaGetDevice(&dev));
    TRIS_REQUIRE(dev >= 0 && dev < 64, TRIS_ERR_UNSUPPORTED, "tris_moe_layer_last_status: device ordinal %d", dev);
    std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
    if (g_static_scratch_ptr[dev] == nullptr) {  // never used on this device: nothing can have been reported
      *status_out = TRIS_OK;
      return TRIS_OK;
    }
    base = static_cast<char*>(g_static_scratch_ptr[dev]);
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int32_t word = 0;
  TRIS_CUDA(cudaMemcpyAsync(&word, base + kStatusWordOffset, sizeof(word), cudaMemcpyDeviceToHost, s));
  TRIS_CUDA(cudaStreamSynchronize(s));
  if (clear && word != 0) TRIS_CUDA(cudaMemsetAsync(base + kStatusWordOffset, 0, sizeof(word), s));
  *status_out = word;
  return TRIS_OK;
}
