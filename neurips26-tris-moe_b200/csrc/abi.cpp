// Host-only part of the C ABI: version, status strings, thread-local error text and the
// block Golomb-Rice encoder.
#include <atomic>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <vector>

#include "../../include/trismoe_b200.h"

namespace tris {

static thread_local char g_last_error[512] = "";

void set_last_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
}

int fail(int status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  return status;
}

int check_cuda(cudaError_t err, const char* what) {
  if (err == cudaSuccess) return TRIS_OK;
  snprintf(g_last_error, sizeof(g_last_error), "%s: %s (%s)", what, cudaGetErrorName(err), cudaGetErrorString(err));
  return TRIS_ERR_CUDA;
}

}  // namespace tris

namespace {
std::atomic<int> g_programmatic_launch{0};
}
namespace tris {
bool programmatic_launch_default() { return g_programmatic_launch.load(std::memory_order_relaxed) != 0; }
}  // namespace tris

extern "C" int tris_set_programmatic_launch(int32_t enable) {
  return g_programmatic_launch.exchange(enable ? 1 : 0, std::memory_order_relaxed);
}

extern "C" int tris_abi_version(void) { return TRIS_B200_ABI_VERSION; }
extern "C" int tris_compact3_kernel_abi_version(void) { return TRIS_COMPACT3_KERNEL_ABI_VERSION; }

extern "C" const char* tris_status_string(int status) {
  switch (status) {
    case TRIS_OK: return "ok";
    case TRIS_ERR_INVALID_ARG: return "invalid argument";
    case TRIS_ERR_UNSUPPORTED: return "unsupported shape or layout";
    case TRIS_ERR_CUDA: return "CUDA error";
    case TRIS_ERR_CORRUPT: return "corrupt payload";
    case TRIS_ERR_WORKSPACE: return "workspace too small";
    case TRIS_ERR_TIMEOUT: return "device-side wait timed out";
    default: return "unknown status";
  }
}

extern "C" const char* tris_last_error(void) { return tris::g_last_error; }

// ---- block Golomb-Rice encoder -------------------------------------------------------------
// Format (QL:3763-3859 of the TriS-MoE tree): blocks iterate k_block outer, out_block
// inner; a block is the 128 words [2 packed rows][64 outputs] (zeros outside the matrix);
// positions of ones in flat order -> zero-run lengths -> for the k in 0..7 with the fewest
// bits (lowest k on ties): run>>k zeros, a one, the low k bits LSB first, packed LSB first
// into 32-bit words.  A block whose code needs >= 128 words is stored verbatim with
// meta = 16; otherwise meta = k | one_count << 8.
namespace {
struct BitWriter {
  std::vector<uint32_t>& words;
  uint32_t cur = 0;
  int fill = 0;
  explicit BitWriter(std::vector<uint32_t>& w) : words(w) {}
  void zeros(int n) {
    while (n > 0) {
      const int take = (32 - fill < n) ? 32 - fill : n;
      fill += take;
      n -= take;
      if (fill == 32) flush();
    }
  }
  void bits(uint32_t value, int n) {  // n <= 8, LSB first
    for (int i = 0; i < n; ++i) {
      if ((value >> i) & 1u) cur |= 1u << fill;
      if (++fill == 32) flush();
    }
  }
  void flush() {
    words.push_back(cur);
    cur = 0;
    fill = 0;
  }
  void finish() {
    if (fill != 0) flush();
  }
};
}  // namespace

extern "C" int tris_block_gr_encode_host(const int32_t* dense_words, int32_t packed_rows, int32_t out_features,
                                         int32_t force_raw, int32_t* words_out, int64_t words_capacity,
                                         int32_t* offsets_out, int32_t* meta_out, int64_t* num_words) {
  return tris_block_gr_encode_host_k(dense_words, packed_rows, out_features, force_raw, 0, TRIS_GR_MAX_K, words_out,
                                     words_capacity, offsets_out, meta_out, num_words);
}

extern "C" int tris_block_gr_encode_host_k(const int32_t* dense_words, int32_t packed_rows, int32_t out_features,
                                           int32_t force_raw, int32_t k_min, int32_t k_max, int32_t* words_out,
                                           int64_t words_capacity, int32_t* offsets_out, int32_t* meta_out,
                                           int64_t* num_words) {
  if (!dense_words || !words_out || !offsets_out || !meta_out || !num_words)
    return tris::fail(TRIS_ERR_INVALID_ARG, "tris_block_gr_encode_host: null pointer");
  if (k_min < 0 || k_max > TRIS_GR_MAX_K || k_min > k_max)
    return tris::fail(TRIS_ERR_INVALID_ARG, "tris_block_gr_encode_host: k range [%d, %d] outside [0, %d]", k_min, k_max,
                      TRIS_GR_MAX_K);
  if (packed_rows < 0 || out_features < 0)
    return tris::fail(TRIS_ERR_INVALID_ARG, "tris_block_gr_encode_host: negative dims");
  const int nkb = (packed_rows + TRIS_GR_BLOCK_PACKED_ROWS - 1) / TRIS_GR_BLOCK_PACKED_ROWS;
  const int nob = (out_features + TRIS_GR_BLOCK_OUT - 1) / TRIS_GR_BLOCK_OUT;
  int64_t total = 0;
  int blk = 0;
  offsets_out[0] = 0;
  std::vector<int> runs;
  std::vector<uint32_t> coded;
  uint32_t block[TRIS_GR_BLOCK_WORDS];
  for (int kb = 0; kb < nkb; ++kb) {
    for (int ob = 0; ob < nob; ++ob, ++blk) {
      runs.clear();
      int prev = -1;
      for (int lr = 0; lr < TRIS_GR_BLOCK_PACKED_ROWS; ++lr) {
        const int p = kb * TRIS_GR_BLOCK_PACKED_ROWS + lr;
        for (int lo = 0; lo < TRIS_GR_BLOCK_OUT; ++lo) {
          const int o = ob * TRIS_GR_BLOCK_OUT + lo;
          uint32_t w = 0;
          if (p < packed_rows && o < out_features)
            w = static_cast<uint32_t>(dense_words[static_cast<int64_t>(p) * out_features + o]);
          const int wi = lr * TRIS_GR_BLOCK_OUT + lo;
          block[wi] = w;
          while (w) {
            const int bit = __builtin_ctz(w);
            const int pos = wi * 32 + bit;
            runs.push_back(pos - prev - 1);
            prev = pos;
            w &= w - 1;
          }
        }
      }
      int best_k = 0;
      int64_t best_bits = static_cast<int64_t>(TRIS_GR_BLOCK_WORDS) * 32 + 1;
      bool have = false;
      for (int k = k_min; k <= k_max; ++k) {
        int64_t bits = 0;
        for (int r : runs) bits += (r >> k) + 1 + k;
        if (bits < best_bits) {
          best_bits = bits;
          best_k = k;
          have = true;
        }
      }
      const int64_t coded_words = have ? (best_bits + 31) / 32 : TRIS_GR_BLOCK_WORDS;
      const bool raw = force_raw || !have || coded_words >= TRIS_GR_BLOCK_WORDS;
      const int64_t need = raw ? TRIS_GR_BLOCK_WORDS : coded_words;
      if (total + need > words_capacity)
        return tris::fail(TRIS_ERR_WORKSPACE, "tris_block_gr_encode_host: words_out too small (%lld needed so far)",
                          static_cast<long long>(total + need));
      if (raw) {
        memcpy(words_out + total, block, sizeof(block));
        meta_out[blk] = TRIS_GR_META_RAW_FLAG;
      } else {
        coded.clear();
        BitWriter bw(coded);
        for (int r : runs) {
          bw.zeros(r >> best_k);
          bw.bits(1u, 1);
          bw.bits(static_cast<uint32_t>(r) & ((1u << best_k) - 1u), best_k);
        }
        bw.finish();
        if (!coded.empty()) memcpy(words_out + total, coded.data(), coded.size() * sizeof(uint32_t));
        meta_out[blk] = best_k | (static_cast<int32_t>(runs.size()) << TRIS_GR_META_ONE_COUNT_SHIFT);
      }
      total += need;
      offsets_out[blk + 1] = static_cast<int32_t>(total);
    }
  }
  *num_words = total;
  return TRIS_OK;
}
