// Expands a block-level mask classification (what MaskInfo encodes) into the per-CTA work
// lists the 128x128-tile kernels walk.  Host only, no CUDA.
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <new>
#include <numeric>
#include <vector>

#include "../../include/splash_b200.h"

namespace {

constexpr int kTile = 128;

struct Entry {
  int32_t tile, state, pid0, pid1;
};

}  // namespace

extern "C" {

int splash_schedule_build(const int32_t* block_state, const int32_t* partial_id, int32_t n_q_blocks,
                          int32_t n_kv_blocks, int32_t block_q, int32_t block_kv, int32_t kind,
                          SplashScheduleOut* out) {
  if (out == nullptr) return SPLASH_ERR_INVALID_ARGUMENT;
  std::memset(out, 0, sizeof(*out));
  if (block_state == nullptr || n_q_blocks <= 0 || n_kv_blocks <= 0) return SPLASH_ERR_INVALID_ARGUMENT;
  if (block_q <= 0 || block_kv <= 0 || block_q % kTile != 0 || block_kv % kTile != 0)
    return SPLASH_ERR_INVALID_ARGUMENT;
  if (kind < 0 || kind > 2) return SPLASH_ERR_INVALID_ARGUMENT;

  const int64_t tq = (int64_t)n_q_blocks * (block_q / kTile);    // q tiles
  const int64_t tkv = (int64_t)n_kv_blocks * (block_kv / kTile); // kv tiles
  const int fq = block_q / kTile, fkv = block_kv / kTile;
  auto state_of = [&](int64_t qt, int64_t kt) -> int32_t {
    return block_state[(qt / fq) * n_kv_blocks + (kt / fkv)];
  };
  auto pid_of = [&](int64_t qt, int64_t kt) -> int32_t {
    if (partial_id == nullptr) return -1;
    return partial_id[(qt / fq) * n_kv_blocks + (kt / fkv)];
  };

  std::vector<int32_t> row_ptr;
  std::vector<Entry> entries;
  try {
    if (kind == 0) {
      const int64_t n_rows = (tq + 1) / 2;
      row_ptr.reserve(n_rows + 1);
      row_ptr.push_back(0);
      for (int64_t r = 0; r < n_rows; ++r) {
        const int64_t q0 = 2 * r, q1 = 2 * r + 1;
        for (int64_t kt = 0; kt < tkv; ++kt) {
          const int32_t s0 = state_of(q0, kt);
          const int32_t s1 = q1 < tq ? state_of(q1, kt) : 0;
          if (s0 == 0 && s1 == 0) continue;
          Entry e;
          e.tile = (int32_t)kt;
          e.state = (s0 & 3) | ((s1 & 3) << 2);
          e.pid0 = s0 == 1 ? pid_of(q0, kt) : -1;
          e.pid1 = s1 == 1 ? pid_of(q1, kt) : -1;
          entries.push_back(e);
        }
        row_ptr.push_back((int32_t)entries.size());
      }
    } else if (kind == 1) {
      row_ptr.reserve(tq + 1);
      row_ptr.push_back(0);
      for (int64_t qt = 0; qt < tq; ++qt) {
        for (int64_t kt = 0; kt < tkv; ++kt) {
          const int32_t s0 = state_of(qt, kt);
          if (s0 == 0) continue;
          entries.push_back(Entry{(int32_t)kt, s0 & 3, s0 == 1 ? pid_of(qt, kt) : -1, -1});
        }
        row_ptr.push_back((int32_t)entries.size());
      }
    } else {
      row_ptr.reserve(tkv + 1);
      row_ptr.push_back(0);
      for (int64_t kt = 0; kt < tkv; ++kt) {
        for (int64_t qt = 0; qt < tq; ++qt) {
          const int32_t s0 = state_of(qt, kt);
          if (s0 == 0) continue;
          entries.push_back(Entry{(int32_t)qt, s0 & 3, s0 == 1 ? pid_of(qt, kt) : -1, -1});
        }
        row_ptr.push_back((int32_t)entries.size());
      }
    }
  } catch (const std::bad_alloc&) {
    return SPLASH_ERR_OUT_OF_MEMORY;
  }
  if (entries.size() > (size_t)0x7fffffff) return SPLASH_ERR_TOO_LARGE;

  out->n_rows = (int32_t)(row_ptr.size() - 1);
  out->n_entries = (int64_t)entries.size();
  out->row_ptr = static_cast<int32_t*>(std::malloc(row_ptr.size() * sizeof(int32_t)));
  out->entries = static_cast<int32_t*>(std::malloc((entries.size() + 1) * sizeof(Entry)));
  out->row_order = static_cast<int32_t*>(std::malloc((size_t)out->n_rows * sizeof(int32_t)));
  if (out->row_ptr == nullptr || out->entries == nullptr || out->row_order == nullptr) {
    splash_schedule_free(out);
    return SPLASH_ERR_OUT_OF_MEMORY;
  }
  std::memcpy(out->row_ptr, row_ptr.data(), row_ptr.size() * sizeof(int32_t));
  // Longest rows first: a grid launched in this order ends on its shortest CTAs.
  std::iota(out->row_order, out->row_order + out->n_rows, 0);
  std::stable_sort(out->row_order, out->row_order + out->n_rows, [&](int32_t a, int32_t b) {
    return row_ptr[a + 1] - row_ptr[a] > row_ptr[b + 1] - row_ptr[b];
  });
  if (!entries.empty()) std::memcpy(out->entries, entries.data(), entries.size() * sizeof(Entry));
  return SPLASH_OK;
}

void splash_schedule_free(SplashScheduleOut* out) {
  if (out == nullptr) return;
  std::free(out->row_ptr);
  std::free(out->entries);
  std::free(out->row_order);
  std::memset(out, 0, sizeof(*out));
}

}  // extern "C"
