// Native MaskInfo builder (host only).
//
// Produces the block-sparse tables of the reference's `_process_mask`
// (tokamax/_src/ops/experimental/tpu/splash_attention/splash_attention_mask_info.py:357-570)
// bit for bit, but classifies blocks analytically instead of materialising every
// (block_q x block_kv) chunk: the lazy masks (causal, local window, chunked causal) keep, for
// query row i, the key interval [lo(i), hi(i)] with lo and hi non-decreasing in i, so a block is
// classified from the intervals of its first and last row, and only blocks the boundary crosses
// are looked at row by row.  Composite masks (AND / OR trees) combine child classifications and
// materialise a block only when that is unavoidable, i.e. when it is partially masked.
//
// Table semantics reproduced here (file:line in the reference module above):
//   block states 0 empty / 1 partial / 2 full in a global q-major scan        :453-468
//   partial blocks deduplicated by content, ids in first-seen order            :447-468
//   all-full shortcut                                                          :470-480
//   per (q shard, kv shard) metadata, dkv transposition, empty-row extension   :183-228, :494-511
//   mask_next "partial block at or after this step", one advance per step      :208-225
//   -1 padding of dynamic-grid shards to the longest shard                     :521-535
#include <algorithm>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <new>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/splash_b200.h"

namespace {

struct Interval {
  int64_t lo, hi;  // inclusive; lo > hi means empty
};

constexpr int64_t kNegInf = INT64_MIN / 4;
constexpr int64_t kPosInf = INT64_MAX / 4;

inline int64_t floordiv(int64_t a, int64_t b) {
  int64_t q = a / b;
  if ((a % b != 0) && ((a < 0) != (b < 0))) --q;
  return q;
}

inline Interval row_interval(const SplashMaskFn& fn, int64_t i) {
  Interval iv{kNegInf, kPosInf};
  switch (fn.kind) {
    case SPLASH_MASK_CAUSAL:
      iv.hi = i + fn.offset;
      break;
    case SPLASH_MASK_LOCAL:
      if (fn.has_left) iv.lo = i + fn.offset - fn.left;
      if (fn.has_right) iv.hi = i + fn.offset + fn.right;
      break;
    case SPLASH_MASK_CHUNKED:
      iv.lo = floordiv(i, fn.chunk) * fn.chunk;
      iv.hi = i;
      break;
    default:
      break;
  }
  return iv;
}

struct Builder {
  const SplashMaskNode* nodes;
  int32_t n_nodes;
  int64_t q_len, kv_len;
  int32_t bq, bkv;

  // 0 empty / 1 partial / 2 full for block (qb, kb) of node n.
  int state(int32_t n, int64_t qb, int64_t kb, std::vector<uint8_t>* scratch) const {
    const SplashMaskNode& nd = nodes[n];
    const int64_t r0 = qb * bq, r1 = r0 + bq, c0 = kb * bkv, c1 = c0 + bkv;
    switch (nd.kind) {
      case SPLASH_NODE_FULL:
        return 2;
      case SPLASH_NODE_CAUSAL:
      case SPLASH_NODE_LOCAL:
      case SPLASH_NODE_CHUNKED: {
        const Interval first = row_interval(nd.fn, r0), last = row_interval(nd.fn, r1 - 1);
        if (last.lo <= c0 && first.hi >= c1 - 1) return 2;   // every row covers the block
        if (last.hi < c0 || first.lo > c1 - 1) return 0;     // no row reaches the block
        bool any = false, all = true;
        for (int64_t i = r0; i < r1; ++i) {
          const Interval iv = row_interval(nd.fn, i);
          const int64_t lo = std::max(iv.lo, c0), hi = std::min(iv.hi, c1 - 1);
          if (lo <= hi) any = true;
          if (!(iv.lo <= c0 && iv.hi >= c1 - 1)) all = false;
          if (any && !all) return 1;
        }
        return any ? (all ? 2 : 1) : 0;
      }
      case SPLASH_NODE_DENSE: {
        bool any = false, all = true;
        for (int64_t i = r0; i < r1; ++i) {
          const uint8_t* row = nd.dense + i * kv_len + c0;
          for (int64_t j = 0; j < bkv; ++j) {
            if (row[j]) any = true; else all = false;
          }
          if (any && !all) return 1;
        }
        return any ? (all ? 2 : 1) : 0;
      }
      case SPLASH_NODE_AND:
      case SPLASH_NODE_OR: {
        const int a = state(nd.left_child, qb, kb, scratch);
        const int b = state(nd.right_child, qb, kb, scratch);
        if (nd.kind == SPLASH_NODE_AND) {
          if (a == 0 || b == 0) return 0;
          if (a == 2) return b;
          if (b == 2) return a;
        } else {
          if (a == 2 || b == 2) return 2;
          if (a == 0) return b;
          if (b == 0) return a;
        }
        // both partial: only the contents decide
        std::vector<uint8_t> buf((size_t)bq * bkv);
        materialize(n, qb, kb, buf.data());
        bool any = false, all = true;
        for (uint8_t x : buf) {
          if (x) any = true; else all = false;
        }
        return any ? (all ? 2 : 1) : 0;
      }
      default:
        return 0;
    }
  }

  // Fills out[bq * bkv] (row-major, 0/1) with block (qb, kb) of node n.
  void materialize(int32_t n, int64_t qb, int64_t kb, uint8_t* out) const {
    const SplashMaskNode& nd = nodes[n];
    const int64_t r0 = qb * bq, c0 = kb * bkv;
    switch (nd.kind) {
      case SPLASH_NODE_FULL:
        std::memset(out, 1, (size_t)bq * bkv);
        break;
      case SPLASH_NODE_CAUSAL:
      case SPLASH_NODE_LOCAL:
      case SPLASH_NODE_CHUNKED:
        for (int64_t i = 0; i < bq; ++i) {
          const Interval iv = row_interval(nd.fn, r0 + i);
          uint8_t* row = out + i * bkv;
          for (int64_t j = 0; j < bkv; ++j) row[j] = (c0 + j >= iv.lo && c0 + j <= iv.hi) ? 1 : 0;
        }
        break;
      case SPLASH_NODE_DENSE:
        for (int64_t i = 0; i < bq; ++i) {
          const uint8_t* src = nd.dense + (r0 + i) * kv_len + c0;
          uint8_t* row = out + i * bkv;
          for (int64_t j = 0; j < bkv; ++j) row[j] = src[j] ? 1 : 0;
        }
        break;
      case SPLASH_NODE_AND:
      case SPLASH_NODE_OR: {
        std::vector<uint8_t> rhs((size_t)bq * bkv);
        materialize(nd.left_child, qb, kb, out);
        materialize(nd.right_child, qb, kb, rhs.data());
        const size_t nel = (size_t)bq * bkv;
        if (nd.kind == SPLASH_NODE_AND) {
          for (size_t t = 0; t < nel; ++t) out[t] &= rhs[t];
        } else {
          for (size_t t = 0; t < nel; ++t) out[t] |= rhs[t];
        }
        break;
      }
      default:
        std::memset(out, 0, (size_t)bq * bkv);
    }
  }
};

struct ShardMeta {
  std::vector<int32_t> rows, cols, mask_next, block_mask;
  int32_t grid_size = 0;
};

// state / pid: the shard's slice, already in walking orientation (transposed for dkv),
// R x Cn row-major.
void shard_metadata(const std::vector<int32_t>& state, const std::vector<int32_t>& pid, int64_t R,
                    int64_t Cn, bool is_dkv, bool dynamic_grid, ShardMeta* m) {
  std::vector<int64_t> walk;  // linear indices r * Cn + c in iteration order
  if (dynamic_grid) {
    for (int64_t r = 0; r < R; ++r) {
      bool any = false;
      for (int64_t c = 0; c < Cn; ++c) any = any || state[r * Cn + c] > 0;
      for (int64_t c = 0; c < Cn; ++c) {
        const bool active = state[r * Cn + c] > 0 || (is_dkv && !any && c == 0);
        if (active) {
          walk.push_back(r * Cn + c);
          m->rows.push_back((int32_t)r);
          m->cols.push_back((int32_t)c);
          m->block_mask.push_back(state[r * Cn + c]);
        }
      }
    }
    m->grid_size = (int32_t)walk.size();
  } else {
    walk.resize((size_t)(R * Cn));
    for (int64_t t = 0; t < R * Cn; ++t) walk[(size_t)t] = t;
    m->block_mask = state;
  }
  std::vector<int64_t> partial;  // linear indices with a partial id, row-major
  for (int64_t t = 0; t < R * Cn; ++t)
    if (pid[(size_t)t] != -1) partial.push_back(t);
  if (partial.empty()) {
    // The reference sizes this array by the block_mask it has at that point.
    m->mask_next.assign(m->block_mask.size(), -1);
    return;
  }
  // The reference walks the partial blocks with a Python iterator: one advance per step that lies
  // beyond the current one; once the iterator has run out it stays run out, so every later step
  // falls back to the FIRST partial block (it does not go round again).
  size_t cur = 0;
  bool exhausted = false;
  m->mask_next.reserve(walk.size());
  for (int64_t idx : walk) {
    if (idx > partial[cur]) {  // lexicographic (r, c) order == linear order
      if (!exhausted && cur + 1 < partial.size()) {
        ++cur;
      } else {
        exhausted = true;
        cur = 0;
      }
    }
    m->mask_next.push_back(pid[(size_t)partial[cur]]);
  }
}

template <typename T>
T* dup(const std::vector<T>& v) {
  T* p = static_cast<T*>(std::malloc(std::max<size_t>(v.size(), 1) * sizeof(T)));
  if (p && !v.empty()) std::memcpy(p, v.data(), v.size() * sizeof(T));
  return p;
}

}  // namespace

extern "C" {

void splash_maskinfo_free(SplashMaskInfoOut* out) {
  if (out == nullptr) return;
  std::free(out->mask_next);
  std::free(out->active_rows);
  std::free(out->active_cols);
  std::free(out->block_mask);
  std::free(out->num_active_blocks);
  std::free(out->partial_mask_blocks);
  std::memset(out, 0, sizeof(*out));
}

int splash_maskinfo_build(const SplashMaskNode* nodes, int32_t n_nodes, int64_t q_len,
                          int64_t kv_len, int32_t block_q, int32_t block_kv, int32_t is_dkv,
                          int32_t q_seq_shards, int32_t kv_seq_shards, int32_t return_dynamic_grid,
                          SplashMaskInfoOut* out) {
  if (out == nullptr) return SPLASH_ERR_INVALID_ARGUMENT;
  std::memset(out, 0, sizeof(*out));
  if (nodes == nullptr || n_nodes <= 0 || q_len <= 0 || kv_len <= 0 || block_q <= 0 || block_kv <= 0 ||
      q_seq_shards <= 0 || kv_seq_shards <= 0)
    return SPLASH_ERR_INVALID_ARGUMENT;
  if (q_len % block_q != 0 || kv_len % block_kv != 0) return SPLASH_ERR_INVALID_ARGUMENT;
  if (q_len % q_seq_shards != 0 || kv_len % kv_seq_shards != 0) return SPLASH_ERR_INVALID_ARGUMENT;
  if ((q_len / q_seq_shards) % block_q != 0 || (kv_len / kv_seq_shards) % block_kv != 0)
    return SPLASH_ERR_INVALID_ARGUMENT;
  for (int32_t i = 0; i < n_nodes; ++i) {
    const SplashMaskNode& nd = nodes[i];
    if (nd.kind < SPLASH_NODE_FULL || nd.kind > SPLASH_NODE_OR) return SPLASH_ERR_INVALID_ARGUMENT;
    if (nd.kind == SPLASH_NODE_AND || nd.kind == SPLASH_NODE_OR) {
      if (nd.left_child < 0 || nd.left_child >= i || nd.right_child < 0 || nd.right_child >= i)
        return SPLASH_ERR_INVALID_ARGUMENT;
    }
    if (nd.kind == SPLASH_NODE_DENSE && nd.dense == nullptr) return SPLASH_ERR_INVALID_ARGUMENT;
    if (nd.kind == SPLASH_NODE_CHUNKED && nd.fn.chunk <= 0) return SPLASH_ERR_INVALID_ARGUMENT;
    if (nd.kind == SPLASH_NODE_CAUSAL || nd.kind == SPLASH_NODE_LOCAL || nd.kind == SPLASH_NODE_CHUNKED) {
      if (nd.fn.kind != nd.kind) return SPLASH_ERR_INVALID_ARGUMENT;
    }
  }

  try {
    const int64_t nq = q_len / block_q, nkv = kv_len / block_kv;
    const int32_t root = n_nodes - 1;
    const bool root_is_lazy = nodes[root].kind == SPLASH_NODE_CAUSAL ||
                              nodes[root].kind == SPLASH_NODE_LOCAL ||
                              nodes[root].kind == SPLASH_NODE_CHUNKED;
    Builder b{nodes, n_nodes, q_len, kv_len, block_q, block_kv};

    std::vector<int32_t> state((size_t)(nq * nkv), 0), pid((size_t)(nq * nkv), -1);
    std::unordered_map<std::string, int32_t> seen;
    std::vector<std::string> unique_blocks;
    std::vector<uint8_t> buf((size_t)block_q * block_kv);
    bool all_full = true;
    int32_t lazy_partial_count = 0;
    for (int64_t qb = 0; qb < nq; ++qb) {
      for (int64_t kb = 0; kb < nkv; ++kb) {
        const int s = b.state(root, qb, kb, nullptr);
        state[(size_t)(qb * nkv + kb)] = s;
        if (s != 2) all_full = false;
        if (s == 1) {
          if (root_is_lazy) {
            // Contents are never emitted for a bare lazy mask; only "is partial" matters.
            pid[(size_t)(qb * nkv + kb)] = 0;
            ++lazy_partial_count;
          } else {
            b.materialize(root, qb, kb, buf.data());
            std::string key(reinterpret_cast<const char*>(buf.data()), buf.size());
            auto it = seen.find(key);
            int32_t id;
            if (it == seen.end()) {
              id = (int32_t)unique_blocks.size();
              seen.emplace(key, id);
              unique_blocks.push_back(std::move(key));
            } else {
              id = it->second;
            }
            pid[(size_t)(qb * nkv + kb)] = id;
          }
        }
      }
    }
    if (all_full) {
      out->all_full = 1;
      return SPLASH_OK;
    }
    const bool have_partial = root_is_lazy ? lazy_partial_count > 0 : !unique_blocks.empty();

    // per-shard metadata
    const int64_t qps = nq / q_seq_shards, kps = nkv / kv_seq_shards;
    std::vector<ShardMeta> shards;
    for (int32_t qs = 0; qs < q_seq_shards; ++qs) {
      for (int32_t ks = 0; ks < kv_seq_shards; ++ks) {
        const int64_t R = is_dkv ? kps : qps, Cn = is_dkv ? qps : kps;
        std::vector<int32_t> st((size_t)(R * Cn)), pd((size_t)(R * Cn));
        for (int64_t r = 0; r < qps; ++r)
          for (int64_t c = 0; c < kps; ++c) {
            const size_t src = (size_t)((qs * qps + r) * nkv + (ks * kps + c));
            const size_t dst = is_dkv ? (size_t)(c * Cn + r) : (size_t)(r * Cn + c);
            st[dst] = state[src];
            pd[dst] = pid[src];
          }
        ShardMeta m;
        shard_metadata(st, pd, R, Cn, is_dkv != 0, return_dynamic_grid != 0, &m);
        shards.push_back(std::move(m));
      }
    }

    std::vector<int32_t> rows, cols, mnext, bmask, nact;
    if (return_dynamic_grid) {
      int32_t max_size = 0;
      for (const ShardMeta& m : shards) max_size = std::max(max_size, m.grid_size);
      auto append_padded = [&](std::vector<int32_t>& dst, const std::vector<int32_t>& src) {
        dst.insert(dst.end(), src.begin(), src.end());
        dst.insert(dst.end(), (size_t)max_size - src.size(), -1);
      };
      for (const ShardMeta& m : shards) {
        append_padded(rows, m.rows);
        append_padded(cols, m.cols);
        append_padded(mnext, m.mask_next);
        append_padded(bmask, m.block_mask);
        nact.push_back(m.grid_size);
      }
    } else {
      for (const ShardMeta& m : shards) {
        mnext.insert(mnext.end(), m.mask_next.begin(), m.mask_next.end());
        bmask.insert(bmask.end(), m.block_mask.begin(), m.block_mask.end());
      }
    }

    out->n_entries = (int64_t)bmask.size();
    out->n_shards = (int32_t)shards.size();
    out->block_mask = dup(bmask);
    bool oom = out->block_mask == nullptr;
    if (return_dynamic_grid) {
      out->active_rows = dup(rows);
      out->active_cols = dup(cols);
      out->num_active_blocks = dup(nact);
      oom = oom || !out->active_rows || !out->active_cols || !out->num_active_blocks;
    }
    if (have_partial && !root_is_lazy) {
      out->mask_next = dup(mnext);
      out->n_partial = (int32_t)unique_blocks.size();
      const size_t blk = (size_t)block_q * block_kv;
      out->partial_mask_blocks = static_cast<int8_t*>(std::malloc(unique_blocks.size() * blk));
      oom = oom || !out->mask_next || !out->partial_mask_blocks;
      if (!oom) {
        for (size_t u = 0; u < unique_blocks.size(); ++u) {
          int8_t* dst = out->partial_mask_blocks + u * blk;
          const char* src = unique_blocks[u].data();
          if (!is_dkv) {
            std::memcpy(dst, src, blk);
          } else {  // stored transposed: [bkv, bq]
            for (int32_t i = 0; i < block_q; ++i)
              for (int32_t j = 0; j < block_kv; ++j) dst[(size_t)j * block_q + i] = src[(size_t)i * block_kv + j];
          }
        }
      }
    }
    if (oom) {
      splash_maskinfo_free(out);
      return SPLASH_ERR_OUT_OF_MEMORY;
    }
    return SPLASH_OK;
  } catch (const std::bad_alloc&) {
    splash_maskinfo_free(out);
    return SPLASH_ERR_OUT_OF_MEMORY;
  }
}

}  // extern "C"
