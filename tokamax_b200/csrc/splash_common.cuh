// Definitions shared by the forward / dq / dkv kernels and their host launchers.
#pragma once

#include <cuda.h>  // CUtensorMap (types only; the encoder is fetched through the runtime)
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cstdint>

#include "../../include/splash_b200.h"
#include "sm100_ptx.cuh"

namespace sb {

constexpr int kTile = 128;          // q and kv tile edge the MMAs work on
constexpr int kHeadDim = 128;       // head dimension of the bf16 kernels
constexpr int kTileBytes = kTile * kHeadDim * 2;   // one bf16 operand tile: 32 KiB
constexpr int kHalfBytes = kTileBytes / 2;         // one 64-column (128-byte) swizzle half
constexpr float kMaskedLogit = -1.0e30f;           // raw logit given to masked positions
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// Per-row key interval kept by an in-kernel mask function (see SplashMaskFn).
struct RowInterval {
  int lo, hi;
};

__device__ __forceinline__ RowInterval mask_fn_interval(const SplashMaskFn& fn, int qi) {
  RowInterval iv;
  iv.lo = INT32_MIN;
  iv.hi = INT32_MAX;
  if (fn.kind == SPLASH_MASK_CAUSAL) {
    iv.hi = qi + fn.offset;
  } else if (fn.kind == SPLASH_MASK_LOCAL) {
    if (fn.has_left) iv.lo = qi + fn.offset - fn.left;
    if (fn.has_right) iv.hi = qi + fn.offset + fn.right;
  } else if (fn.kind == SPLASH_MASK_CHUNKED) {
    iv.lo = (qi / fn.chunk) * fn.chunk;
    iv.hi = qi;
  }
  return iv;
}

// Same mask function seen from a key: the queries i that keep key j form an interval too, but
// the dkv kernel simply evaluates lo(i) <= j <= hi(i) per element, so no inverse is needed.

// Which (row, group) a CTA of a 1-D grid of n_rows * n_groups blocks works on.  A group is a
// (batch, head) pair.  Groups are taken chunk_groups at a time; inside a chunk the launch order
// runs through the rows longest first (row_order, or `fallback_reversed` index order), all groups
// of the chunk side by side.  A chunk small enough for its streamed operands to stay in L2 keeps
// DRAM traffic near the compulsory minimum, while the grid still drains on short CTAs.
struct CtaWork {
  int row, group;
};
__device__ __forceinline__ CtaWork cta_work_at(unsigned block, const int32_t* row_order, int n_rows, int n_groups,
                                               int chunk_groups, bool fallback_reversed) {
  const unsigned per_chunk = (unsigned)n_rows * (unsigned)chunk_groups;
  const unsigned chunk = block / per_chunk;
  const unsigned rem = block - chunk * per_chunk;
  const unsigned first = chunk * (unsigned)chunk_groups;
  const unsigned here = min((unsigned)chunk_groups, (unsigned)n_groups - first);
  const unsigned pos = rem / here;
  CtaWork w;
  w.group = (int)(first + (rem - pos * here));
  w.row = row_order ? row_order[pos] : (fallback_reversed ? n_rows - 1 - (int)pos : (int)pos);
  return w;
}
__device__ __forceinline__ CtaWork cta_work(const int32_t* row_order, int n_rows, int n_groups,
                                            int chunk_groups, bool fallback_reversed) {
  return cta_work_at(blockIdx.x, row_order, n_rows, n_groups, chunk_groups, fallback_reversed);
}
// Groups per chunk so that `bytes_per_group` of streamed operands of one chunk fill about half
// of a 126 MB L2, in whole multiples of `align` (heads sharing a kv head stay together).
inline int chunk_groups_for(int64_t bytes_per_group, int64_t n_groups, int64_t align) {
  int64_t g = (int64_t)(64ll << 20) / (bytes_per_group > 0 ? bytes_per_group : 1);
  g = g / align * align;
  if (g < align) g = align;
  if (g > n_groups) g = n_groups;
  return (int)g;
}

// Address of row `s` of local head `h` in the rank that owns it (see SplashPeerOutput).
__device__ __forceinline__ __nv_bfloat16* peer_row(const SplashPeerOutput& po, int batch, int h, int s) {
  const int64_t peer = s / po.rows_per_peer;
  const int64_t local = s - peer * po.rows_per_peer;
  uint8_t* base = reinterpret_cast<uint8_t*>(po.ptrs[peer]) + po.base_bytes;
  return reinterpret_cast<__nv_bfloat16*>(base) + (int64_t)batch * po.stride_b + (int64_t)(po.head0 + h) * po.stride_h +
         local * po.stride_s;
}
inline int check_peer_output(const SplashPeerOutput& po, int64_t rows, int64_t head_dim) {
  if (po.ptrs == nullptr) return SPLASH_OK;
  if (po.rows_per_peer <= 0 || rows % po.rows_per_peer != 0 || po.head0 < 0 || po.base_bytes < 0 ||
      po.base_bytes % 16 != 0 || po.stride_s < head_dim || po.stride_b % 8 != 0 || po.stride_h % 8 != 0 ||
      po.stride_s % 8 != 0)
    return SPLASH_ERR_INVALID_ARGUMENT;
  return SPLASH_OK;
}

// Host-side helpers (defined in splash_host.cu).
int make_tile_tensor_map(CUtensorMap* out, const SplashTensor& t, int box_rows);
int check_bf16_tensor(const SplashTensor& t);
int check_e4m3_tensor(const SplashTensor& t);

}  // namespace sb
