// Parameters and helpers shared by the backward kernels (128-wide tiles: splash_bwd_sm100.cu;
// head dims above 128: splash_bwd_wide_sm100.cu).
#pragma once

#include "splash_common.cuh"

namespace sb {

constexpr int kBwdThreads = 384;  // 8 compute warps + TMA warp + MMA warp + 2 idle warps that
                                  // complete the third warpgroup for the register hand-over
constexpr int kComputeRegs = 224;
constexpr int kIssueRegs = 56;

struct BwdParams {
  // outputs (dq kernel: dq; dkv kernel: dk, dv)
  __nv_bfloat16* out0;
  int64_t out0_sb, out0_sh, out0_ss;
  __nv_bfloat16* out1;
  int64_t out1_sb, out1_sh, out1_ss;
  SplashPeerOutput out0_peer, out1_peer;  // second destinations in other ranks' memory (ptrs == nullptr: none)
  const float* nlse2;  // [B, Hq, Sq]  -logsumexp * log2(e)
  const float* delta;  // [B, Hq, Sq]  -sum_d(o * do)
  const int32_t* q_seg;
  const int32_t* kv_seg;
  const int32_t* q_sequence;
  const int32_t* row_ptr;
  const int4* entries;
  const int32_t* row_order;    // launch order of the rows (longest first) or nullptr
  const int32_t* row_end;      // per batch row [batch, n_rows] or nullptr
  int64_t entries_per_batch;   // 0: one list shared by all batch rows
  const int8_t* pmb;
  int pm_bq, pm_bkv;
  SplashMaskFn fn;
  int q_len, kv_len, q_heads, kv_heads, n_rows;
  int d_qk, d_v;               // real columns of q / k / dq / dk and of v / o / do / dv (<= 128)
  int nk_qk, nk_v;             // K = 16 slices with real columns in contractions over d_qk / d_v
  int n_groups, chunk_groups;  // (batch, head) pairs of the grid; how many share a launch chunk
  // soft-cap variants: logits = cap * tanh(scale * q k^T / cap); dS gains the factor 1 - tanh^2
  float soft_cap, softcap_a;   // cap; scale / cap
  float scale, scale_log2;
  uint32_t* err;
  // fused form only: fp32 dQ image, one 128 x 128 tile per (batch, q head, q tile), each tile
  // stored as [col / 4][row][col % 4] so that one warp's vector red covers 512 contiguous bytes
  float* dq_acc;
};

// Column offset (32-bit TMEM columns) at which compute warpgroup w stores its 32 packed bf16
// columns: inside the 64 fp32 columns it has itself read, so the two warpgroups never race.
__device__ __forceinline__ uint32_t packed_col(int w) { return (uint32_t)(w * 64); }
// TMEM column of the A operand for K-slice k (16 values) of a tile written that way.
__device__ __forceinline__ uint32_t packed_a_col(int k) {
  return (uint32_t)((k >> 2) * 64 + (k & 3) * 8);
}

// 32 columns of a row, starting at column `col0` of a tensor that has `cols` columns: chunks of
// eight that lie beyond the tensor's last column (head dims below 128) are not stored.
__device__ __forceinline__ void store_row_half(__nv_bfloat16* dst, const uint32_t (&v)[32],
                                               float mul, int col0 = 0, int cols = kHeadDim) {
  uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (col0 + 8 * j >= cols) break;
    uint4 w;
    w.x = pack_bf16(__uint_as_float(v[8 * j + 0]) * mul, __uint_as_float(v[8 * j + 1]) * mul);
    w.y = pack_bf16(__uint_as_float(v[8 * j + 2]) * mul, __uint_as_float(v[8 * j + 3]) * mul);
    w.z = pack_bf16(__uint_as_float(v[8 * j + 4]) * mul, __uint_as_float(v[8 * j + 5]) * mul);
    w.w = pack_bf16(__uint_as_float(v[8 * j + 6]) * mul, __uint_as_float(v[8 * j + 7]) * mul);
    d4[j] = w;
  }
}

// Backward for head dims above 128 (defined in splash_bwd_wide_sm100.cu).  `p` carries the fields
// that do not depend on the pass; the launcher fills outputs and schedules per pass.
int launch_bwd_wide(const CUtensorMap& tm_q, const CUtensorMap& tm_do, const CUtensorMap& tm_k,
                    const CUtensorMap& tm_v, BwdParams p, const SplashBwdArgs& a, bool soft_cap,
                    uint32_t launch_mask, cudaStream_t stream);

}  // namespace sb
