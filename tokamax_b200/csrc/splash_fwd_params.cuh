// Parameters and constants shared by the forward kernels (128-wide tiles: splash_fwd_sm100.cu;
// head dims above 128: splash_fwd_wide_sm100.cu).
#pragma once

#include "splash_common.cuh"

namespace sb {

constexpr int kFwdStages = 4;
constexpr int kFwdThreads = 384;  // 3 warpgroups: softmax 0, softmax 1, {TMA, MMA, 2 idle warps}
constexpr int kSoftmaxRegs = 224;  // setmaxnreg targets: 2*128*224 + 128*56 <= 64K registers
constexpr int kIssueRegs = 56;
constexpr float kRescaleThreshold = 8.0f;  // log2 units
// Lower bound of the running maximum (log2 units).  A row whose entries so far are all masked
// would otherwise take the scaled masked logit as its maximum and turn its masked entries into
// exp2(rounding error of a 1e29-sized product); with the floor they stay exactly zero, l stays 0,
// and a row that never meets a live key ends as zeros with logsumexp = mask_value.
constexpr float kLogitFloor = -1.0e6f;
constexpr float kMinScaleLog2 = 1.0e-20f;  // keeps kMaskedLogit * scale far below kLogitFloor
constexpr float kFp8RescaleThreshold = 2.0f;  // e4m3 P must stay below 448 = 2^8.8
constexpr float kFp8PShift = 6.0f;            // P is stored as 2^6 * exp2(s - m) * (v scale ratio <= 1)
constexpr int kFp8TileBytes = kTile * kHeadDim;  // 16 KiB

struct FwdParams {
  __nv_bfloat16* o;
  int64_t o_sb, o_sh, o_ss;
  SplashPeerOutput o_peer;  // second destination of o in other ranks' memory (ptrs == nullptr: none)
  int d_v;  // columns of v / o (<= 128; the tile's remaining columns are zeros and are not stored)
  int nk_qk;  // K = 16 slices of q k^T that hold real columns: ceil(d_qk / 16); the rest are zeros and are skipped
  int d_qk;   // columns of q / k: at most 64 -> the second 64-column half of their tiles is never loaded or read
  float* lse;
  float* maxl;
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
  int q_len, kv_len, q_heads, kv_heads, n_q_tiles, n_rows;
  int n_groups, chunk_groups;  // (batch, q head) pairs; how many of them share a launch chunk
  float scale, scale_log2, mask_value;
  uint32_t* err;
  // e4m3 variant only: one scale per (batch, head, 128-token tile)
  const float* q_scale;
  const float* k_scale;
  const float* v_scale;
  int n_kv_tiles;
  const float* sinks;            // [q_heads] or nullptr
  const float* max_logit_value;  // [q_heads] or nullptr
  // soft-cap variant: logits = cap * tanh(scale * q k^T / cap)
  float soft_cap, softcap_a;     // cap; scale / cap
};

// Launches the forward for head dims above 128 (defined in splash_fwd_wide_sm100.cu); `p` and the
// tensor maps are those the 128-wide launcher prepared.
int launch_fwd_wide(const CUtensorMap& tm_q, const CUtensorMap& tm_k, const CUtensorMap& tm_v,
                    const FwdParams& p, bool soft_cap, cudaStream_t stream);

}  // namespace sb
