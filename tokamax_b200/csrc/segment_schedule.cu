// Segment-aware schedules: drop, per batch row, the 128x128 tiles whose q and kv segment-id
// ranges cannot contain an equal pair, and mark the tiles that lie inside one segment (all ids of
// the q tile and of the kv tile equal), for which the kernels skip the per-element comparison.  Two small HBM-bound kernels: tile ranges, then a
// per-row stream compaction of the schedule entries.  Results of attention are unchanged (the
// dropped tiles are fully masked by the segment mask); only skipped work differs.
#include "splash_common.cuh"

namespace sb {

constexpr int kSegThreads = 128;

// [min, max] of the segment ids of every 128-token tile: out[b][tile] (q tiles then kv tiles).
__global__ void __launch_bounds__(kSegThreads)
splash_segment_ranges_kernel(const int32_t* __restrict__ q_seg, const int32_t* __restrict__ kv_seg,
                             int q_len, int kv_len, int2* __restrict__ q_rng, int2* __restrict__ kv_rng) {
  const int nq = q_len / kTile, nkv = kv_len / kTile;
  const int b = blockIdx.y;
  int t = blockIdx.x;
  const int32_t* src;
  int2* dst;
  if (t < nq) {
    src = q_seg + (int64_t)b * q_len + (int64_t)t * kTile;
    dst = q_rng + (int64_t)b * nq + t;
  } else {
    t -= nq;
    if (t >= nkv) return;
    src = kv_seg + (int64_t)b * kv_len + (int64_t)t * kTile;
    dst = kv_rng + (int64_t)b * nkv + t;
  }
  const int v = src[threadIdx.x];
  int lo = v, hi = v;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, off));
    hi = max(hi, __shfl_xor_sync(0xffffffffu, hi, off));
  }
  __shared__ int s_lo[kSegThreads / 32], s_hi[kSegThreads / 32];
  if ((threadIdx.x & 31) == 0) {
    s_lo[threadIdx.x >> 5] = lo;
    s_hi[threadIdx.x >> 5] = hi;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
#pragma unroll
    for (int w = 1; w < kSegThreads / 32; ++w) {
      lo = min(lo, s_lo[w]);
      hi = max(hi, s_hi[w]);
    }
    *dst = make_int2(lo, hi);
  }
}

__device__ __forceinline__ bool ranges_overlap(int2 a, int2 b) { return !(a.y < b.x || a.x > b.y); }
// every token of both tiles carries one and the same id: the segment mask keeps the whole tile
__device__ __forceinline__ bool same_segment(int2 a, int2 b) { return a.x == a.y && b.x == b.y && a.x == b.x; }

// One block per (schedule row, batch row): keeps the entries that can still hold an unmasked
// pair, in order, at the start of the row's slot of the per-batch copy.
__global__ void __launch_bounds__(kSegThreads)
splash_segment_filter_kernel(const int32_t* __restrict__ row_ptr, const int4* __restrict__ entries, int n_rows,
                             int64_t n_entries, int kind, int n_q_tiles, int n_kv_tiles,
                             const int2* __restrict__ q_rng, const int2* __restrict__ kv_rng,
                             int4* __restrict__ out_entries, int32_t* __restrict__ row_end) {
  const int row = blockIdx.x, b = blockIdx.y;
  const int ebeg = row_ptr[row], eend = row_ptr[row + 1];
  const int2* qr = q_rng + (int64_t)b * n_q_tiles;
  const int2* kr = kv_rng + (int64_t)b * n_kv_tiles;
  int4* out = out_entries + (int64_t)b * n_entries;
  __shared__ int warp_count[kSegThreads / 32];
  __shared__ int base;
  if (threadIdx.x == 0) base = ebeg;
  __syncthreads();
  for (int e0 = ebeg; e0 < eend; e0 += kSegThreads) {
    const int e = e0 + threadIdx.x;
    int4 ent = make_int4(0, 0, -1, -1);
    bool keep = false;
    if (e < eend) {
      ent = entries[e];
      int s0 = ent.y & 3, s1 = (ent.y >> 2) & 3;
      int u0 = 0, u1 = 0;  // SPLASH_ENTRY_ONE_SEGMENT_*: the kernels skip the per-element id comparison
      if (kind == 0) {  // row = pair of q tiles, entry = kv tile
        const int2 k = kr[ent.x];
        if (s0 && !ranges_overlap(qr[2 * row], k)) s0 = 0;
        if (s1 && (2 * row + 1 >= n_q_tiles || !ranges_overlap(qr[2 * row + 1], k))) s1 = 0;
        u0 = s0 && same_segment(qr[2 * row], k);
        u1 = s1 && same_segment(qr[2 * row + 1], k);
      } else if (kind == 1) {  // row = q tile, entry = kv tile
        if (s0 && !ranges_overlap(qr[row], kr[ent.x])) s0 = 0;
        s1 = 0;
        u0 = s0 && same_segment(qr[row], kr[ent.x]);
      } else {  // row = kv tile, entry = q tile
        if (s0 && !ranges_overlap(qr[ent.x], kr[row])) s0 = 0;
        s1 = 0;
        u0 = s0 && same_segment(qr[ent.x], kr[row]);
      }
      ent.y = s0 | (s1 << 2) | (u0 << 4) | (u1 << 5);
      if (s0 == 0) ent.z = -1;
      if (s1 == 0) ent.w = -1;
      keep = (s0 | s1) != 0;
    }
    const unsigned ballot = __ballot_sync(0xffffffffu, keep);
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    if (lane == 0) warp_count[w] = __popc(ballot);
    __syncthreads();
    int offset = base;
    for (int i = 0; i < w; ++i) offset += warp_count[i];
    if (keep) out[offset + __popc(ballot & ((1u << lane) - 1u))] = ent;
    __syncthreads();
    if (threadIdx.x == 0) {
      int total = 0;
      for (int i = 0; i < kSegThreads / 32; ++i) total += warp_count[i];
      base += total;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) row_end[(int64_t)b * n_rows + row] = base;
}

static size_t align256(size_t n) { return (n + 255) & ~(size_t)255; }

}  // namespace sb

extern "C" {

size_t splash_segment_schedule_bytes(int64_t batch, int64_t q_len, int64_t kv_len, int32_t n_rows,
                                     int64_t n_entries) {
  if (batch <= 0 || q_len <= 0 || kv_len <= 0 || n_rows <= 0 || n_entries < 0) return 0;
  const size_t nq = (size_t)(q_len / sb::kTile), nkv = (size_t)(kv_len / sb::kTile);
  return sb::align256((size_t)batch * nq * sizeof(int2)) + sb::align256((size_t)batch * nkv * sizeof(int2)) +
         sb::align256((size_t)batch * (size_t)n_rows * sizeof(int32_t)) +
         sb::align256((size_t)batch * (size_t)(n_entries > 0 ? n_entries : 1) * sizeof(int4));
}

int splash_segment_schedule(const SplashDeviceSchedule* in, int32_t kind, const int32_t* q_segment_ids,
                            const int32_t* kv_segment_ids, int64_t batch, int64_t q_len, int64_t kv_len,
                            void* workspace, size_t workspace_bytes, SplashDeviceSchedule* out,
                            void* cuda_stream) {
  if (in == nullptr || out == nullptr || workspace == nullptr || q_segment_ids == nullptr ||
      kv_segment_ids == nullptr)
    return SPLASH_ERR_INVALID_ARGUMENT;
  if (kind < 0 || kind > 2 || batch <= 0 || batch > 65535 || q_len <= 0 || kv_len <= 0 ||
      q_len % sb::kTile != 0 || kv_len % sb::kTile != 0)
    return SPLASH_ERR_INVALID_ARGUMENT;
  if (in->row_ptr == nullptr || in->entries == nullptr || in->n_rows <= 0 || in->n_entries < 0 ||
      in->row_end != nullptr || in->entries_per_batch != 0)
    return SPLASH_ERR_INVALID_ARGUMENT;
  const int nq = (int)(q_len / sb::kTile), nkv = (int)(kv_len / sb::kTile);
  const int expect_rows = kind == 0 ? (nq + 1) / 2 : (kind == 1 ? nq : nkv);
  if (in->n_rows != expect_rows) return SPLASH_ERR_INVALID_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return SPLASH_ERR_INVALID_ARGUMENT;
  if (workspace_bytes < splash_segment_schedule_bytes(batch, q_len, kv_len, in->n_rows, in->n_entries))
    return SPLASH_ERR_INVALID_ARGUMENT;

  uint8_t* ws = static_cast<uint8_t*>(workspace);
  int2* q_rng = reinterpret_cast<int2*>(ws);
  ws += sb::align256((size_t)batch * nq * sizeof(int2));
  int2* kv_rng = reinterpret_cast<int2*>(ws);
  ws += sb::align256((size_t)batch * nkv * sizeof(int2));
  int32_t* row_end = reinterpret_cast<int32_t*>(ws);
  ws += sb::align256((size_t)batch * in->n_rows * sizeof(int32_t));
  int4* entries = reinterpret_cast<int4*>(ws);

  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  sb::splash_segment_ranges_kernel<<<dim3((unsigned)(nq + nkv), (unsigned)batch), sb::kSegThreads, 0, stream>>>(
      q_segment_ids, kv_segment_ids, (int)q_len, (int)kv_len, q_rng, kv_rng);
  if (cudaGetLastError() != cudaSuccess) return SPLASH_ERR_CUDA;
  sb::splash_segment_filter_kernel<<<dim3((unsigned)in->n_rows, (unsigned)batch), sb::kSegThreads, 0, stream>>>(
      in->row_ptr, reinterpret_cast<const int4*>(in->entries), in->n_rows, in->n_entries, kind, nq, nkv, q_rng,
      kv_rng, entries, row_end);
  if (cudaGetLastError() != cudaSuccess) return SPLASH_ERR_CUDA;

  *out = *in;
  out->entries = reinterpret_cast<const int32_t*>(entries);
  out->row_end = row_end;
  out->entries_per_batch = in->n_entries;
  return SPLASH_OK;
}

}  // extern "C"
