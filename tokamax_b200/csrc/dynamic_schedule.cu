// Schedules for a mask that is data on the device (a bool / int8 array [q_len, kv_len]) and may
// change from call to call: nothing of it goes through the host.  Two HBM-bound kernels: the state
// (0 empty, 1 partial, 2 full) of every 128x128 tile, then one work list per schedule row written
// at a fixed stride with its end stored in `row_end`.  The attention kernels read partially masked
// tiles straight from the mask: the whole array is passed as a single "partial block" of shape
// [q_len, kv_len] (transposed for the dkv kernel), so no per-block copy is made either.
//
// Counterpart of the reference's `_process_dynamic_mask`
// (tokamax/_src/ops/experimental/tpu/splash_attention/splash_attention_mask_info.py:231-350), which
// builds fixed-size tables from a runtime mask with XLA ops and keeps every block as a partial block.
#include "splash_common.cuh"

namespace sb {

constexpr int kDynThreads = 128;

// One CTA per 128x128 tile, one thread per row (128 bytes = eight 16-byte loads).
__global__ void __launch_bounds__(kDynThreads)
splash_mask_tile_state_kernel(const uint8_t* __restrict__ mask, int64_t row_stride, int n_kv_tiles,
                              int32_t* __restrict__ states) {
  const int kt = blockIdx.x, qt = blockIdx.y;
  const uint4* row = reinterpret_cast<const uint4*>(mask + ((int64_t)qt * kTile + threadIdx.x) * row_stride +
                                                    (int64_t)kt * kTile);
  bool any = false, all = true;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint4 v = __ldg(row + i);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      any |= w[j] != 0u;
      all &= ((w[j] - 0x01010101u) & ~w[j] & 0x80808080u) == 0u;  // no zero byte in the word
    }
  }
  const int warp_any = __any_sync(0xffffffffu, any);
  const int warp_all = __all_sync(0xffffffffu, all);
  __shared__ int s_any[kDynThreads / 32], s_all[kDynThreads / 32];
  if ((threadIdx.x & 31) == 0) {
    s_any[threadIdx.x >> 5] = warp_any;
    s_all[threadIdx.x >> 5] = warp_all;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int a = 0, f = 1;
#pragma unroll
    for (int w = 0; w < kDynThreads / 32; ++w) {
      a |= s_any[w];
      f &= s_all[w];
    }
    states[(int64_t)qt * n_kv_tiles + kt] = a ? (f ? 2 : 1) : 0;
  }
}

// One CTA per schedule row: compacts the live tiles of the row, in order, into its fixed-stride
// slot.  kind 0: row = pair of q tiles, entries = kv tiles; kind 1: row = q tile; kind 2: row = kv
// tile, entries = q tiles.  Partial tiles get block id 0 (the whole mask is the one block).
__global__ void __launch_bounds__(kDynThreads)
splash_dynamic_schedule_kernel(const int32_t* __restrict__ states, int n_q_tiles, int n_kv_tiles, int kind,
                               int n_cols, int batch, int n_rows, int32_t* __restrict__ row_ptr,
                               int32_t* __restrict__ row_end, int4* __restrict__ entries) {
  const int row = blockIdx.x;
  const int begin = row * n_cols;
  __shared__ int warp_count[kDynThreads / 32];
  __shared__ int base;
  if (threadIdx.x == 0) base = begin;
  __syncthreads();
  for (int c0 = 0; c0 < n_cols; c0 += kDynThreads) {
    const int c = c0 + threadIdx.x;
    int s0 = 0, s1 = 0;
    if (c < n_cols) {
      if (kind == 0) {
        s0 = states[(int64_t)(2 * row) * n_kv_tiles + c];
        if (2 * row + 1 < n_q_tiles) s1 = states[(int64_t)(2 * row + 1) * n_kv_tiles + c];
      } else if (kind == 1) {
        s0 = states[(int64_t)row * n_kv_tiles + c];
      } else {
        s0 = states[(int64_t)c * n_kv_tiles + row];
      }
    }
    const bool keep = (s0 | s1) != 0;
    const unsigned ballot = __ballot_sync(0xffffffffu, keep);
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    if (lane == 0) warp_count[w] = __popc(ballot);
    __syncthreads();
    int offset = base;
    for (int i = 0; i < w; ++i) offset += warp_count[i];
    if (keep)
      entries[offset + __popc(ballot & ((1u << lane) - 1u))] =
          make_int4(c, s0 | (s1 << 2), s0 == 1 ? 0 : -1, s1 == 1 ? 0 : -1);
    __syncthreads();
    if (threadIdx.x == 0) {
      int total = 0;
      for (int i = 0; i < kDynThreads / 32; ++i) total += warp_count[i];
      base += total;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    row_ptr[row] = begin;
    if (row == n_rows - 1) row_ptr[n_rows] = n_rows * n_cols;
    for (int b = 0; b < batch; ++b) row_end[(int64_t)b * n_rows + row] = base;
  }
}

static size_t dyn_align256(size_t n) { return (n + 255) & ~(size_t)255; }

static bool dyn_shape(int64_t q_len, int64_t kv_len, int32_t kind, int64_t* n_rows, int64_t* n_cols) {
  if (q_len <= 0 || kv_len <= 0 || q_len % kTile != 0 || kv_len % kTile != 0 || kind < 0 || kind > 2) return false;
  const int64_t nq = q_len / kTile, nkv = kv_len / kTile;
  *n_rows = kind == 0 ? (nq + 1) / 2 : (kind == 1 ? nq : nkv);
  *n_cols = kind == 2 ? nq : nkv;
  return true;
}

}  // namespace sb

extern "C" {

int splash_mask_tile_states(const void* mask, int64_t row_stride_bytes, int64_t q_len, int64_t kv_len,
                            int32_t* states, void* cuda_stream) {
  if (mask == nullptr || states == nullptr) return SPLASH_ERR_INVALID_ARGUMENT;
  if (q_len <= 0 || kv_len <= 0 || q_len % sb::kTile != 0 || kv_len % sb::kTile != 0)
    return SPLASH_ERR_INVALID_ARGUMENT;
  if (row_stride_bytes < kv_len || row_stride_bytes % 16 != 0 || (reinterpret_cast<uintptr_t>(mask) & 15u) != 0)
    return SPLASH_ERR_INVALID_ARGUMENT;
  const int64_t nq = q_len / sb::kTile, nkv = kv_len / sb::kTile;
  if (nq > 65535 || nkv > 0x7fffffff) return SPLASH_ERR_TOO_LARGE;
  sb::splash_mask_tile_state_kernel<<<dim3((unsigned)nkv, (unsigned)nq), sb::kDynThreads, 0,
                                      static_cast<cudaStream_t>(cuda_stream)>>>(
      static_cast<const uint8_t*>(mask), row_stride_bytes, (int)nkv, states);
  return cudaGetLastError() == cudaSuccess ? SPLASH_OK : SPLASH_ERR_CUDA;
}

size_t splash_dynamic_schedule_bytes(int64_t q_len, int64_t kv_len, int32_t kind, int64_t batch) {
  int64_t n_rows, n_cols;
  if (batch <= 0 || !sb::dyn_shape(q_len, kv_len, kind, &n_rows, &n_cols)) return 0;
  return sb::dyn_align256((size_t)(n_rows + 1) * sizeof(int32_t)) +
         sb::dyn_align256((size_t)batch * (size_t)n_rows * sizeof(int32_t)) +
         sb::dyn_align256((size_t)n_rows * (size_t)n_cols * sizeof(int4));
}

int splash_dynamic_schedule(const int32_t* states, int64_t q_len, int64_t kv_len, int32_t kind, int64_t batch,
                            const void* partial_blocks, void* workspace, size_t workspace_bytes,
                            SplashDeviceSchedule* out, void* cuda_stream) {
  int64_t n_rows, n_cols;
  if (states == nullptr || workspace == nullptr || out == nullptr || partial_blocks == nullptr || batch <= 0 ||
      batch > 65535 || !sb::dyn_shape(q_len, kv_len, kind, &n_rows, &n_cols))
    return SPLASH_ERR_INVALID_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0 ||
      workspace_bytes < splash_dynamic_schedule_bytes(q_len, kv_len, kind, batch))
    return SPLASH_ERR_INVALID_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(partial_blocks) & 15u) != 0) return SPLASH_ERR_INVALID_ARGUMENT;
  if (n_rows * n_cols > 0x7fffffffll || q_len > 0x7fffffffll || kv_len > 0x7fffffffll) return SPLASH_ERR_TOO_LARGE;

  uint8_t* ws = static_cast<uint8_t*>(workspace);
  int32_t* row_ptr = reinterpret_cast<int32_t*>(ws);
  ws += sb::dyn_align256((size_t)(n_rows + 1) * sizeof(int32_t));
  int32_t* row_end = reinterpret_cast<int32_t*>(ws);
  ws += sb::dyn_align256((size_t)batch * (size_t)n_rows * sizeof(int32_t));
  int4* entries = reinterpret_cast<int4*>(ws);

  sb::splash_dynamic_schedule_kernel<<<(unsigned)n_rows, sb::kDynThreads, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
      states, (int)(q_len / sb::kTile), (int)(kv_len / sb::kTile), kind, (int)n_cols, (int)batch, (int)n_rows, row_ptr,
      row_end, entries);
  if (cudaGetLastError() != cudaSuccess) return SPLASH_ERR_CUDA;

  out->row_ptr = row_ptr;
  out->entries = reinterpret_cast<const int32_t*>(entries);
  out->n_rows = (int32_t)n_rows;
  out->partial_mask_blocks = static_cast<const int8_t*>(partial_blocks);
  out->block_q = (int32_t)q_len;   // the whole mask is the single partial block
  out->block_kv = (int32_t)kv_len;
  out->n_entries = n_rows * n_cols;
  out->row_end = row_end;
  out->entries_per_batch = 0;      // one list shared by all batch rows
  out->row_order = nullptr;
  return SPLASH_OK;
}

}  // extern "C"
