// Ring attention: fold one step's partial result into the running pair, in one pass.
//   lse_new = log(exp(lse_acc) + exp(lse_i));  o_acc = o_acc * exp(lse_acc - lse_new) + o_i * exp(lse_i - lse_new)
// HBM-bound elementwise work: per row it reads 128 fp32 + 128 bf16 + two floats and writes 128 fp32
// + one float (1288 bytes); one warp per row, 16-byte accesses.  Same arithmetic as the (m, l, o)
// carry of the reference's ring (ring_attention_kernel.py:150-158), written on logsumexp.
#include "splash_common.cuh"

namespace sb {

__global__ void __launch_bounds__(256)
splash_ring_merge_kernel(float* __restrict__ o_acc, float* __restrict__ lse_acc, const __nv_bfloat16* __restrict__ o_i,
                         const float* __restrict__ lse_i, int64_t n_rows) {
  const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  const int lane = threadIdx.x & 31;
  const float a = lse_acc[row], b = lse_i[row];
  const float m = fmaxf(a, b);
  float wa = 0.f, wb = 0.f, lse = m;
  if (m > -INFINITY) {  // both -inf: nothing merged yet and nothing to merge
    const float ea = __expf(a - m), eb = __expf(b - m);
    const float inv = 1.0f / (ea + eb);
    wa = ea * inv;
    wb = eb * inv;
    lse = m + __logf(ea + eb);
  }
  float4* acc = reinterpret_cast<float4*>(o_acc + row * kHeadDim) + lane;
  const uint2 raw = __ldg(reinterpret_cast<const uint2*>(o_i + row * kHeadDim) + lane);
  const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
  const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  float4 v = *acc;
  v.x = v.x * wa + __bfloat162float(lo.x) * wb;
  v.y = v.y * wa + __bfloat162float(lo.y) * wb;
  v.z = v.z * wa + __bfloat162float(hi.x) * wb;
  v.w = v.w * wa + __bfloat162float(hi.y) * wb;
  *acc = v;
  if (lane == 0) lse_acc[row] = lse;
}

}  // namespace sb

extern "C" int splash_ring_merge(float* o_acc, float* lse_acc, const void* o_i, const float* lse_i, int64_t n_rows,
                                 int64_t head_dim, void* cuda_stream) {
  if (o_acc == nullptr || lse_acc == nullptr || o_i == nullptr || lse_i == nullptr || n_rows <= 0)
    return SPLASH_ERR_INVALID_ARGUMENT;
  if (head_dim != sb::kHeadDim) return SPLASH_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(o_acc) & 15u) != 0 || (reinterpret_cast<uintptr_t>(o_i) & 7u) != 0)
    return SPLASH_ERR_INVALID_ARGUMENT;
  const int64_t blocks = (n_rows + 7) / 8;
  if (blocks > 0x7fffffffll) return SPLASH_ERR_TOO_LARGE;
  sb::splash_ring_merge_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
      o_acc, lse_acc, static_cast<const __nv_bfloat16*>(o_i), lse_i, n_rows);
  return cudaGetLastError() == cudaSuccess ? SPLASH_OK : SPLASH_ERR_CUDA;
}
