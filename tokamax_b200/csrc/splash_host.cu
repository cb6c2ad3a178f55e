// Host side of the C ABI: argument checks, TMA tensor maps, status strings, error read-back.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "splash_common.cuh"

namespace sb {

int launch_fwd(const SplashFwdArgs& a, cudaStream_t stream);
int launch_fwd_fp8(const SplashFwdFp8Args& a, cudaStream_t stream);
int launch_bwd(const SplashBwdArgs& a, cudaStream_t stream);
int launch_bwd_static_scratch(const SplashBwdArgs& a, cudaStream_t stream);
size_t bwd_workspace_bytes(int64_t batch, int64_t q_heads, int64_t q_len);
size_t bwd_fused_workspace_bytes(int64_t batch, int64_t q_heads, int64_t q_len);

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static std::mutex mu;
  static EncodeTiledFn fn = nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (fn == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

int check_bf16_tensor(const SplashTensor& t) {
  if (t.data == nullptr) return SPLASH_ERR_INVALID_ARGUMENT;
  if (t.dtype != SPLASH_BF16) return SPLASH_ERR_UNSUPPORTED;
  if (t.stride[3] != 1) return SPLASH_ERR_INVALID_ARGUMENT;
  for (int i = 0; i < 4; ++i)
    if (t.size[i] <= 0) return SPLASH_ERR_INVALID_ARGUMENT;
  for (int i = 0; i < 3; ++i)
    if (t.stride[i] % 8 != 0 || t.stride[i] < 0) return SPLASH_ERR_INVALID_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(t.data) & 15u) != 0) return SPLASH_ERR_INVALID_ARGUMENT;
  return SPLASH_OK;
}

int check_e4m3_tensor(const SplashTensor& t) {
  if (t.data == nullptr) return SPLASH_ERR_INVALID_ARGUMENT;
  if (t.dtype != SPLASH_F8E4M3) return SPLASH_ERR_UNSUPPORTED;
  if (t.stride[3] != 1) return SPLASH_ERR_INVALID_ARGUMENT;
  for (int i = 0; i < 4; ++i)
    if (t.size[i] <= 0) return SPLASH_ERR_INVALID_ARGUMENT;
  for (int i = 0; i < 3; ++i)
    if (t.stride[i] % 16 != 0 || t.stride[i] < 0) return SPLASH_ERR_INVALID_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(t.data) & 15u) != 0) return SPLASH_ERR_INVALID_ARGUMENT;
  return SPLASH_OK;
}

// Tensor map over (head_dim, seq, heads, batch) with a (128 bytes x box_rows) box and 128-byte
// swizzle.  bf16: 64 columns, one swizzle half of an MMA operand tile; e4m3: all 128 columns.
int make_tile_tensor_map(CUtensorMap* out, const SplashTensor& t, int box_rows) {
  EncodeTiledFn enc = get_encode_fn();
  if (enc == nullptr) return SPLASH_ERR_NO_DEVICE;
  const bool fp8 = t.dtype == SPLASH_F8E4M3;
  const cuuint64_t esize = fp8 ? 1u : 2u;
  const cuuint64_t dims[4] = {(cuuint64_t)t.size[3], (cuuint64_t)t.size[2], (cuuint64_t)t.size[1],
                              (cuuint64_t)t.size[0]};
  // A size-1 dimension may carry any stride; give it a legal one.
  auto stride_bytes = [&](int i) -> cuuint64_t {
    cuuint64_t s = (cuuint64_t)t.stride[i] * esize;
    if (s == 0) s = 16;
    return s;
  };
  const cuuint64_t strides[3] = {stride_bytes(2), stride_bytes(1), stride_bytes(0)};
  const cuuint32_t box[4] = {fp8 ? 128u : 64u, (cuuint32_t)box_rows, 1u, 1u};
  const cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
  CUresult r = enc(out, fp8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, t.data,
                   dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS && std::getenv("SPLASH_DEBUG") != nullptr)
    std::fprintf(stderr, "splash_b200: cuTensorMapEncodeTiled failed (%d): sizes %lld %lld %lld %lld strides %lld %lld %lld box rows %d\n",
                 (int)r, (long long)t.size[0], (long long)t.size[1], (long long)t.size[2], (long long)t.size[3],
                 (long long)t.stride[0], (long long)t.stride[1], (long long)t.stride[2], box_rows);
  return r == CUDA_SUCCESS ? SPLASH_OK : SPLASH_ERR_CUDA;
}

// One thread waits, through the same mbar_wait the attention kernels use, on a barrier that
// nothing ever arrives on; the wait gives up after `limit_cycles` and the kernel returns.
__global__ void bounded_wait_probe_kernel(uint32_t* err, long long limit_cycles, uint32_t tag) {
  __shared__ uint64_t bar;
  __shared__ uint32_t flag;
  if (threadIdx.x == 0) {
    flag = 0;
    mbar_init(&bar, 1);
    mbar_fence_init();
    AbortCtx ab{&flag, err, limit_cycles};
    (void)mbar_wait(&bar, 0, ab, tag);
  }
}

}  // namespace sb

extern "C" {

int splash_probe_bounded_wait(uint32_t* error_record, int64_t limit_cycles, uint32_t tag, void* cuda_stream) {
  if (error_record == nullptr || limit_cycles <= 0 || limit_cycles > 100000000ll) return SPLASH_ERR_INVALID_ARGUMENT;
  sb::bounded_wait_probe_kernel<<<1, 32, 0, static_cast<cudaStream_t>(cuda_stream)>>>(error_record, (long long)limit_cycles, tag);
  return cudaGetLastError() == cudaSuccess ? SPLASH_OK : SPLASH_ERR_CUDA;
}

int splash_fwd(const SplashFwdArgs* args, void* cuda_stream) {
  if (args == nullptr) return SPLASH_ERR_INVALID_ARGUMENT;
  return sb::launch_fwd(*args, static_cast<cudaStream_t>(cuda_stream));
}

int splash_fwd_fp8(const SplashFwdFp8Args* args, void* cuda_stream) {
  if (args == nullptr) return SPLASH_ERR_INVALID_ARGUMENT;
  return sb::launch_fwd_fp8(*args, static_cast<cudaStream_t>(cuda_stream));
}

size_t splash_bwd_workspace_bytes(int64_t batch, int64_t q_heads, int64_t q_len) {
  return sb::bwd_workspace_bytes(batch, q_heads, q_len);
}

size_t splash_bwd_fused_workspace_bytes(int64_t batch, int64_t q_heads, int64_t q_len) {
  return sb::bwd_fused_workspace_bytes(batch, q_heads, q_len);
}

int splash_bwd(const SplashBwdArgs* args, void* cuda_stream) {
  if (args == nullptr) return SPLASH_ERR_INVALID_ARGUMENT;
  return sb::launch_bwd(*args, static_cast<cudaStream_t>(cuda_stream));
}

int splash_bwd_static_scratch(const SplashBwdArgs* args, void* cuda_stream) {
  if (args == nullptr) return SPLASH_ERR_INVALID_ARGUMENT;
  return sb::launch_bwd_static_scratch(*args, static_cast<cudaStream_t>(cuda_stream));
}

int splash_read_error(const uint32_t* error_record, void* cuda_stream, uint32_t record_out[4]) {
  if (error_record == nullptr) return SPLASH_ERR_INVALID_ARGUMENT;
  uint32_t host[4] = {0, 0, 0, 0};
  cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
  if (cudaMemcpyAsync(host, error_record, sizeof(host), cudaMemcpyDeviceToHost, s) != cudaSuccess)
    return SPLASH_ERR_CUDA;
  if (cudaStreamSynchronize(s) != cudaSuccess) return SPLASH_ERR_CUDA;
  if (record_out != nullptr) std::memcpy(record_out, host, sizeof(host));
  return host[0] == 0 ? SPLASH_OK : SPLASH_ERR_KERNEL_TIMEOUT;
}

const char* splash_status_str(int status) {
  switch (status) {
    case SPLASH_OK: return "ok";
    case SPLASH_ERR_INVALID_ARGUMENT: return "invalid argument (shape, stride, alignment or table)";
    case SPLASH_ERR_UNSUPPORTED: return "unsupported configuration (NotImplementedError)";
    case SPLASH_ERR_CUDA: return "CUDA call failed";
    case SPLASH_ERR_NO_DEVICE: return "no usable sm_100 device or driver entry point";
    case SPLASH_ERR_KERNEL_TIMEOUT: return "device-side bounded wait ran out";
    case SPLASH_ERR_OUT_OF_MEMORY: return "host allocation failed";
    case SPLASH_ERR_TOO_LARGE:
      return "size beyond a built-in limit (grid dimension, or SPLASH_STATIC_SCRATCH_MAX_ROWS for the "
             "static-scratch backward)";
    default: return "unknown status";
  }
}

const char* splash_version(void) { return "splash_b200 0.1 sm_100a"; }

}  // extern "C"
