// XLA custom-call (jax.ffi) adapter over the C ABI of include/splash_b200.h.
//
// The reference reaches its kernels from JAX through `pl.pallas_call`
// (tokamax/_src/ops/experimental/tpu/splash_attention/splash_attention_kernel.py:888, :1840); the
// counterpart for a CUDA library is an XLA FFI handler per entry point.  This translation unit is
// that adapter and nothing else: every handler copies buffers and attributes into SplashFwdArgs /
// SplashBwdArgs and calls splash_fwd / splash_bwd on the stream XLA hands it.
//
// It needs XLA's header-only FFI API ("xla/ffi/api/ffi.h", shipped with jaxlib under
// jaxlib/include).  Where that header is not on the include path the handlers are compiled out and
// only the two introspection functions at the bottom remain, so the library builds the same with
// or without XLA.  The operand / result / attribute order of each handler is spelled out ONCE, in
// the SPLASH_FFI_* lists below: the handler signatures, the binding builders and the strings the
// Python side reads back (splash_xla_ffi_signature) are all generated from them.
//
// Conventions of the handlers
//   * q / k / v / o / do / dq / dk / dv are dense row-major rank-4 buffers; attribute `layout`
//     says which: 0 = [batch, heads, seq, head_dim], 1 = [batch, seq, heads, head_dim] (the Op
//     layout of tokamax/_src/ops/attention/base.py:564-584, read in place through strides).
//   * An optional operand is passed as a buffer with zero elements and arrives as NULL.
//   * Schedules are the arrays of SplashDeviceSchedule (built on the host by
//     splash_schedule_build and passed as int32 operands).
//   * `error_record` is a u32[4] result; the handler clears it on the stream before the launch.
//     The caller reads it after the computation (word 0 != 0: a bounded device wait ran out).
//   * A non-zero SplashStatus becomes an ffi::Error (UNSUPPORTED -> kUnimplemented, so the
//     dispatcher of tokamax/_src/ops/attention/api.py:187-192 can fall through).
#include <cstdint>
#include <cstring>

#include "../../include/splash_b200.h"

// name lists: X(kind, C++ type, name)
#define SPLASH_FFI_FWD_OPERANDS(X)                                                                  \
  X(any, q) X(any, k) X(any, v) X(s32, q_segment_ids) X(s32, kv_segment_ids) X(s32, q_sequence)      \
  X(s32, sched_row_ptr) X(s32, sched_entries) X(s32, sched_row_order) X(s8, sched_partial_mask_blocks) \
  X(s32, sched_row_end) X(f32, sinks) X(f32, max_logit_value)
#define SPLASH_FFI_FWD_RESULTS(X) X(any, o) X(f32, logsumexp) X(f32, max_logits) X(u32, error_record)
#define SPLASH_FFI_FWD_ATTRS(X)                                                                      \
  X(int32_t, layout) X(float, scale) X(float, mask_value) X(float, soft_cap) X(int32_t, sched_block_q) \
  X(int32_t, sched_block_kv) X(int64_t, sched_entries_per_batch) X(int32_t, mask_kind)               \
  X(int32_t, mask_offset) X(int32_t, mask_left) X(int32_t, mask_right) X(int32_t, mask_has_left)     \
  X(int32_t, mask_has_right) X(int32_t, mask_chunk)

#define SPLASH_FFI_BWD_OPERANDS(X)                                                                  \
  X(any, q) X(any, k) X(any, v) X(any, o) X(any, d_o) X(f32, logsumexp) X(s32, q_segment_ids)        \
  X(s32, kv_segment_ids) X(s32, q_sequence)                                                          \
  X(s32, dq_row_ptr) X(s32, dq_entries) X(s32, dq_row_order) X(s8, dq_partial_mask_blocks) X(s32, dq_row_end) \
  X(s32, dkv_row_ptr) X(s32, dkv_entries) X(s32, dkv_row_order) X(s8, dkv_partial_mask_blocks) X(s32, dkv_row_end)
#define SPLASH_FFI_BWD_RESULTS(X) X(any, dq) X(any, dk) X(any, dv) X(u8, workspace) X(u32, error_record)
#define SPLASH_FFI_BWD_ATTRS(X)                                                                      \
  X(int32_t, layout) X(float, scale) X(float, soft_cap) X(int32_t, flags) X(int32_t, sched_block_q)   \
  X(int32_t, sched_block_kv) X(int64_t, dq_entries_per_batch) X(int64_t, dkv_entries_per_batch)       \
  X(int32_t, mask_kind) X(int32_t, mask_offset) X(int32_t, mask_left) X(int32_t, mask_right)          \
  X(int32_t, mask_has_left) X(int32_t, mask_has_right) X(int32_t, mask_chunk)

#if defined(__has_include)
#if __has_include("xla/ffi/api/ffi.h")
#define SPLASH_HAVE_XLA_FFI 1
#endif
#endif

#ifdef SPLASH_HAVE_XLA_FFI
#include <cuda_runtime.h>

#include "xla/ffi/api/ffi.h"

namespace {
namespace ffi = xla::ffi;

using any_arg = ffi::AnyBuffer;
using s32_arg = ffi::Buffer<ffi::S32>;
using s8_arg = ffi::Buffer<ffi::S8>;
using u8_arg = ffi::Buffer<ffi::U8>;
using u32_arg = ffi::Buffer<ffi::U32>;
using f32_arg = ffi::Buffer<ffi::F32>;

// Dense rank-4 XLA buffer -> (batch, heads, seq, head_dim) view with element strides.
bool View(const ffi::AnyBuffer& b, int32_t layout, SplashTensor* t) {
  auto d = b.dimensions();
  if (d.size() != 4) return false;
  t->data = b.untyped_data();
  t->dtype = b.element_type() == ffi::BF16 ? SPLASH_BF16 : (b.element_type() == ffi::F8E4M3FN ? SPLASH_F8E4M3 : -1);
  if (layout == 0) {  // [B, H, S, D]
    t->size[0] = d[0]; t->size[1] = d[1]; t->size[2] = d[2]; t->size[3] = d[3];
    t->stride[3] = 1; t->stride[2] = d[3]; t->stride[1] = d[2] * d[3]; t->stride[0] = d[1] * d[2] * d[3];
  } else {            // [B, S, H, D]
    t->size[0] = d[0]; t->size[1] = d[2]; t->size[2] = d[1]; t->size[3] = d[3];
    t->stride[3] = 1; t->stride[1] = d[3]; t->stride[2] = d[2] * d[3]; t->stride[0] = d[1] * d[2] * d[3];
  }
  return t->dtype >= 0;
}

template <typename B>
auto* OrNull(B& b) {
  return b.element_count() == 0 ? nullptr : b.typed_data();
}

SplashDeviceSchedule Schedule(s32_arg& row_ptr, s32_arg& entries, s32_arg& row_order, s8_arg& pmb, s32_arg& row_end,
                              int32_t block_q, int32_t block_kv, int64_t entries_per_batch) {
  SplashDeviceSchedule s;
  std::memset(&s, 0, sizeof(s));
  s.row_ptr = OrNull(row_ptr);
  s.entries = OrNull(entries);
  s.n_rows = row_ptr.element_count() > 0 ? (int32_t)row_ptr.element_count() - 1 : 0;
  s.partial_mask_blocks = OrNull(pmb);
  s.block_q = block_q;
  s.block_kv = block_kv;
  s.n_entries = (int64_t)entries.element_count() / 4;
  s.row_end = OrNull(row_end);
  s.entries_per_batch = entries_per_batch;
  s.row_order = OrNull(row_order);
  return s;
}

ffi::Error ToError(int st) {
  if (st == SPLASH_OK) return ffi::Error::Success();
  const ffi::ErrorCode code = st == SPLASH_ERR_UNSUPPORTED ? ffi::ErrorCode::kUnimplemented
                              : st == SPLASH_ERR_INVALID_ARGUMENT ? ffi::ErrorCode::kInvalidArgument
                              : st == SPLASH_ERR_TOO_LARGE ? ffi::ErrorCode::kOutOfRange
                                                           : ffi::ErrorCode::kInternal;
  return ffi::Error(code, splash_status_str(st));
}

// Each list element expands with a LEADING comma, after the stream parameter every handler has.
#define SPLASH_ARG_PARAM(kind, name) , kind##_arg name
#define SPLASH_RET_PARAM(kind, name) , ffi::Result<kind##_arg> name
#define SPLASH_ATTR_PARAM(type, name) , type name

ffi::Error SplashFwdImpl(cudaStream_t stream SPLASH_FFI_FWD_OPERANDS(SPLASH_ARG_PARAM)
                             SPLASH_FFI_FWD_RESULTS(SPLASH_RET_PARAM) SPLASH_FFI_FWD_ATTRS(SPLASH_ATTR_PARAM)) {
  SplashFwdArgs a;
  std::memset(&a, 0, sizeof(a));
  if (!View(q, layout, &a.q) || !View(k, layout, &a.k) || !View(v, layout, &a.v) || !View(*o, layout, &a.o))
    return ffi::Error(ffi::ErrorCode::kInvalidArgument, "q / k / v / o must be rank-4 bf16 (or e4m3) buffers");
  a.logsumexp = OrNull(*logsumexp);
  a.max_logits = OrNull(*max_logits);
  a.q_segment_ids = OrNull(q_segment_ids);
  a.kv_segment_ids = OrNull(kv_segment_ids);
  a.q_sequence = OrNull(q_sequence);
  a.sched = Schedule(sched_row_ptr, sched_entries, sched_row_order, sched_partial_mask_blocks, sched_row_end,
                     sched_block_q, sched_block_kv, sched_entries_per_batch);
  a.mask_fn.kind = mask_kind;
  a.mask_fn.offset = mask_offset;
  a.mask_fn.left = mask_left;
  a.mask_fn.right = mask_right;
  a.mask_fn.has_left = mask_has_left;
  a.mask_fn.has_right = mask_has_right;
  a.mask_fn.chunk = mask_chunk;
  a.scale = scale;
  a.mask_value = mask_value;
  a.error_record = error_record->typed_data();
  a.sinks = OrNull(sinks);
  a.max_logit_value = OrNull(max_logit_value);
  a.soft_cap = soft_cap;
  if (cudaMemsetAsync(a.error_record, 0, 4 * sizeof(uint32_t), stream) != cudaSuccess) return ToError(SPLASH_ERR_CUDA);
  return ToError(splash_fwd(&a, stream));
}

ffi::Error SplashBwdImpl(cudaStream_t stream SPLASH_FFI_BWD_OPERANDS(SPLASH_ARG_PARAM)
                             SPLASH_FFI_BWD_RESULTS(SPLASH_RET_PARAM) SPLASH_FFI_BWD_ATTRS(SPLASH_ATTR_PARAM)) {
  SplashBwdArgs a;
  std::memset(&a, 0, sizeof(a));
  if (!View(q, layout, &a.q) || !View(k, layout, &a.k) || !View(v, layout, &a.v) || !View(o, layout, &a.o) ||
      !View(d_o, layout, &a.d_o) || !View(*dq, layout, &a.dq) || !View(*dk, layout, &a.dk) || !View(*dv, layout, &a.dv))
    return ffi::Error(ffi::ErrorCode::kInvalidArgument, "q / k / v / o / do / dq / dk / dv must be rank-4 bf16 buffers");
  a.logsumexp = OrNull(logsumexp);
  a.q_segment_ids = OrNull(q_segment_ids);
  a.kv_segment_ids = OrNull(kv_segment_ids);
  a.q_sequence = OrNull(q_sequence);
  a.sched_dq = Schedule(dq_row_ptr, dq_entries, dq_row_order, dq_partial_mask_blocks, dq_row_end, sched_block_q,
                        sched_block_kv, dq_entries_per_batch);
  a.sched_dkv = Schedule(dkv_row_ptr, dkv_entries, dkv_row_order, dkv_partial_mask_blocks, dkv_row_end, sched_block_q,
                         sched_block_kv, dkv_entries_per_batch);
  a.mask_fn.kind = mask_kind;
  a.mask_fn.offset = mask_offset;
  a.mask_fn.left = mask_left;
  a.mask_fn.right = mask_right;
  a.mask_fn.has_left = mask_has_left;
  a.mask_fn.has_right = mask_has_right;
  a.mask_fn.chunk = mask_chunk;
  a.scale = scale;
  a.workspace = workspace->typed_data();  // XLA allocations are at least 256-byte aligned
  a.workspace_bytes = workspace->element_count();
  a.error_record = error_record->typed_data();
  a.launch_mask = 0;
  a.soft_cap = soft_cap;
  a.flags = (uint32_t)flags;
  if (cudaMemsetAsync(a.error_record, 0, 4 * sizeof(uint32_t), stream) != cudaSuccess) return ToError(SPLASH_ERR_CUDA);
  return ToError(splash_bwd(&a, stream));
}

#define SPLASH_BIND_ARG(kind, name) .Arg<kind##_arg>()
#define SPLASH_BIND_RET(kind, name) .Ret<kind##_arg>()
#define SPLASH_BIND_ATTR(type, name) .Attr<type>(#name)

}  // namespace

// Registered from Python with jax.ffi.register_ffi_target("splash_b200_fwd" / "splash_b200_bwd",
// jax.ffi.pycapsule(lib.SplashFwd / lib.SplashBwd), platform="CUDA").
XLA_FFI_DEFINE_HANDLER_SYMBOL(SplashFwd, SplashFwdImpl,
                              ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>() SPLASH_FFI_FWD_OPERANDS(
                                  SPLASH_BIND_ARG) SPLASH_FFI_FWD_RESULTS(SPLASH_BIND_RET) SPLASH_FFI_FWD_ATTRS(SPLASH_BIND_ATTR));
XLA_FFI_DEFINE_HANDLER_SYMBOL(SplashBwd, SplashBwdImpl,
                              ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>() SPLASH_FFI_BWD_OPERANDS(
                                  SPLASH_BIND_ARG) SPLASH_FFI_BWD_RESULTS(SPLASH_BIND_RET) SPLASH_FFI_BWD_ATTRS(SPLASH_BIND_ATTR));
#endif  // SPLASH_HAVE_XLA_FFI

// ------------------------------------------------------------------------------------------
// introspection (always built)
// ------------------------------------------------------------------------------------------
#define SPLASH_NAME_KIND(kind, name) #name ":" #kind ","
extern "C" {

// 1 if this library was built with the XLA FFI handlers (SplashFwd / SplashBwd exported), else 0.
int splash_xla_ffi_compiled(void) {
#ifdef SPLASH_HAVE_XLA_FFI
  return 1;
#else
  return 0;
#endif
}

// The handlers' operand / result / attribute lists, in binding order, as
// "operands=name:kind,...;results=...;attrs=name:type,...;" — which: 0 forward, 1 backward.
// The Python side builds its jax.ffi.ffi_call argument lists from the same names.
const char* splash_xla_ffi_signature(int which) {
  if (which == 0)
    return "operands=" SPLASH_FFI_FWD_OPERANDS(SPLASH_NAME_KIND) ";results=" SPLASH_FFI_FWD_RESULTS(SPLASH_NAME_KIND)
           ";attrs=" SPLASH_FFI_FWD_ATTRS(SPLASH_NAME_KIND) ";";
  if (which == 1)
    return "operands=" SPLASH_FFI_BWD_OPERANDS(SPLASH_NAME_KIND) ";results=" SPLASH_FFI_BWD_RESULTS(SPLASH_NAME_KIND)
           ";attrs=" SPLASH_FFI_BWD_ATTRS(SPLASH_NAME_KIND) ";";
  return "";
}

}  // extern "C"
