// Test driver: includes the FFI adapter as part of this translation unit (built against the stub
// ffi.h next to this file), replaces the C ABI entry points with recorders, calls both handlers with
// fake buffers and checks what reached SplashFwdArgs / SplashBwdArgs.  Prints "OK" on success.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

int g_stub_memsets = 0;  // counted by the stand-in cuda_runtime.h next to this file

#include "../../tokamax_b200/csrc/splash_xla_ffi.cc"

static SplashFwdArgs g_fwd;
static SplashBwdArgs g_bwd;
static void* g_stream = nullptr;
static int g_ret = 0;
extern "C" int splash_fwd(const SplashFwdArgs* a, void* s) { g_fwd = *a; g_stream = s; return g_ret; }
extern "C" int splash_bwd(const SplashBwdArgs* a, void* s) { g_bwd = *a; g_stream = s; return g_ret; }
extern "C" const char* splash_status_str(int) { return "status text"; }

#define CHECK(c) do { if (!(c)) { std::printf("FAILED line %d: %s\n", __LINE__, #c); return 1; } } while (0)

int main() {
  namespace ffi = xla::ffi;
  const int64_t B = 2, H = 8, Hkv = 2, S = 256, D = 128;
  std::vector<char> mem(1 << 16);
  char* base = mem.data();
  auto buf = [&](int off, std::vector<int64_t> dims) { return ffi::AnyBuffer(base + off, ffi::BF16, dims); };
  auto s32 = [&](int off, std::vector<int64_t> dims) { return ffi::Buffer<ffi::S32>(base + off, dims); };
  auto f32 = [&](int off, std::vector<int64_t> dims) { return ffi::Buffer<ffi::F32>(base + off, dims); };
  ffi::Buffer<ffi::S8> no_pmb(nullptr, {0});
  ffi::Buffer<ffi::S32> none(nullptr, {0});
  ffi::Buffer<ffi::F32> nonef(nullptr, {0});
  uint32_t err[4] = {9, 9, 9, 9};
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(0x1234);

  // forward, Op layout [B, S, H, D]
  ffi::Error e = SplashFwdImpl(stream, buf(0, {B, S, H, D}), buf(64, {B, S, Hkv, D}), buf(128, {B, S, Hkv, D}),
                               none, none, none, s32(256, {3}), s32(320, {12}), s32(384, {2}), no_pmb, none, nonef, nonef,
                               ffi::Result<ffi::AnyBuffer>(buf(512, {B, S, H, D})),
                               ffi::Result<ffi::Buffer<ffi::F32>>(f32(576, {B, H, S})),
                               ffi::Result<ffi::Buffer<ffi::F32>>(f32(640, {B, H, S})),
                               ffi::Result<ffi::Buffer<ffi::U32>>(ffi::Buffer<ffi::U32>(err, {4})),
                               /*layout=*/1, /*scale=*/0.25f, /*mask_value=*/-1e30f, /*soft_cap=*/0.f, 128, 128, 0,
                               SPLASH_MASK_LOCAL, 1, 2, 3, 1, 0, 0);
  CHECK(e.success());
  CHECK(g_stream == (void*)stream && g_stub_memsets == 1 && err[0] == 0 && err[3] == 0);
  CHECK(g_fwd.q.data == base && g_fwd.q.size[0] == B && g_fwd.q.size[1] == H && g_fwd.q.size[2] == S && g_fwd.q.size[3] == D);
  CHECK(g_fwd.q.stride[3] == 1 && g_fwd.q.stride[1] == D && g_fwd.q.stride[2] == H * D && g_fwd.q.stride[0] == S * H * D);
  CHECK(g_fwd.k.size[1] == Hkv && g_fwd.k.stride[2] == Hkv * D && g_fwd.o.data == base + 512);
  CHECK(g_fwd.q_segment_ids == nullptr && g_fwd.q_sequence == nullptr && g_fwd.sinks == nullptr);
  CHECK(g_fwd.sched.row_ptr == (const int32_t*)(base + 256) && g_fwd.sched.n_rows == 2 && g_fwd.sched.n_entries == 3);
  CHECK(g_fwd.sched.row_order == (const int32_t*)(base + 384) && g_fwd.sched.partial_mask_blocks == nullptr);
  CHECK(g_fwd.mask_fn.kind == SPLASH_MASK_LOCAL && g_fwd.mask_fn.offset == 1 && g_fwd.mask_fn.left == 2 &&
        g_fwd.mask_fn.right == 3 && g_fwd.mask_fn.has_left == 1 && g_fwd.mask_fn.has_right == 0);
  CHECK(g_fwd.scale == 0.25f && g_fwd.error_record == err && g_fwd.logsumexp == (float*)(base + 576));

  // backward, splash layout [B, H, S, D]; unsupported status must map to kUnimplemented
  std::vector<uint8_t> ws(4096);
  g_ret = SPLASH_ERR_UNSUPPORTED;
  e = SplashBwdImpl(stream, buf(0, {B, H, S, D}), buf(64, {B, Hkv, S, D}), buf(128, {B, Hkv, S, D}), buf(512, {B, H, S, D}),
                    buf(700, {B, H, S, D}), f32(576, {B, H, S}), none, none, none,
                    s32(256, {3}), s32(320, {12}), s32(384, {2}), no_pmb, none,
                    s32(800, {3}), s32(864, {8}), s32(928, {2}), no_pmb, none,
                    ffi::Result<ffi::AnyBuffer>(buf(1024, {B, H, S, D})), ffi::Result<ffi::AnyBuffer>(buf(1088, {B, Hkv, S, D})),
                    ffi::Result<ffi::AnyBuffer>(buf(1152, {B, Hkv, S, D})),
                    ffi::Result<ffi::Buffer<ffi::U8>>(ffi::Buffer<ffi::U8>(ws.data(), {(int64_t)ws.size()})),
                    ffi::Result<ffi::Buffer<ffi::U32>>(ffi::Buffer<ffi::U32>(err, {4})),
                    /*layout=*/0, 0.5f, 0.f, /*flags=*/SPLASH_BWD_FUSED_DQ, 128, 128, 0, 0, SPLASH_MASK_CAUSAL, 0, 0, 0, 0, 0, 0);
  CHECK(!e.success() && e.code() == ffi::ErrorCode::kUnimplemented && e.message() == "status text");
  CHECK(g_bwd.q.stride[1] == S * D && g_bwd.q.stride[2] == D && g_bwd.d_o.data == base + 700);
  CHECK(g_bwd.dk.size[1] == Hkv && g_bwd.workspace == ws.data() && g_bwd.workspace_bytes == ws.size());
  CHECK(g_bwd.sched_dq.n_entries == 3 && g_bwd.sched_dkv.n_entries == 2 && g_bwd.sched_dkv.row_ptr == (const int32_t*)(base + 800));
  CHECK(g_bwd.flags == SPLASH_BWD_FUSED_DQ && g_bwd.launch_mask == 0 && g_bwd.mask_fn.kind == SPLASH_MASK_CAUSAL);
  CHECK(g_bwd.scale == 0.5f && g_bwd.logsumexp == (const float*)(base + 576));

  // the bindings list as many operands / results / attributes as the signature strings name
  auto count = [](const char* sig, const char* key) {
    const char* p = std::strstr(sig, key);
    int n = 0;
    for (p += std::strlen(key); *p != ';'; ++p) n += *p == ',';
    return n;
  };
  const xla::ffi::Binding* fb = SplashFwd_binding();
  const xla::ffi::Binding* bb = SplashBwd_binding();
  CHECK(fb->n_ctx == 1 && fb->n_args == count(splash_xla_ffi_signature(0), "operands=") &&
        fb->n_rets == count(splash_xla_ffi_signature(0), "results=") &&
        (int)fb->attrs.size() == count(splash_xla_ffi_signature(0), "attrs="));
  CHECK(bb->n_ctx == 1 && bb->n_args == count(splash_xla_ffi_signature(1), "operands=") &&
        bb->n_rets == count(splash_xla_ffi_signature(1), "results=") &&
        (int)bb->attrs.size() == count(splash_xla_ffi_signature(1), "attrs="));
  CHECK(fb->attrs[0] == "layout" && bb->attrs[3] == "flags");
  CHECK(splash_xla_ffi_compiled() == 1);
  std::printf("OK\n");
  return 0;
}
