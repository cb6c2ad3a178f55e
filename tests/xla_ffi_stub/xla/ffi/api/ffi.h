// Minimal stand-in for XLA's "xla/ffi/api/ffi.h", for tests only: just enough of the API's shape
// (AnyBuffer, Buffer<dtype>, Result<>, Error, the Bind() builder and the handler macro) for
// tokamax_b200/csrc/splash_xla_ffi.cc to compile, and for a test to call a handler with fake
// buffers and look at what it passes to the C ABI.  It is NOT the real header: argument decoding,
// call frames and registration are absent.
#ifndef TESTS_XLA_FFI_STUB_H_
#define TESTS_XLA_FFI_STUB_H_
#include <cstddef>
#include <cstdint>
#include <string>
#include <tuple>
#include <utility>
#include <vector>

namespace xla {
namespace ffi {

enum DataType { S8, U8, S32, U32, F32, BF16, F8E4M3FN };
template <DataType> struct NativeType;
template <> struct NativeType<S8> { using type = int8_t; };
template <> struct NativeType<U8> { using type = uint8_t; };
template <> struct NativeType<S32> { using type = int32_t; };
template <> struct NativeType<U32> { using type = uint32_t; };
template <> struct NativeType<F32> { using type = float; };

struct Span {
  std::vector<int64_t> v;
  size_t size() const { return v.size(); }
  int64_t operator[](size_t i) const { return v[i]; }
};

class AnyBuffer {
 public:
  AnyBuffer() = default;
  AnyBuffer(void* data, DataType t, std::vector<int64_t> dims) : data_(data), type_(t), dims_{std::move(dims)} {}
  void* untyped_data() const { return data_; }
  DataType element_type() const { return type_; }
  const Span& dimensions() const { return dims_; }
  size_t element_count() const {
    size_t n = 1;
    for (int64_t d : dims_.v) n *= (size_t)d;
    return n;
  }

 private:
  void* data_ = nullptr;
  DataType type_ = BF16;
  Span dims_;
};

template <DataType T>
class Buffer : public AnyBuffer {
 public:
  Buffer() = default;
  Buffer(void* data, std::vector<int64_t> dims) : AnyBuffer(data, T, std::move(dims)) {}
  typename NativeType<T>::type* typed_data() const { return static_cast<typename NativeType<T>::type*>(untyped_data()); }
};

template <typename B>
class Result {
 public:
  Result() = default;
  explicit Result(B b) : b_(std::move(b)) {}
  B& operator*() { return b_; }
  B* operator->() { return &b_; }

 private:
  B b_;
};

enum class ErrorCode { kOk, kInvalidArgument, kUnimplemented, kOutOfRange, kInternal };
class Error {
 public:
  Error() = default;
  Error(ErrorCode c, std::string m) : code_(c), msg_(std::move(m)) {}
  static Error Success() { return Error(); }
  bool success() const { return code_ == ErrorCode::kOk; }
  ErrorCode code() const { return code_; }
  const std::string& message() const { return msg_; }

 private:
  ErrorCode code_ = ErrorCode::kOk;
  std::string msg_;
};

template <typename T> struct PlatformStream {};

// Builder that only records how many of each kind were bound and the attribute names.
struct Binding {
  int n_ctx = 0, n_args = 0, n_rets = 0;
  std::vector<std::string> attrs;
  template <typename T> Binding Ctx() { ++n_ctx; return *this; }
  template <typename T> Binding Arg() { ++n_args; return *this; }
  template <typename T> Binding Ret() { ++n_rets; return *this; }
  template <typename T> Binding Attr(const char* name) { attrs.emplace_back(name); return *this; }
};
struct Ffi {
  static Binding Bind() { return Binding(); }
};

}  // namespace ffi
}  // namespace xla

// The real macro defines an exported XLA_FFI_Handler; here it exports the binding description so
// a test can compare it with the handler's parameter list.
#define XLA_FFI_DEFINE_HANDLER_SYMBOL(name, impl, binding)                                  \
  extern "C" const ::xla::ffi::Binding* name##_binding() {                                  \
    static const ::xla::ffi::Binding b = (binding);                                         \
    return &b;                                                                               \
  }                                                                                          \
  extern "C" void* name##_impl_address() { return reinterpret_cast<void*>(&impl); }
#endif  // TESTS_XLA_FFI_STUB_H_
