// TEST STAND-IN, not XLA's header: the part of the `xla::ffi` surface that
// train_gpt_b200/xla_ffi/xla_ffi.cc uses, declared just far enough for `g++ -fsyntax-only` to
// type-check the handlers on a machine without jaxlib.  It checks the handlers against THIS
// reading of the API (buffer accessors, binding chain, handler macro), nothing more.
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>
#include <type_traits>

namespace xla::ffi {

enum DataType { BF16, F8E4M3FN, F32, S32, U8, U32 };
enum class ErrorCode { kOk, kInvalidArgument, kInternal };

class Error {
 public:
  Error() = default;
  Error(ErrorCode, std::string) {}
  static Error Success() { return Error(); }
};

template <typename T>
struct Span {
  const T* p = nullptr;
  size_t n = 0;
  size_t size() const { return n; }
  const T& operator[](size_t i) const { return p[i]; }
  const T& back() const { return p[n - 1]; }
};

template <DataType> struct NativeOf { using type = void; };
template <> struct NativeOf<F32> { using type = float; };
template <> struct NativeOf<S32> { using type = int32_t; };
template <> struct NativeOf<U8> { using type = uint8_t; };
template <> struct NativeOf<U32> { using type = uint32_t; };
template <> struct NativeOf<BF16> { using type = uint16_t; };
template <> struct NativeOf<F8E4M3FN> { using type = uint8_t; };

template <DataType D>
class Buffer {
 public:
  using Native = typename NativeOf<D>::type;
  Span<int64_t> dimensions() const { return {}; }
  size_t element_count() const { return 0; }
  void* untyped_data() const { return nullptr; }
  Native* typed_data() const { return nullptr; }
};

template <typename T>
class Result {
 public:
  T* operator->() { return &v_; }
  T& operator*() { return v_; }
 private:
  T v_;
};
template <DataType D> using ResultBuffer = Result<Buffer<D>>;

template <typename T> struct PlatformStream {};

template <typename... Ts>
struct Binding {
  template <typename T> constexpr Binding<Ts..., T> Ctx() const { return {}; }
  template <typename T> constexpr Binding<Ts..., T> Arg() const { return {}; }
  template <typename T> constexpr Binding<Ts..., Result<T>> Ret() const { return {}; }
  template <typename T> constexpr Binding<Ts..., T> Attr(const char*) const { return {}; }
};
struct Ffi {
  static constexpr Binding<> Bind() { return {}; }
};

// what a context / argument / result / attribute hands the implementation function
template <typename T> struct Decoded { using type = T; };
template <typename S> struct Decoded<PlatformStream<S>> { using type = S; };

template <typename... Ts, typename Fn>
constexpr bool Invocable(Binding<Ts...>, Fn fn) {
  return std::is_invocable_r_v<Error, Fn, typename Decoded<Ts>::type...>;
}

}  // namespace xla::ffi

// the real macro defines an exported XLA_FFI_Handler; the stand-in checks that the implementation
// can be called with what the binding decodes, and defines a symbol of the same name
#define XLA_FFI_DEFINE_HANDLER_SYMBOL(name, impl, binding)                                             \
  static_assert(::xla::ffi::Invocable(binding, impl), #impl " does not match its binding");           \
  extern "C" int name() { return 0; }
