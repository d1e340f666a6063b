// Declarations-only stand-in for jaxlib's xla/ffi/api/ffi.h, just enough of the public
// API for a syntax and type check of ffi/bsx_ffi.cc on a machine without jaxlib.  It
// defines nothing that runs; a real build uses the header jaxlib ships.
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>

#include <cuda_runtime_api.h>

namespace xla::ffi {

enum class DataType { INVALID, PRED, S8, S16, S32, S64, U8, U16, U32, U64, F16, F32, F64, BF16 };
inline constexpr DataType PRED = DataType::PRED, S32 = DataType::S32, S64 = DataType::S64, U8 = DataType::U8,
                          U32 = DataType::U32, F32 = DataType::F32;

template <typename T>
struct Span {
  const T* ptr;
  size_t n;
  size_t size() const { return n; }
  const T& operator[](size_t i) const { return ptr[i]; }
};

class Error {
 public:
  static Error Success();
  static Error Internal(std::string message);
  static Error InvalidArgument(std::string message);
};

class AnyBuffer {
 public:
  DataType element_type() const;
  Span<int64_t> dimensions() const;
  size_t element_count() const;
  size_t size_bytes() const;
  void* untyped_data() const;
};

template <DataType dtype>
class Buffer {
 public:
  Span<int64_t> dimensions() const;
  size_t element_count() const;
  float* typed_data() const;
  void* untyped_data() const;
};

template <typename T>
class Result {
 public:
  T* operator->();
  T& operator*();
};

template <typename T>
struct PlatformStream {};

template <typename... Ts>
struct Binding {
  template <typename T>
  Binding<Ts..., T> Ctx() &&;
  template <typename T>
  Binding<Ts..., T> Arg() &&;
  template <typename T>
  Binding<Ts..., Result<T>> Ret() &&;
  template <typename T>
  Binding<Ts..., T> Attr(const char* name) &&;
};

struct Ffi {
  static Binding<> Bind();
};

// What the real macro checks at compile time: the implementation is callable with the
// decoded operand types of the binding.
template <typename T>
struct Decoded { using type = T; };
template <typename T>
struct Decoded<PlatformStream<T>> { using type = T; };

template <typename Fn, typename... Ts>
constexpr bool CallableWith(Fn*, Binding<Ts...>*) {
  return std::is_invocable_r_v<Error, Fn, typename Decoded<Ts>::type...>;
}

}  // namespace xla::ffi

#include <type_traits>
#define XLA_FFI_DEFINE_HANDLER_SYMBOL(name, impl, binding)                                                  \
  static_assert(::xla::ffi::CallableWith(&impl, static_cast<decltype(binding)*>(nullptr)),                  \
                "handler signature does not match its binding");                                            \
  extern "C" void* name(void* call_frame) { return call_frame; }
