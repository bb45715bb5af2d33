// STAND-IN for jaxlib's xla/ffi/api/ffi.h, for compile checks only (tests/test_ffi_compile.py).
//
// jaxlib is not installable where this repository is built, so its headers are not available.  This file declares the
// small part of the XLA FFI C++ binding API that lewi_surge_b200/csrc/ffi_xla.cc uses, with the argument-passing rules
// of the real header (Ctx<PlatformStream<S>> passes S; Arg<T> passes T; Ret<T> passes Result<T>; Attr<T> passes T), so
// that the handlers' signatures are type-checked against their bindings and against include/lewi_moe.h.  It is not an
// implementation of the FFI and nothing built from it is ever loaded.
#pragma once

#include <cstddef>
#include <cstdint>
#include <string>
#include <type_traits>

namespace xla {
namespace ffi {

enum class DataType { PRED, S8, S16, S32, S64, U8, U16, U32, U64, F16, F32, F64, BF16 };
constexpr DataType S32 = DataType::S32;
constexpr DataType U8 = DataType::U8;
constexpr DataType F32 = DataType::F32;
constexpr DataType BF16 = DataType::BF16;

enum class ErrorCode { kOk, kInvalidArgument, kInternal };

class Error {
 public:
  Error() = default;
  Error(ErrorCode, std::string) {}
  static Error Success() { return Error(); }
};

template <typename T>
class Span {
 public:
  const T& operator[](size_t i) const { return data_[i]; }
  size_t size() const { return size_; }
  const T* data_ = nullptr;
  size_t size_ = 0;
};

template <DataType> struct NativeOf { using type = void; };
template <> struct NativeOf<DataType::S32> { using type = int32_t; };
template <> struct NativeOf<DataType::U8> { using type = uint8_t; };
template <> struct NativeOf<DataType::F32> { using type = float; };
template <> struct NativeOf<DataType::BF16> { using type = uint16_t; };

class AnyBuffer {
 public:
  void* untyped_data() const { return nullptr; }
  DataType element_type() const { return DataType::F32; }
  Span<int64_t> dimensions() const { return {}; }
  size_t element_count() const { return 0; }
  size_t size_bytes() const { return 0; }
};

template <DataType dt>
class Buffer {
 public:
  using T = typename NativeOf<dt>::type;
  T* typed_data() const { return nullptr; }
  void* untyped_data() const { return nullptr; }
  Span<int64_t> dimensions() const { return {}; }
  size_t element_count() const { return 0; }
  size_t size_bytes() const { return 0; }
};

template <typename T>
class Result {
 public:
  T* operator->() { return &value_; }
  T& operator*() { return value_; }
  T value_;
};
template <DataType dt>
using ResultBuffer = Result<Buffer<dt>>;

template <typename S>
struct PlatformStream {};

template <typename... Passed>
struct Binding {
  template <typename C>
  struct CtxOf { using type = C; };
  template <typename S>
  struct CtxOf<PlatformStream<S>> { using type = S; };
  template <typename C>
  Binding<Passed..., typename CtxOf<C>::type> Ctx() const { return {}; }
  template <typename T>
  Binding<Passed..., T> Arg() const { return {}; }
  template <typename T>
  Binding<Passed..., Result<T>> Ret() const { return {}; }
  template <typename T>
  Binding<Passed..., T> Attr(const char*) const { return {}; }
  template <typename Fn>
  static constexpr bool Accepts() { return std::is_invocable_r_v<Error, Fn, Passed...>; }
};

struct Ffi {
  static Binding<> Bind() { return {}; }
};

}  // namespace ffi
}  // namespace xla

// The real macro defines an exported XLA_FFI_Handler; here it checks that `fn` takes exactly what the binding passes.
#define XLA_FFI_DEFINE_HANDLER_SYMBOL(name, fn, binding)                                                       \
  static_assert(decltype(binding)::template Accepts<decltype(&fn)>(), #name ": handler signature != binding"); \
  extern "C" const void* const name = nullptr
