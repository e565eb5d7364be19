// Test double of the parts of jaxlib's `xla/ffi/api/ffi.h` that tokamax_b200/csrc/xla_ffi_shim.cc
// uses: just enough declarations for a compiler to type-check the shim (buffer accessors, the
// error type, the binding builder and the handler macro).  It defines no behaviour and is not
// part of the product; the real header comes with jaxlib (`jax.ffi.include_dir()`).
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>

namespace xla {
namespace ffi {

enum class DataType { BF16, F16, F32, F8E4M3FN, S8, S32 };
enum class ErrorCode { kInvalidArgument, kUnimplemented, kInternal };

struct Dims {
  const int64_t* data_;
  size_t size_;
  size_t size() const { return size_; }
  int64_t operator[](size_t i) const { return data_[i]; }
};

class AnyBuffer {
 public:
  Dims dimensions() const;
  void* untyped_data() const;
  DataType element_type() const;
  size_t size_bytes() const;
  size_t element_count() const;
};

template <DataType T> struct NativeOf { using type = void; };
template <> struct NativeOf<DataType::S32> { using type = int32_t; };
template <> struct NativeOf<DataType::F32> { using type = float; };

template <DataType T>
class Buffer {
 public:
  Dims dimensions() const;
  typename NativeOf<T>::type* typed_data() const;
  size_t element_count() const;
};

template <typename T>
class Result {
 public:
  T* operator->() const;
  T& operator*() const;
};

class Error {
 public:
  Error(ErrorCode, std::string);
  static Error Success();
  static Error InvalidArgument(std::string);
  static Error Internal(std::string);
};

template <typename T> struct PlatformStream {};

struct Binding {
  template <typename T> Binding Ctx() const { return *this; }
  template <typename T> Binding Arg() const { return *this; }
  template <typename T> Binding Ret() const { return *this; }
  template <typename T> Binding Attr(const char*) const { return *this; }
};
struct Ffi {
  static Binding Bind() { return Binding(); }
};

}  // namespace ffi
}  // namespace xla

#define XLA_FFI_DEFINE_HANDLER_SYMBOL(sym, impl, binding) \
  [[maybe_unused]] static auto sym##_binding = (binding);                  \
  void* sym = reinterpret_cast<void*>(&impl)
