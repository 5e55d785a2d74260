// Compile-only stand-in for jaxlib's xla/ffi/api/ffi.h, for tests/test_xla_ffi_source.py.
//
// It declares just the names csrc/wkv6_xla_ffi.cc uses, with the shapes that file assumes, so that the handlers can be
// type-checked (against this library's C ABI above all: argument counts and types of wkv6_forward / wkv6_backward) where
// JAX is not installed.  It is not the real header and proves nothing about it; nothing here is ever linked or run.
#pragma once

#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

namespace xla {
namespace ffi {

enum class DataType { INVALID, PRED, S8, S16, S32, S64, U8, U16, U32, U64, F16, F32, F64, BF16 };
enum class ErrorCode { kOk, kInvalidArgument, kInternal };

class Error {
 public:
    Error() = default;
    Error(ErrorCode code, std::string message) : code_(code), message_(std::move(message)) {}
    static Error Success() { return Error(); }
    bool failure() const { return code_ != ErrorCode::kOk; }
    bool success() const { return code_ == ErrorCode::kOk; }

 private:
    ErrorCode code_ = ErrorCode::kOk;
    std::string message_;
};

template <typename T>
struct Span {
    const T *ptr = nullptr;
    size_t n = 0;
    size_t size() const { return n; }
    const T &operator[](size_t i) const { return ptr[i]; }
};

class AnyBuffer {
 public:
    Span<int64_t> dimensions() const { return {}; }
    DataType element_type() const { return DataType::INVALID; }
    void *untyped_data() const { return nullptr; }
    size_t size_bytes() const { return 0; }
    size_t element_count() const { return 0; }
};

template <typename T>
class Result {
 public:
    T *operator->() { return &value_; }
    const T *operator->() const { return &value_; }

 private:
    T value_;
};

template <typename T>
struct PlatformStream {};

template <typename... Ts>
class Binding {
 public:
    template <typename T> Binding<Ts..., T> Ctx() const { return {}; }
    template <typename T> Binding<Ts..., T> Arg() const { return {}; }
    template <typename T> Binding<Ts..., T> Ret() const { return {}; }
    template <typename T> Binding<Ts..., T> Attr(const char *) const { return {}; }
};

struct Ffi {
    static Binding<> Bind() { return {}; }
};

}  // namespace ffi
}  // namespace xla

// The real macro defines an extern "C" symbol that decodes a call frame and invokes `impl`; here it only forces the
// implementation to be odr-used with the binding, so that the compiler checks it exists.
#define XLA_FFI_DEFINE_HANDLER_SYMBOL(name, impl, binding)                    \
    extern "C" const void *name() {                                           \
        (void)(binding);                                                      \
        return reinterpret_cast<const void *>(&impl);                         \
    }
