// Typed XLA FFI handlers for the WKV6 op (XLA_FFI_DEFINE_HANDLER_SYMBOL), on the C ABI of this library.
//
// They replace the three legacy custom calls of the reference (rwkv_kernel/jax_kernel/kernels.h:44-53,
// rwkv_kernels.cu:451-508; registered in gpu_ops.cpp:20-29 and lowered from jax_rwkv_kernel.py:75-111,202-217):
// shapes and dtypes come from the buffers, the head size is an attribute instead of a field of the opaque blob,
// failures come back as ffi::Error instead of an exception, and the checkpoint / scratch buffers the chunked
// kernels need are ordinary results.
//
//   wkv6_ffi_forward             (r, k, v, w, u)                     -> (y, ckpt)              attr head_size
//   wkv6_ffi_backward            (r, k, v, w, u, gy, ckpt)           -> (gr, gk, gv, gw, gu, ws)   attr head_size
//   wkv6_ffi_forward_with_state  (r, k, v, w, u, s, map)             -> (y, ys)                attr head_size, has_state
// r, k, v, w, gy, y, g*: [B, T, C];  u: [H, N];  gu: [B, H, N];  ckpt: [B, H, ceil(T/64), 4096] bf16 (any shape when the
// problem resolves to the sequential variant);  ws: bytes >= wkv6_backward_workspace_bytes;  s: [kinds, H, N, N],
// map: int64 [B], ys: [B, H, N, N] in the layout S[b][h][key][value].
//
// This file needs xla/ffi/api/ffi.h, which ships with jaxlib (jax.ffi.include_dir()).  The build compiles it only
// when that directory exists; without it the library exports the legacy handlers only.  It has not been compiled
// or run where this library was developed (no JAX there).
#include <cuda_runtime_api.h>

#include <cstdint>
#include <string>

#include "../../include/wkv6_b200.h"
#include "xla/ffi/api/ffi.h"

namespace ffi = xla::ffi;

namespace {

int dtype_code(ffi::DataType t) {
    switch (t) {
        case ffi::DataType::BF16: return WKV6_BF16;
        case ffi::DataType::F16: return WKV6_F16;
        case ffi::DataType::F32: return WKV6_F32;
        default: return -1;
    }
}

ffi::Error invalid(const std::string &msg) { return ffi::Error(ffi::ErrorCode::kInvalidArgument, msg); }

ffi::Error from_rc(int rc) {
    if (rc == WKV6_OK) return ffi::Error::Success();
    return ffi::Error(rc == WKV6_ERR_INVALID ? ffi::ErrorCode::kInvalidArgument : ffi::ErrorCode::kInternal,
                      std::string(wkv6_last_error()));
}

// Problem description from the buffers of one call.
ffi::Error describe(const ffi::AnyBuffer &r, const ffi::AnyBuffer &u, ffi::DataType y_type, int64_t head_size,
                    wkv6_problem *p) {
    auto dims = r.dimensions();
    if (dims.size() != 3) return invalid("r must be [B, T, C]");
    if (head_size <= 0 || dims[2] % head_size) return invalid("C is not a multiple of head_size");
    *p = wkv6_problem{};
    p->B = static_cast<int32_t>(dims[0]);
    p->T = static_cast<int32_t>(dims[1]);
    p->H = static_cast<int32_t>(dims[2] / head_size);
    p->N = static_cast<int32_t>(head_size);
    p->x_dtype = dtype_code(r.element_type());
    p->y_dtype = dtype_code(y_type);
    p->u_dtype = dtype_code(u.element_type());
    p->gu_dtype = p->y_dtype;
    p->s_dtype = p->y_dtype;
    p->variant = WKV6_VARIANT_AUTO;
    if (p->x_dtype < 0 || p->y_dtype < 0 || p->u_dtype < 0) return invalid("dtypes must be bf16, f16 or f32");
    if (static_cast<int64_t>(u.element_count()) != dims[2]) return invalid("u must hold H*N values");
    return ffi::Error::Success();
}

ffi::Error ForwardImpl(cudaStream_t stream, ffi::AnyBuffer r, ffi::AnyBuffer k, ffi::AnyBuffer v, ffi::AnyBuffer w,
                       ffi::AnyBuffer u, ffi::Result<ffi::AnyBuffer> y, ffi::Result<ffi::AnyBuffer> ckpt,
                       int64_t head_size) {
    wkv6_problem p;
    if (auto e = describe(r, u, y->element_type(), head_size, &p); e.failure()) return e;
    const size_t need = wkv6_ckpt_bytes(&p);
    if (need > ckpt->size_bytes()) return invalid("the checkpoint result is smaller than wkv6_ckpt_bytes");
    return from_rc(wkv6_forward(&p, r.untyped_data(), k.untyped_data(), v.untyped_data(), w.untyped_data(), u.untyped_data(),
                                y->untyped_data(), nullptr, nullptr, 0, nullptr, need ? ckpt->untyped_data() : nullptr,
                                stream));
}

ffi::Error BackwardImpl(cudaStream_t stream, ffi::AnyBuffer r, ffi::AnyBuffer k, ffi::AnyBuffer v, ffi::AnyBuffer w,
                        ffi::AnyBuffer u, ffi::AnyBuffer gy, ffi::AnyBuffer ckpt, ffi::Result<ffi::AnyBuffer> gr,
                        ffi::Result<ffi::AnyBuffer> gk, ffi::Result<ffi::AnyBuffer> gv, ffi::Result<ffi::AnyBuffer> gw,
                        ffi::Result<ffi::AnyBuffer> gu, ffi::Result<ffi::AnyBuffer> ws, int64_t head_size) {
    wkv6_problem p;
    if (auto e = describe(r, u, gy.element_type(), head_size, &p); e.failure()) return e;
    p.gu_dtype = dtype_code(gu->element_type());
    if (p.gu_dtype < 0) return invalid("gu must be bf16, f16 or f32");
    const bool have_ckpt = wkv6_ckpt_bytes(&p) != 0;
    if (have_ckpt && ckpt.size_bytes() < wkv6_ckpt_bytes(&p)) return invalid("the checkpoint operand is smaller than wkv6_ckpt_bytes");
    const size_t need = wkv6_backward_workspace_bytes(&p, have_ckpt ? 1 : 0);
    if (need > ws->size_bytes()) return invalid("the scratch result is smaller than wkv6_backward_workspace_bytes");
    return from_rc(wkv6_backward(&p, r.untyped_data(), k.untyped_data(), v.untyped_data(), w.untyped_data(), u.untyped_data(),
                                 gy.untyped_data(), gr->untyped_data(), gk->untyped_data(), gv->untyped_data(),
                                 gw->untyped_data(), gu->untyped_data(), have_ckpt ? ckpt.untyped_data() : nullptr,
                                 need ? ws->untyped_data() : nullptr, ws->size_bytes(), stream));
}

ffi::Error ForwardWithStateImpl(cudaStream_t stream, ffi::AnyBuffer r, ffi::AnyBuffer k, ffi::AnyBuffer v, ffi::AnyBuffer w,
                                ffi::AnyBuffer u, ffi::AnyBuffer s, ffi::AnyBuffer map, ffi::Result<ffi::AnyBuffer> y,
                                ffi::Result<ffi::AnyBuffer> ys, int64_t head_size, bool has_state) {
    wkv6_problem p;
    if (auto e = describe(r, u, y->element_type(), head_size, &p); e.failure()) return e;
    p.s_dtype = dtype_code(ys->element_type());
    if (p.s_dtype != WKV6_F32 && p.s_dtype != WKV6_BF16) return invalid("states must be f32 or bf16");
    const void *s_in = nullptr;
    const int64_t *s_map = nullptr;
    int32_t kinds = 0;
    if (has_state) {
        if (s.element_type() != ys->element_type()) return invalid("initial and returned states must share a dtype");
        if (map.element_type() != ffi::DataType::S64) return invalid("state_map must be int64 (enable jax_enable_x64)");
        if (s.dimensions().size() != 4 || static_cast<int64_t>(map.element_count()) != p.B) return invalid("bad state shapes");
        s_in = s.untyped_data();
        s_map = static_cast<const int64_t *>(map.untyped_data());
        kinds = static_cast<int32_t>(s.dimensions()[0]);
    }
    return from_rc(wkv6_forward(&p, r.untyped_data(), k.untyped_data(), v.untyped_data(), w.untyped_data(), u.untyped_data(),
                                y->untyped_data(), s_in, s_map, kinds, ys->untyped_data(), nullptr, stream));
}

}  // namespace

XLA_FFI_DEFINE_HANDLER_SYMBOL(wkv6_ffi_forward, ForwardImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()   // r
                                  .Arg<ffi::AnyBuffer>()   // k
                                  .Arg<ffi::AnyBuffer>()   // v
                                  .Arg<ffi::AnyBuffer>()   // w
                                  .Arg<ffi::AnyBuffer>()   // u
                                  .Ret<ffi::AnyBuffer>()   // y
                                  .Ret<ffi::AnyBuffer>()   // ckpt
                                  .Attr<int64_t>("head_size"));

XLA_FFI_DEFINE_HANDLER_SYMBOL(wkv6_ffi_backward, BackwardImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()   // r
                                  .Arg<ffi::AnyBuffer>()   // k
                                  .Arg<ffi::AnyBuffer>()   // v
                                  .Arg<ffi::AnyBuffer>()   // w
                                  .Arg<ffi::AnyBuffer>()   // u
                                  .Arg<ffi::AnyBuffer>()   // gy
                                  .Arg<ffi::AnyBuffer>()   // ckpt
                                  .Ret<ffi::AnyBuffer>()   // gr
                                  .Ret<ffi::AnyBuffer>()   // gk
                                  .Ret<ffi::AnyBuffer>()   // gv
                                  .Ret<ffi::AnyBuffer>()   // gw
                                  .Ret<ffi::AnyBuffer>()   // gu
                                  .Ret<ffi::AnyBuffer>()   // ws
                                  .Attr<int64_t>("head_size"));

XLA_FFI_DEFINE_HANDLER_SYMBOL(wkv6_ffi_forward_with_state, ForwardWithStateImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()   // r
                                  .Arg<ffi::AnyBuffer>()   // k
                                  .Arg<ffi::AnyBuffer>()   // v
                                  .Arg<ffi::AnyBuffer>()   // w
                                  .Arg<ffi::AnyBuffer>()   // u
                                  .Arg<ffi::AnyBuffer>()   // s
                                  .Arg<ffi::AnyBuffer>()   // map
                                  .Ret<ffi::AnyBuffer>()   // y
                                  .Ret<ffi::AnyBuffer>()   // ys
                                  .Attr<int64_t>("head_size")
                                  .Attr<bool>("has_state"));
