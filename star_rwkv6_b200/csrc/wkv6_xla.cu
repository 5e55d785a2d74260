// XLA legacy custom-call entry points with the reference's symbol names, buffer orders and 28-byte descriptor
// (rwkv_kernel/jax_kernel/kernels.h:30-53, rwkv_kernels.cu:451-508), implemented on the C ABI of this library.
//   wkv_forward             buffers = [r, k, v, w, u, y]
//   wkv_backward            buffers = [r, k, v, w, u, gy, gr, gk, gv, gw, gu]        gu is [B, C] in the output dtype
//   wkv_forward_with_state  S = 1:   [map, r, k, v, w, u, s, y, ys]      S = 0: [r, k, v, w, u, y, ys]
// XLA owns every buffer and this ABI has no workspace and no status channel.  A lowering that keeps the reference's
// eleven backward buffers therefore gets the sequential variant (dense fp32: no scratch at all; otherwise the
// library's built-in scratch, one slice of batch rows / heads after the other when the problem is larger than that
// array).  A lowering that can declare two more buffers reaches the chunked tensor-core kernels:
//   wkv_forward_ckpt        buffers = [r, k, v, w, u, y, ckpt]        ckpt: extra result, kept as a residual of the vjp
//   wkv_backward_ws         buffers = [r, k, v, w, u, gy, ckpt, gr, gk, gv, gw, gu, ws]   ws: extra result (scratch)
// with ckpt = [B, H, ceil(T/64), 4096] bf16 and ws = [B, H, 64] int32 (dummies of any size when the problem resolves to
// the sequential variant, whose scratch then also lives in ws: [B, T, C] fp32).  Failures are reported the way the
// reference reports a bad descriptor, by throwing std::runtime_error.  The extern "C" twins return the error code
// instead.  States are S[b][h][key][value].
#include <cstring>
#include <stdexcept>

#include "wkv6_internal.h"

namespace gpu_ops {

enum ElementType { BF16, F16, F32 };

struct WKVDescriptor {
    int B;
    int T;
    int C;
    int H;
    bool S;
    ElementType x_type;
    ElementType y_type;
};
static_assert(sizeof(WKVDescriptor) == 28, "descriptor layout must match the reference's");

static int unpack(const char *opaque, std::size_t len, WKVDescriptor *d, wkv6_problem *p) {
    if (opaque == nullptr || len != sizeof(WKVDescriptor)) return wkv6::fail(WKV6_ERR_INVALID, "Invalid opaque object size");
    std::memcpy(d, opaque, sizeof(WKVDescriptor));
    if (d->H <= 0 || d->C % d->H) return wkv6::fail(WKV6_ERR_INVALID, "C=%d is not a multiple of H=%d", d->C, d->H);
    std::memset(p, 0, sizeof(*p));
    p->B = d->B; p->T = d->T; p->H = d->H; p->N = d->C / d->H;
    p->x_dtype = d->x_type; p->y_dtype = d->y_type;
    p->u_dtype = d->x_type; p->gu_dtype = d->y_type; p->s_dtype = d->y_type;
    p->variant = WKV6_VARIANT_AUTO;
    return WKV6_OK;
}

static int forward_impl(cudaStream_t st, void **b, const char *opaque, std::size_t len) {
    WKVDescriptor d; wkv6_problem p;
    if (int rc = unpack(opaque, len, &d, &p)) return rc;
    return wkv6_forward(&p, b[0], b[1], b[2], b[3], b[4], b[5], nullptr, nullptr, 0, nullptr, nullptr, st);
}

static int forward_state_impl(cudaStream_t st, void **b, const char *opaque, std::size_t len) {
    WKVDescriptor d; wkv6_problem p;
    if (int rc = unpack(opaque, len, &d, &p)) return rc;
    if (d.S)  // the descriptor does not carry the number of initial states: at most B, selected by the map
        return wkv6_forward(&p, b[1], b[2], b[3], b[4], b[5], b[7], b[6], static_cast<const int64_t *>(b[0]), d.B, b[8],
                            nullptr, st);
    return wkv6_forward(&p, b[0], b[1], b[2], b[3], b[4], b[5], nullptr, nullptr, 0, b[6], nullptr, st);
}

static inline const void *at(const void *base, size_t elems, int dtype) {
    return static_cast<const char *>(base) + elems * wkv6::dtype_size(dtype);
}
static inline void *at(void *base, size_t elems, int dtype) {
    return static_cast<char *>(base) + elems * wkv6::dtype_size(dtype);
}

// Eleven buffers, no scratch from the caller: the sequential backward on the library's built-in array.  A problem
// larger than the array is cut into slices that fit - whole batch rows, or head groups of one row - and the slices
// run one after the other on the stream (which also keeps the shared array free of overlapping users).  What
// remains out of reach is a single head of a single row beyond the array: T * N * 4 bytes > 32 MiB.
static int backward_impl(cudaStream_t st, void **b, const char *opaque, std::size_t len) {
    WKVDescriptor d; wkv6_problem p;
    if (int rc = unpack(opaque, len, &d, &p)) return rc;
    p.variant = WKV6_VARIANT_SEQ;
    if (wkv6_backward_workspace_bytes(&p, 0) == 0)
        return wkv6_backward(&p, b[0], b[1], b[2], b[3], b[4], b[5], b[6], b[7], b[8], b[9], b[10], nullptr, nullptr, 0, st);
    const size_t cap = wkv6_static_scratch_bytes() / sizeof(float);  // (token, channel) pairs per call
    const size_t row = (size_t)p.T * d.C;
    if ((size_t)p.B * row <= cap)
        return wkv6_backward_static_scratch(&p, b[0], b[1], b[2], b[3], b[4], b[5], b[6], b[7], b[8], b[9], b[10], st);
    if (p.B == 0 || p.T == 0) return WKV6_OK;
    const int N = p.N, H = p.H, C = d.C;
    int rows_per = (int)(cap / row), heads_per = H;
    if (rows_per == 0) {
        rows_per = 1;
        heads_per = (int)(cap / ((size_t)p.T * N));
        if (heads_per == 0)
            return wkv6::fail(WKV6_ERR_WORKSPACE, "one head of one row (T=%d, N=%d) needs %zu bytes of scratch, beyond the built-in %zu: "
                              "lower to wkv_backward_ws, which takes its scratch as a buffer", p.T, N, (size_t)p.T * N * 4,
                              wkv6_static_scratch_bytes());
    }
    for (int b0 = 0; b0 < p.B; b0 += rows_per) {
        for (int h0 = 0; h0 < H; h0 += heads_per) {
            wkv6_problem q = p;
            q.B = (b0 + rows_per <= p.B) ? rows_per : p.B - b0;
            q.H = (h0 + heads_per <= H) ? heads_per : H - h0;
            q.row_stride = C;
            q.batch_stride = (int64_t)p.T * C;
            const size_t off = (size_t)b0 * row + (size_t)h0 * N;          // first element of the slice in a [B,T,C] tensor
            const size_t goff = (size_t)b0 * C + (size_t)h0 * N;           // ... and in gu [B,C] (heads are cut only when q.B == 1)
            int rc = wkv6_backward_static_scratch(&q, at((const void *)b[0], off, p.x_dtype), at((const void *)b[1], off, p.x_dtype),
                                                  at((const void *)b[2], off, p.x_dtype), at((const void *)b[3], off, p.x_dtype),
                                                  at((const void *)b[4], (size_t)h0 * N, p.u_dtype), at((const void *)b[5], off, p.y_dtype),
                                                  at(b[6], off, p.y_dtype), at(b[7], off, p.y_dtype), at(b[8], off, p.y_dtype),
                                                  at(b[9], off, p.y_dtype), at(b[10], goff, p.gu_dtype), st);
            if (rc) return rc;
        }
    }
    return WKV6_OK;
}

// The extended forms: the lowering declares the checkpoint buffer as an extra result of the forward and hands it,
// with a scratch result, to the backward; both then run whatever variant AUTO resolves to (the chunked kernels for
// bf16 and head size 64).
static int forward_ckpt_impl(cudaStream_t st, void **b, const char *opaque, std::size_t len) {
    WKVDescriptor d; wkv6_problem p;
    if (int rc = unpack(opaque, len, &d, &p)) return rc;
    void *ckpt = wkv6_ckpt_bytes(&p) ? b[6] : nullptr;
    return wkv6_forward(&p, b[0], b[1], b[2], b[3], b[4], b[5], nullptr, nullptr, 0, nullptr, ckpt, st);
}

static int backward_ws_impl(cudaStream_t st, void **b, const char *opaque, std::size_t len) {
    WKVDescriptor d; wkv6_problem p;
    if (int rc = unpack(opaque, len, &d, &p)) return rc;
    const bool have_ckpt = wkv6_ckpt_bytes(&p) != 0;
    const size_t ws_bytes = wkv6_backward_workspace_bytes(&p, have_ckpt ? 1 : 0);  // the lowering sized b[12] with wkv6_xla_buffer_bytes
    return wkv6_backward(&p, b[0], b[1], b[2], b[3], b[4], b[5], b[7], b[8], b[9], b[10], b[11], have_ckpt ? b[6] : nullptr,
                         ws_bytes ? b[12] : nullptr, ws_bytes, st);
}

static void raise_on(int rc) {
    if (rc != WKV6_OK) throw std::runtime_error(wkv6_last_error());
}

__attribute__((visibility("default")))
void rwkv_forward_fn(cudaStream_t stream, void **buffers, const char *opaque, std::size_t opaque_len) {
    raise_on(forward_impl(stream, buffers, opaque, opaque_len));
}
__attribute__((visibility("default")))
void rwkv_backward_fn(cudaStream_t stream, void **buffers, const char *opaque, std::size_t opaque_len) {
    raise_on(backward_impl(stream, buffers, opaque, opaque_len));
}
__attribute__((visibility("default")))
void rwkv_forward_with_state_fn(cudaStream_t stream, void **buffers, const char *opaque, std::size_t opaque_len) {
    raise_on(forward_state_impl(stream, buffers, opaque, opaque_len));
}

__attribute__((visibility("default")))
void rwkv_forward_ckpt_fn(cudaStream_t stream, void **buffers, const char *opaque, std::size_t opaque_len) {
    raise_on(forward_ckpt_impl(stream, buffers, opaque, opaque_len));
}
__attribute__((visibility("default")))
void rwkv_backward_ws_fn(cudaStream_t stream, void **buffers, const char *opaque, std::size_t opaque_len) {
    raise_on(backward_ws_impl(stream, buffers, opaque, opaque_len));
}

}  // namespace gpu_ops

extern "C" {

WKV6_API int wkv6_xla_forward_ckpt(void *stream, void **buffers, const char *opaque, size_t opaque_len) {
    return gpu_ops::forward_ckpt_impl(static_cast<cudaStream_t>(stream), buffers, opaque, opaque_len);
}
WKV6_API int wkv6_xla_backward_ws(void *stream, void **buffers, const char *opaque, size_t opaque_len) {
    return gpu_ops::backward_ws_impl(static_cast<cudaStream_t>(stream), buffers, opaque, opaque_len);
}
// Bytes the extended lowerings must give the two extra buffers (which = 0: ckpt result of wkv_forward_ckpt,
// 1: ws result of wkv_backward_ws) for the problem a descriptor describes; never 0, so that no zero-sized buffer
// has to be declared.
WKV6_API size_t wkv6_xla_buffer_bytes(const char *opaque, size_t opaque_len, int which) {
    gpu_ops::WKVDescriptor d; wkv6_problem p;
    if (gpu_ops::unpack(opaque, opaque_len, &d, &p)) return 0;
    const size_t ck = wkv6_ckpt_bytes(&p);
    const size_t n = which == 0 ? ck : wkv6_backward_workspace_bytes(&p, ck ? 1 : 0);
    return n < 16 ? 16 : n;
}

WKV6_API int wkv6_xla_forward(void *stream, void **buffers, const char *opaque, size_t opaque_len) {
    return gpu_ops::forward_impl(static_cast<cudaStream_t>(stream), buffers, opaque, opaque_len);
}
WKV6_API int wkv6_xla_backward(void *stream, void **buffers, const char *opaque, size_t opaque_len) {
    return gpu_ops::backward_impl(static_cast<cudaStream_t>(stream), buffers, opaque, opaque_len);
}
WKV6_API int wkv6_xla_forward_with_state(void *stream, void **buffers, const char *opaque, size_t opaque_len) {
    return gpu_ops::forward_state_impl(static_cast<cudaStream_t>(stream), buffers, opaque, opaque_len);
}
WKV6_API int wkv6_xla_descriptor(int B, int T, int C, int H, int S, int x_type, int y_type, char *out, size_t out_len) {
    if (out == nullptr || out_len < sizeof(gpu_ops::WKVDescriptor)) return wkv6::fail(WKV6_ERR_INVALID, "descriptor buffer too small");
    gpu_ops::WKVDescriptor d;
    std::memset(&d, 0, sizeof(d));
    d.B = B; d.T = T; d.C = C; d.H = H; d.S = S != 0;
    d.x_type = static_cast<gpu_ops::ElementType>(x_type);
    d.y_type = static_cast<gpu_ops::ElementType>(y_type);
    std::memcpy(out, &d, sizeof(d));
    return (int)sizeof(d);
}
// Addresses of the C++ handlers, for wrapping in "xla._CUSTOM_CALL_TARGET" capsules.
WKV6_API void *wkv6_xla_target(int which) {
    switch (which) {
        case 0: return reinterpret_cast<void *>(&gpu_ops::rwkv_forward_fn);
        case 1: return reinterpret_cast<void *>(&gpu_ops::rwkv_backward_fn);
        case 2: return reinterpret_cast<void *>(&gpu_ops::rwkv_forward_with_state_fn);
        case 3: return reinterpret_cast<void *>(&gpu_ops::rwkv_forward_ckpt_fn);
        case 4: return reinterpret_cast<void *>(&gpu_ops::rwkv_backward_ws_fn);
        default: return nullptr;
    }
}

}  // extern "C"
