// XLA legacy custom-call entry points with the reference's symbol names, buffer orders and 28-byte descriptor
// (rwkv_kernel/jax_kernel/kernels.h:30-53, rwkv_kernels.cu:451-508), implemented on the C ABI of this library.
//   wkv_forward             buffers = [r, k, v, w, u, y]
//   wkv_backward            buffers = [r, k, v, w, u, gy, gr, gk, gv, gw, gu]        gu is [B, C] in the output dtype
//   wkv_forward_with_state  S = 1:   [map, r, k, v, w, u, s, y, ys]      S = 0: [r, k, v, w, u, y, ys]
// XLA owns every buffer and this ABI has no workspace and no status channel: the backward therefore uses the
// sequential variant (dense fp32: no scratch at all; otherwise the library's built-in scratch), and failures are
// reported the way the reference reports a bad descriptor, by throwing std::runtime_error.  The extern "C"
// twins return the error code instead.  States are S[b][h][key][value].
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

static int backward_impl(cudaStream_t st, void **b, const char *opaque, std::size_t len) {
    WKVDescriptor d; wkv6_problem p;
    if (int rc = unpack(opaque, len, &d, &p)) return rc;
    p.variant = WKV6_VARIANT_SEQ;
    if (wkv6_backward_workspace_bytes(&p, 0) == 0)
        return wkv6_backward(&p, b[0], b[1], b[2], b[3], b[4], b[5], b[6], b[7], b[8], b[9], b[10], nullptr, nullptr, 0, st);
    return wkv6_backward_static_scratch(&p, b[0], b[1], b[2], b[3], b[4], b[5], b[6], b[7], b[8], b[9], b[10], st);
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

}  // namespace gpu_ops

extern "C" {

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
        default: return nullptr;
    }
}

}  // extern "C"
