// wkv6_backward_static_scratch: the sequential backward for callers that cannot hand the library any scratch
// memory.  The scratch the sequential backward needs (one fp32 value per (token, channel), see wkv6_seq.cuh)
// lives in a fixed device array that is part of the library image, so the call allocates nothing.
#include <mutex>

#include "wkv6_internal.h"

namespace wkv6 {

// 32 MiB = 8 388 608 (token, channel) pairs, e.g. B=1, T=4096, C=2048.  Every GPU that loads the library
// holds this array until the process exits.
constexpr size_t kStaticScratchBytes = size_t(32) << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// In host code the name g_static_scratch is only a handle; the device address has to be asked for, once per
// device, with that device current.
static int static_scratch_address(void **out) {
    constexpr int kMaxDevices = 64;
    static std::mutex mu;
    static void *addr[kMaxDevices] = {};
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (dev < 0 || dev >= kMaxDevices) return fail(WKV6_ERR_UNSUPPORTED, "device ordinal %d is beyond %d", dev, kMaxDevices);
    std::lock_guard<std::mutex> lock(mu);
    if (addr[dev] == nullptr) {
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(static scratch)");
        addr[dev] = p;
    }
    *out = addr[dev];
    return WKV6_OK;
}

}  // namespace wkv6

using namespace wkv6;

extern "C" __attribute__((visibility("default")))
size_t wkv6_static_scratch_bytes(void) { return kStaticScratchBytes; }

extern "C" __attribute__((visibility("default")))
int wkv6_backward_static_scratch(const wkv6_problem *p, const void *r, const void *k, const void *v, const void *w,
                                 const void *u, const void *gy, void *gr, void *gk, void *gv, void *gw, void *gu,
                                 void *stream) {
    if (p == nullptr) return fail(WKV6_ERR_INVALID, "problem is NULL");
    wkv6_problem q = *p;
    q.variant = WKV6_VARIANT_SEQ;  // the kernel this entry point is a variant of
    Dims d;
    int rc = validate(&q, &d);
    if (rc) return rc;
    if (q.B == 0 || q.H == 0) return WKV6_OK;
    const void *ins[] = {r, k, v, w, gy};
    void *outs[] = {gr, gk, gv, gw};
    if (u == nullptr || gu == nullptr) return fail(WKV6_ERR_INVALID, "u or gu is NULL");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (q.T == 0) {
        cudaError_t e = cudaMemsetAsync(gu, 0, (size_t)q.B * d.C * dtype_size(q.gu_dtype), st);
        return e == cudaSuccess ? WKV6_OK : cuda_fail(e, "cudaMemsetAsync(gu)");
    }
    for (const void *ptr : ins)
        if (ptr == nullptr || reinterpret_cast<uintptr_t>(ptr) % 16) return fail(WKV6_ERR_INVALID, "an input pointer is NULL or not 16-byte aligned");
    for (void *ptr : outs)
        if (ptr == nullptr || reinterpret_cast<uintptr_t>(ptr) % 16) return fail(WKV6_ERR_INVALID, "an output pointer is NULL or not 16-byte aligned");
    const size_t need = seq_backward_workspace(&q, d);  // 0 for dense fp32 problems: they stage inside gw
    if (need > kStaticScratchBytes)
        return fail(WKV6_ERR_WORKSPACE,
                    "B*T*H*N = %zu (token, channel) pairs need %zu bytes of scratch; the built-in scratch holds %zu bytes "
                    "(%zu pairs) - use wkv6_backward with a caller workspace for larger problems",
                    need / sizeof(float), need, kStaticScratchBytes, kStaticScratchBytes / sizeof(float));
    void *scratch = nullptr;
    if (need > 0) {
        rc = static_scratch_address(&scratch);
        if (rc) return rc;
    }
    // Nothing in the scratch has to start at zero: the ascending sweep writes every element the descending sweep reads.
    // (Dense fp32 problems stage that data inside the gw output instead and leave the array untouched.)
    return seq_backward(&q, d, r, k, v, w, u, gy, gr, gk, gv, gw, gu, scratch, need > 0 ? kStaticScratchBytes : 0, st);
}
