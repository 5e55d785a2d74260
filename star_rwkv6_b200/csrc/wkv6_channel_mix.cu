// Element-wise stages of the channel-mix block over whole sequences, one launch per direction:
//   relu_sq      out = max(x, 0)^2                       gx = gout * 2 max(x, 0)
//   sigmoid_mul  out = sigmoid(r) * kv                   gr = gout * kv * s (1 - s),  gkv = gout * s,  s = sigmoid(r)
// They are the activations of the reference's ChannelMix (rwkv6_model.py:47-48 relu_square on dense_key, :83 sigmoid on
// dense_receptance, :64 `o = r * kv`), which a framework evaluates as two to three kernels per direction with a round
// trip through HBM each (relu, square, their backward pair; sigmoid, multiply, and three backward kernels).  Each kernel
// here reads its operands once and writes its results once: 4 / 6 bytes per element (relu_sq forward / backward) and
// 6 / 10 bytes (sigmoid_mul) in bf16.  HBM-bound; eight elements (one 16-byte access in bf16) per thread and step,
// grid of 8 x 148 CTAs walking the array with a grid stride.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "wkv6_internal.h"

namespace wkv6 {

template <typename T> struct CmVec;
template <> struct CmVec<__nv_bfloat16> {
    static __device__ __forceinline__ void load(const void *p, size_t i, float (&f)[8]) {
        const uint4 q = *reinterpret_cast<const uint4 *>(static_cast<const __nv_bfloat16 *>(p) + i);
        const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&q);
#pragma unroll
        for (int e = 0; e < 4; ++e) { const float2 t = __bfloat1622float2(h[e]); f[2 * e] = t.x; f[2 * e + 1] = t.y; }
    }
    static __device__ __forceinline__ void store(void *p, size_t i, const float (&f)[8]) {
        uint4 q;
        __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&q);
#pragma unroll
        for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(f[2 * e], f[2 * e + 1]);
        *reinterpret_cast<uint4 *>(static_cast<__nv_bfloat16 *>(p) + i) = q;
    }
    static __device__ __forceinline__ float load1(const void *p, size_t i) { return __bfloat162float(static_cast<const __nv_bfloat16 *>(p)[i]); }
    static __device__ __forceinline__ void store1(void *p, size_t i, float x) { static_cast<__nv_bfloat16 *>(p)[i] = __float2bfloat16_rn(x); }
};
template <> struct CmVec<__half> {
    static __device__ __forceinline__ void load(const void *p, size_t i, float (&f)[8]) {
        const uint4 q = *reinterpret_cast<const uint4 *>(static_cast<const __half *>(p) + i);
        const __half2 *h = reinterpret_cast<const __half2 *>(&q);
#pragma unroll
        for (int e = 0; e < 4; ++e) { const float2 t = __half22float2(h[e]); f[2 * e] = t.x; f[2 * e + 1] = t.y; }
    }
    static __device__ __forceinline__ void store(void *p, size_t i, const float (&f)[8]) {
        uint4 q;
        __half2 *h = reinterpret_cast<__half2 *>(&q);
#pragma unroll
        for (int e = 0; e < 4; ++e) h[e] = __floats2half2_rn(f[2 * e], f[2 * e + 1]);
        *reinterpret_cast<uint4 *>(static_cast<__half *>(p) + i) = q;
    }
    static __device__ __forceinline__ float load1(const void *p, size_t i) { return __half2float(static_cast<const __half *>(p)[i]); }
    static __device__ __forceinline__ void store1(void *p, size_t i, float x) { static_cast<__half *>(p)[i] = __float2half_rn(x); }
};
template <> struct CmVec<float> {
    static __device__ __forceinline__ void load(const void *p, size_t i, float (&f)[8]) {
        const float4 a = *reinterpret_cast<const float4 *>(static_cast<const float *>(p) + i);
        const float4 b = *reinterpret_cast<const float4 *>(static_cast<const float *>(p) + i + 4);
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    }
    static __device__ __forceinline__ void store(void *p, size_t i, const float (&f)[8]) {
        *reinterpret_cast<float4 *>(static_cast<float *>(p) + i) = make_float4(f[0], f[1], f[2], f[3]);
        *reinterpret_cast<float4 *>(static_cast<float *>(p) + i + 4) = make_float4(f[4], f[5], f[6], f[7]);
    }
    static __device__ __forceinline__ float load1(const void *p, size_t i) { return static_cast<const float *>(p)[i]; }
    static __device__ __forceinline__ void store1(void *p, size_t i, float x) { static_cast<float *>(p)[i] = x; }
};

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

// MODE 0: relu_sq forward (a = x -> o0)          MODE 1: relu_sq backward (a = x, b = gout -> o0 = gx)
// MODE 2: sigmoid_mul forward (a = r, b = kv -> o0)   MODE 3: sigmoid_mul backward (a = r, b = kv, c = gout -> o0 = gr, o1 = gkv)
template <int MODE>
__device__ __forceinline__ void cm_apply(float a, float b, float c, float &o0, float &o1) {
    if (MODE == 0) { const float v = fmaxf(a, 0.f); o0 = v * v; }
    if (MODE == 1) { o0 = b * 2.f * fmaxf(a, 0.f); }
    if (MODE == 2) { o0 = sigmoidf_(a) * b; }
    if (MODE == 3) { const float s = sigmoidf_(a); o0 = c * b * s * (1.f - s); o1 = c * s; }
}

template <typename T, int MODE>
__global__ void __launch_bounds__(256) channel_mix_elementwise_kernel(size_t n, const void *__restrict__ a, const void *__restrict__ b,
                                                                      const void *__restrict__ c, void *__restrict__ o0,
                                                                      void *__restrict__ o1) {
    const size_t nvec = n / 8;
    for (size_t v = (size_t)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += (size_t)gridDim.x * blockDim.x) {
        float fa[8], fb[8], fc[8], r0[8], r1[8];
        CmVec<T>::load(a, v * 8, fa);
        if (MODE >= 1) CmVec<T>::load(b, v * 8, fb);
        if (MODE == 3) CmVec<T>::load(c, v * 8, fc);
#pragma unroll
        for (int e = 0; e < 8; ++e) cm_apply<MODE>(fa[e], MODE >= 1 ? fb[e] : 0.f, MODE == 3 ? fc[e] : 0.f, r0[e], r1[e]);
        CmVec<T>::store(o0, v * 8, r0);
        if (MODE == 3) CmVec<T>::store(o1, v * 8, r1);
    }
    // ragged tail (n not a multiple of 8): one thread per element
    const size_t i = nvec * 8 + (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        float r0, r1;
        cm_apply<MODE>(CmVec<T>::load1(a, i), MODE >= 1 ? CmVec<T>::load1(b, i) : 0.f, MODE == 3 ? CmVec<T>::load1(c, i) : 0.f, r0, r1);
        CmVec<T>::store1(o0, i, r0);
        if (MODE == 3) CmVec<T>::store1(o1, i, r1);
    }
}

template <int MODE>
static int cm_launch(const char *what, int64_t n, int32_t dtype, const void *a, const void *b, const void *c, void *o0, void *o1,
                     void *stream) {
    if (dtype != WKV6_BF16 && dtype != WKV6_F16 && dtype != WKV6_F32) return fail(WKV6_ERR_INVALID, "%s: unknown dtype code %d", what, dtype);
    if (n < 0) return fail(WKV6_ERR_INVALID, "%s: n=%lld", what, (long long)n);
    if (n == 0) return WKV6_OK;
    const void *ptrs[] = {a, MODE >= 1 ? b : a, MODE == 3 ? c : a, o0, MODE == 3 ? o1 : o0};
    for (const void *p : ptrs)
        if (p == nullptr || reinterpret_cast<uintptr_t>(p) % 16) return fail(WKV6_ERR_INVALID, "%s: a pointer is NULL or not 16-byte aligned", what);
    const size_t nvec = (size_t)n / 8;
    size_t blocks = (nvec + 255) / 256;
    if (blocks > 8 * 148) blocks = 8 * 148;
    if (blocks == 0) blocks = 1;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == WKV6_BF16) channel_mix_elementwise_kernel<__nv_bfloat16, MODE><<<(unsigned)blocks, 256, 0, st>>>((size_t)n, a, b, c, o0, o1);
    else if (dtype == WKV6_F16) channel_mix_elementwise_kernel<__half, MODE><<<(unsigned)blocks, 256, 0, st>>>((size_t)n, a, b, c, o0, o1);
    else channel_mix_elementwise_kernel<float, MODE><<<(unsigned)blocks, 256, 0, st>>>((size_t)n, a, b, c, o0, o1);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? WKV6_OK : cuda_fail(e, what);
}

}  // namespace wkv6

using namespace wkv6;

extern "C" {

int wkv6_relu_sq_forward(int64_t n, int32_t dtype, const void *x, void *out, void *stream) {
    return cm_launch<0>("wkv6_relu_sq_forward", n, dtype, x, nullptr, nullptr, out, nullptr, stream);
}
int wkv6_relu_sq_backward(int64_t n, int32_t dtype, const void *x, const void *gout, void *gx, void *stream) {
    return cm_launch<1>("wkv6_relu_sq_backward", n, dtype, x, gout, nullptr, gx, nullptr, stream);
}
int wkv6_sigmoid_mul_forward(int64_t n, int32_t dtype, const void *r, const void *kv, void *out, void *stream) {
    return cm_launch<2>("wkv6_sigmoid_mul_forward", n, dtype, r, kv, nullptr, out, nullptr, stream);
}
int wkv6_sigmoid_mul_backward(int64_t n, int32_t dtype, const void *r, const void *kv, const void *gout, void *gr, void *gkv,
                              void *stream) {
    return cm_launch<3>("wkv6_sigmoid_mul_backward", n, dtype, r, kv, gout, gr, gkv, stream);
}

}  // extern "C"
