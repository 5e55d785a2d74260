// Output stage of the time-mix block, fused: per-head normalisation of the WKV output followed by the gate,
//   out[b,t,h,n] = (scale[h,n] * (y[b,t,h,n] - mean) * rstd + offset[h,n]) * g[b,t,h,n],
// mean and variance over the N = 64 channels of one head of one token, rstd = 1 / sqrt(var + eps).  This is
// GroupNorm.call (rwkv6_model.py:93-99: LayerNormalization(epsilon=64e-5) over the head dimension, then the
// [H,N] scale and offset) followed by `x * g` (rwkv6_model.py:158-160), which the reference runs as separate
// element-wise framework ops with an HBM round trip each.  Forward: 6 bytes per (token, channel) in bf16
// (y, g in; out out); backward: 10 bytes (y, g, gout in; gy, gg out) plus the [H,N] parameter gradients.
//
// One CTA thread owns eight adjacent channels of a row (one 16-byte load in bf16), eight threads one head; a CTA
// covers all H*N channels of a row and walks rows with a grid stride, so a thread always meets the same (head,
// channels) and can keep its share of the parameter gradients in registers.  Those partial sums go to a workspace
// [grid][2][H*N] and a second kernel adds them in a fixed order (bit-identical reruns; no atomics).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "wkv6_internal.h"
#include "wkv6_seq.cuh"

namespace wkv6 {

constexpr int kGnVec = 8;  // channels per thread

template <typename T> struct Vec8;
template <> struct Vec8<__nv_bfloat16> {
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
};
template <> struct Vec8<__half> {
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
};
template <> struct Vec8<float> {
    static __device__ __forceinline__ void load(const void *p, size_t i, float (&f)[8]) {
        const float4 a = *reinterpret_cast<const float4 *>(static_cast<const float *>(p) + i);
        const float4 b = *reinterpret_cast<const float4 *>(static_cast<const float *>(p) + i + 4);
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    }
    static __device__ __forceinline__ void store(void *p, size_t i, const float (&f)[8]) {
        *reinterpret_cast<float4 *>(static_cast<float *>(p) + i) = make_float4(f[0], f[1], f[2], f[3]);
        *reinterpret_cast<float4 *>(static_cast<float *>(p) + i + 4) = make_float4(f[4], f[5], f[6], f[7]);
    }
};

// sum over the eight threads (64 channels) of one head
__device__ __forceinline__ float head_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    v += __shfl_xor_sync(0xffffffffu, v, 4);
    return v;
}

// mean and 1/sqrt(var + eps) of the head this thread belongs to, two passes over the registers
__device__ __forceinline__ void head_stats(const float (&y)[8], float eps, float &mean, float &rstd) {
    float s = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) s += y[e];
    mean = head_sum(s) * (1.0f / 64.0f);
    float q = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) { const float d = y[e] - mean; q = fmaf(d, d, q); }
    rstd = rsqrtf(head_sum(q) * (1.0f / 64.0f) + eps);
}

// SILU: g is the gate projection before its activation and the kernel applies silu(g) = g sigmoid(g) itself
// (rwkv6_model.py:147 `g = silu(dense_g(xg))`), so that the activated gate never exists in memory.
template <typename T, bool SILU>
__global__ void __launch_bounds__(1024) gn_gate_fwd_kernel(int64_t rows, int C, float eps, const void *__restrict__ y,
                                                           const void *__restrict__ g, const float *__restrict__ scale,
                                                           const float *__restrict__ offset, void *__restrict__ out) {
    const int c0 = threadIdx.x * kGnVec;  // this thread's first channel
    const bool live = c0 < C;             // the block is padded to whole warps; padding threads only take part in the shuffles
    float sc[8] = {}, of[8] = {};
    if (live) {
        Vec8<float>::load(scale, c0, sc);
        Vec8<float>::load(offset, c0, of);
    }
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const size_t i = (size_t)row * C + c0;
        float yv[8] = {}, gv[8] = {}, o[8];
        if (live) {
            Vec8<T>::load(y, i, yv);
            Vec8<T>::load(g, i, gv);
        }
        float mean, rstd;
        head_stats(yv, eps, mean, rstd);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float gate = SILU ? gv[e] / (1.f + __expf(-gv[e])) : gv[e];
            o[e] = fmaf((yv[e] - mean) * rstd, sc[e], of[e]) * gate;
        }
        if (live) Vec8<T>::store(out, i, o);
    }
}

template <typename T, bool SILU>
__global__ void __launch_bounds__(1024) gn_gate_bwd_kernel(int64_t rows, int C, float eps, const void *__restrict__ y,
                                                           const void *__restrict__ g, const float *__restrict__ scale,
                                                           const float *__restrict__ offset, const void *__restrict__ gout,
                                                           void *__restrict__ gy, void *__restrict__ gg,
                                                           float *__restrict__ partial) {
    const int c0 = threadIdx.x * kGnVec;
    const bool live = c0 < C;
    float sc[8] = {}, of[8] = {}, dsc[8], dof[8];
    if (live) {
        Vec8<float>::load(scale, c0, sc);
        Vec8<float>::load(offset, c0, of);
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) dsc[e] = dof[e] = 0.f;
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const size_t i = (size_t)row * C + c0;
        float yv[8] = {}, gv[8] = {}, go[8] = {}, dy[8], dg[8];
        if (live) {
            Vec8<T>::load(y, i, yv);
            Vec8<T>::load(g, i, gv);
            Vec8<T>::load(gout, i, go);
        }
        float mean, rstd;
        head_stats(yv, eps, mean, rstd);
        // x^ = (y - mean) rstd;  out = (scale x^ + offset) g;  dx^ = gout g scale
        float s1 = 0.f, s2 = 0.f, xh[8], dx[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            xh[e] = (yv[e] - mean) * rstd;
            float gate = gv[e], dgate = 1.f;  // silu(g) = g s, its derivative s (1 + g (1 - s)), s = sigmoid(g)
            if (SILU) {
                const float sg = 1.f / (1.f + __expf(-gv[e]));
                gate = gv[e] * sg;
                dgate = sg * fmaf(gv[e], 1.f - sg, 1.f);
            }
            const float gog = go[e] * gate;
            dg[e] = go[e] * fmaf(xh[e], sc[e], of[e]) * dgate;
            dx[e] = gog * sc[e];
            dsc[e] = fmaf(gog, xh[e], dsc[e]);
            dof[e] += gog;
            s1 += dx[e];
            s2 = fmaf(dx[e], xh[e], s2);
        }
        s1 = head_sum(s1) * (1.0f / 64.0f);
        s2 = head_sum(s2) * (1.0f / 64.0f);
#pragma unroll
        for (int e = 0; e < 8; ++e) dy[e] = rstd * (dx[e] - s1 - xh[e] * s2);
        if (live) {
            Vec8<T>::store(gy, i, dy);
            Vec8<T>::store(gg, i, dg);
        }
    }
    if (live) {
        float *p = partial + (size_t)blockIdx.x * 2 * C;
        Vec8<float>::store(p, c0, dsc);
        Vec8<float>::store(p + C, c0, dof);
    }
}

// gscale[c] = sum over the CTAs' partial sums in a fixed order (reruns are bit-identical): 32 columns x 8 row groups per
// block, group g adds the partial sums g, g + 8, ... and the eight group sums are added in group order.
__global__ void __launch_bounds__(256) gn_gate_reduce_kernel(int nparts, int C, const float *__restrict__ partial,
                                                             float *__restrict__ gscale, float *__restrict__ goffset) {
    __shared__ float sred[8][33];
    const int cx = threadIdx.x & 31, grp = threadIdx.x >> 5;
    const int c = blockIdx.x * 32 + cx;
    float s = 0.f;
    if (c < 2 * C) {
#pragma unroll 8
        for (int pidx = grp; pidx < nparts; pidx += 8) s += partial[(size_t)pidx * 2 * C + c];
    }
    sred[grp][cx] = s;
    __syncthreads();
    if (grp == 0 && c < 2 * C) {
        float t = sred[0][cx];
#pragma unroll
        for (int g2 = 1; g2 < 8; ++g2) t += sred[g2][cx];
        if (c < C) gscale[c] = t; else goffset[c - C] = t;
    }
}

static int gn_grid(int64_t rows) {
    const int64_t cap = 148 * 4;
    return (int)(rows < cap ? rows : cap);
}

static int gn_check(int64_t rows, int H, int N, int dtype, const char *what) {
    if (rows < 0 || H < 1) return fail(WKV6_ERR_INVALID, "%s: rows=%lld H=%d", what, (long long)rows, H);
    if (N != 64) return fail(WKV6_ERR_UNSUPPORTED, "%s is built for head size 64, got %d", what, N);
    if ((int64_t)H * N / kGnVec > 1024) return fail(WKV6_ERR_UNSUPPORTED, "%s: H*N = %d exceeds 8192", what, H * N);
    if (dtype != WKV6_BF16 && dtype != WKV6_F16 && dtype != WKV6_F32) return fail(WKV6_ERR_INVALID, "%s: bad dtype %d", what, dtype);
    return WKV6_OK;
}

}  // namespace wkv6

using namespace wkv6;

#define GN_PTR(p) \
    if ((p) == nullptr || reinterpret_cast<uintptr_t>(p) % 16) return fail(WKV6_ERR_INVALID, #p " is NULL or not 16-byte aligned")

extern "C" {

extern "C++" {
template <bool SILU>
static int gn_forward_impl(int64_t rows, int32_t H, int32_t N, int32_t dtype, float eps, const void *y, const void *g,
                           const float *scale, const float *offset, void *out, void *stream) {
    int rc = gn_check(rows, H, N, dtype, "wkv6_groupnorm_gate_forward");
    if (rc) return rc;
    if (rows == 0) return WKV6_OK;
    GN_PTR(y); GN_PTR(g); GN_PTR(scale); GN_PTR(offset); GN_PTR(out);
    const int C = H * N, threads = (C / kGnVec + 31) / 32 * 32, grid = gn_grid(rows);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == WKV6_BF16) gn_gate_fwd_kernel<__nv_bfloat16, SILU><<<grid, threads, 0, st>>>(rows, C, eps, y, g, scale, offset, out);
    else if (dtype == WKV6_F16) gn_gate_fwd_kernel<__half, SILU><<<grid, threads, 0, st>>>(rows, C, eps, y, g, scale, offset, out);
    else gn_gate_fwd_kernel<float, SILU><<<grid, threads, 0, st>>>(rows, C, eps, y, g, scale, offset, out);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? WKV6_OK : cuda_fail(e, "gn_gate_fwd_kernel launch");
}
}  // extern "C++"

__attribute__((visibility("default")))
int wkv6_groupnorm_gate_forward(int64_t rows, int32_t H, int32_t N, int32_t dtype, float eps, const void *y, const void *g,
                                const float *scale, const float *offset, void *out, void *stream) {
    return gn_forward_impl<false>(rows, H, N, dtype, eps, y, g, scale, offset, out, stream);
}
__attribute__((visibility("default")))
int wkv6_groupnorm_silu_gate_forward(int64_t rows, int32_t H, int32_t N, int32_t dtype, float eps, const void *y, const void *g_raw,
                                     const float *scale, const float *offset, void *out, void *stream) {
    return gn_forward_impl<true>(rows, H, N, dtype, eps, y, g_raw, scale, offset, out, stream);
}

__attribute__((visibility("default")))
size_t wkv6_groupnorm_gate_workspace_bytes(int64_t rows, int32_t H, int32_t N) {
    if (rows <= 0 || H < 1 || N < 1) return 0;
    return (size_t)gn_grid(rows) * 2 * H * N * sizeof(float);
}

extern "C++" {
template <bool SILU>
static int gn_backward_impl(int64_t rows, int32_t H, int32_t N, int32_t dtype, float eps, const void *y, const void *g,
                            const float *scale, const float *offset, const void *gout, void *gy, void *gg,
                            float *gscale, float *goffset, void *workspace, size_t workspace_bytes, void *stream) {
    int rc = gn_check(rows, H, N, dtype, "wkv6_groupnorm_gate_backward");
    if (rc) return rc;
    GN_PTR(gscale); GN_PTR(goffset);
    const int C = H * N, threads = (C / kGnVec + 31) / 32 * 32;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (rows == 0) {
        cudaError_t e = cudaMemsetAsync(gscale, 0, (size_t)C * sizeof(float), st);
        if (e == cudaSuccess) e = cudaMemsetAsync(goffset, 0, (size_t)C * sizeof(float), st);
        return e == cudaSuccess ? WKV6_OK : cuda_fail(e, "cudaMemsetAsync(parameter gradients)");
    }
    GN_PTR(y); GN_PTR(g); GN_PTR(scale); GN_PTR(offset); GN_PTR(gout); GN_PTR(gy); GN_PTR(gg);
    const size_t need = wkv6_groupnorm_gate_workspace_bytes(rows, H, N);
    if (workspace == nullptr || workspace_bytes < need || reinterpret_cast<uintptr_t>(workspace) % 16)
        return fail(WKV6_ERR_WORKSPACE, "groupnorm_gate backward workspace: need %zu bytes (16-byte aligned), got %zu", need,
                    workspace ? workspace_bytes : (size_t)0);
    const int grid = gn_grid(rows);
    float *partial = static_cast<float *>(workspace);
    if (dtype == WKV6_BF16)
        gn_gate_bwd_kernel<__nv_bfloat16, SILU><<<grid, threads, 0, st>>>(rows, C, eps, y, g, scale, offset, gout, gy, gg, partial);
    else if (dtype == WKV6_F16)
        gn_gate_bwd_kernel<__half, SILU><<<grid, threads, 0, st>>>(rows, C, eps, y, g, scale, offset, gout, gy, gg, partial);
    else
        gn_gate_bwd_kernel<float, SILU><<<grid, threads, 0, st>>>(rows, C, eps, y, g, scale, offset, gout, gy, gg, partial);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "gn_gate_bwd_kernel launch");
    gn_gate_reduce_kernel<<<(2 * C + 31) / 32, 256, 0, st>>>(grid, C, partial, gscale, goffset);
    e = cudaGetLastError();
    return e == cudaSuccess ? WKV6_OK : cuda_fail(e, "gn_gate_reduce_kernel launch");
}
}  // extern "C++"

__attribute__((visibility("default")))
int wkv6_groupnorm_gate_backward(int64_t rows, int32_t H, int32_t N, int32_t dtype, float eps, const void *y, const void *g,
                                 const float *scale, const float *offset, const void *gout, void *gy, void *gg,
                                 float *gscale, float *goffset, void *workspace, size_t workspace_bytes, void *stream) {
    return gn_backward_impl<false>(rows, H, N, dtype, eps, y, g, scale, offset, gout, gy, gg, gscale, goffset, workspace,
                                   workspace_bytes, stream);
}
__attribute__((visibility("default")))
int wkv6_groupnorm_silu_gate_backward(int64_t rows, int32_t H, int32_t N, int32_t dtype, float eps, const void *y,
                                      const void *g_raw, const float *scale, const float *offset, const void *gout, void *gy,
                                      void *gg_raw, float *gscale, float *goffset, void *workspace, size_t workspace_bytes,
                                      void *stream) {
    return gn_backward_impl<true>(rows, H, N, dtype, eps, y, g_raw, scale, offset, gout, gy, gg_raw, gscale, goffset, workspace,
                                  workspace_bytes, stream);
}

}  // extern "C"
