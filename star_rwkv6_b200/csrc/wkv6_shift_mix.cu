// Input stage of the time-mix block: the token-shift interpolations
//   out_j[b,t,c] = x[b,t,c] + (x[b,t-1,c] - x[b,t,c]) * m_j[b,t,c],      x[b,-1,:] = 0,
// for j = 0..nmix-1, where m_j is either one vector per channel (time_mix_x: TimeMix.call, rwkv6_model.py:135-138,
// with TimeShift = pad-and-subtract, :37-44) or a full tensor (the five data-dependent mixes built from the low-rank
// projections, rwkv6_model.py:141-146).  The reference runs them as separate framework ops (a padded copy, a
// subtraction, and per mix a multiply and an add); here one kernel per direction reads x once and every m_j once.
//
// A thread owns eight adjacent channels and walks a run of consecutive tokens of one batch row, carrying the
// neighbouring token in registers: the forward walks up (carrying x[t-1]), the backward walks down (carrying
// gs[t+1] = sum_j gout_j[t+1] m_j[t+1], the gradient that reaches x[t] through the shift).  Bytes per (token,
// channel) in bf16: vector mix 4 forward / 6 backward; five tensor mixes 22 forward / 34 backward.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "wkv6_internal.h"

namespace wkv6 {

constexpr int kRun = 32;  // tokens a thread walks; the carried neighbour is re-read once per run

template <typename T> struct V8;
template <> struct V8<__nv_bfloat16> {
    static __device__ __forceinline__ void ld(const void *p, size_t i, float (&f)[8]) {
        const uint4 q = *reinterpret_cast<const uint4 *>(static_cast<const __nv_bfloat16 *>(p) + i);
        const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&q);
#pragma unroll
        for (int e = 0; e < 4; ++e) { const float2 t = __bfloat1622float2(h[e]); f[2 * e] = t.x; f[2 * e + 1] = t.y; }
    }
    static __device__ __forceinline__ void st(void *p, size_t i, const float (&f)[8]) {
        uint4 q;
        __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&q);
#pragma unroll
        for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(f[2 * e], f[2 * e + 1]);
        *reinterpret_cast<uint4 *>(static_cast<__nv_bfloat16 *>(p) + i) = q;
    }
};
template <> struct V8<__half> {
    static __device__ __forceinline__ void ld(const void *p, size_t i, float (&f)[8]) {
        const uint4 q = *reinterpret_cast<const uint4 *>(static_cast<const __half *>(p) + i);
        const __half2 *h = reinterpret_cast<const __half2 *>(&q);
#pragma unroll
        for (int e = 0; e < 4; ++e) { const float2 t = __half22float2(h[e]); f[2 * e] = t.x; f[2 * e + 1] = t.y; }
    }
    static __device__ __forceinline__ void st(void *p, size_t i, const float (&f)[8]) {
        uint4 q;
        __half2 *h = reinterpret_cast<__half2 *>(&q);
#pragma unroll
        for (int e = 0; e < 4; ++e) h[e] = __floats2half2_rn(f[2 * e], f[2 * e + 1]);
        *reinterpret_cast<uint4 *>(static_cast<__half *>(p) + i) = q;
    }
};
template <> struct V8<float> {
    static __device__ __forceinline__ void ld(const void *p, size_t i, float (&f)[8]) {
        const float4 a = *reinterpret_cast<const float4 *>(static_cast<const float *>(p) + i);
        const float4 b = *reinterpret_cast<const float4 *>(static_cast<const float *>(p) + i + 4);
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    }
    static __device__ __forceinline__ void st(void *p, size_t i, const float (&f)[8]) {
        *reinterpret_cast<float4 *>(static_cast<float *>(p) + i) = make_float4(f[0], f[1], f[2], f[3]);
        *reinterpret_cast<float4 *>(static_cast<float *>(p) + i + 4) = make_float4(f[4], f[5], f[6], f[7]);
    }
};

// Work item = (batch row b, run of kRun tokens, channel octet).  Items are laid out octet-fastest so that a warp
// reads 512 contiguous bytes of a token.
struct ShiftGeom {
    int B, T, C, runs, octets;
    size_t items;
};
__host__ __device__ inline ShiftGeom shift_geom(int B, int T, int C) {
    ShiftGeom g;
    g.B = B; g.T = T; g.C = C; g.runs = (T + kRun - 1) / kRun; g.octets = C / 8;
    g.items = (size_t)B * g.runs * g.octets;
    return g;
}

// VEC: m is one fp32 vector [C] (nmix == 1), else m and out are dense [nmix][B][T][C] of the activation dtype
template <typename T, bool VEC, int NMIX>
__global__ void __launch_bounds__(256) shift_mix_fwd_kernel(ShiftGeom g, const void *__restrict__ x, const void *__restrict__ m,
                                                            void *__restrict__ out) {
    const size_t item = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (item >= g.items) return;
    const int oct = (int)(item % g.octets);
    const int run = (int)((item / g.octets) % g.runs);
    const int b = (int)(item / ((size_t)g.octets * g.runs));
    const int t0 = run * kRun, t1 = min(t0 + kRun, g.T);
    const size_t plane = (size_t)g.B * g.T * g.C;
    float mv[8] = {};
    if (VEC) V8<float>::ld(m, (size_t)oct * 8, mv);
    float prev[8] = {};
    if (t0 > 0) V8<T>::ld(x, ((size_t)b * g.T + t0 - 1) * g.C + oct * 8, prev);
    for (int t = t0; t < t1; ++t) {
        const size_t i = ((size_t)b * g.T + t) * g.C + oct * 8;
        float xv[8];
        V8<T>::ld(x, i, xv);
#pragma unroll
        for (int j = 0; j < NMIX; ++j) {
            float o[8];
            if (!VEC) V8<T>::ld(m, (size_t)j * plane + i, mv);
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] = fmaf(prev[e] - xv[e], mv[e], xv[e]);
            V8<T>::st(out, (size_t)j * plane + i, o);
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) prev[e] = xv[e];
    }
}

// gx[t] = sum_j gout_j[t] (1 - m_j[t]) + gs[t+1],  gs[t] = sum_j gout_j[t] m_j[t]  (gs beyond the last token is 0);
// gm_j[t] = gout_j[t] (x[t-1] - x[t])  (tensor mixes: written out; vector mix: summed over rows into partial[item-run][C])
template <typename T, bool VEC, int NMIX>
__global__ void __launch_bounds__(256) shift_mix_bwd_kernel(ShiftGeom g, const void *__restrict__ x, const void *__restrict__ m,
                                                            const void *__restrict__ gout, void *__restrict__ gx,
                                                            void *__restrict__ gm, float *__restrict__ partial) {
    const size_t item = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (item >= g.items) return;
    const int oct = (int)(item % g.octets);
    const int run = (int)((item / g.octets) % g.runs);
    const int b = (int)(item / ((size_t)g.octets * g.runs));
    const int t0 = run * kRun, t1 = min(t0 + kRun, g.T);
    const size_t plane = (size_t)g.B * g.T * g.C;
    float mv[8] = {};
    if (VEC) V8<float>::ld(m, (size_t)oct * 8, mv);
    // gs of the token after this run
    float gs_next[8] = {};
    if (t1 < g.T) {
        const size_t i = ((size_t)b * g.T + t1) * g.C + oct * 8;
#pragma unroll
        for (int j = 0; j < NMIX; ++j) {
            float go[8];
            V8<T>::ld(gout, (size_t)j * plane + i, go);
            if (!VEC) V8<T>::ld(m, (size_t)j * plane + i, mv);
#pragma unroll
            for (int e = 0; e < 8; ++e) gs_next[e] = fmaf(go[e], mv[e], gs_next[e]);
        }
    }
    float xcur[8], gmsum[8] = {};
    V8<T>::ld(x, ((size_t)b * g.T + t1 - 1) * g.C + oct * 8, xcur);
    for (int t = t1 - 1; t >= t0; --t) {
        const size_t i = ((size_t)b * g.T + t) * g.C + oct * 8;
        float xprev[8] = {};
        if (t > 0) V8<T>::ld(x, i - g.C, xprev);
        float acc[8], gs[8] = {};
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = gs_next[e];
#pragma unroll
        for (int j = 0; j < NMIX; ++j) {
            float go[8];
            V8<T>::ld(gout, (size_t)j * plane + i, go);
            if (!VEC) V8<T>::ld(m, (size_t)j * plane + i, mv);
            float gmj[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float gom = go[e] * mv[e];
                gs[e] += gom;
                acc[e] += go[e] - gom;
                gmj[e] = go[e] * (xprev[e] - xcur[e]);
                if (VEC) gmsum[e] += gmj[e];
            }
            if (!VEC) V8<T>::st(gm, (size_t)j * plane + i, gmj);
        }
        V8<T>::st(gx, i, acc);
#pragma unroll
        for (int e = 0; e < 8; ++e) { gs_next[e] = gs[e]; xcur[e] = xprev[e]; }
    }
    if (VEC) V8<float>::st(partial, ((size_t)b * g.runs + run) * g.C + oct * 8, gmsum);
}

// gmu[c] = sum of the per-(batch row, run) partial sums in a fixed order: 32 columns x 8 row groups per block, group g
// adds the partial sums g, g + 8, ... and the eight group sums are added in group order.
__global__ void __launch_bounds__(256) shift_mix_reduce_kernel(int nparts, int C, const float *__restrict__ partial,
                                                               float *__restrict__ gmu) {
    __shared__ float sred[8][33];
    const int cx = threadIdx.x & 31, grp = threadIdx.x >> 5;
    const int c = blockIdx.x * 32 + cx;
    float s = 0.f;
    if (c < C) {
#pragma unroll 8
        for (int p = grp; p < nparts; p += 8) s += partial[(size_t)p * C + c];
    }
    sred[grp][cx] = s;
    __syncthreads();
    if (grp == 0 && c < C) {
        float t = sred[0][cx];
#pragma unroll
        for (int g2 = 1; g2 < 8; ++g2) t += sred[g2][cx];
        gmu[c] = t;
    }
}

static int shift_check(int B, int T, int C, int dtype, int nmix, const char *what) {
    if (B < 0 || T < 0 || C < 8 || C % 8) return fail(WKV6_ERR_INVALID, "%s: B=%d T=%d C=%d (C must be a positive multiple of 8)", what, B, T, C);
    if (nmix != 1 && nmix != 5) return fail(WKV6_ERR_UNSUPPORTED, "%s: nmix must be 1 or 5, got %d", what, nmix);
    if (dtype != WKV6_BF16 && dtype != WKV6_F16 && dtype != WKV6_F32) return fail(WKV6_ERR_INVALID, "%s: bad dtype %d", what, dtype);
    return WKV6_OK;
}

}  // namespace wkv6

using namespace wkv6;

#define SM_PTR(p) \
    if ((p) == nullptr || reinterpret_cast<uintptr_t>(p) % 16) return fail(WKV6_ERR_INVALID, #p " is NULL or not 16-byte aligned")

#define SM_DISPATCH(KERNEL, VEC, NMIX, ...)                                                                  \
    do {                                                                                                      \
        if (dtype == WKV6_BF16) KERNEL<__nv_bfloat16, VEC, NMIX><<<grid, 256, 0, st>>>(__VA_ARGS__);           \
        else if (dtype == WKV6_F16) KERNEL<__half, VEC, NMIX><<<grid, 256, 0, st>>>(__VA_ARGS__);              \
        else KERNEL<float, VEC, NMIX><<<grid, 256, 0, st>>>(__VA_ARGS__);                                      \
    } while (0)

extern "C" {

__attribute__((visibility("default")))
int wkv6_shift_mix_forward(int32_t B, int32_t T, int32_t C, int32_t dtype, int32_t nmix, int32_t m_is_vector, const void *x,
                           const void *m, void *out, void *stream) {
    int rc = shift_check(B, T, C, dtype, nmix, "wkv6_shift_mix_forward");
    if (rc) return rc;
    if (m_is_vector && nmix != 1) return fail(WKV6_ERR_INVALID, "a vector mix has nmix == 1");
    if (B == 0 || T == 0) return WKV6_OK;
    SM_PTR(x); SM_PTR(m); SM_PTR(out);
    const ShiftGeom g = shift_geom(B, T, C);
    const unsigned grid = (unsigned)((g.items + 255) / 256);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (m_is_vector) SM_DISPATCH(shift_mix_fwd_kernel, true, 1, g, x, m, out);
    else if (nmix == 1) SM_DISPATCH(shift_mix_fwd_kernel, false, 1, g, x, m, out);
    else SM_DISPATCH(shift_mix_fwd_kernel, false, 5, g, x, m, out);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? WKV6_OK : cuda_fail(e, "shift_mix_fwd_kernel launch");
}

__attribute__((visibility("default")))
size_t wkv6_shift_mix_workspace_bytes(int32_t B, int32_t T, int32_t C, int32_t m_is_vector) {
    if (!m_is_vector || B <= 0 || T <= 0 || C <= 0) return 0;
    return (size_t)B * ((T + kRun - 1) / kRun) * C * sizeof(float);
}

__attribute__((visibility("default")))
int wkv6_shift_mix_backward(int32_t B, int32_t T, int32_t C, int32_t dtype, int32_t nmix, int32_t m_is_vector, const void *x,
                            const void *m, const void *gout, void *gx, void *gm, void *workspace, size_t workspace_bytes,
                            void *stream) {
    int rc = shift_check(B, T, C, dtype, nmix, "wkv6_shift_mix_backward");
    if (rc) return rc;
    if (m_is_vector && nmix != 1) return fail(WKV6_ERR_INVALID, "a vector mix has nmix == 1");
    SM_PTR(gm);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (B == 0 || T == 0) {
        if (m_is_vector) {
            cudaError_t e0 = cudaMemsetAsync(gm, 0, (size_t)C * sizeof(float), st);
            if (e0 != cudaSuccess) return cuda_fail(e0, "cudaMemsetAsync(gmu)");
        }
        return WKV6_OK;
    }
    SM_PTR(x); SM_PTR(m); SM_PTR(gout); SM_PTR(gx);
    const ShiftGeom g = shift_geom(B, T, C);
    const unsigned grid = (unsigned)((g.items + 255) / 256);
    float *partial = nullptr;
    if (m_is_vector) {
        const size_t need = wkv6_shift_mix_workspace_bytes(B, T, C, 1);
        if (workspace == nullptr || workspace_bytes < need || reinterpret_cast<uintptr_t>(workspace) % 16)
            return fail(WKV6_ERR_WORKSPACE, "shift_mix backward workspace: need %zu bytes (16-byte aligned), got %zu", need,
                        workspace ? workspace_bytes : (size_t)0);
        partial = static_cast<float *>(workspace);
        SM_DISPATCH(shift_mix_bwd_kernel, true, 1, g, x, m, gout, gx, nullptr, partial);
    } else if (nmix == 1) {
        SM_DISPATCH(shift_mix_bwd_kernel, false, 1, g, x, m, gout, gx, gm, nullptr);
    } else {
        SM_DISPATCH(shift_mix_bwd_kernel, false, 5, g, x, m, gout, gx, gm, nullptr);
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "shift_mix_bwd_kernel launch");
    if (m_is_vector) {
        shift_mix_reduce_kernel<<<(C + 31) / 32, 256, 0, st>>>(B * g.runs, C, partial, static_cast<float *>(gm));
        e = cudaGetLastError();
        if (e != cudaSuccess) return cuda_fail(e, "shift_mix_reduce_kernel launch");
    }
    return WKV6_OK;
}

}  // extern "C"
