// Element-wise stages of one decode step (T = 1) of an RWKV-6 block, fused so that a layer costs a handful of launches
// besides its matrix products.  At T = 1 every tensor is [B, D] (a few hundred KB), so each stage is bound by launch
// latency, not by bandwidth; what counts is their number.  Expressions: the reference's time-mix and channel-mix blocks
// (rwkv6_model.py:128-160 and :48-83; the same in rwkv_v6_demo.py:102-150, 174-183) evaluated for one token, with the
// previous token carried in `prev`.
//
//   ln_shift_mix     xa = LayerNorm(x); xs = prev - xa; prev <- xa; mix_i = xa + xs * mu_i   (i < 2)
//   lora_mix         out_m = xa + xs * (bias_m + tanh(h[:, m]) B_m),  m < 5   (the five data-dependent interpolations)
//   relu_sq          out = max(x, 0)^2
//   sigmoid_mul_add  out = x + sigmoid(r) * kv
//   (the per-head GroupNorm * SiLU gate behind the recurrence is fused into the decode kernel itself: wkv6_decode.cu)
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdint>
#include <initializer_list>
#include <type_traits>

#include "wkv6_internal.h"
#include "wkv6_seq.cuh"

namespace wkv6 {

constexpr int kStageThreads = 256;
constexpr int kStageMaxPer = 32;  // channels per thread of the row kernel: D <= 8192

__device__ __forceinline__ float block_sum_256(float x, float *scratch) {
    x = warp_sum(x);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();  // scratch may still be read from a previous call
    if (lane == 0) scratch[warp] = x;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < kStageThreads / 32; ++i) t += scratch[i];
    return t;
}

template <typename T> struct Pair;
template <> struct Pair<float> {
    static __device__ __forceinline__ float2 load(const void *p, size_t i) { return *reinterpret_cast<const float2 *>(static_cast<const float *>(p) + i); }
    static __device__ __forceinline__ void store(void *p, size_t i, float2 v) { *reinterpret_cast<float2 *>(static_cast<float *>(p) + i) = v; }
    static __device__ __forceinline__ float round(float x) { return x; }
};
template <> struct Pair<__nv_bfloat16> {
    static __device__ __forceinline__ float2 load(const void *p, size_t i) {
        return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(static_cast<const __nv_bfloat16 *>(p) + i));
    }
    static __device__ __forceinline__ void store(void *p, size_t i, float2 v) {
        *reinterpret_cast<__nv_bfloat162 *>(static_cast<__nv_bfloat16 *>(p) + i) = __float22bfloat162_rn(v);
    }
    static __device__ __forceinline__ float round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
};
template <> struct Pair<__half> {
    static __device__ __forceinline__ float2 load(const void *p, size_t i) {
        return __half22float2(*reinterpret_cast<const __half2 *>(static_cast<const __half *>(p) + i));
    }
    static __device__ __forceinline__ void store(void *p, size_t i, float2 v) {
        *reinterpret_cast<__half2 *>(static_cast<__half *>(p) + i) = __float22half2_rn(v);
    }
    static __device__ __forceinline__ float round(float x) { return __half2float(__float2half_rn(x)); }
};

// One CTA per batch row; a thread owns pairs of neighbouring channels (pair index tid + 256 j).  xa_out / xs_out / mix1
// may be NULL.  D even, D <= 8192.
template <typename T>
__global__ void __launch_bounds__(kStageThreads) decode_ln_shift_mix_kernel(int D, const void *x, const void *ln_w,
                                                                          const void *ln_b, float eps, void *prev,
                                                                          const float *mu0, const float *mu1, void *xa_out,
                                                                          void *xs_out, void *mix0, void *mix1) {
    __shared__ float scratch[kStageThreads / 32];
    constexpr int kPairs = kStageMaxPer / 2;
    const size_t row = (size_t)blockIdx.x * D;
    const int npairs = D / 2;
    float2 v[kPairs], pv[kPairs];
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < kPairs; ++j) {
        const int i = threadIdx.x + j * kStageThreads;
        v[j] = i < npairs ? Pair<T>::load(x, row + 2 * i) : make_float2(0.f, 0.f);
        pv[j] = i < npairs ? Pair<T>::load(prev, row + 2 * i) : make_float2(0.f, 0.f);
        s += v[j].x + v[j].y;
    }
    const float mean = block_sum_256(s, scratch) / D;
    float q = 0.f;
#pragma unroll
    for (int j = 0; j < kPairs; ++j) {
        const int i = threadIdx.x + j * kStageThreads;
        if (i < npairs) {
            const float cx = v[j].x - mean, cy = v[j].y - mean;
            q += cx * cx + cy * cy;
        }
    }
    const float rstd = rsqrtf(block_sum_256(q, scratch) / D + eps);
#pragma unroll
    for (int j = 0; j < kPairs; ++j) {
        const int i = threadIdx.x + j * kStageThreads;
        if (i < npairs) {
            const float2 lw = Pair<T>::load(ln_w, 2 * i), lb = Pair<T>::load(ln_b, 2 * i);
            const float2 m0 = *reinterpret_cast<const float2 *>(mu0 + 2 * i);
            // the normalised value is rounded to the activation dtype first, as a separate LayerNorm would leave it
            const float2 xa = make_float2(Pair<T>::round((v[j].x - mean) * rstd * lw.x + lb.x),
                                          Pair<T>::round((v[j].y - mean) * rstd * lw.y + lb.y));
            const float2 xs = make_float2(pv[j].x - xa.x, pv[j].y - xa.y);
            const size_t o = row + 2 * i;
            Pair<T>::store(prev, o, xa);
            if (xa_out) Pair<T>::store(xa_out, o, xa);
            if (xs_out) Pair<T>::store(xs_out, o, xs);
            Pair<T>::store(mix0, o, make_float2(fmaf(xs.x, m0.x, xa.x), fmaf(xs.y, m0.y, xa.y)));
            if (mix1) {
                const float2 m1 = *reinterpret_cast<const float2 *>(mu1 + 2 * i);
                Pair<T>::store(mix1, o, make_float2(fmaf(xs.x, m1.x, xa.x), fmaf(xs.y, m1.y, xa.y)));
            }
        }
    }
}

struct Perm5 { int v[5]; };

// grid (ceil(D / 256), ceil(B / 4), 5), 128 threads: a thread owns two neighbouring channels of one mix m for up to four
// batch rows, so that the R weight rows it needs are independent loads the compiler keeps in flight together.
// h [B, 5R] (the x_mix A product, before tanh), wb [5, R, D], bias [5, D], xa / xs [B, D], out [5, B, D]; D even.
// The result of mix m is written to out[perm.v[m]].
constexpr int kLoraRows = 4;
template <typename T>
__global__ void __launch_bounds__(128) decode_lora_mix_kernel(int B, int D, int R, const void *h, const void *wb,
                                                              const void *bias, const void *xa, const void *xs, void *out,
                                                              Perm5 perm) {
    extern __shared__ float sh[];  // [kLoraRows][R] tanh(h) of this mix
    const int m = blockIdx.z, b0 = blockIdx.y * kLoraRows, nb = min(kLoraRows, B - b0);
    for (int i = threadIdx.x; i < kLoraRows * R; i += blockDim.x) {
        const int rb = i / R, j = i - rb * R;
        sh[i] = rb < nb ? tanhf(load_any(h, sizeof(T) == 4 ? WKV6_F32 : (std::is_same<T, __half>::value ? WKV6_F16 : WKV6_BF16),
                                         (size_t)(b0 + rb) * 5 * R + m * R + j))
                        : 0.f;
    }
    __syncthreads();
    const int d = 2 * (blockIdx.x * blockDim.x + threadIdx.x);
    if (d >= D) return;
    float2 acc[kLoraRows];
#pragma unroll
    for (int rb = 0; rb < kLoraRows; ++rb) acc[rb] = make_float2(0.f, 0.f);
    const size_t wbase = (size_t)m * R * D + d;
#pragma unroll 8
    for (int j = 0; j < R; ++j) {
        const float2 wgt = Pair<T>::load(wb, wbase + (size_t)j * D);
#pragma unroll
        for (int rb = 0; rb < kLoraRows; ++rb) {
            const float hv = sh[rb * R + j];
            acc[rb].x = fmaf(hv, wgt.x, acc[rb].x);
            acc[rb].y = fmaf(hv, wgt.y, acc[rb].y);
        }
    }
    const float2 bm = Pair<T>::load(bias, (size_t)m * D + d);
#pragma unroll
    for (int rb = 0; rb < kLoraRows; ++rb)
        if (rb < nb) {
            const size_t o = (size_t)(b0 + rb) * D + d;
            const float2 a2 = Pair<T>::load(xa, o), s2 = Pair<T>::load(xs, o);
            // l = bias + tanh(.) B rounded to the activation dtype, as the separate matrix product leaves it
            const float lx = Pair<T>::round(bm.x + acc[rb].x), ly = Pair<T>::round(bm.y + acc[rb].y);
            Pair<T>::store(out, (size_t)perm.v[m] * B * D + o, make_float2(fmaf(s2.x, lx, a2.x), fmaf(s2.y, ly, a2.y)));
        }
}

__global__ void __launch_bounds__(256) decode_relu_sq_kernel(size_t n, int dt, const void *x, void *out) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        const float v = fmaxf(load_any(x, dt, i), 0.f);
        store_any(out, dt, i, v * v);
    }
}

__global__ void __launch_bounds__(256) decode_sigmoid_mul_add_kernel(size_t n, int dt, const void *x, const void *r,
                                                                     const void *kv, void *out) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        const float sg = 1.f / (1.f + __expf(-load_any(r, dt, i)));
        store_any(out, dt, i, fmaf(sg, load_any(kv, dt, i), load_any(x, dt, i)));
    }
}

// the kernels move pairs of elements: every tensor pointer must be aligned to two elements (fp32 vectors to 8 bytes)
static bool pair_aligned(int dt, std::initializer_list<const void *> ptrs) {
    const uintptr_t a = 2 * dtype_size(dt);
    for (const void *p : ptrs)
        if (p != nullptr && reinterpret_cast<uintptr_t>(p) % a) return false;
    return true;
}

static int check_dtype(int dt, const char *what) {
    if (dt != WKV6_BF16 && dt != WKV6_F16 && dt != WKV6_F32) return fail(WKV6_ERR_INVALID, "%s: bad dtype %d", what, dt);
    return WKV6_OK;
}

}  // namespace wkv6

using namespace wkv6;

extern "C" {

int wkv6_decode_ln_shift_mix(int32_t B, int32_t D, int32_t dtype, float eps, const void *x, const void *ln_w,
                             const void *ln_b, void *prev, const float *mu0, const float *mu1, void *xa_out, void *xs_out,
                             void *mix0, void *mix1, void *stream) {
    int rc = check_dtype(dtype, "wkv6_decode_ln_shift_mix");
    if (rc) return rc;
    if (B < 0 || D < 2 || D % 2 || D > kStageThreads * kStageMaxPer)
        return fail(WKV6_ERR_UNSUPPORTED, "wkv6_decode_ln_shift_mix: B=%d D=%d (D even, D <= %d)", B, D, kStageThreads * kStageMaxPer);
    if (B == 0) return WKV6_OK;
    if (!x || !ln_w || !ln_b || !prev || !mu0 || !mix0) return fail(WKV6_ERR_INVALID, "wkv6_decode_ln_shift_mix: NULL argument");
    if (mix1 != nullptr && mu1 == nullptr) return fail(WKV6_ERR_INVALID, "wkv6_decode_ln_shift_mix: mix1 without mu1");
    if (!pair_aligned(dtype, {x, ln_w, ln_b, prev, xa_out, xs_out, mix0, mix1}) || !pair_aligned(WKV6_F32, {mu0, mu1}))
        return fail(WKV6_ERR_INVALID, "wkv6_decode_ln_shift_mix: a pointer is not aligned to two elements");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == WKV6_F32)
        decode_ln_shift_mix_kernel<float><<<B, kStageThreads, 0, st>>>(D, x, ln_w, ln_b, eps, prev, mu0, mu1, xa_out, xs_out, mix0, mix1);
    else if (dtype == WKV6_BF16)
        decode_ln_shift_mix_kernel<__nv_bfloat16><<<B, kStageThreads, 0, st>>>(D, x, ln_w, ln_b, eps, prev, mu0, mu1, xa_out, xs_out, mix0, mix1);
    else
        decode_ln_shift_mix_kernel<__half><<<B, kStageThreads, 0, st>>>(D, x, ln_w, ln_b, eps, prev, mu0, mu1, xa_out, xs_out, mix0, mix1);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? WKV6_OK : cuda_fail(e, "decode_ln_shift_mix_kernel launch");
}

int wkv6_decode_lora_mix(int32_t B, int32_t D, int32_t R, int32_t dtype, const void *h, const void *wb, const void *bias,
                         const void *xa, const void *xs, void *out, const int32_t *perm, void *stream) {
    int rc = check_dtype(dtype, "wkv6_decode_lora_mix");
    if (rc) return rc;
    if (B < 0 || D < 2 || D % 2 || R < 1 || R > 256)
        return fail(WKV6_ERR_UNSUPPORTED, "wkv6_decode_lora_mix: B=%d D=%d R=%d (D even, R <= 256)", B, D, R);
    if (B == 0) return WKV6_OK;
    if (!h || !wb || !bias || !xa || !xs || !out) return fail(WKV6_ERR_INVALID, "wkv6_decode_lora_mix: NULL argument");
    if (!pair_aligned(dtype, {wb, bias, xa, xs, out}))
        return fail(WKV6_ERR_INVALID, "wkv6_decode_lora_mix: a pointer is not aligned to two elements");
    Perm5 pm;
    bool seen[5] = {false, false, false, false, false};
    for (int m = 0; m < 5; ++m) {
        pm.v[m] = perm ? perm[m] : m;
        if (pm.v[m] < 0 || pm.v[m] > 4 || seen[pm.v[m]]) return fail(WKV6_ERR_INVALID, "wkv6_decode_lora_mix: perm is not a permutation of 0..4");
        seen[pm.v[m]] = true;
    }
    const dim3 grid((D / 2 + 127) / 128, (B + kLoraRows - 1) / kLoraRows, 5);
    const size_t smem = kLoraRows * R * sizeof(float);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == WKV6_F32) decode_lora_mix_kernel<float><<<grid, 128, smem, st>>>(B, D, R, h, wb, bias, xa, xs, out, pm);
    else if (dtype == WKV6_BF16) decode_lora_mix_kernel<__nv_bfloat16><<<grid, 128, smem, st>>>(B, D, R, h, wb, bias, xa, xs, out, pm);
    else decode_lora_mix_kernel<__half><<<grid, 128, smem, st>>>(B, D, R, h, wb, bias, xa, xs, out, pm);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? WKV6_OK : cuda_fail(e, "decode_lora_mix_kernel launch");
}

int wkv6_decode_relu_sq(int64_t n, int32_t dtype, const void *x, void *out, void *stream) {
    int rc = check_dtype(dtype, "wkv6_decode_relu_sq");
    if (rc) return rc;
    if (n < 0) return fail(WKV6_ERR_INVALID, "wkv6_decode_relu_sq: n=%lld", (long long)n);
    if (n == 0) return WKV6_OK;
    if (!x || !out) return fail(WKV6_ERR_INVALID, "wkv6_decode_relu_sq: NULL argument");
    decode_relu_sq_kernel<<<(unsigned)((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>((size_t)n, dtype, x, out);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? WKV6_OK : cuda_fail(e, "decode_relu_sq_kernel launch");
}

int wkv6_decode_sigmoid_mul_add(int64_t n, int32_t dtype, const void *x, const void *r, const void *kv, void *out,
                                void *stream) {
    int rc = check_dtype(dtype, "wkv6_decode_sigmoid_mul_add");
    if (rc) return rc;
    if (n < 0) return fail(WKV6_ERR_INVALID, "wkv6_decode_sigmoid_mul_add: n=%lld", (long long)n);
    if (n == 0) return WKV6_OK;
    if (!x || !r || !kv || !out) return fail(WKV6_ERR_INVALID, "wkv6_decode_sigmoid_mul_add: NULL argument");
    decode_sigmoid_mul_add_kernel<<<(unsigned)((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>((size_t)n, dtype, x, r, kv,
                                                                                                            out);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? WKV6_OK : cuda_fail(e, "decode_sigmoid_mul_add_kernel launch");
}

}  // extern "C"
