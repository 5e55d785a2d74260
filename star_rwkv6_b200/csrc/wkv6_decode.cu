// Single-token state update (decode step): y = r (u k v^T + S), S <- diag(exp(-exp(w))) S + k v^T for every
// (batch, head), with the fp32 state [B,H,64,64] (key, value) streamed once from and once to HBM.  This is the
// T = 1 case of the reference's with-state kernel (rwkv_kernel/jax_kernel/rwkv_kernels.cu:165-190), whose state
// traffic (2*B*H*N*N*4 bytes per step) is all that matters at this size.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "wkv6_internal.h"
#include "wkv6_seq.cuh"

namespace wkv6 {

// Optional output stage (GATE): the per-head GroupNorm of the reference's time-mix block and its gate
// (rwkv6_model.py:158-160 with g = silu(dense_g(xg)), :147), out = (GroupNorm(y) * scale + offset) * silu(g_raw), applied
// to the 64 outputs of this (batch, head) while they are still in shared memory.
struct DecodeGate {
    const void *g_raw;   // [B, H*64] gate projection before SiLU, x_dtype
    const float *scale;  // [H, 64]
    const float *offset; // [H, 64]
    float eps;
};

// 256 threads per (b, h): thread = (row group ig = tid / 16, column quad jq = tid % 16); rows ig, ig+16, ig+32, ig+48.
template <bool GATE>
__global__ void __launch_bounds__(256) decode_kernel(int H, int x_dtype, int y_dtype, int u_dtype, const void *r,
                                                     const void *k, const void *v, const void *w, const void *u,
                                                     const float *s_in, const int64_t *s_map, int s_kinds, float *s_out,
                                                     void *y, DecodeGate gate) {
    __shared__ float sR[64], sK[64], sD[64], sU[64];
    __shared__ __align__(16) float sV[64];
    __shared__ __align__(16) float sY[16][64];
    const int tid = threadIdx.x, bh = blockIdx.x, b = bh / H, h = bh % H;
    const int jq = tid & 15, ig = tid >> 4;
    size_t in_base = 0;
    if (s_in != nullptr) {
        int64_t kind = s_map ? s_map[b] : (s_kinds == 1 ? 0 : b);
        kind = kind < 0 ? 0 : (kind >= s_kinds ? s_kinds - 1 : kind);
        in_base = ((size_t)kind * H + h) * 4096;
    }
    // The state rows are requested first, so that they travel while the operands are staged.  All four are loaded
    // before the first store: s_in may alias s_out (in-place update), which would
    // otherwise force every load to wait for the store before it; a thread only ever writes what it has read.
    float4 st4[4];
#pragma unroll
    for (int m = 0; m < 4; ++m)
        st4[m] = s_in ? __ldcs(reinterpret_cast<const float4 *>(s_in + in_base + (size_t)(ig + 16 * m) * 64 + 4 * jq))
                      : make_float4(0.f, 0.f, 0.f, 0.f);
    if (tid < 64) {
        const size_t o = (size_t)bh * 64 + tid;
        sR[tid] = load_any(r, x_dtype, o);
        sK[tid] = load_any(k, x_dtype, o);
        sV[tid] = load_any(v, x_dtype, o);
        sD[tid] = expf(-expf(load_any(w, x_dtype, o)));
        sU[tid] = load_any(u, u_dtype, (size_t)h * 64 + tid);
    }
    __syncthreads();
    const float4 v4 = *reinterpret_cast<const float4 *>(&sV[4 * jq]);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int m = 0; m < 4; ++m) {
        const int i = ig + 16 * m;
        float4 s = st4[m];
        const float ri = sR[i], ki = sK[i], di = sD[i], uk = sU[i] * ki;
        acc.x = fmaf(ri, fmaf(uk, v4.x, s.x), acc.x); s.x = fmaf(di, s.x, ki * v4.x);
        acc.y = fmaf(ri, fmaf(uk, v4.y, s.y), acc.y); s.y = fmaf(di, s.y, ki * v4.y);
        acc.z = fmaf(ri, fmaf(uk, v4.z, s.z), acc.z); s.z = fmaf(di, s.z, ki * v4.z);
        acc.w = fmaf(ri, fmaf(uk, v4.w, s.w), acc.w); s.w = fmaf(di, s.w, ki * v4.w);
        __stcs(reinterpret_cast<float4 *>(s_out + (size_t)bh * 4096 + (size_t)i * 64 + 4 * jq), s);
    }
    *reinterpret_cast<float4 *>(&sY[ig][4 * jq]) = acc;
    __syncthreads();
    float t = 0.f;
    if (tid < 64) {
#pragma unroll
        for (int g = 0; g < 16; ++g) t += sY[g][tid];
    }
    if (!GATE) {
        if (tid < 64) store_any(y, y_dtype, (size_t)bh * 64 + tid, t);
        return;
    }
    // GroupNorm over the 64 outputs (two warps), on the values as the ungated kernel would have stored them
    __shared__ float sRed[4];
    t = round_to(t, y_dtype);
    const float s1 = warp_sum(t);
    if (tid < 64 && (tid & 31) == 0) sRed[tid >> 5] = s1;
    __syncthreads();
    const float mean = (sRed[0] + sRed[1]) * (1.f / 64.f);
    const float c = tid < 64 ? t - mean : 0.f;
    const float s2 = warp_sum(c * c);
    if (tid < 64 && (tid & 31) == 0) sRed[2 + (tid >> 5)] = s2;
    __syncthreads();
    if (tid < 64) {
        const float rstd = rsqrtf((sRed[2] + sRed[3]) * (1.f / 64.f) + gate.eps);
        const size_t o = (size_t)bh * 64 + tid;
        const float gr = load_any(gate.g_raw, x_dtype, o);
        const float sg = round_to(gr / (1.f + __expf(-gr)), x_dtype);
        store_any(y, y_dtype, o, fmaf(c * rstd, gate.scale[h * 64 + tid], gate.offset[h * 64 + tid]) * sg);
    }
}

}  // namespace wkv6

using namespace wkv6;

static int decode_launch(const wkv6_problem *p, const void *r, const void *k, const void *v, const void *w, const void *u,
                         void *y, const float *s_in, const int64_t *s_map, int32_t s_kinds, float *s_out,
                         const DecodeGate *gate, void *stream) {
    Dims d;
    int rc = validate(p, &d);
    if (rc) return rc;
    if (p->T != 1) return fail(WKV6_ERR_INVALID, "wkv6_decode handles T == 1, got T=%d", p->T);
    if (p->N != 64) return fail(WKV6_ERR_UNSUPPORTED, "wkv6_decode is built for N == 64");
    if (!d.dense) return fail(WKV6_ERR_UNSUPPORTED, "wkv6_decode needs dense [B,1,H*N] tensors");
    if (p->B == 0 || p->H == 0) return WKV6_OK;
    if (!r || !k || !v || !w || !u || !y || !s_out) return fail(WKV6_ERR_INVALID, "NULL argument");
    if (s_in == nullptr && s_map != nullptr) return fail(WKV6_ERR_INVALID, "s_map given without s_in");
    if (s_in != nullptr) {
        if (s_kinds < 1 || s_kinds > p->B) return fail(WKV6_ERR_INVALID, "s_kinds=%d must be in [1, B=%d]", s_kinds, p->B);
        if (s_map == nullptr && s_kinds != 1 && s_kinds != p->B)
            return fail(WKV6_ERR_INVALID, "s_map is required when s_kinds (%d) is neither 1 nor B (%d)", s_kinds, p->B);
        if (reinterpret_cast<uintptr_t>(s_in) % 16) return fail(WKV6_ERR_INVALID, "s_in is not 16-byte aligned");
    }
    if (reinterpret_cast<uintptr_t>(s_out) % 16) return fail(WKV6_ERR_INVALID, "s_out is not 16-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (gate != nullptr) {
        if (!gate->g_raw || !gate->scale || !gate->offset) return fail(WKV6_ERR_INVALID, "wkv6_decode_gated: NULL gate argument");
        decode_kernel<true><<<p->B * p->H, 256, 0, st>>>(p->H, p->x_dtype, p->y_dtype, p->u_dtype, r, k, v, w, u, s_in, s_map,
                                                         s_kinds, s_out, y, *gate);
    } else {
        decode_kernel<false><<<p->B * p->H, 256, 0, st>>>(p->H, p->x_dtype, p->y_dtype, p->u_dtype, r, k, v, w, u, s_in, s_map,
                                                          s_kinds, s_out, y, DecodeGate{nullptr, nullptr, nullptr, 0.f});
    }
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? WKV6_OK : cuda_fail(e, "decode_kernel launch");
}

extern "C" int wkv6_decode(const wkv6_problem *p, const void *r, const void *k, const void *v, const void *w,
                           const void *u, void *y, const float *s_in, const int64_t *s_map, int32_t s_kinds,
                           float *s_out, void *stream) {
    return decode_launch(p, r, k, v, w, u, y, s_in, s_map, s_kinds, s_out, nullptr, stream);
}

extern "C" int wkv6_decode_gated(const wkv6_problem *p, const void *r, const void *k, const void *v, const void *w,
                                 const void *u, const void *g_raw, const float *gn_scale, const float *gn_offset, float eps,
                                 void *out, const float *s_in, const int64_t *s_map, int32_t s_kinds, float *s_out,
                                 void *stream) {
    const DecodeGate gate{g_raw, gn_scale, gn_offset, eps};
    return decode_launch(p, r, k, v, w, u, out, s_in, s_map, s_kinds, s_out, &gate, stream);
}
