// Sequential (register-state) WKV6 kernels for sm_100a.
//
// One CTA per (batch, head) pair, 4*N threads.  The N x N state is spread over
// the CTA as N columns (or rows) x 4 quarters, N/4 fp32 values per thread, so a
// time step costs three FP32 instructions per state element and one 4-lane
// shuffle reduction; r/k/v/w tiles of 32 time steps are staged through shared
// memory with 128-bit coalesced global loads that are issued one tile ahead.
// All arithmetic is fp32 with precise expf: this is the variant used for fp32
// inputs and the correctness anchor of the chunked tensor-core variant.
//
// Two kernel templates cover the forward and the three backward sweeps:
//   column kernel  out_t[j] = sum_i P_t[i] S[i][j] + X_t[j] c_t,  S[i][j] = d_t[i] S[i][j] + Q_t[i] X_t[j]
//                  c_t = sum_i u[i] P_t[i] Q_t[i]
//        forward : P=r Q=k X=v  out=y   time ascending   (reference: rwkv_kernels.cu:107-160)
//        gv      : P=k Q=r X=gy out=gv  time descending  (reference: rwkv_kernels.cu:295-338)
//   row kernel     out_t[i] = sum_j S[i][j] Y_t[j] + u[i] Q_t[i] (X_t . Y_t),  S[i][j] = d_t[i] S[i][j] + Q_t[i] X_t[j]
//        gr, gu  : Q=k X=v  Y=gy time ascending   (reference: rwkv_kernels.cu:205-250)
//        gk, gw  : Q=r X=gy Y=v  time descending  (reference: rwkv_kernels.cu:252-293, 340-407)
// gw does not use the reference's per-thread T-long local array.  With
// Z_t[i] = sum_j S_t[i][j] A_t[i][j] (A = reverse state) one has
//   r_t gr_t - k_t gk_t = Z_{t-1} - Z_t   and   gw_t = -exp(w_t) (Z_t - k_t sum_j A_t[i][j] v_t[j]),
// so the ascending sweep leaves x_t = r_t*gr_t in an fp32 scratch tensor and the
// descending sweep accumulates Z in double precision.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/wkv6_b200.h"

namespace wkv6 {

constexpr int kSeqTile = 32;  // time steps staged per tile

template <typename T> __device__ __forceinline__ void load8(const T *p, float (&f)[8]);
template <> __device__ __forceinline__ void load8<float>(const float *p, float (&f)[8]) {
    const float4 a = __ldg(reinterpret_cast<const float4 *>(p));
    const float4 b = __ldg(reinterpret_cast<const float4 *>(p) + 1);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
template <> __device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16 *p, float (&f)[8]) {
    const uint4 raw = __ldg(reinterpret_cast<const uint4 *>(p));
    const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&raw);
#pragma unroll
    for (int e = 0; e < 4; ++e) { const float2 t = __bfloat1622float2(h[e]); f[2 * e] = t.x; f[2 * e + 1] = t.y; }
}
template <> __device__ __forceinline__ void load8<__half>(const __half *p, float (&f)[8]) {
    const uint4 raw = __ldg(reinterpret_cast<const uint4 *>(p));
    const __half2 *h = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
    for (int e = 0; e < 4; ++e) { const float2 t = __half22float2(h[e]); f[2 * e] = t.x; f[2 * e + 1] = t.y; }
}

template <typename T> __device__ __forceinline__ void store8(T *p, const float *f);
template <> __device__ __forceinline__ void store8<float>(float *p, const float *f) {
    reinterpret_cast<float4 *>(p)[0] = make_float4(f[0], f[1], f[2], f[3]);
    reinterpret_cast<float4 *>(p)[1] = make_float4(f[4], f[5], f[6], f[7]);
}
template <> __device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16 *p, const float *f) {
    uint4 raw;
    __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&raw);
#pragma unroll
    for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(f[2 * e], f[2 * e + 1]);
    *reinterpret_cast<uint4 *>(p) = raw;
}
template <> __device__ __forceinline__ void store8<__half>(__half *p, const float *f) {
    uint4 raw;
    __half2 *h = reinterpret_cast<__half2 *>(&raw);
#pragma unroll
    for (int e = 0; e < 4; ++e) h[e] = __floats2half2_rn(f[2 * e], f[2 * e + 1]);
    *reinterpret_cast<uint4 *>(p) = raw;
}

// Small tensors (u, gu, states) are typed at run time.
__device__ __forceinline__ float load_any(const void *p, int dtype, size_t i) {
    if (dtype == WKV6_F32) return static_cast<const float *>(p)[i];
    if (dtype == WKV6_BF16) return __bfloat162float(static_cast<const __nv_bfloat16 *>(p)[i]);
    return __half2float(static_cast<const __half *>(p)[i]);
}
__device__ __forceinline__ void store_any(void *p, int dtype, size_t i, float x) {
    if (dtype == WKV6_F32) static_cast<float *>(p)[i] = x;
    else if (dtype == WKV6_BF16) static_cast<__nv_bfloat16 *>(p)[i] = __float2bfloat16_rn(x);
    else static_cast<__half *>(p)[i] = __float2half_rn(x);
}

// x rounded to the storage dtype (what a store followed by a load would give)
__device__ __forceinline__ float round_to(float x, int dtype) {
    if (dtype == WKV6_BF16) return __bfloat162float(__float2bfloat16_rn(x));
    if (dtype == WKV6_F16) return __half2float(__float2half_rn(x));
    return x;
}

__device__ __forceinline__ float quad_sum(float x) {
    x += __shfl_xor_sync(0xffffffffu, x, 1);
    x += __shfl_xor_sync(0xffffffffu, x, 2);
    return x;
}
__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
}

// Position of element i of an N-vector whose four quarters are read with 128-bit
// loads by the four lanes of a quad: each quarter is padded by 4 floats so that the
// four 16-byte reads of one instruction fall into different banks.
template <int N> struct QuarterLayout {
    static constexpr int Q = N / 4;
    static constexpr int PAD = (Q % 4 == 0) ? 4 : 0;
    static constexpr int ROW = 4 * (Q + PAD);
    __device__ static __forceinline__ int pos(int i) { return i + PAD * (i / Q); }
};

struct SeqColArgs {
    const void *P, *Q, *W, *X;  // [B,T,H*N] strided
    const void *u;              // [H,N]
    void *out;                  // [B,T,H*N] strided
    const void *s_in;           // optional [kinds,H,N,N]
    const int64_t *s_map;       // optional [B]
    void *s_out;                // optional [B,H,N,N]
    int s_kinds, s_dtype, u_dtype;
    int B, T, H;
    int64_t ld, bs;
};

template <typename Tx, typename TX, typename Ty, int N, bool REVERSE>
__global__ void __launch_bounds__(4 * N) seq_col_kernel(const SeqColArgs a) {
    using L = QuarterLayout<N>;
    constexpr int TT = kSeqTile, NT = 4 * N, KQ = N / 4, ROW = L::ROW;
    __shared__ __align__(16) float sP[TT * ROW];
    __shared__ __align__(16) float sQ[TT * ROW];
    __shared__ __align__(16) float sD[TT * ROW];
    __shared__ __align__(16) float sX[TT * N];
    __shared__ __align__(16) float sO[TT * N];
    __shared__ float sC[TT];
    __shared__ float sU[N];

    const int tid = threadIdx.x, q = tid & 3, j = tid >> 2;
    const int b = blockIdx.x / a.H, h = blockIdx.x % a.H;
    const int lane = tid & 31, warp = tid >> 5;
    const size_t base = (size_t)b * a.bs + (size_t)h * N;
    const Tx *gP = static_cast<const Tx *>(a.P) + base;
    const Tx *gQ = static_cast<const Tx *>(a.Q) + base;
    const Tx *gW = static_cast<const Tx *>(a.W) + base;
    const TX *gX = static_cast<const TX *>(a.X) + base;
    Ty *gO = static_cast<Ty *>(a.out) + base;

    if (tid < N) sU[tid] = load_any(a.u, a.u_dtype, (size_t)h * N + tid);

    float S[KQ];
    if (a.s_in != nullptr) {
        int64_t kind = a.s_map ? a.s_map[b] : (a.s_kinds == 1 ? 0 : b);
        kind = kind < 0 ? 0 : (kind >= a.s_kinds ? a.s_kinds - 1 : kind);
        const size_t so = ((size_t)kind * a.H + h) * N * N;
#pragma unroll
        for (int ii = 0; ii < KQ; ++ii) S[ii] = load_any(a.s_in, a.s_dtype, so + (size_t)(q * KQ + ii) * N + j);
    } else {
#pragma unroll
        for (int ii = 0; ii < KQ; ++ii) S[ii] = 0.f;
    }

    // this thread stages 8 contiguous elements of one row of each tile
    const int srow = (tid * 8) / N, scol = (tid * 8) % N;
    const int ntiles = (a.T + TT - 1) / TT;
    float fP[8], fQ[8], fW[8], fX[8];
    auto fetch = [&](int tile) {
        const int t = tile * TT + srow;
        if (t < a.T) {
            const size_t o = (size_t)t * a.ld + scol;
            load8<Tx>(gP + o, fP); load8<Tx>(gQ + o, fQ); load8<Tx>(gW + o, fW); load8<TX>(gX + o, fX);
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) { fP[e] = 0.f; fQ[e] = 0.f; fW[e] = 0.f; fX[e] = 0.f; }
        }
    };
    fetch(REVERSE ? ntiles - 1 : 0);

    for (int it = 0; it < ntiles; ++it) {
        const int tile = REVERSE ? ntiles - 1 - it : it;
        const int t0 = tile * TT;
        const int cnt = min(TT, a.T - t0);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const int p = srow * ROW + L::pos(scol + e);
            sP[p] = fP[e];
            sQ[p] = fQ[e];
            sD[p] = expf(-expf(fW[e]));
            sX[srow * N + scol + e] = fX[e];
        }
        __syncthreads();
        if (it + 1 < ntiles) fetch(REVERSE ? tile - 1 : tile + 1);
        for (int row = warp; row < cnt; row += NT / 32) {
            float part = 0.f;
            for (int i = lane; i < N; i += 32) part += sU[i] * sP[row * ROW + L::pos(i)] * sQ[row * ROW + L::pos(i)];
            part = warp_sum(part);
            if (lane == 0) sC[row] = part;
        }
        __syncthreads();
        for (int s = 0; s < cnt; ++s) {
            const int tt = REVERSE ? cnt - 1 - s : s;
            const float xj = sX[tt * N + j];
            const float *rp = sP + tt * ROW + q * (KQ + L::PAD);
            const float *rq = sQ + tt * ROW + q * (KQ + L::PAD);
            const float *rd = sD + tt * ROW + q * (KQ + L::PAD);
            float acc = 0.f;
            if constexpr (KQ % 4 == 0) {
#pragma unroll
                for (int ii = 0; ii < KQ; ii += 4) {
                    const float4 p4 = *reinterpret_cast<const float4 *>(rp + ii);
                    const float4 q4 = *reinterpret_cast<const float4 *>(rq + ii);
                    const float4 d4 = *reinterpret_cast<const float4 *>(rd + ii);
                    acc = fmaf(p4.x, S[ii + 0], acc); S[ii + 0] = fmaf(S[ii + 0], d4.x, q4.x * xj);
                    acc = fmaf(p4.y, S[ii + 1], acc); S[ii + 1] = fmaf(S[ii + 1], d4.y, q4.y * xj);
                    acc = fmaf(p4.z, S[ii + 2], acc); S[ii + 2] = fmaf(S[ii + 2], d4.z, q4.z * xj);
                    acc = fmaf(p4.w, S[ii + 3], acc); S[ii + 3] = fmaf(S[ii + 3], d4.w, q4.w * xj);
                }
            } else {
#pragma unroll
                for (int ii = 0; ii < KQ; ++ii) {
                    acc = fmaf(rp[ii], S[ii], acc);
                    S[ii] = fmaf(S[ii], rd[ii], rq[ii] * xj);
                }
            }
            acc = quad_sum(acc);
            if (q == 0) sO[tt * N + j] = fmaf(xj, sC[tt], acc);
        }
        __syncthreads();
        if (t0 + srow < a.T) store8<Ty>(gO + (size_t)(t0 + srow) * a.ld + scol, sO + srow * N + scol);
    }

    if (a.s_out != nullptr) {
        const size_t so = ((size_t)b * a.H + h) * N * N;
#pragma unroll
        for (int ii = 0; ii < KQ; ++ii) store_any(a.s_out, a.s_dtype, so + (size_t)(q * KQ + ii) * N + j, S[ii]);
    }
}

struct SeqRowArgs {
    const void *r, *k, *w, *v, *gy;  // [B,T,H*N] strided
    const void *u;                   // [H,N]
    void *out;                       // gr (MODE 0) or gk (MODE 1)
    void *gw;                        // MODE 1
    void *gu;                        // MODE 0: [B,H,N]
    float *x;                        // fp32 scratch [B,T,H*N] dense: written by MODE 0, read by MODE 1
    int u_dtype, gu_dtype;
    int B, T, H;
    int64_t ld, bs;
};

template <int N> constexpr int seq_row_smem_bytes() {
    return (kSeqTile * N * 7 + kSeqTile * QuarterLayout<N>::ROW * 2 + kSeqTile + N) * (int)sizeof(float);
}

// MODE 0: ascending time, writes gr, gu and x = r*gr.  MODE 1: descending time, reads x, writes gk and gw.
template <typename Tx, typename Ty, int N, int MODE>
__global__ void __launch_bounds__(4 * N) seq_row_kernel(const SeqRowArgs a) {
    using L = QuarterLayout<N>;
    constexpr int TT = kSeqTile, NT = 4 * N, VQ = N / 4, ROW = L::ROW;
    constexpr bool REVERSE = (MODE == 1);
    extern __shared__ __align__(16) float smem[];
    float *sR = smem;                 // [TT][N]
    float *sK = sR + TT * N;          // [TT][N]
    float *sD = sK + TT * N;          // [TT][N]   decay
    float *sE = sD + TT * N;          // [TT][N]   exp(w)
    float *sXi = sE + TT * N;         // [TT][N]   x read back (MODE 1)
    float *sO1 = sXi + TT * N;        // [TT][N]
    float *sO2 = sO1 + TT * N;        // [TT][N]
    float *sV = sO2 + TT * N;         // [TT][ROW] quarter-padded
    float *sG = sV + TT * ROW;        // [TT][ROW] quarter-padded
    float *sVG = sG + TT * ROW;       // [TT]
    float *sU = sVG + TT;             // [N]

    const int tid = threadIdx.x, q = tid & 3, i = tid >> 2;
    const int b = blockIdx.x / a.H, h = blockIdx.x % a.H;
    const int lane = tid & 31, warp = tid >> 5;
    const size_t base = (size_t)b * a.bs + (size_t)h * N;
    const size_t xbase = ((size_t)b * a.T) * ((size_t)a.H * N) + (size_t)h * N;
    const size_t xld = (size_t)a.H * N;
    const Tx *gR = static_cast<const Tx *>(a.r) + base;
    const Tx *gK = static_cast<const Tx *>(a.k) + base;
    const Tx *gW = static_cast<const Tx *>(a.w) + base;
    const Tx *gV = static_cast<const Tx *>(a.v) + base;
    const Ty *gG = static_cast<const Ty *>(a.gy) + base;
    Ty *gO = static_cast<Ty *>(a.out) + base;
    Ty *gGW = (MODE == 1) ? static_cast<Ty *>(a.gw) + base : nullptr;
    float *gXs = a.x + xbase;

    if (tid < N) sU[tid] = load_any(a.u, a.u_dtype, (size_t)h * N + tid);
    __syncthreads();
    const float ui = sU[i];

    float S[VQ];
#pragma unroll
    for (int jj = 0; jj < VQ; ++jj) S[jj] = 0.f;
    float gu_acc = 0.f;
    double z = 0.0;

    const int srow = (tid * 8) / N, scol = (tid * 8) % N;
    const int ntiles = (a.T + TT - 1) / TT;
    float fR[8], fK[8], fW[8], fV[8], fG[8], fX[8];
    auto fetch = [&](int tile) {
        const int t = tile * TT + srow;
        if (t < a.T) {
            const size_t o = (size_t)t * a.ld + scol;
            load8<Tx>(gR + o, fR); load8<Tx>(gK + o, fK); load8<Tx>(gW + o, fW); load8<Tx>(gV + o, fV);
            load8<Ty>(gG + o, fG);
            if (MODE == 1) {
                // plain loads: x was written by the preceding kernel, and in fp32 mode it aliases gw
                const float4 x0 = *reinterpret_cast<const float4 *>(gXs + (size_t)t * xld + scol);
                const float4 x1 = *reinterpret_cast<const float4 *>(gXs + (size_t)t * xld + scol + 4);
                fX[0] = x0.x; fX[1] = x0.y; fX[2] = x0.z; fX[3] = x0.w;
                fX[4] = x1.x; fX[5] = x1.y; fX[6] = x1.z; fX[7] = x1.w;
            }
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) { fR[e] = 0.f; fK[e] = 0.f; fW[e] = 0.f; fV[e] = 0.f; fG[e] = 0.f; fX[e] = 0.f; }
        }
    };
    fetch(REVERSE ? ntiles - 1 : 0);

    for (int it = 0; it < ntiles; ++it) {
        const int tile = REVERSE ? ntiles - 1 - it : it;
        const int t0 = tile * TT;
        const int cnt = min(TT, a.T - t0);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const int p = srow * N + scol + e;
            const float ew = expf(fW[e]);
            sR[p] = fR[e];
            sK[p] = fK[e];
            sE[p] = ew;
            sD[p] = expf(-ew);
            if (MODE == 1) sXi[p] = fX[e];
            const int pp = srow * ROW + L::pos(scol + e);
            sV[pp] = fV[e];
            sG[pp] = fG[e];
        }
        __syncthreads();
        if (it + 1 < ntiles) fetch(REVERSE ? tile - 1 : tile + 1);
        for (int row = warp; row < cnt; row += NT / 32) {
            float part = 0.f;
            for (int jx = lane; jx < N; jx += 32) part += sV[row * ROW + L::pos(jx)] * sG[row * ROW + L::pos(jx)];
            part = warp_sum(part);
            if (lane == 0) sVG[row] = part;
        }
        __syncthreads();
        for (int s = 0; s < cnt; ++s) {
            const int tt = REVERSE ? cnt - 1 - s : s;
            const float ri = sR[tt * N + i], ki = sK[tt * N + i], di = sD[tt * N + i];
            const float qi = (MODE == 0) ? ki : ri;  // the factor entering the state update
            const float *rv = sV + tt * ROW + q * (VQ + L::PAD);
            const float *rg = sG + tt * ROW + q * (VQ + L::PAD);
            const float *ry = (MODE == 0) ? rg : rv;  // dotted with the state
            const float *rx = (MODE == 0) ? rv : rg;  // enters the state update
            float acc = 0.f;
            if constexpr (VQ % 4 == 0) {
#pragma unroll
                for (int jj = 0; jj < VQ; jj += 4) {
                    const float4 y4 = *reinterpret_cast<const float4 *>(ry + jj);
                    const float4 x4 = *reinterpret_cast<const float4 *>(rx + jj);
                    acc = fmaf(S[jj + 0], y4.x, acc); S[jj + 0] = fmaf(S[jj + 0], di, qi * x4.x);
                    acc = fmaf(S[jj + 1], y4.y, acc); S[jj + 1] = fmaf(S[jj + 1], di, qi * x4.y);
                    acc = fmaf(S[jj + 2], y4.z, acc); S[jj + 2] = fmaf(S[jj + 2], di, qi * x4.z);
                    acc = fmaf(S[jj + 3], y4.w, acc); S[jj + 3] = fmaf(S[jj + 3], di, qi * x4.w);
                }
            } else {
#pragma unroll
                for (int jj = 0; jj < VQ; ++jj) {
                    acc = fmaf(S[jj], ry[jj], acc);
                    S[jj] = fmaf(S[jj], di, qi * rx[jj]);
                }
            }
            acc = quad_sum(acc);
            const float vg = sVG[tt];
            if (MODE == 0) {
                const float gr = fmaf(ui * ki, vg, acc);
                if (q == 0) {
                    sO1[tt * N + i] = gr;
                    sO2[tt * N + i] = ri * gr;
                    gu_acc = fmaf(ri * ki, vg, gu_acc);
                }
            } else {
                const float gk = fmaf(ui * ri, vg, acc);
                if (q == 0) {
                    // Z_t - k_t * sum_j A_t[i][j] v_t[j], then Z_{t-1} = Z_t + r_t gr_t - k_t gk_t
                    const float gcore = (float)(z - (double)ki * (double)acc);
                    sO1[tt * N + i] = gk;
                    // at t = 0 the state before the step is the zero initial state: gw is exactly 0
                    sO2[tt * N + i] = (t0 + tt == 0) ? 0.f : -sE[tt * N + i] * gcore;
                    z += (double)sXi[tt * N + i] - (double)ki * (double)gk;
                }
            }
        }
        __syncthreads();
        if (t0 + srow < a.T) {
            const size_t o = (size_t)(t0 + srow) * a.ld + scol;
            store8<Ty>(gO + o, sO1 + srow * N + scol);
            if (MODE == 0) {
                float *xp = gXs + (size_t)(t0 + srow) * xld + scol;
                reinterpret_cast<float4 *>(xp)[0] = *reinterpret_cast<const float4 *>(sO2 + srow * N + scol);
                reinterpret_cast<float4 *>(xp)[1] = *reinterpret_cast<const float4 *>(sO2 + srow * N + scol + 4);
            } else {
                store8<Ty>(gGW + o, sO2 + srow * N + scol);
            }
        }
    }
    if (MODE == 0 && q == 0) store_any(a.gu, a.gu_dtype, ((size_t)b * a.H + h) * N + i, gu_acc);
}

}  // namespace wkv6
