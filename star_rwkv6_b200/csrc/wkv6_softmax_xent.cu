// Next-token loss of the language-model head in one pass over the logits: for every row (token) the softmax
// cross-entropy against its target id and, in the same kernel, the gradient with respect to the logits, written over
// the logits themselves:   loss[row] = logsumexp(z) - z[target];   z <- (softmax(z) - onehot(target)) * scale.
// bf16 logits [rows, V], fp32 arithmetic.  A training step of the 1.6B-shape model has 32768 x 65536 logits (4.3 GB in
// bf16): the framework path copies them to fp32, writes fp32 log-probabilities, reads them back in the backward and
// converts the gradient to bf16 again (about 65 GB of traffic, 20 ms); this kernel reads a row once into registers and
// writes the gradient once (8.6 GB).  One CTA of 512 threads per row, 16-byte loads, two block reductions.
// The reference has no trainer (its trainer files are empty); this belongs to the training step built around the op.
#include <cuda_bf16.h>

#include <cstdint>

#include "wkv6_internal.h"

namespace wkv6 {

constexpr int kXentThreads = 512;
constexpr int kXentVecs = 16;  // 16-byte vectors per thread: V <= 512 * 16 * 8 = 65536

__device__ __forceinline__ float xent_block_reduce(float x, bool is_max, float *scratch) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float y = __shfl_xor_sync(0xffffffffu, x, o);
        x = is_max ? fmaxf(x, y) : x + y;
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) scratch[warp] = x;
    __syncthreads();
    float t = scratch[0];
#pragma unroll
    for (int i = 1; i < kXentThreads / 32; ++i) t = is_max ? fmaxf(t, scratch[i]) : t + scratch[i];
    return t;
}

__global__ void __launch_bounds__(kXentThreads) softmax_xent_kernel(int V, __nv_bfloat16 *__restrict__ logits,
                                                                    const int64_t *__restrict__ targets, float scale,
                                                                    float *__restrict__ loss) {
    __shared__ float scratch[kXentThreads / 32];
    const size_t row = blockIdx.x;
    uint4 *zrow = reinterpret_cast<uint4 *>(logits + row * (size_t)V);
    const int nvec = V >> 3;
    uint4 z[kXentVecs];
    float mx = -3.0e38f;
#pragma unroll
    for (int j = 0; j < kXentVecs; ++j) {
        const int i = threadIdx.x + j * kXentThreads;
        if (i < nvec) {
            z[j] = zrow[i];
            const __nv_bfloat162 *p = reinterpret_cast<const __nv_bfloat162 *>(&z[j]);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __bfloat1622float2(p[e]);
                mx = fmaxf(mx, fmaxf(f.x, f.y));
            }
        }
    }
    mx = xent_block_reduce(mx, true, scratch);
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < kXentVecs; ++j) {
        const int i = threadIdx.x + j * kXentThreads;
        if (i < nvec) {
            const __nv_bfloat162 *p = reinterpret_cast<const __nv_bfloat162 *>(&z[j]);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __bfloat1622float2(p[e]);
                sum += __expf(f.x - mx) + __expf(f.y - mx);
            }
        }
    }
    sum = xent_block_reduce(sum, false, scratch);
    const float inv = 1.f / sum;
    int64_t tgt = targets[row];
    const bool ignore = tgt < 0 || tgt >= V;  // such rows contribute neither loss nor gradient
    if (threadIdx.x == 0)
        loss[row] = ignore ? 0.f : (mx + __logf(sum)) - __bfloat162float(logits[row * (size_t)V + tgt]);
    __syncthreads();  // the target logit is read before any thread overwrites the row
    const float sc = ignore ? 0.f : scale;
#pragma unroll
    for (int j = 0; j < kXentVecs; ++j) {
        const int i = threadIdx.x + j * kXentThreads;
        if (i < nvec) {
            __nv_bfloat162 *p = reinterpret_cast<__nv_bfloat162 *>(&z[j]);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __bfloat1622float2(p[e]);
                const int c = 8 * i + 2 * e;
                float gx = __expf(f.x - mx) * inv, gy = __expf(f.y - mx) * inv;
                if (c == tgt) gx -= 1.f;
                if (c + 1 == tgt) gy -= 1.f;
                p[e] = __floats2bfloat162_rn(gx * sc, gy * sc);
            }
            zrow[i] = z[j];
        }
    }
}

}  // namespace wkv6

using namespace wkv6;

extern "C" int wkv6_softmax_xent_bf16(int64_t rows, int32_t V, void *logits_inout, const int64_t *targets, float scale,
                                      float *loss, void *stream) {
    if (rows < 0 || V < 8 || V % 8 || V > kXentThreads * kXentVecs * 8)
        return fail(WKV6_ERR_UNSUPPORTED, "wkv6_softmax_xent_bf16: rows=%lld V=%d (V a multiple of 8, at most %d)", (long long)rows, V,
                    kXentThreads * kXentVecs * 8);
    if (rows == 0) return WKV6_OK;
    if (rows > 2147483647LL) return fail(WKV6_ERR_UNSUPPORTED, "wkv6_softmax_xent_bf16: too many rows");
    if (!logits_inout || !targets || !loss) return fail(WKV6_ERR_INVALID, "wkv6_softmax_xent_bf16: NULL argument");
    if (reinterpret_cast<uintptr_t>(logits_inout) % 16) return fail(WKV6_ERR_INVALID, "wkv6_softmax_xent_bf16: logits must be 16-byte aligned");
    softmax_xent_kernel<<<(unsigned)rows, kXentThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        V, static_cast<__nv_bfloat16 *>(logits_inout), targets, scale, loss);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? WKV6_OK : cuda_fail(e, "softmax_xent_kernel launch");
}
