// Host side of the chunked tensor-core variant: TMA descriptors, launches, workspace sizes.
#include <atomic>
#include <utility>
#include <cuda.h>
#include <cudaTypedefs.h>

#include "wkv6_chunk_bwd.cuh"
#include "wkv6_chunk_bwd_wide.cuh"
#include "wkv6_chunk_fwd.cuh"
#include "wkv6_chunk_summary.cuh"
#include "wkv6_internal.h"

namespace wkv6 {

// SMs of the current device (looked up once per device).
static int sm_count() {
    static std::atomic<int> cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    int n = cached[dev].load();
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev].store(n);
    }
    return n;
}

// Launch with programmatic stream serialization: the kernel's CTAs may become resident while the kernel before it in the
// stream drains.  A kernel launched this way calls ptx::grid_dependency_wait() before its first access to global
// memory, so whatever ran before it has completed by then.  Used for the general backward behind the fast one (its
// launch, which normally finds every flag at zero, then costs 1.5 us instead of 4.5); chaining the other kernels of a
// split step the same way measured no gain.
template <typename... KArgs, typename... Args>
static cudaError_t launch_behind(void (*kernel)(KArgs...), unsigned grid, unsigned block, size_t smem, cudaStream_t st,
                                 Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(block);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// Test hook (wkv6_debug_inject): chunk index whose input tiles the forward never requests, -1 = off.
static std::atomic<int> g_skip_load_chunk{-1};

static PFN_cuTensorMapEncodeTiled_v12000 get_encode() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = []() -> PFN_cuTensorMapEncodeTiled_v12000 {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            return nullptr;
        return reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
    }();
    return fn;
}

// [B][T][C] bf16 tensor seen as (channel, token, batch row); one box is 64 channels x 64 tokens, 128-byte swizzled.
// The driver-API encoder needs a CUDA context current on the calling thread.  A thread that has made no runtime call
// yet (an autograd worker, an XLA host thread) has none: bind the runtime's context of the current device once.
static int ensure_context() {
    static thread_local bool bound = false;
    if (bound) return WKV6_OK;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaSetDevice(dev);
    if (e != cudaSuccess) return cuda_fail(e, "binding the CUDA context to the calling thread");
    bound = true;
    return WKV6_OK;
}

static int make_map(CUtensorMap *m, const void *base, const wkv6_problem *p, const Dims &d, const char *what) {
    if (int rc = ensure_context()) return rc;
    auto enc = get_encode();
    if (!enc) return fail(WKV6_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[3] = {(cuuint64_t)d.C, (cuuint64_t)p->T, (cuuint64_t)p->B};
    cuuint64_t strides[2] = {(cuuint64_t)d.ld * 2, (cuuint64_t)d.bs * 2};
    cuuint32_t box[3] = {64, (cuuint32_t)kChunk, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void *>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(WKV6_ERR_CUDA, "cuTensorMapEncodeTiled(%s) failed with CUresult %d", what, (int)r);
    return WKV6_OK;
}

// The same tensor with the token axis split as token = 16 I + 2 j + p and walked in the order (j, p, I): one box is
// 64 channels x (8 j x 2 p x 4 I), so tile row 16 I + 8 p + j holds token 16 I + 2 j + p of the chunk (the order
// chunk_bwd_wide_kernel<true> works in).  Needs T % 16 == 0; blocks I past the end of the sequence read as zeros
// and are not written.
static int make_map_paired(CUtensorMap *m, const void *base, const wkv6_problem *p, const Dims &d, const char *what) {
    if (int rc = ensure_context()) return rc;
    auto enc = get_encode();
    if (!enc) return fail(WKV6_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[5] = {(cuuint64_t)d.C, 8, 2, (cuuint64_t)(p->T / 16), (cuuint64_t)p->B};
    cuuint64_t strides[4] = {(cuuint64_t)d.ld * 4, (cuuint64_t)d.ld * 2, (cuuint64_t)d.ld * 32, (cuuint64_t)d.bs * 2};
    cuuint32_t box[5] = {64, 8, 2, 4, 1};
    cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void *>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(WKV6_ERR_CUDA, "cuTensorMapEncodeTiled(%s, paired tokens) failed with CUresult %d", what, (int)r);
    return WKV6_OK;
}

bool chunk_supported(const wkv6_problem *p) {
    return p->N == 64 && p->x_dtype == WKV6_BF16 && p->y_dtype == WKV6_BF16 && p->T >= 1;
}

size_t chunk_ckpt_bytes(const wkv6_problem *p) {
    const size_t nchunks = ((size_t)p->T + kChunk - 1) / kChunk;
    return (size_t)p->B * p->H * nchunks * 4096 * sizeof(__nv_bfloat16);
}

int chunk_forward(const wkv6_problem *p, const Dims &d, const void *r, const void *k, const void *v, const void *w,
                  const void *u, void *y, const void *s_in, const int64_t *s_map, int s_kinds, void *s_out,
                  void *ckpt, cudaStream_t st) {
    CUtensorMap mr, mk, mv, mw, my;
    int rc;
    if ((rc = make_map(&mr, r, p, d, "r"))) return rc;
    if ((rc = make_map(&mk, k, p, d, "k"))) return rc;
    if ((rc = make_map(&mv, v, p, d, "v"))) return rc;
    if ((rc = make_map(&mw, w, p, d, "w"))) return rc;
    if ((rc = make_map(&my, y ? y : r, p, d, "y"))) return rc;  // y == NULL: states only, the map is never used
    ChunkFwdArgs a{};
    a.u = u; a.u_dtype = p->u_dtype; a.s_in = s_in; a.s_map = s_map; a.s_kinds = s_kinds; a.s_dtype = p->s_dtype;
    a.s_out = s_out; a.write_y = (y != nullptr); a.ckpt = static_cast<__nv_bfloat16 *>(ckpt);
    a.reverse_state = false; a.dec_out = nullptr; a.B = p->B; a.T = p->T; a.H = p->H;
    a.skip_load_chunk = g_skip_load_chunk.load() + 1;
    cudaError_t e = cudaFuncSetAttribute(chunk_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         ChunkFwdSmem::kAlloc);
    if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(chunk_fwd_kernel)");
    chunk_fwd_kernel<<<p->B * p->H, 256, ChunkFwdSmem::kAlloc, st>>>(mr, mk, mv, mw, my, a);
    e = cudaGetLastError();
    return e == cudaSuccess ? WKV6_OK : cuda_fail(e, "chunk_fwd_kernel launch");
}

// Workspace of the backward: one word per sequence for the hand-over between the fast and the general kernel, then,
// without a checkpoint buffer from the forward, room for the chunk-start states, which the backward first rebuilds
// with the forward kernel (its y output suppressed).
static size_t flag_bytes(const wkv6_problem *p) { return (((size_t)p->B * p->H * sizeof(int)) + 255) & ~(size_t)255; }
size_t chunk_backward_workspace(const wkv6_problem *p, const Dims &, int have_ckpt) {
    return flag_bytes(p) + (have_ckpt ? 0 : chunk_ckpt_bytes(p));
}

int chunk_backward(const wkv6_problem *p, const Dims &d, const void *r, const void *k, const void *v, const void *w,
                   const void *u, const void *gy, void *gr, void *gk, void *gv, void *gw, void *gu, const void *ckpt,
                   void *ws, size_t ws_bytes, cudaStream_t st) {
    return chunk_backward_seeded(p, d, r, k, v, w, u, gy, gr, gk, gv, gw, gu, ckpt, nullptr, ws, ws_bytes, st);
}

int chunk_backward_seeded(const wkv6_problem *p, const Dims &d, const void *r, const void *k, const void *v,
                          const void *w, const void *u, const void *gy, void *gr, void *gk, void *gv, void *gw,
                          void *gu, const void *ckpt, const float *ab_in, void *ws, size_t ws_bytes, cudaStream_t st) {
    int rc;
    // A caller that passes no workspace although it holds the checkpoints still gets a result: from the general kernel alone.
    int *flags = (ws != nullptr && ws_bytes >= flag_bytes(p)) ? static_cast<int *>(ws) : nullptr;
    if (ckpt == nullptr) {
        const size_t need = flag_bytes(p) + chunk_ckpt_bytes(p);
        if (ws == nullptr || ws_bytes < need)
            return fail(WKV6_ERR_WORKSPACE, "backward workspace: need %zu bytes, got %zu", need, ws ? ws_bytes : (size_t)0);
        void *area = static_cast<uint8_t *>(ws) + flag_bytes(p);
        if ((rc = chunk_forward(p, d, r, k, v, w, u, nullptr, nullptr, nullptr, 0, nullptr, area, st))) return rc;
        ckpt = area;
    }
    CUtensorMap mr, mk, mv, mw, mgy, mgr, mgk, mgv, mgw;
    if ((rc = make_map(&mr, r, p, d, "r"))) return rc;
    if ((rc = make_map(&mk, k, p, d, "k"))) return rc;
    if ((rc = make_map(&mv, v, p, d, "v"))) return rc;
    if ((rc = make_map(&mw, w, p, d, "w"))) return rc;
    if ((rc = make_map(&mgy, gy, p, d, "gy"))) return rc;
    if ((rc = make_map(&mgr, gr, p, d, "gr"))) return rc;
    if ((rc = make_map(&mgk, gk, p, d, "gk"))) return rc;
    if ((rc = make_map(&mgv, gv, p, d, "gv"))) return rc;
    if ((rc = make_map(&mgw, gw, p, d, "gw"))) return rc;
    ChunkBwdArgs a{};
    a.u = u; a.u_dtype = p->u_dtype; a.gu = gu; a.gu_dtype = p->gu_dtype;
    a.ckpt = static_cast<const __nv_bfloat16 *>(ckpt); a.B = p->B; a.T = p->T; a.H = p->H;
    a.ab_in = ab_in; a.zero_init = (ab_in == nullptr);  // a seeded call is one segment of a longer sequence
    a.flags = flags;
    cudaError_t e;
    if (flags != nullptr) {  // the fast kernel first; it marks the sequences it has to leave to the general one
        if (p->T % 16 == 0) {  // adjacent tokens per thread (see the kernel)
            CUtensorMap pr, pk, pv, pw, pgy, pgr, pgk, pgv, pgw;
            if ((rc = make_map_paired(&pr, r, p, d, "r"))) return rc;
            if ((rc = make_map_paired(&pk, k, p, d, "k"))) return rc;
            if ((rc = make_map_paired(&pv, v, p, d, "v"))) return rc;
            if ((rc = make_map_paired(&pw, w, p, d, "w"))) return rc;
            if ((rc = make_map_paired(&pgy, gy, p, d, "gy"))) return rc;
            if ((rc = make_map_paired(&pgr, gr, p, d, "gr"))) return rc;
            if ((rc = make_map_paired(&pgk, gk, p, d, "gk"))) return rc;
            if ((rc = make_map_paired(&pgv, gv, p, d, "gv"))) return rc;
            if ((rc = make_map_paired(&pgw, gw, p, d, "gw"))) return rc;
            e = cudaFuncSetAttribute(chunk_bwd_wide_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, WideBwdSmem::kAlloc);
            if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(chunk_bwd_wide_kernel)");
            chunk_bwd_wide_kernel<true><<<p->B * p->H, 256, WideBwdSmem::kAlloc, st>>>(pr, pk, pv, pw, pgy, pgr, pgk, pgv, pgw, a);
        } else {
            e = cudaFuncSetAttribute(chunk_bwd_wide_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, WideBwdSmem::kAlloc);
            if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(chunk_bwd_wide_kernel)");
            chunk_bwd_wide_kernel<false><<<p->B * p->H, 256, WideBwdSmem::kAlloc, st>>>(mr, mk, mv, mw, mgy, mgr, mgk, mgv, mgw, a);
        }
        e = cudaGetLastError();
        if (e != cudaSuccess) return cuda_fail(e, "chunk_bwd_wide_kernel launch");
    }
    auto general = (int64_t)p->B * p->H <= sm_count() ? chunk_bwd_kernel<1> : chunk_bwd_kernel<2>;
    e = cudaFuncSetAttribute(general, cudaFuncAttributeMaxDynamicSharedMemorySize, ChunkBwdSmem::kAlloc);
    if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(chunk_bwd_kernel)");
    e = launch_behind(general, (unsigned)(p->B * p->H), 256, ChunkBwdSmem::kAlloc, st, mr, mk, mv, mw, mgy, mgr, mgk, mgv, mgw, a);
    return e == cudaSuccess ? WKV6_OK : cuda_fail(e, "chunk_bwd_kernel launch");
}

// Summary of every sequence as an affine map of the state: log2 of the total decay per key channel and the state
// the sequence builds from zero.  Forward direction: x1 = k, x2 = v.  Reverse direction (the backward's state):
// x1 = r, x2 = gy.  A kernel of its own (wkv6_chunk_summary.cuh): one scaled operand and one product per chunk.
int chunk_segment_summary(const wkv6_problem *p, const Dims &d, const void *x1, const void *x2, const void *w,
                          bool reverse, float *b_out, float *dec_log2_out, int skip_mod, int skip_rem, cudaStream_t st) {
    CUtensorMap m1, m2, mw;
    int rc;
    if ((rc = make_map(&m1, x1, p, d, "x1"))) return rc;
    if ((rc = make_map(&m2, x2, p, d, "x2"))) return rc;
    if ((rc = make_map(&mw, w, p, d, "w"))) return rc;
    ChunkFwdArgs a{};
    a.u = nullptr; a.u_dtype = WKV6_F32; a.s_dtype = WKV6_F32; a.s_out = b_out; a.B = p->B; a.T = p->T; a.H = p->H;
    a.write_y = false; a.reverse_state = reverse; a.dec_out = dec_log2_out;
    a.skip_mod = skip_mod; a.skip_rem = skip_rem;
    cudaError_t e = cudaFuncSetAttribute(chunk_summary_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         ChunkSumSmem::kAlloc);
    if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(chunk_summary_kernel)");
    chunk_summary_kernel<<<p->B * p->H, 256, ChunkSumSmem::kAlloc, st>>>(m1, m2, mw, a);
    e = cudaGetLastError();
    return e == cudaSuccess ? WKV6_OK : cuda_fail(e, "chunk_summary_kernel launch");
}

// Exclusive scan of affine state maps over the G segments of each sequence:
//   forward : S_in[g] = state entering segment g      = 2^{dec[g-1]} S_in[g-1] + b[g-1],  S_in[0] = s0 (or 0)
//   reverse : A_in[g] = reverse state entering at the end of segment g = 2^{dec[g+1]} A_in[g+1] + b[g+1],  A_in[G-1] = 0
// Segment g of sequence (b, h) sits at batch index b*G + g of the [B*G, H, ...] summary arrays.
__global__ void state_scan_kernel(int B, int H, int G, const float *__restrict__ dec, const float *__restrict__ bsum,
                                  const float *__restrict__ s0, float *__restrict__ out, float *__restrict__ last,
                                  bool reverse) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;  // over B*H*64*64
    if (idx >= (size_t)B * H * 4096) return;
    const int ij = (int)(idx & 4095), i = ij >> 6;
    const int h = (int)((idx >> 12) % H), b = (int)(idx / ((size_t)H * 4096));
    float s = (!reverse && s0 != nullptr) ? s0[idx] : 0.f;
    // eight segments at a time: their loads do not depend on the running state, so they are all requested before the
    // first of them is folded in (one memory round trip per eight segments instead of one per segment)
    for (int g0 = 0; g0 < G; g0 += 8) {
        float d8[8], b8[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const int gg = g0 + e;
            if (gg < G) {
                const size_t seq = ((size_t)(b * G + (reverse ? G - 1 - gg : gg)) * H + h);
                d8[e] = dec[seq * 64 + i];
                b8[e] = bsum[seq * 4096 + ij];
            }
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const int gg = g0 + e;
            if (gg < G) {
                const size_t seq = ((size_t)(b * G + (reverse ? G - 1 - gg : gg)) * H + h);
                out[seq * 4096 + ij] = s;
                s = fmaf(exp2f(d8[e]), s, b8[e]);
            }
        }
    }
    if (last != nullptr) last[idx] = s;
}

int chunk_state_scan(int B, int H, int G, const float *dec, const float *bsum, const float *s0, float *out, float *last,
                     bool reverse, cudaStream_t st) {
    const size_t n = (size_t)B * H * 4096;
    if (n == 0 || G <= 0) return WKV6_OK;
    state_scan_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(B, H, G, dec, bsum, s0, out, last, reverse);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? WKV6_OK : cuda_fail(e, "state_scan_kernel launch");
}

__global__ void sum_rows_kernel(const float *__restrict__ in, long long rows, long long n, float *__restrict__ out) {
    const long long j = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= n) return;
    float s = 0.f;
    long long r0 = 0;
    for (; r0 + 8 <= rows; r0 += 8) {  // eight independent loads in flight, added in row order
        float v8[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) v8[e] = in[(r0 + e) * n + j];
#pragma unroll
        for (int e = 0; e < 8; ++e) s += v8[e];
    }
    for (; r0 < rows; ++r0) s += in[r0 * n + j];
    out[j] = s;
}

int chunk_sum_rows(const float *in, int64_t rows, int64_t n, float *out, cudaStream_t st) {
    sum_rows_kernel<<<(unsigned)((n + 127) / 128), 128, 0, st>>>(in, rows, n, out);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? WKV6_OK : cuda_fail(e, "sum_rows_kernel launch");
}

// Read and clear: the word reports what happened since the previous query.  (cudaMemcpyFromSymbol synchronises.)
int chunk_status() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_chunk_status, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) {
        const int zero = 0;
        if (cudaMemcpyToSymbol(g_chunk_status, &zero, sizeof(int)) != cudaSuccess) return -1;
    }
    return v;
}

// Test hook behind wkv6_debug_inject: the time limit of the in-kernel waits and the chunk whose loads the forward skips.
int chunk_debug_inject(int skip_load_chunk, long long wait_limit_ms) {
    const unsigned long long ns = wait_limit_ms > 0 ? (unsigned long long)wait_limit_ms * 1000000ull : 1000000000ull;
    cudaError_t e = cudaMemcpyToSymbol(ptx::g_wait_limit_ns, &ns, sizeof(ns));
    g_skip_load_chunk.store(skip_load_chunk);  // travels to the forward kernel as an argument of its next launches
    return e == cudaSuccess ? WKV6_OK : cuda_fail(e, "cudaMemcpyToSymbol(debug hooks)");
}

}  // namespace wkv6

#ifdef WKV6_TIMING
extern "C" __attribute__((visibility("default"))) int wkv6_debug_timing(long long *out) {
    return (int)cudaMemcpyFromSymbol(out, wkv6::g_chunk_timing, sizeof(long long) * 64 * 16 * 8);
}
extern "C" __attribute__((visibility("default"))) int wkv6_debug_cta_times(long long *out) {
    return (int)cudaMemcpyFromSymbol(out, wkv6::g_cta_times, sizeof(long long) * 1024 * 8);
}
extern "C" __attribute__((visibility("default"))) int wkv6_debug_cta_sm(int *out) {
    return (int)cudaMemcpyFromSymbol(out, wkv6::g_cta_sm, sizeof(int) * 1024);
}
#endif
