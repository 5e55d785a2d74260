// C ABI of the B200 WKV6 library: argument validation, variant choice, launches.
// Declarations and the contract of every entry point: include/wkv6_b200.h.
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "wkv6_internal.h"
#include "wkv6_seq.cuh"

namespace wkv6 {

static thread_local char g_err[512] = "";

int fail(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int cuda_fail(cudaError_t e, const char *what) {
    return fail(WKV6_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

size_t dtype_size(int dt) { return dt == WKV6_F32 ? 4 : 2; }

static bool dtype_ok(int dt) { return dt == WKV6_BF16 || dt == WKV6_F16 || dt == WKV6_F32; }

int validate(const wkv6_problem *p, Dims *d) {
    if (p == nullptr) return fail(WKV6_ERR_INVALID, "problem is NULL");
    if (p->B < 0 || p->T < 0 || p->H < 0) return fail(WKV6_ERR_INVALID, "negative B/T/H (%d,%d,%d)", p->B, p->T, p->H);
    if (p->N != 8 && p->N != 16 && p->N != 32 && p->N != 64)
        return fail(WKV6_ERR_UNSUPPORTED, "head size N=%d is not one of 8,16,32,64", p->N);
    if (!dtype_ok(p->x_dtype) || !dtype_ok(p->y_dtype) || !dtype_ok(p->u_dtype) || !dtype_ok(p->gu_dtype) ||
        !dtype_ok(p->s_dtype))
        return fail(WKV6_ERR_INVALID, "unknown dtype code");
    const bool combo = (p->x_dtype == WKV6_F32 && p->y_dtype == WKV6_F32) ||
                       (p->x_dtype == WKV6_BF16 && p->y_dtype == WKV6_BF16) ||
                       (p->x_dtype == WKV6_F16 && p->y_dtype == WKV6_F32) ||
                       (p->x_dtype == WKV6_BF16 && p->y_dtype == WKV6_F32);
    if (!combo) return fail(WKV6_ERR_UNSUPPORTED, "unsupported (x_dtype,y_dtype)=(%d,%d)", p->x_dtype, p->y_dtype);
    if (p->variant < WKV6_VARIANT_AUTO || p->variant > WKV6_VARIANT_CHUNK)
        return fail(WKV6_ERR_INVALID, "unknown variant %d", p->variant);
    const int64_t C = (int64_t)p->H * p->N;
    d->C = C;
    d->ld = p->row_stride ? p->row_stride : C;
    d->bs = p->batch_stride ? p->batch_stride : (int64_t)p->T * d->ld;
    if (d->ld < C) return fail(WKV6_ERR_INVALID, "row_stride %lld < H*N %lld", (long long)d->ld, (long long)C);
    if (d->ld % 8 || d->bs % 8) return fail(WKV6_ERR_INVALID, "row_stride and batch_stride must be multiples of 8 elements");
    d->dense = (d->ld == C) && (d->bs == (int64_t)p->T * C);
    return WKV6_OK;
}

static int check_ptr(const void *ptr, const char *name) {
    if (ptr == nullptr) return fail(WKV6_ERR_INVALID, "%s is NULL", name);
    if (reinterpret_cast<uintptr_t>(ptr) % 16) return fail(WKV6_ERR_INVALID, "%s is not 16-byte aligned", name);
    return WKV6_OK;
}

#define WKV6_CHECK_PTR(ptr) do { int rc_ = check_ptr(ptr, #ptr); if (rc_) return rc_; } while (0)

int resolve_variant(const wkv6_problem *p) {
    if (p->variant == WKV6_VARIANT_SEQ) return WKV6_VARIANT_SEQ;
    const bool chunk_ok = chunk_supported(p);
    if (p->variant == WKV6_VARIANT_CHUNK) return chunk_ok ? (int)WKV6_VARIANT_CHUNK : (int)WKV6_ERR_UNSUPPORTED;
    return chunk_ok ? WKV6_VARIANT_CHUNK : WKV6_VARIANT_SEQ;
}

// ---- sequential variant -------------------------------------------------------------------------

template <typename Tx, typename TX, typename Ty, int N, bool REV>
static int launch_col(const SeqColArgs &a, cudaStream_t st) {
    seq_col_kernel<Tx, TX, Ty, N, REV><<<a.B * a.H, 4 * N, 0, st>>>(a);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? WKV6_OK : cuda_fail(e, "seq_col_kernel launch");
}

template <typename Tx, typename Ty, int N, int MODE>
static int launch_row(const SeqRowArgs &a, cudaStream_t st) {
    constexpr int smem = seq_row_smem_bytes<N>();
    auto kern = seq_row_kernel<Tx, Ty, N, MODE>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(seq_row_kernel)");
    }
    kern<<<a.B * a.H, 4 * N, smem, st>>>(a);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? WKV6_OK : cuda_fail(e, "seq_row_kernel launch");
}

template <typename Tx, typename Ty, int N>
static int seq_forward_t(const SeqColArgs &a, cudaStream_t st) {
    return launch_col<Tx, Tx, Ty, N, false>(a, st);
}

template <typename Tx, typename Ty, int N>
static int seq_backward_t(const SeqRowArgs &ra, const SeqColArgs &ca, void *gk, cudaStream_t st) {
    int rc = launch_row<Tx, Ty, N, 0>(ra, st);  // gr, gu, x
    if (rc) return rc;
    SeqRowArgs rb = ra;
    rb.out = gk;
    rc = launch_row<Tx, Ty, N, 1>(rb, st);      // gk, gw
    if (rc) return rc;
    return launch_col<Tx, Ty, Ty, N, true>(ca, st);
}

#define WKV6_DISPATCH_N(N_, Tx, Ty, CALL)                    \
    switch (N_) {                                            \
        case 8: { constexpr int kN = 8; return CALL(Tx, Ty, kN); }   \
        case 16: { constexpr int kN = 16; return CALL(Tx, Ty, kN); } \
        case 32: { constexpr int kN = 32; return CALL(Tx, Ty, kN); } \
        default: { constexpr int kN = 64; return CALL(Tx, Ty, kN); } \
    }

#define WKV6_DISPATCH(p, CALL)                                                                   \
    do {                                                                                         \
        if ((p)->x_dtype == WKV6_F32) { WKV6_DISPATCH_N((p)->N, float, float, CALL) }            \
        else if ((p)->x_dtype == WKV6_F16) { WKV6_DISPATCH_N((p)->N, __half, float, CALL) }      \
        else if ((p)->y_dtype == WKV6_BF16) { WKV6_DISPATCH_N((p)->N, __nv_bfloat16, __nv_bfloat16, CALL) } \
        else { WKV6_DISPATCH_N((p)->N, __nv_bfloat16, float, CALL) }                             \
    } while (0)

static int seq_forward(const wkv6_problem *p, const Dims &d, const void *r, const void *k, const void *v,
                       const void *w, const void *u, void *y, const void *s_in, const int64_t *s_map,
                       int s_kinds, void *s_out, cudaStream_t st) {
    SeqColArgs a{};
    a.P = r; a.Q = k; a.W = w; a.X = v; a.u = u; a.out = y;
    a.s_in = s_in; a.s_map = s_map; a.s_out = s_out; a.s_kinds = s_kinds; a.s_dtype = p->s_dtype;
    a.u_dtype = p->u_dtype; a.B = p->B; a.T = p->T; a.H = p->H; a.ld = d.ld; a.bs = d.bs;
#define CALL_FWD(Tx, Ty, kN) seq_forward_t<Tx, Ty, kN>(a, st)
    WKV6_DISPATCH(p, CALL_FWD);
#undef CALL_FWD
}

size_t seq_backward_workspace(const wkv6_problem *p, const Dims &d) {
    if (p->y_dtype == WKV6_F32 && d.dense) return 0;  // x = r*gr is staged in the gw buffer itself
    return (size_t)p->B * p->T * d.C * sizeof(float);
}

static int seq_backward(const wkv6_problem *p, const Dims &d, const void *r, const void *k, const void *v,
                        const void *w, const void *u, const void *gy, void *gr, void *gk, void *gv, void *gw,
                        void *gu, void *ws, size_t ws_bytes, cudaStream_t st) {
    const size_t need = seq_backward_workspace(p, d);
    if (need > 0 && (ws == nullptr || ws_bytes < need))
        return fail(WKV6_ERR_WORKSPACE, "backward workspace: need %zu bytes, got %zu", need, ws ? ws_bytes : (size_t)0);
    SeqRowArgs ra{};
    ra.r = r; ra.k = k; ra.w = w; ra.v = v; ra.gy = gy; ra.u = u; ra.out = gr; ra.gw = gw; ra.gu = gu;
    ra.x = need ? static_cast<float *>(ws) : static_cast<float *>(gw);
    ra.u_dtype = p->u_dtype; ra.gu_dtype = p->gu_dtype; ra.B = p->B; ra.T = p->T; ra.H = p->H; ra.ld = d.ld; ra.bs = d.bs;
    SeqColArgs ca{};
    ca.P = k; ca.Q = r; ca.W = w; ca.X = gy; ca.u = u; ca.out = gv; ca.u_dtype = p->u_dtype;
    ca.s_dtype = WKV6_F32; ca.B = p->B; ca.T = p->T; ca.H = p->H; ca.ld = d.ld; ca.bs = d.bs;
#define CALL_BWD(Tx, Ty, kN) seq_backward_t<Tx, Ty, kN>(ra, ca, gk, st)
    WKV6_DISPATCH(p, CALL_BWD);
#undef CALL_BWD
}

}  // namespace wkv6

using namespace wkv6;

extern "C" {

const char *wkv6_last_error(void) { return g_err; }

const char *wkv6_version(void) { return "wkv6_b200 0.1 (sm_100a)"; }

int wkv6_resolve_variant(const wkv6_problem *p) {
    Dims d;
    int rc = validate(p, &d);
    if (rc) return rc;
    rc = resolve_variant(p);
    if (rc < 0) return fail(rc, "the chunked variant needs N == 64, bf16 r/k/v/w and T a multiple of its chunk length");
    return rc;
}

int wkv6_forward(const wkv6_problem *p, const void *r, const void *k, const void *v, const void *w, const void *u,
                 void *y, const void *s_in, const int64_t *s_map, int32_t s_kinds, void *s_out, void *ckpt,
                 void *stream) {
    Dims d;
    int rc = validate(p, &d);
    if (rc) return rc;
    if (s_in == nullptr && s_map != nullptr) return fail(WKV6_ERR_INVALID, "s_map given without s_in");
    if (s_in != nullptr) {
        if (s_kinds < 1 || s_kinds > p->B) return fail(WKV6_ERR_INVALID, "s_kinds=%d must be in [1, B=%d]", s_kinds, p->B);
        if (s_map == nullptr && s_kinds != 1 && s_kinds != p->B)
            return fail(WKV6_ERR_INVALID, "s_map is required when s_kinds (%d) is neither 1 nor B (%d)", s_kinds, p->B);
    }
    if (p->B == 0 || p->T == 0 || p->H == 0) {
        // nothing to compute; a requested final state equals the initial one only for T == 0, which the
        // host wrappers handle before calling in.
        return WKV6_OK;
    }
    WKV6_CHECK_PTR(r); WKV6_CHECK_PTR(k); WKV6_CHECK_PTR(v); WKV6_CHECK_PTR(w); WKV6_CHECK_PTR(y);
    if (u == nullptr) return fail(WKV6_ERR_INVALID, "u is NULL");
    const int variant = resolve_variant(p);
    if (variant < 0) return fail(variant, "the chunked variant does not cover this problem");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (variant == WKV6_VARIANT_CHUNK) return chunk_forward(p, d, r, k, v, w, u, y, s_in, s_map, s_kinds, s_out, ckpt, st);
    return seq_forward(p, d, r, k, v, w, u, y, s_in, s_map, s_kinds, s_out, st);
}

size_t wkv6_ckpt_bytes(const wkv6_problem *p) {
    Dims d;
    if (validate(p, &d)) return 0;
    if (resolve_variant(p) != WKV6_VARIANT_CHUNK) return 0;
    return chunk_ckpt_bytes(p);
}

size_t wkv6_backward_workspace_bytes(const wkv6_problem *p, int have_ckpt) {
    Dims d;
    if (validate(p, &d)) return 0;
    if (resolve_variant(p) == WKV6_VARIANT_CHUNK) return chunk_backward_workspace(p, d, have_ckpt);
    return seq_backward_workspace(p, d);
}

int wkv6_backward(const wkv6_problem *p, const void *r, const void *k, const void *v, const void *w, const void *u,
                  const void *gy, void *gr, void *gk, void *gv, void *gw, void *gu, const void *ckpt,
                  void *workspace, size_t workspace_bytes, void *stream) {
    Dims d;
    int rc = validate(p, &d);
    if (rc) return rc;
    if (p->B == 0 || p->H == 0) return WKV6_OK;
    if (gu == nullptr) return fail(WKV6_ERR_INVALID, "gu is NULL");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (p->T == 0) {
        cudaError_t e = cudaMemsetAsync(gu, 0, (size_t)p->B * d.C * dtype_size(p->gu_dtype), st);
        return e == cudaSuccess ? WKV6_OK : cuda_fail(e, "cudaMemsetAsync(gu)");
    }
    WKV6_CHECK_PTR(r); WKV6_CHECK_PTR(k); WKV6_CHECK_PTR(v); WKV6_CHECK_PTR(w); WKV6_CHECK_PTR(gy);
    WKV6_CHECK_PTR(gr); WKV6_CHECK_PTR(gk); WKV6_CHECK_PTR(gv); WKV6_CHECK_PTR(gw);
    if (u == nullptr) return fail(WKV6_ERR_INVALID, "u is NULL");
    if (workspace != nullptr && reinterpret_cast<uintptr_t>(workspace) % 16)
        return fail(WKV6_ERR_INVALID, "workspace is not 16-byte aligned");
    const int variant = resolve_variant(p);
    if (variant < 0) return fail(variant, "the chunked variant does not cover this problem");
    if (variant == WKV6_VARIANT_CHUNK)
        return chunk_backward(p, d, r, k, v, w, u, gy, gr, gk, gv, gw, gu, ckpt, workspace, workspace_bytes, st);
    return seq_backward(p, d, r, k, v, w, u, gy, gr, gk, gv, gw, gu, workspace, workspace_bytes, st);
}

}  // extern "C"
