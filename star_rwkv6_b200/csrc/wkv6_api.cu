// C ABI of the B200 WKV6 library: argument validation, variant choice, launches.
// Declarations and the contract of every entry point: include/wkv6_b200.h.
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "wkv6_internal.h"

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

}  // namespace wkv6

using namespace wkv6;

extern "C" {

const char *wkv6_last_error(void) { return g_err; }

const char *wkv6_version(void) { return "wkv6_b200 0.1 (sm_100a)"; }

int wkv6_device_status(void) { return chunk_status(); }

int wkv6_debug_inject(int32_t skip_load_chunk, int64_t wait_limit_ms) { return chunk_debug_inject(skip_load_chunk, wait_limit_ms); }

int wkv6_copy_2d_async(void *dst, size_t dst_pitch, const void *src, size_t src_pitch, size_t width_bytes, size_t rows,
                       int32_t to_host, void *stream) {
    if (width_bytes == 0 || rows == 0) return WKV6_OK;
    if (dst == nullptr || src == nullptr) return fail(WKV6_ERR_INVALID, "wkv6_copy_2d_async: NULL pointer");
    if (dst_pitch < width_bytes || src_pitch < width_bytes)
        return fail(WKV6_ERR_INVALID, "wkv6_copy_2d_async: a pitch is smaller than the line width");
    const cudaMemcpyKind kind = to_host ? cudaMemcpyDeviceToHost : cudaMemcpyHostToDevice;
    cudaError_t e;
    if (dst_pitch == width_bytes && src_pitch == width_bytes)  // one contiguous block: a plain copy
        e = cudaMemcpyAsync(dst, src, width_bytes * rows, kind, static_cast<cudaStream_t>(stream));
    else
        e = cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, width_bytes, rows, kind, static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? WKV6_OK : cuda_fail(e, "cudaMemcpy2DAsync");
}

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

int wkv6_segment_summary(const wkv6_problem *p, const void *x1, const void *x2, const void *w, int reverse,
                         float *state_out, float *dec_log2_out, void *stream) {
    Dims d;
    int rc = validate(p, &d);
    if (rc) return rc;
    if (!chunk_supported(p)) return fail(WKV6_ERR_UNSUPPORTED, "segment summaries need the chunked variant (N == 64, bf16)");
    if (p->B == 0 || p->H == 0) return WKV6_OK;
    WKV6_CHECK_PTR(x1); WKV6_CHECK_PTR(x2); WKV6_CHECK_PTR(w); WKV6_CHECK_PTR(state_out); WKV6_CHECK_PTR(dec_log2_out);
    return chunk_segment_summary(p, d, x1, x2, w, reverse != 0, state_out, dec_log2_out, 0, 0, static_cast<cudaStream_t>(stream));
}

int wkv6_segment_summary_for_scan(const wkv6_problem *p, const void *x1, const void *x2, const void *w, int reverse, int32_t G,
                                  float *state_out, float *dec_log2_out, void *stream) {
    Dims d;
    int rc = validate(p, &d);
    if (rc) return rc;
    if (!chunk_supported(p)) return fail(WKV6_ERR_UNSUPPORTED, "segment summaries need the chunked variant (N == 64, bf16)");
    if (G < 1 || p->B % G != 0) return fail(WKV6_ERR_INVALID, "wkv6_segment_summary_for_scan: B=%d is not a multiple of G=%d", p->B, G);
    if (p->B == 0 || p->H == 0) return WKV6_OK;
    WKV6_CHECK_PTR(x1); WKV6_CHECK_PTR(x2); WKV6_CHECK_PTR(w); WKV6_CHECK_PTR(state_out); WKV6_CHECK_PTR(dec_log2_out);
    return chunk_segment_summary(p, d, x1, x2, w, reverse != 0, state_out, dec_log2_out, G, reverse ? 0 : G - 1,
                                 static_cast<cudaStream_t>(stream));
}

int wkv6_state_scan(int32_t B, int32_t H, int32_t N, int32_t G, const float *dec_log2, const float *state_sum,
                    const float *s0, float *state_in_out, float *last_out, int reverse, void *stream) {
    if (N != 64) return fail(WKV6_ERR_UNSUPPORTED, "state scan is built for N == 64");
    if (B < 0 || H < 0 || G < 1) return fail(WKV6_ERR_INVALID, "bad B/H/G (%d,%d,%d)", B, H, G);
    if (dec_log2 == nullptr || state_sum == nullptr || state_in_out == nullptr) return fail(WKV6_ERR_INVALID, "NULL argument");
    return chunk_state_scan(B, H, G, dec_log2, state_sum, s0, state_in_out, last_out, reverse != 0, static_cast<cudaStream_t>(stream));
}

int wkv6_sum_rows(const float *in, int64_t rows, int64_t n, float *out, void *stream) {
    if (rows < 0 || n < 0) return fail(WKV6_ERR_INVALID, "wkv6_sum_rows: rows=%lld n=%lld", (long long)rows, (long long)n);
    if (n == 0) return WKV6_OK;
    if (in == nullptr && rows > 0) return fail(WKV6_ERR_INVALID, "wkv6_sum_rows: NULL input");
    if (out == nullptr) return fail(WKV6_ERR_INVALID, "wkv6_sum_rows: NULL output");
    return chunk_sum_rows(in, rows, n, out, static_cast<cudaStream_t>(stream));
}

int wkv6_backward_seeded(const wkv6_problem *p, const void *r, const void *k, const void *v, const void *w, const void *u,
                         const void *gy, void *gr, void *gk, void *gv, void *gw, void *gu, const void *ckpt,
                         const float *ab_in, void *workspace, size_t workspace_bytes, void *stream) {
    Dims d;
    int rc = validate(p, &d);
    if (rc) return rc;
    if (!chunk_supported(p)) return fail(WKV6_ERR_UNSUPPORTED, "the seeded backward needs the chunked variant (N == 64, bf16)");
    if (ckpt == nullptr) return fail(WKV6_ERR_INVALID, "the seeded backward needs the checkpoints of the matching forward");
    if (p->B == 0 || p->H == 0 || p->T == 0) return WKV6_OK;
    WKV6_CHECK_PTR(r); WKV6_CHECK_PTR(k); WKV6_CHECK_PTR(v); WKV6_CHECK_PTR(w); WKV6_CHECK_PTR(gy);
    WKV6_CHECK_PTR(gr); WKV6_CHECK_PTR(gk); WKV6_CHECK_PTR(gv); WKV6_CHECK_PTR(gw);
    if (u == nullptr || gu == nullptr) return fail(WKV6_ERR_INVALID, "u or gu is NULL");
    if (workspace != nullptr && reinterpret_cast<uintptr_t>(workspace) % 16)
        return fail(WKV6_ERR_INVALID, "workspace is not 16-byte aligned");
    return chunk_backward_seeded(p, d, r, k, v, w, u, gy, gr, gk, gv, gw, gu, ckpt, ab_in, workspace, workspace_bytes,
                                 static_cast<cudaStream_t>(stream));
}

}  // extern "C"
