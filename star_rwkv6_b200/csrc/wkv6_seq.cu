// Host side of the sequential variant: argument packing, dtype / head-size dispatch, launches.
#include "wkv6_internal.h"
#include "wkv6_seq.cuh"

namespace wkv6 {

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

int seq_forward(const wkv6_problem *p, const Dims &d, const void *r, const void *k, const void *v,
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

int seq_backward(const wkv6_problem *p, const Dims &d, const void *r, const void *k, const void *v,
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
