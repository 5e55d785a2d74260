// Host side of the chunked tensor-core variant: TMA descriptors, launches, workspace sizes.
#include <cuda.h>
#include <cudaTypedefs.h>

#include "wkv6_chunk_bwd.cuh"
#include "wkv6_chunk_fwd.cuh"
#include "wkv6_internal.h"

namespace wkv6 {

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
static int make_map(CUtensorMap *m, const void *base, const wkv6_problem *p, const Dims &d, const char *what) {
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
    a.s_out = s_out; a.write_y = (y != nullptr); a.ckpt = static_cast<__nv_bfloat16 *>(ckpt); a.B = p->B; a.T = p->T; a.H = p->H;
    cudaError_t e = cudaFuncSetAttribute(chunk_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         ChunkFwdSmem::kAlloc);
    if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(chunk_fwd_kernel)");
    chunk_fwd_kernel<<<p->B * p->H, 256, ChunkFwdSmem::kAlloc, st>>>(mr, mk, mv, mw, my, a);
    e = cudaGetLastError();
    return e == cudaSuccess ? WKV6_OK : cuda_fail(e, "chunk_fwd_kernel launch");
}

// Without a checkpoint buffer from the forward, the backward first rebuilds the chunk-start states with the
// forward kernel (its y output suppressed) inside the workspace.
size_t chunk_backward_workspace(const wkv6_problem *p, const Dims &, int have_ckpt) {
    return have_ckpt ? 0 : chunk_ckpt_bytes(p);
}

int chunk_backward(const wkv6_problem *p, const Dims &d, const void *r, const void *k, const void *v, const void *w,
                   const void *u, const void *gy, void *gr, void *gk, void *gv, void *gw, void *gu, const void *ckpt,
                   void *ws, size_t ws_bytes, cudaStream_t st) {
    int rc;
    if (ckpt == nullptr) {
        const size_t need = chunk_ckpt_bytes(p);
        if (ws == nullptr || ws_bytes < need)
            return fail(WKV6_ERR_WORKSPACE, "backward workspace: need %zu bytes, got %zu", need, ws ? ws_bytes : (size_t)0);
        if ((rc = chunk_forward(p, d, r, k, v, w, u, nullptr, nullptr, nullptr, 0, nullptr, ws, st))) return rc;
        ckpt = ws;
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
    cudaError_t e = cudaFuncSetAttribute(chunk_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         ChunkBwdSmem::kAlloc);
    if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(chunk_bwd_kernel)");
    chunk_bwd_kernel<<<p->B * p->H, 256, ChunkBwdSmem::kAlloc, st>>>(mr, mk, mv, mw, mgy, mgr, mgk, mgv, mgw, a);
    e = cudaGetLastError();
    return e == cudaSuccess ? WKV6_OK : cuda_fail(e, "chunk_bwd_kernel launch");
}

int chunk_status() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_chunk_status, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

}  // namespace wkv6

#ifdef WKV6_TIMING
extern "C" __attribute__((visibility("default"))) int wkv6_debug_timing(long long *out) {
    return (int)cudaMemcpyFromSymbol(out, wkv6::g_chunk_timing, sizeof(long long) * 64 * 16);
}
#endif
