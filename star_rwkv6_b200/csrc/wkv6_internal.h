// Declarations shared by the translation units of the library (not part of the public ABI).
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "../../include/wkv6_b200.h"

namespace wkv6 {

struct Dims {
    int64_t C;    // H*N
    int64_t ld;   // resolved row stride (elements)
    int64_t bs;   // resolved batch stride (elements)
    bool dense;   // ld == C and bs == T*C
};

int fail(int code, const char *fmt, ...);
int cuda_fail(cudaError_t e, const char *what);
size_t dtype_size(int dt);
int validate(const wkv6_problem *p, Dims *d);

// sequential variant (wkv6_seq.cu)
int seq_forward(const wkv6_problem *p, const Dims &d, const void *r, const void *k, const void *v, const void *w,
                const void *u, void *y, const void *s_in, const int64_t *s_map, int s_kinds, void *s_out,
                cudaStream_t st);
size_t seq_backward_workspace(const wkv6_problem *p, const Dims &d);
int seq_backward(const wkv6_problem *p, const Dims &d, const void *r, const void *k, const void *v, const void *w,
                 const void *u, const void *gy, void *gr, void *gk, void *gv, void *gw, void *gu, void *ws,
                 size_t ws_bytes, cudaStream_t st);

// chunked tensor-core variant (wkv6_chunk.cu)
bool chunk_supported(const wkv6_problem *p);
int chunk_status();
int chunk_debug_inject(int skip_load_chunk, long long wait_limit_ms);
size_t chunk_ckpt_bytes(const wkv6_problem *p);
int chunk_sum_rows(const float *in, int64_t rows, int64_t n, float *out, cudaStream_t st);
size_t chunk_backward_workspace(const wkv6_problem *p, const Dims &d, int have_ckpt);
int chunk_forward(const wkv6_problem *p, const Dims &d, const void *r, const void *k, const void *v, const void *w,
                  const void *u, void *y, const void *s_in, const int64_t *s_map, int s_kinds, void *s_out,
                  void *ckpt, cudaStream_t st);
int chunk_backward(const wkv6_problem *p, const Dims &d, const void *r, const void *k, const void *v, const void *w,
                   const void *u, const void *gy, void *gr, void *gk, void *gv, void *gw, void *gu, const void *ckpt,
                   void *ws, size_t ws_bytes, cudaStream_t st);

int chunk_backward_seeded(const wkv6_problem *p, const Dims &d, const void *r, const void *k, const void *v,
                          const void *w, const void *u, const void *gy, void *gr, void *gk, void *gv, void *gw,
                          void *gu, const void *ckpt, const float *ab_in, void *ws, size_t ws_bytes, cudaStream_t st);
int chunk_segment_summary(const wkv6_problem *p, const Dims &d, const void *x1, const void *x2, const void *w,
                          bool reverse, float *b_out, float *dec_log2_out, int skip_mod, int skip_rem, cudaStream_t st);
int chunk_state_scan(int B, int H, int G, const float *dec, const float *bsum, const float *s0, float *out, float *last,
                     bool reverse, cudaStream_t st);
int resolve_variant(const wkv6_problem *p);

}  // namespace wkv6
