/*
 * wkv6_b200 — C ABI of the B200 (sm_100a) RWKV-6 WKV recurrence.
 *
 * Plain pointers and sizes only; every function enqueues work on the CUDA
 * stream it is given and returns without synchronising.  Nothing here
 * allocates device memory: outputs, checkpoints and workspaces are the
 * caller's.  All entry points return WKV6_OK (0) or a negative error code;
 * wkv6_last_error() gives the message of the last failure on the calling
 * thread.
 *
 * Tensor conventions
 *   r, k, v, w, gy, y, gr, gk, gv, gw : [B, T, H*N], element (b, t, c) at
 *        b*batch_stride + t*row_stride + c   (strides in elements; 0 selects the
 *        dense value).  A head-sharded view of a wider tensor is expressed by a
 *        row_stride larger than H*N, with no copy.
 *   u    : [H, N]
 *   gu   : [B, H, N]  per batch row; the caller sums over B, exactly as the
 *        reference does outside its kernels.
 *   state: S[b, h, key, value], N*N contiguous values per (b, h).  This is the
 *        layout of the reference's non-CUDA operator
 *        (rwkv_kernel/ops_rwkv_kernal.py:85-91).
 *   y_t[j]   = sum_i r_t[i] * (u[i]*k_t[i]*v_t[j] + S_{t-1}[i][j])
 *   S_t[i][j] = exp(-exp(w_t[i])) * S_{t-1}[i][j] + k_t[i]*v_t[j]
 */
#ifndef WKV6_B200_H_
#define WKV6_B200_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define WKV6_API __attribute__((visibility("default")))
#else
#define WKV6_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* Element types.  Values equal the reference's gpu_ops::ElementType
 * (rwkv_kernel/jax_kernel/kernels.h:30). */
enum { WKV6_BF16 = 0, WKV6_F16 = 1, WKV6_F32 = 2 };

/* Kernel variants.  AUTO picks per shape and dtype. */
enum { WKV6_VARIANT_AUTO = 0, WKV6_VARIANT_SEQ = 1, WKV6_VARIANT_CHUNK = 2 };

enum {
    WKV6_OK = 0,
    WKV6_ERR_INVALID = -1,     /* bad shape, dtype combination, null pointer, misalignment */
    WKV6_ERR_UNSUPPORTED = -2, /* valid request that no compiled kernel covers */
    WKV6_ERR_WORKSPACE = -3,   /* workspace / checkpoint buffer missing or too small */
    WKV6_ERR_CUDA = -4         /* a CUDA runtime call failed; message carries cudaGetErrorString */
};

/* Problem description shared by all entry points.  Replaces the compile-time
 * _N_/_T_ macros and the WKVDescriptor blob of the reference
 * (rwkv_kernel/jax_kernel/kernels.h:24-42): N and T are runtime values. */
typedef struct wkv6_problem {
    int32_t B, T, H, N;   /* N (head size) in {8, 16, 32, 64}; the chunked variant needs N == 64 */
    int32_t x_dtype;      /* r, k, v, w */
    int32_t y_dtype;      /* y, gy, gr, gk, gv, gw.  Allowed (x, y): (F32,F32) (BF16,BF16) (F16,F32) (BF16,F32) */
    int32_t u_dtype;      /* u: F32, or the same as x_dtype */
    int32_t gu_dtype;     /* gu: F32 or y_dtype */
    int32_t s_dtype;      /* s_in / s_out: F32 or BF16 */
    int32_t variant;      /* WKV6_VARIANT_* */
    int64_t row_stride;   /* elements between consecutive tokens; 0 = H*N */
    int64_t batch_stride; /* elements between batch rows; 0 = T*row_stride */
} wkv6_problem;

WKV6_API const char *wkv6_last_error(void);
WKV6_API const char *wkv6_version(void);

/* Error word of the device kernels on the current device: 0, or the code of a bounded in-kernel wait that
 * ran out (the kernel then unwinds - it drains its outstanding copies, frees its tensor memory, returns - and
 * leaves its outputs undefined).  Every wait is limited to one second of the GPU's global timer.  The call
 * synchronises the device and clears the word: it reports what happened since the previous query.  The
 * reference has no counterpart: its kernels contain no waits. */
WKV6_API int wkv6_device_status(void);

/* Host-side failure injection for tests of the error path above; no counterpart in the reference.
 * wait_limit_ms > 0 sets the time limit of the in-kernel waits on the current device (0 restores one second), and
 * skip_load_chunk >= 0 makes every later launch of the chunked forward (from this process, on any device) never
 * request the input tiles of that 64-token chunk, so that the wait for them runs out with nothing in flight (-1
 * restores normal operation).  The kernel then returns normally with wkv6_device_status() != 0; nothing faults,
 * traps or hangs.  Synchronises the device. */
WKV6_API int wkv6_debug_inject(int32_t skip_load_chunk, int64_t wait_limit_ms);

/* Which variant AUTO resolves to for this problem (WKV6_VARIANT_SEQ / _CHUNK), or a negative error. */
WKV6_API int wkv6_resolve_variant(const wkv6_problem *p);

/*
 * Forward.  Replaces kernel_forward / kernel_forward_state and their host launchers
 * (rwkv_kernel/jax_kernel/rwkv_kernels.cu:107-203, 413-433; rwkv_kernel/torch_kernel/wkv6_cuda.cu:12-107, 323-339).
 *   s_in   : optional [s_kinds, H, N, N] initial states (NULL = zero state)
 *   s_map  : optional int64[B] device array, row b starts from s_in[s_map[b]]; NULL = identity when
 *            s_kinds == B, all-zero when s_kinds == 1.  Values must lie in [0, s_kinds): the caller
 *            validates them (the kernel clamps instead of trapping).
 *   s_out  : optional [B, H, N, N] final states
 *   ckpt   : optional checkpoint buffer of wkv6_ckpt_bytes(p) bytes.  When given, the forward stores what
 *            the backward of the same variant needs so that it does not recompute it.
 */
WKV6_API int wkv6_forward(const wkv6_problem *p, const void *r, const void *k, const void *v, const void *w,
                 const void *u, void *y, const void *s_in, const int64_t *s_map, int32_t s_kinds,
                 void *s_out, void *ckpt, void *stream);

WKV6_API size_t wkv6_ckpt_bytes(const wkv6_problem *p);

/*
 * Backward: gradients of sum(y*gy) with respect to r, k, v, w, u for a zero initial state; no gradient
 * flows through a returned state.  Replaces kernel_backward_101/102/103/201 and HostApplyGradient
 * (rwkv_kernel/jax_kernel/rwkv_kernels.cu:205-407, 435-444; rwkv_kernel/torch_kernel/wkv6_cuda.cu:112-314, 341-353).
 * Every element of gr, gk, gv, gw, gu is written.
 *   ckpt      : the buffer a forward of the same problem filled, or NULL (then the backward rebuilds it
 *               inside the workspace)
 *   workspace : wkv6_backward_workspace_bytes(p, ckpt != NULL) bytes of device scratch (may be NULL when 0).
 *               The chunked variant keeps one word per sequence there, with which its fast kernel (one decay
 *               reference point per chunk) hands the sequences it cannot finish to the general kernel; with a
 *               ckpt buffer but no workspace the call still succeeds, through the general kernel alone, slower.
 */
WKV6_API int wkv6_backward(const wkv6_problem *p, const void *r, const void *k, const void *v, const void *w,
                  const void *u, const void *gy, void *gr, void *gk, void *gv, void *gw, void *gu,
                  const void *ckpt, void *workspace, size_t workspace_bytes, void *stream);

WKV6_API size_t wkv6_backward_workspace_bytes(const wkv6_problem *p, int have_ckpt);

/*
 * Backward without any caller-provided scratch.  It has no counterpart in the reference.
 *
 * Some hosts of this library may not allocate device memory around a call and have no buffer to lend it: a
 * handler for XLA's legacy custom-call ABI sees only the operand and result buffers XLA planned
 * (rwkv_backward_fn has eleven of them and no workspace), and code running under a fixed memory plan or inside
 * a region where the CUDA allocator must not be entered is in the same position.  For them this entry point
 * runs the sequential backward (always that variant, whatever p->variant says) with its fp32 scratch - one
 * value per (token, channel) - taken from an array that is compiled into the library image.
 *
 *   - Limit: B*T*H*N <= wkv6_static_scratch_bytes()/4 = 8 388 608 (32 MiB of scratch).  Larger problems are
 *     rejected with WKV6_ERR_WORKSPACE and a message; use wkv6_backward with a workspace for them.
 *   - The array costs 32 MiB on every GPU that loads the library, for the life of the process.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress); make that
 *     first call outside any stream capture.  No call allocates or frees memory.
 *   - All calls on one device share the one array and it keeps whatever the last call left in it.  Nothing in it
 *     needs clearing between calls (each call overwrites what it later reads), but two calls whose kernels
 *     overlap on the GPU - different streams, or different host threads - would corrupt each other: order them.
 * Arguments and results are those of wkv6_backward.
 */
WKV6_API int wkv6_backward_static_scratch(const wkv6_problem *p, const void *r, const void *k, const void *v,
                                          const void *w, const void *u, const void *gy, void *gr, void *gk, void *gv,
                                          void *gw, void *gu, void *stream);
WKV6_API size_t wkv6_static_scratch_bytes(void);

/*
 * Decode step: the T == 1 case of the forward with state, as its own streaming kernel (one read and one write of
 * the fp32 state [B,H,N,N], N == 64).  Replaces kernel_forward_state at T = 1
 * (rwkv_kernel/jax_kernel/rwkv_kernels.cu:165-190).  s_in may be NULL (zero state) and may equal s_out (in-place
 * update, the serving loop's case) as long as no s_map row is shared between batch rows.
 */
WKV6_API int wkv6_decode(const wkv6_problem *p, const void *r, const void *k, const void *v, const void *w,
                         const void *u, void *y, const float *s_in, const int64_t *s_map, int32_t s_kinds,
                         float *s_out, void *stream);

/*
 * Decode step with the output stage of the time-mix block fused behind the recurrence:
 *   out = (GroupNorm_per_head(y) * gn_scale + gn_offset) * silu(g_raw)
 * (rwkv6_model.py:147 g = silu(dense_g(xg)), :158-160 group_norm then the gate; GroupNorm :84-114 with eps 64e-5).
 * g_raw is the gate projection before SiLU, [B,1,H*N] of x_dtype; gn_scale / gn_offset are fp32 [H,N].
 * All other arguments as wkv6_decode.
 */
WKV6_API int wkv6_decode_gated(const wkv6_problem *p, const void *r, const void *k, const void *v, const void *w,
                               const void *u, const void *g_raw, const float *gn_scale, const float *gn_offset, float eps,
                               void *out, const float *s_in, const int64_t *s_map, int32_t s_kinds, float *s_out,
                               void *stream);

/*
 * Element-wise stages of a decode step (T == 1) around the matrix products of an RWKV-6 block, one launch each;
 * every tensor is dense [B, D] of `dtype` (WKV6_F32 / WKV6_BF16 / WKV6_F16) unless stated.  The reference evaluates
 * these expressions with framework operations over whole sequences (rwkv6_model.py:37-44,128-146 time shift and
 * mixes; :48-83 channel mix); at one token per step they are pure launch latency, so they are fused here.
 *   wkv6_decode_ln_shift_mix: xa = LayerNorm(x; ln_w, ln_b, eps); xs = prev - xa; prev <- xa (in place);
 *       mix0 = xa + xs * mu0, mix1 = xa + xs * mu1 (mu fp32 [D]; mix1 / mu1, xa_out and xs_out may be NULL). D even, D <= 8192.
 *   wkv6_decode_lora_mix: h [B, 5R] is x_mix A before tanh (A = the five dense_a kernels side by side);
 *       out[perm[m]] = xa + xs * (bias[m] + tanh(h[:, mR:(m+1)R]) wb[m]),  wb [5, R, D], bias [5, D], out [5, B, D];
 *       perm (host pointer to 5 ints, NULL = identity) lets the caller order the outputs for its next products.  D even.
 *       Tensor pointers of these two calls must be aligned to two elements (mu to 8 bytes).
 *   wkv6_decode_relu_sq: out = max(x, 0)^2 over n elements (channel-mix key activation, rwkv6_model.py:47-48,73).
 *   wkv6_decode_sigmoid_mul_add: out = x + sigmoid(r) * kv over n elements (channel-mix output plus the residual).
 */
WKV6_API int wkv6_decode_ln_shift_mix(int32_t B, int32_t D, int32_t dtype, float eps, const void *x, const void *ln_w,
                                      const void *ln_b, void *prev, const float *mu0, const float *mu1, void *xa_out,
                                      void *xs_out, void *mix0, void *mix1, void *stream);
WKV6_API int wkv6_decode_lora_mix(int32_t B, int32_t D, int32_t R, int32_t dtype, const void *h, const void *wb,
                                  const void *bias, const void *xa, const void *xs, void *out, const int32_t *perm,
                                  void *stream);
WKV6_API int wkv6_decode_relu_sq(int64_t n, int32_t dtype, const void *x, void *out, void *stream);
WKV6_API int wkv6_decode_sigmoid_mul_add(int64_t n, int32_t dtype, const void *x, const void *r, const void *kv, void *out,
                                         void *stream);

/*
 * Language-model loss in one pass over bf16 logits [rows, V] (fp32 arithmetic): loss[row] = logsumexp(z) - z[target]
 * and, over the logits themselves, the gradient  z <- (softmax(z) - onehot(target)) * scale  (scale = 1 / rows for a
 * mean loss).  Rows whose target lies outside [0, V) give zero loss and gradient.  V a multiple of 8, at most 65536;
 * logits 16-byte aligned.  No counterpart in the reference (its trainer files are empty); used by the training step
 * around the op, where it replaces about 65 GB of framework traffic per step by 8.6 GB.
 */
WKV6_API int wkv6_softmax_xent_bf16(int64_t rows, int32_t V, void *logits_inout, const int64_t *targets, float scale,
                                    float *loss, void *stream);

/*
 * Sequence splitting along T (no counterpart in the reference, whose kernels cap T at a compile-time constant and
 * never split a sequence; sequences of 131072 tokens need it).  A sequence cut into G segments is
 * handled as a batch of B*G shorter sequences (a dense [B, G*Tseg, C] tensor is a [B*G, Tseg, C] tensor) whose
 * segment g starts from the state the segments before it produce:
 *   1. wkv6_segment_summary: per segment, the state it builds from zero (state_out [B*G,H,N,N] fp32) and the log2
 *      of its total decay per key channel (dec_log2_out [B*G,H,N]).  reverse = 0: x1 = k, x2 = v (forward state).
 *      reverse = 1: x1 = r, x2 = gy (the reverse state of the backward).
 *   2. wkv6_state_scan: exclusive scan over g of the maps S -> 2^dec S + state (ascending g, seeded with s0
 *      [B,H,N,N] or zero; descending g when reverse).  state_in_out[b*G+g] = state entering segment g;
 *      last_out (optional, [B,H,N,N]) = state after the last segment.  Across GPUs the summaries of all ranks are
 *      gathered (they are small: H*(N*N+N)*4 bytes per segment) and every rank runs the same scan.
 *   3. wkv6_forward on the [B*G, Tseg, C] problem with s_in = the scanned states (and a ckpt buffer), and
 *      wkv6_backward_seeded with ab_in = the scanned reverse states [B*G,H,N,N] fp32, that ckpt buffer and a
 *      workspace of wkv6_backward_workspace_bytes(p, 1) bytes.
 * Chunked variant only (N == 64, bf16 r,k,v,w,y).
 */
WKV6_API int wkv6_segment_summary(const wkv6_problem *p, const void *x1, const void *x2, const void *w, int reverse,
                                  float *state_out, float *dec_log2_out, void *stream);
/* The same for a caller that only needs the states ENTERING the segments (an exclusive scan that does not return the
 * state after the last segment): the problem holds G segments per sequence (p->B = sequences * G, segment g of sequence s
 * at batch row s*G + g), and the one segment per sequence whose summary such a scan never reads is left out - the last
 * one when reverse = 0, the first when reverse = 1.  Its rows of state_out and dec_log2_out are not written.  With
 * reverse = 1 dec_log2_out holds exactly the decays the descending scan needs, so the backward no longer depends on the
 * forward's summary. */
WKV6_API int wkv6_segment_summary_for_scan(const wkv6_problem *p, const void *x1, const void *x2, const void *w, int reverse,
                                           int32_t G, float *state_out, float *dec_log2_out, void *stream);
WKV6_API int wkv6_state_scan(int32_t B, int32_t H, int32_t N, int32_t G, const float *dec_log2, const float *state_sum,
                             const float *s0, float *state_in_out, float *last_out, int reverse, void *stream);
WKV6_API int wkv6_backward_seeded(const wkv6_problem *p, const void *r, const void *k, const void *v, const void *w,
                                  const void *u, const void *gy, void *gr, void *gk, void *gv, void *gw, void *gu,
                                  const void *ckpt, const float *ab_in, void *workspace, size_t workspace_bytes,
                                  void *stream);
/* out[j] = sum over the rows of in[rows][n] (fp32, rows added in ascending order): the per-segment gu rows of
 * wkv6_backward_seeded summed into the [H, N] gradient of u (the reference sums its per-batch-row gu the same way,
 * jax_rwkv_kernel.py:202).  One small launch. */
WKV6_API int wkv6_sum_rows(const float *in, int64_t rows, int64_t n, float *out, void *stream);

/*
 * Output stage of the time-mix block, fused: per-head normalisation of the WKV output, then the gate:
 *   out[row,h,n] = (scale[h,n] * (y[row,h,n] - mean[row,h]) * rstd[row,h] + offset[h,n]) * g[row,h,n],
 * mean / variance over the N channels of head h of row (= token) `row`, rstd = 1/sqrt(var + eps).  Replaces
 * GroupNorm.call (rwkv6_model.py:93-99; LayerNormalization(epsilon=64e-5) over the head dimension plus the [H,N]
 * scale and offset) and the `x * g` that follows it (rwkv6_model.py:158-160).  rows = B*T; y, g, out, gout, gy, gg
 * are dense [rows, H*N] of one dtype (WKV6_BF16 / WKV6_F16 / WKV6_F32); scale, offset and their gradients are fp32
 * [H,N].  N == 64, H*N <= 8192, all pointers 16-byte aligned.  The backward needs
 * wkv6_groupnorm_gate_workspace_bytes(rows, H, N) bytes of scratch (partial sums of the parameter gradients, added in
 * a fixed order: reruns are bit-identical).
 */
WKV6_API int wkv6_groupnorm_gate_forward(int64_t rows, int32_t H, int32_t N, int32_t dtype, float eps, const void *y,
                                         const void *g, const float *scale, const float *offset, void *out, void *stream);
WKV6_API int wkv6_groupnorm_gate_backward(int64_t rows, int32_t H, int32_t N, int32_t dtype, float eps, const void *y,
                                          const void *g, const float *scale, const float *offset, const void *gout,
                                          void *gy, void *gg, float *gscale, float *goffset, void *workspace,
                                          size_t workspace_bytes, void *stream);
WKV6_API size_t wkv6_groupnorm_gate_workspace_bytes(int64_t rows, int32_t H, int32_t N);
/* The same stage with the gate's activation inside: g_raw is the gate projection before SiLU (rwkv6_model.py:147
 * `g = silu(dense_g(xg))`), out = (...) * silu(g_raw), and the backward returns the gradient of g_raw.  The activated
 * gate is never written to memory.  All other arguments as above. */
WKV6_API int wkv6_groupnorm_silu_gate_forward(int64_t rows, int32_t H, int32_t N, int32_t dtype, float eps, const void *y,
                                              const void *g_raw, const float *scale, const float *offset, void *out,
                                              void *stream);
WKV6_API int wkv6_groupnorm_silu_gate_backward(int64_t rows, int32_t H, int32_t N, int32_t dtype, float eps, const void *y,
                                               const void *g_raw, const float *scale, const float *offset, const void *gout,
                                               void *gy, void *gg_raw, float *gscale, float *goffset, void *workspace,
                                               size_t workspace_bytes, void *stream);

/*
 * Input stage of the time-mix block: token-shift interpolations
 *   out_j[b,t,c] = x[b,t,c] + (x[b,t-1,c] - x[b,t,c]) * m_j[b,t,c],   x[b,-1,:] = 0,   j < nmix,
 * replacing TimeShift (rwkv6_model.py:37-44) plus the multiply-adds of TimeMix.call (rwkv6_model.py:135-146).
 *   m_is_vector = 1 : nmix = 1, m is one fp32 vector [C] (time_mix_x); out is [B,T,C]
 *   m_is_vector = 0 : nmix = 1 or 5, m and out are dense [nmix,B,T,C] of the activation dtype (the data-dependent mixes)
 * x, out, gout, gx are dense [B,T,C] / [nmix,B,T,C] of `dtype`; C a multiple of 8; pointers 16-byte aligned.
 * Backward: gx [B,T,C], gm = gradient of m ([nmix,B,T,C] of `dtype`, or fp32 [C] for the vector form, which needs
 * wkv6_shift_mix_workspace_bytes(B,T,C,1) bytes of scratch; its partial sums are added in a fixed order).
 */
WKV6_API int wkv6_shift_mix_forward(int32_t B, int32_t T, int32_t C, int32_t dtype, int32_t nmix, int32_t m_is_vector,
                                    const void *x, const void *m, void *out, void *stream);
WKV6_API int wkv6_shift_mix_backward(int32_t B, int32_t T, int32_t C, int32_t dtype, int32_t nmix, int32_t m_is_vector,
                                     const void *x, const void *m, const void *gout, void *gx, void *gm, void *workspace,
                                     size_t workspace_bytes, void *stream);
WKV6_API size_t wkv6_shift_mix_workspace_bytes(int32_t B, int32_t T, int32_t C, int32_t m_is_vector);

/*
 * Activations of the channel-mix block over whole sequences, one launch per direction (n elements of `dtype`, dense,
 * pointers 16-byte aligned):
 *   wkv6_relu_sq_forward:      out = max(x, 0)^2          wkv6_relu_sq_backward:      gx = gout * 2 max(x, 0)
 *   wkv6_sigmoid_mul_forward:  out = sigmoid(r) * kv      wkv6_sigmoid_mul_backward:  gr = gout * kv * s (1 - s), gkv = gout * s
 * They replace the framework operations behind the reference's ChannelMix (rwkv6_model.py:47-48 relu_square as the
 * activation of dense_key, :83 sigmoid as the activation of dense_receptance, :64 `o = r * kv`) and their autograd
 * kernels: operands read once, results written once.
 */
WKV6_API int wkv6_relu_sq_forward(int64_t n, int32_t dtype, const void *x, void *out, void *stream);
WKV6_API int wkv6_relu_sq_backward(int64_t n, int32_t dtype, const void *x, const void *gout, void *gx, void *stream);
WKV6_API int wkv6_sigmoid_mul_forward(int64_t n, int32_t dtype, const void *r, const void *kv, void *out, void *stream);
WKV6_API int wkv6_sigmoid_mul_backward(int64_t n, int32_t dtype, const void *r, const void *kv, const void *gout, void *gr,
                                       void *gkv, void *stream);

/*
 * Pitched copy between host and device memory on `stream` (a thin wrapper of cudaMemcpy2DAsync, exported so that a
 * host-side pipeline bound through this ABI needs no second library): `rows` lines of `width_bytes` bytes, line i at
 * dst + i*dst_pitch / src + i*src_pitch.  to_host = 0: host to device, 1: device to host.  A head group of a [T, H*N]
 * activation row in host memory is such a region (pitch H*N elements, width g*N elements).  The reference has no
 * counterpart: its operators take device tensors only.
 */
WKV6_API int wkv6_copy_2d_async(void *dst, size_t dst_pitch, const void *src, size_t src_pitch, size_t width_bytes,
                                size_t rows, int32_t to_host, void *stream);

/*
 * XLA legacy custom-call surface.  The library also exports the C++ symbols gpu_ops::rwkv_forward_fn,
 * gpu_ops::rwkv_backward_fn and gpu_ops::rwkv_forward_with_state_fn with the signature
 *     void f(cudaStream_t stream, void **buffers, const char *opaque, size_t opaque_len)
 * and the buffer orders of the reference (rwkv_kernel/jax_kernel/kernels.h:44-53, rwkv_kernels.cu:451-508);
 * they throw std::runtime_error on failure as the reference does for a bad descriptor.  The functions below are
 * the same handlers with an error code instead of an exception, the descriptor packer that replaces
 * gpu_ops.create_rwkv_descriptor (rwkv_kernel/jax_kernel/gpu_ops.cpp:33-36; returns the blob size, 28), and the
 * handler addresses (0 forward, 1 backward, 2 forward_with_state, 3 forward_ckpt, 4 backward_ws) for
 * "xla._CUSTOM_CALL_TARGET" capsules (replaces gpu_ops.get_rwkv_registrations, gpu_ops.cpp:20-29).
 *
 * wkv_backward keeps the reference's eleven buffers (rwkv_kernels.cu:493-508) and so has no scratch: it runs the
 * sequential kernels on the library's built-in array, in slices when the problem is larger than the array.  The two
 * extended handlers reach the chunked tensor-core kernels for any size by letting the lowering declare two more
 * buffers (the legacy ABI's way to get a workspace: an extra result):
 *   wkv6_xla_forward_ckpt   [r, k, v, w, u, y, ckpt]                            ckpt = extra result, residual of the vjp
 *   wkv6_xla_backward_ws    [r, k, v, w, u, gy, ckpt, gr, gk, gv, gw, gu, ws]   ws = extra result, scratch
 * wkv6_xla_buffer_bytes(descriptor, which) gives the least size of ckpt (which = 0) and ws (which = 1); the shapes
 * [B, H, ceil(T/64), 4096] bf16 and [B, H, 64] int32 always suffice for bf16 inputs with head size 64 and split with
 * the (batch, head) pairs under a partitioning rule.
 */
WKV6_API int wkv6_xla_forward(void *stream, void **buffers, const char *opaque, size_t opaque_len);
WKV6_API int wkv6_xla_backward(void *stream, void **buffers, const char *opaque, size_t opaque_len);
WKV6_API int wkv6_xla_forward_with_state(void *stream, void **buffers, const char *opaque, size_t opaque_len);
WKV6_API int wkv6_xla_forward_ckpt(void *stream, void **buffers, const char *opaque, size_t opaque_len);
WKV6_API int wkv6_xla_backward_ws(void *stream, void **buffers, const char *opaque, size_t opaque_len);
WKV6_API size_t wkv6_xla_buffer_bytes(const char *opaque, size_t opaque_len, int which);
WKV6_API int wkv6_xla_descriptor(int B, int T, int C, int H, int S, int x_type, int y_type, char *out, size_t out_len);
WKV6_API void *wkv6_xla_target(int which);

#ifdef __cplusplus
}
#endif
#endif /* WKV6_B200_H_ */
