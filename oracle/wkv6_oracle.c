/*
 * CPU oracle for the RWKV-6 WKV recurrence, plain C.  TEST INFRASTRUCTURE ONLY:
 * it is the checker for the CUDA path and the timed CPU baseline; no product
 * code path may call it.
 *
 * Restates the reference's non-CUDA operator:
 *   forward loop            rwkv_kernel/ops_rwkv_kernal.py:83-95  (= rwkv_v6_demo.py:27-37)
 *   initial state handling  rwkv_kernel/ops_rwkv_kernal.py:41-72  (resolved by the caller into s_in[B,H,N,N])
 *   gradients               closed forms stated by rwkv_kernel/jax_kernel/rwkv_kernels.cu:205-407,
 *                           which the reference otherwise gets from autograd
 *                           (deprecated_code/wkv_torch.py:56)
 *
 * Layout: r,k,v,w,gy,y,g* are [B,T,H*N] row-major; u is [H,N]; states are
 * S[b,h,key,value].  One (b,h) pair is independent of every other, so the outer
 * loop is an OpenMP parallel-for over B*H.
 *
 * Built twice: REAL=double (the parity oracle) and REAL=float (the CPU baseline,
 * which is the arithmetic width the reference runs its CPU path in).
 */
#include <math.h>
#include <stdlib.h>
#include <string.h>

#ifndef REAL
#define REAL double
#endif
#ifndef SUFFIX
#define SUFFIX f64
#endif
#define CAT_(a, b) a##_##b
#define CAT(a, b) CAT_(a, b)
#define FN(name) CAT(name, SUFFIX)

#if defined(_OPENMP)
#include <omp.h>
int FN(wkv6_oracle_threads)(void) { return omp_get_max_threads(); }
void FN(wkv6_oracle_set_threads)(int n) { if (n > 0) omp_set_num_threads(n); }
#else
int FN(wkv6_oracle_threads)(void) { return 1; }
void FN(wkv6_oracle_set_threads)(int n) { (void)n; }
#endif

static inline REAL decay_of(REAL w) { return (REAL)exp(-exp((double)w)); }

/* y_t[j] = sum_i r_t[i] (u[i] k_t[i] v_t[j] + S[i][j]);  S = d_t S + k_t v_t^T */
int FN(wkv6_oracle_fwd)(int B, int T, int H, int N, const REAL *r, const REAL *k, const REAL *v,
                        const REAL *w, const REAL *u, const REAL *s_in, REAL *y, REAL *s_out)
{
    const long C = (long)H * N;
    int bh;
#pragma omp parallel for schedule(dynamic, 1)
    for (bh = 0; bh < B * H; ++bh) {
        const int b = bh / H, h = bh % H;
        REAL *S = (REAL *)malloc(sizeof(REAL) * N * N);
        if (s_in) memcpy(S, s_in + (long)bh * N * N, sizeof(REAL) * N * N);
        else memset(S, 0, sizeof(REAL) * N * N);
        for (int t = 0; t < T; ++t) {
            const long o = ((long)b * T + t) * C + (long)h * N;
            for (int j = 0; j < N; ++j) y[o + j] = 0;
            for (int i = 0; i < N; ++i) {
                const REAL ri = r[o + i], ki = k[o + i], di = decay_of(w[o + i]);
                const REAL uk = u[h * N + i] * ki;
                REAL *Si = S + (long)i * N;
                for (int j = 0; j < N; ++j) {
                    const REAL vj = v[o + j];
                    y[o + j] += ri * (uk * vj + Si[j]);
                    Si[j] = di * Si[j] + ki * vj;
                }
            }
        }
        if (s_out) memcpy(s_out + (long)bh * N * N, S, sizeof(REAL) * N * N);
        free(S);
    }
    return 0;
}

/*
 * Gradients of sum(y*gy).  gu is per batch row [B,H,N].  gw uses the direct
 * closed form  gw_t[i] = -exp(w_t[i]) d_t[i] sum_j S_{t-1}[i][j] A_t[i][j]
 * with forward states rebuilt from checkpoints every SEG steps.
 */
#define SEG 64
int FN(wkv6_oracle_bwd)(int B, int T, int H, int N, const REAL *r, const REAL *k, const REAL *v,
                        const REAL *w, const REAL *u, const REAL *gy, const REAL *s_in, REAL *gr,
                        REAL *gk, REAL *gv, REAL *gw, REAL *gu)
{
    const long C = (long)H * N;
    const long NN = (long)N * N;
    const int nseg = (T + SEG - 1) / SEG;
    int bh;
#pragma omp parallel for schedule(dynamic, 1)
    for (bh = 0; bh < B * H; ++bh) {
        const int b = bh / H, h = bh % H;
        REAL *ck = (REAL *)malloc(sizeof(REAL) * NN * (nseg + 1)); /* state at the start of each segment */
        REAL *Sp = (REAL *)malloc(sizeof(REAL) * NN * SEG);        /* S_{t-1} for one segment */
        REAL *A = (REAL *)calloc(NN, sizeof(REAL));
        REAL *S = (REAL *)malloc(sizeof(REAL) * NN);
        if (s_in) memcpy(S, s_in + (long)bh * NN, sizeof(REAL) * NN);
        else memset(S, 0, sizeof(REAL) * NN);
        for (int i = 0; i < N; ++i) gu[(long)bh * N + i] = 0;
        /* forward sweep: gr, gu, checkpoints */
        for (int t = 0; t < T; ++t) {
            const long o = ((long)b * T + t) * C + (long)h * N;
            if (t % SEG == 0) memcpy(ck + NN * (t / SEG), S, sizeof(REAL) * NN);
            REAL vg = 0;
            for (int j = 0; j < N; ++j) vg += v[o + j] * gy[o + j];
            for (int i = 0; i < N; ++i) {
                const REAL ki = k[o + i], di = decay_of(w[o + i]);
                REAL *Si = S + (long)i * N;
                REAL acc = 0;
                for (int j = 0; j < N; ++j) {
                    acc += Si[j] * gy[o + j];
                    Si[j] = di * Si[j] + ki * v[o + j];
                }
                gr[o + i] = u[h * N + i] * ki * vg + acc;
                gu[(long)bh * N + i] += r[o + i] * ki * vg;
            }
        }
        /* reverse sweep, segment by segment */
        for (int sg = nseg - 1; sg >= 0; --sg) {
            const int t0 = sg * SEG, t1 = (t0 + SEG < T) ? t0 + SEG : T;
            memcpy(S, ck + NN * sg, sizeof(REAL) * NN);
            for (int t = t0; t < t1; ++t) {
                const long o = ((long)b * T + t) * C + (long)h * N;
                memcpy(Sp + NN * (t - t0), S, sizeof(REAL) * NN);
                for (int i = 0; i < N; ++i) {
                    const REAL ki = k[o + i], di = decay_of(w[o + i]);
                    REAL *Si = S + (long)i * N;
                    for (int j = 0; j < N; ++j) Si[j] = di * Si[j] + ki * v[o + j];
                }
            }
            for (int t = t1 - 1; t >= t0; --t) {
                const long o = ((long)b * T + t) * C + (long)h * N;
                const REAL *Spt = Sp + NN * (t - t0);
                for (int j = 0; j < N; ++j) gv[o + j] = 0;
                for (int i = 0; i < N; ++i) {
                    const REAL ri = r[o + i], ki = k[o + i];
                    const REAL ew = (REAL)exp((double)w[o + i]);
                    const REAL di = (REAL)exp(-(double)ew);
                    const REAL ur = u[h * N + i] * ri;
                    REAL *Ai = A + (long)i * N;
                    REAL acck = 0, accw = 0;
                    for (int j = 0; j < N; ++j) {
                        const REAL m = ur * gy[o + j] + Ai[j];
                        acck += m * v[o + j];
                        gv[o + j] += m * ki;
                        accw += Spt[(long)i * N + j] * Ai[j];
                        Ai[j] = ri * gy[o + j] + di * Ai[j];
                    }
                    gk[o + i] = acck;
                    gw[o + i] = -ew * di * accw;
                }
            }
        }
        free(ck); free(Sp); free(A); free(S);
    }
    return 0;
}
