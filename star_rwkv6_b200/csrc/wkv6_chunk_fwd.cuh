// Chunked WKV6 forward for sm_100a: TMA-fed tcgen05 MMAs over 64-token chunks, fp32 state carried in
// registers across the chunks of one (batch, head) sequence.
//
// Per chunk (tokens t, s in [0,64), key channel i, value channel j, c_t = sum_{sigma<=t} log d_sigma):
//   A[t][s]  = sum_i r_t[i] k_s[i] exp(c_{t-1}[i] - c_s[i])      (s < t),   A[t][t] = sum_i r_t[i] u[i] k_t[i]
//   y_t      = sum_s A[t][s] v_s  +  sum_i r_t[i] exp(c_{t-1}[i]) S_in[i][:]
//   S_out    = diag(exp(c_63)) S_in + sum_s (k_s exp(c_63 - c_s)) (x) v_s
// With a single reference point the diagonal of A (the bonus term) also comes from the tensor core: the operand
// q_t = r_t u exp(c_t - c_rho) times k~_t gives sum_i r_t[i] u[i] k_t[i] on the diagonal of q k~^T (only the diagonal
// blocks are read), and the factor exp(c_63 - c_rho) of the state increment is applied to the rows of the fp32
// accumulator of k~^T v instead of to a second copy of k~.  With per-block reference points that factor differs from
// block to block, so those chunks keep the copy k^ = k~ exp(c_63 - c_rho(J)) and sum the bonus on the CUDA cores.
// The decay exponent of A is split between the two bf16 operands around reference points so that no factor
// can overflow: tokens are grouped in blocks of 16, each block I has the reference rho_I = its 8th token, and
//   r~_t = r_t exp(c_{t-1} - c_rho(I)),   k~_s = k_s exp(c_rho(J) - c_s),
//   A_IJ = r~_I (k~_J exp(c_rho(I) - c_rho(J)))^T        for block pairs J <= I.
// Positive exponents span at most 8 steps; log-decays are clamped at -10 per step (a decay of e^-10, below
// bf16 resolution of anything it multiplies), so every factor stays below e^80.  The block-pair factor is
// folded into extra copies of k~ (one per block distance 1..3), all multiplied by the same r~ in one MMA;
// the epilogue picks, per block pair, the columns of the matching copy.  Chunks with a mild total decay (see
// kWideLimit2; the usual case) use a single reference (half of the chunk's total decay) and skip the copies.
//
// Tensor-memory map (256 columns, M = 64 accumulators occupy 16 lanes of each 32-lane quarter):
//   lanes  0-15: cols [0,64) A for distance 0 | [64,128) y | [128,192) k~^T V (state increment) | [192,256) q k~^T (bonus)
//   lanes 16-31: cols [0,48) A distance 1 | [48,80) distance 2 | [80,96) distance 3
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "sm100_ptx.cuh"
#include "wkv6_seq.cuh"

namespace wkv6 {

constexpr int kChunk = 64;
constexpr int kTile = 8192;  // one [64 x 64] bf16 tile
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kMinLogDecay2 = -10.0f * 1.4426950408889634f;  // clamp of the per-step log2 decay
// A chunk whose total log2 decay stays above this limit in every channel takes one reference point for the whole
// chunk instead of one per 16-token block, and the copies of k~ / r~ for the block distances 1..3 are not needed.
// The reference is not a token position but a value: half of the chunk's total log2 decay (rounded to an integer), so
// that the largest factor of r (at the first token) and of k (at the last) are both 2^{-total/2} <= 2^96, finite in
// bf16 whatever r and k hold and however the decay is distributed over the chunk.  A channel may then lose up to 2^-3
// per token on average (exp(w) up to 2.08, w up to 0.73).  Products of two such factors occur only at masked
// positions (a key after its query), where they may overflow to infinity: every mask is a select, never a
// multiplication, so nothing of them is used.
constexpr float kWideLimit2 = -192.0f;

// device-side error word: 0 = fine, otherwise the code of the wait that ran out (read and cleared by the host)
__device__ int g_chunk_status;

// Phase timestamps of CTA 0 (builds with -DWKV6_TIMING only): g_chunk_timing[chunk][phase][warp] = clock64() of lane 0
#ifdef WKV6_TIMING
__device__ long long g_chunk_timing[64][16][8];
__device__ long long g_cta_times[1024][8];  // per CTA: eight %globaltimer stamps from entry (0) to exit (7)
__device__ int g_cta_sm[1024];              // per CTA: the SM it ran on
#define WKV6_CSTAMP(k) \
    do { \
        if (threadIdx.x == 0 && blockIdx.x < 1024) { \
            g_cta_times[blockIdx.x][(k)] = (long long)ptx::global_timer_ns(); \
            if ((k) == 0) { unsigned sm_; asm volatile("mov.u32 %0, %%smid;" : "=r"(sm_)); g_cta_sm[blockIdx.x] = (int)sm_; } \
        } \
    } while (0)
#define WKV6_TSTAMP(iter, k) \
    do { if (blockIdx.x == 0 && (threadIdx.x & 31) == 0 && (iter) < 64) g_chunk_timing[(iter)][(k)][threadIdx.x >> 5] = clock64(); } while (0)
#else
#define WKV6_TSTAMP(iter, k) do { } while (0)
#define WKV6_CSTAMP(k) do { } while (0)
#endif

struct ChunkFwdSmem {
    static constexpr int kStage = 4 * kTile;                 // r, k, v, w
    static constexpr int oStage0 = 0;
    static constexpr int oKH = 2 * kStage;                   // q = r u exp(c_t - c_rho), operand of the bonus product (per-block mode: k^)
    static constexpr int oKD = oKH + kTile;                  // k~ copies for block distances 1..3: 96 rows
    static constexpr int oAM = oKD + 96 * 128;               // masked A (bf16), later the y tile
    static constexpr int oSB = oAM + kTile;                  // bf16 copy of the state, MN-major B operand
    static constexpr int oHead = oSB + kTile;                // float [4][64]: log-decay sum of the first 8 tokens of a block
    static constexpr int oTot = oHead + 4 * 64 * 4;          // float [4][64]: log-decay sum of the block
    static constexpr int oDtot = oTot + 4 * 64 * 4;          // float [64]: decay over the whole chunk
    static constexpr int oFK = oDtot + 64 * 4;               // float [64]: exp(c_63 - c_rho), scales the state increment rows
    static constexpr int oBonus = oFK + 64 * 4;              // float [64]: sum_i r u k per token (per-block mode only)
    static constexpr int oBar = oBonus + 64 * 4;             // mbarriers: full[2], mma1, mma2
    static constexpr int oSlot = oBar + 4 * 8;
    static constexpr int kBytes = oSlot + 16;
    static constexpr int kAlloc = kBytes;
};

struct ChunkFwdArgs {
    const void *u; int u_dtype;
    const void *s_in; const int64_t *s_map; int s_kinds; int s_dtype; void *s_out;
    __nv_bfloat16 *ckpt;  // optional [B*H][T/64][64*64] bf16 chunk-start states in operand (swizzled) layout
    int B, T, H;
    bool write_y;         // false: only states / checkpoints are produced
    // Used by the summary kernel only (wkv6_chunk_summary.cuh): walk the chunks from last to first and accumulate the
    // reverse state of the backward (x1 = r, x2 = gy); and where to leave log2 of the total decay per key channel.
    bool reverse_state;
    float *dec_out;       // optional [B*H][64]
    int skip_mod, skip_rem;  // summary kernel: sequences (batch rows) with b % skip_mod == skip_rem are left out (0: none)
    // Test hook (wkv6_debug_inject): the forward never requests the input tiles of chunk index skip_load_chunk - 1
    // (0 = off), so the wait for them runs out with no copy outstanding and the kernel takes its error path.
    int skip_load_chunk;
};

__device__ __forceinline__ float ex2f(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float2 ld_bf2(const uint8_t *p) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(p));
}
__device__ __forceinline__ void st_bf2(uint8_t *p, float a, float b) {
    *reinterpret_cast<__nv_bfloat162 *>(p) = __floats2bfloat162_rn(a, b);
}
// packed fp32 pairs (one issue slot for two lanes of work on sm_100)
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
    unsigned long long ra, rb, rc;
    asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(rc) : "l"(ra), "l"(rb));
    float2 c;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(c.x), "=f"(c.y) : "l"(rc));
    return c;
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
    unsigned long long ra, rb, rc;
    asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(rc) : "l"(ra), "l"(rb));
    float2 c;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(c.x), "=f"(c.y) : "l"(rc));
    return c;
}
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
    unsigned long long ra, rb, rc, rd;
    asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rc) : "f"(c.x), "f"(c.y));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(rd) : "l"(ra), "l"(rb), "l"(rc));
    float2 d;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
    return d;
}
__device__ __forceinline__ __nv_bfloat162 to_bf2(float2 a) { return __floats2bfloat162_rn(a.x, a.y); }
__device__ __forceinline__ uint32_t pack_bf2(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&h);
}

__global__ void __launch_bounds__(256, 2) chunk_fwd_kernel(const __grid_constant__ CUtensorMap tm_r,
                                                           const __grid_constant__ CUtensorMap tm_k,
                                                           const __grid_constant__ CUtensorMap tm_v,
                                                           const __grid_constant__ CUtensorMap tm_w,
                                                           const __grid_constant__ CUtensorMap tm_y,
                                                           const ChunkFwdArgs a) {
    using namespace ptx;
    using SM = ChunkFwdSmem;
    // Declared with the alignment the swizzled tiles need, so that the compiler keeps every access in the shared
    // address space with 32-bit addresses; the base is verified once instead of being realigned by pointer math.
    extern __shared__ __align__(1024) uint8_t wkv6_chunk_smem[];
    uint8_t *const smem = wkv6_chunk_smem;
    if ((smem_u32(smem) & 1023u) != 0) {
        if (threadIdx.x == 0) atomicExch(&g_chunk_status, 50);
        return;
    }
    uint8_t *sKH = smem + SM::oKH, *sKD = smem + SM::oKD, *sAM = smem + SM::oAM, *sSB = smem + SM::oSB;
    float *sHead = reinterpret_cast<float *>(smem + SM::oHead);  // [4][64] log2-decay sum of tokens 0..7 of a block
    float *sTail = reinterpret_cast<float *>(smem + SM::oTot);   // [4][64] log2-decay sum of tokens 8..15 of a block
    float *sDtot = reinterpret_cast<float *>(smem + SM::oDtot);
    float *sFK = reinterpret_cast<float *>(smem + SM::oFK);
    float *sBonus = reinterpret_cast<float *>(smem + SM::oBonus);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + SM::oBar);
    uint64_t *bar_full = bars, *bar_mma1 = bars + 2, *bar_mma2 = bars + 3;
    uint32_t *slot = reinterpret_cast<uint32_t *>(smem + SM::oSlot);

    // Thread roles.  Operand pass: warp (w4, half) owns tokens 16*w4 + 8*half .. +7, lane = channel pair.
    // Accumulator passes: warp (w4, half) owns rows 16*w4 + r0 (+8) and the 32 columns 32*half .. +31
    // (fragment layout of tcgen05.ld.16x256b: columns 8n + 2q, +1).
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int w4 = warp & 3, half = warp >> 2, n0 = 4 * half;
    const int q = lane & 3, r0 = lane >> 2;
    const int ta = 16 * w4 + r0;
    const int b = blockIdx.x / a.H, h = blockIdx.x % a.H;
    const int nchunks = (a.T + kChunk - 1) / kChunk;
    WKV6_CSTAMP(0);

    if (tid == 0) {
        mbar_init(&bar_full[0], 4);  // one arrival per loading thread
        mbar_init(&bar_full[1], 4);
        mbar_init(bar_mma1, 2);  // two issuing threads
        mbar_init(bar_mma2, 1);
        fence_mbar_init();
        prefetch_tensormap(&tm_r); prefetch_tensormap(&tm_k); prefetch_tensormap(&tm_v);
        prefetch_tensormap(&tm_w); prefetch_tensormap(&tm_y);
    }
    if (warp == 0) {
        tmem_alloc(slot, 256);
        tmem_relinquish();
    }

    __syncthreads();  // the barriers are initialised: the first two chunks can be requested before the state is read
    WKV6_CSTAMP(1);
    // Issuing a TMA copy keeps a thread busy for on the order of a hundred cycles, so the copies of one chunk are
    // spread over warps: lane 0 of warps 2..5 loads one input tile each, lane 0 of warp 1 issues the stores.  Warp 0,
    // whose first lane issues MMAs, issues none.
    const int load_slot = (lane == 0 && warp >= 2 && warp <= 5) ? warp - 2 : -1;  // 0..3 = r, k, v, w
    const int skip_chunk = a.skip_load_chunk - 1;  // test hook, -1 in normal use
    auto issue_loads = [&](int ic2) {  // every thread calls it; the four loading threads act
        if (load_slot < 0 || ic2 == skip_chunk) return;
        const int c = ic2;
        const int st = ic2 & 1;
        uint8_t *dst = smem + st * SM::kStage + load_slot * kTile;
        const CUtensorMap *tm = load_slot == 0 ? &tm_r : load_slot == 1 ? &tm_k : load_slot == 2 ? &tm_v : &tm_w;
        mbar_expect_tx(&bar_full[st], kTile);
        tma_load_3d(dst, tm, &bar_full[st], h * 64, c * kChunk, b);
    };
    issue_loads(0);
    if (nchunks > 1) issue_loads(1);

    // u of this thread's channel pair (requested before the state so that the two reads overlap)
    float2 u2 = make_float2(0.f, 0.f);
    if (a.u != nullptr) {
        if (a.u_dtype == WKV6_F32) u2 = *reinterpret_cast<const float2 *>(static_cast<const float *>(a.u) + (size_t)h * 64 + 2 * lane);
        else u2 = make_float2(load_any(a.u, a.u_dtype, (size_t)h * 64 + 2 * lane), load_any(a.u, a.u_dtype, (size_t)h * 64 + 2 * lane + 1));
    }
    // state in accumulator-fragment layout: rows i = ta (+8), columns j = 8(n0+nn) + 2q (+1)
    float S[16];
    {
        const bool has = a.s_in != nullptr;
        size_t so = 0;
        if (has) {
            int64_t kind = a.s_map ? a.s_map[b] : (a.s_kinds == 1 ? 0 : b);
            kind = kind < 0 ? 0 : (kind >= a.s_kinds ? a.s_kinds - 1 : kind);
            so = ((size_t)kind * a.H + h) * 4096;
        }
        if (has && a.s_dtype == WKV6_F32) {
            // eight independent 8-byte loads per thread (the generic reader below switches on the dtype per element,
            // which serialises its sixteen loads: 5 us of a launch over short sequences)
            const float *sp = static_cast<const float *>(a.s_in) + so;
#pragma unroll
            for (int nn = 0; nn < 4; ++nn) {
                const int j = 8 * (n0 + nn) + 2 * q;
                const float2 lo2 = *reinterpret_cast<const float2 *>(sp + (size_t)ta * 64 + j);
                const float2 hi2 = *reinterpret_cast<const float2 *>(sp + (size_t)(ta + 8) * 64 + j);
                S[4 * nn] = lo2.x; S[4 * nn + 1] = lo2.y; S[4 * nn + 2] = hi2.x; S[4 * nn + 3] = hi2.y;
            }
        } else {
#pragma unroll
            for (int nn = 0; nn < 4; ++nn) {
                const int j = 8 * (n0 + nn) + 2 * q;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int i = ta + (e >= 2 ? 8 : 0);
                    S[4 * nn + e] = has ? load_any(a.s_in, a.s_dtype, so + (size_t)i * 64 + j + (e & 1)) : 0.f;
                }
            }
        }
#pragma unroll
        for (int nn = 0; nn < 4; ++nn) {
            const int j = 8 * (n0 + nn) + 2 * q;
            *reinterpret_cast<uint32_t *>(sSB + sw128_off(ta, j)) = pack_bf2(S[4 * nn], S[4 * nn + 1]);
            *reinterpret_cast<uint32_t *>(sSB + sw128_off(ta + 8, j)) = pack_bf2(S[4 * nn + 2], S[4 * nn + 3]);
        }
    }

    const __nv_bfloat162 ub = to_bf2(u2);

    WKV6_CSTAMP(2);
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tb = *slot;
    WKV6_CSTAMP(3);
    const uint32_t tmA0 = tb, tmY = tb + 64, tmS = tb + 128, tmAU = tb + 192, tmAD = tb + (16u << 16);
    const uint32_t wl = (uint32_t)(w4 * 32) << 16;  // this warp's TMEM lane quarter
    const uint32_t cb = 8 * n0;                     // first accumulator column of this thread's fragment
    // byte offsets of this thread's fragment elements (rows ta / ta+8, column pairs 8(n0+nn)+2q) in a swizzled tile
    uint32_t foA[4], foB[4];
#pragma unroll
    for (int nn = 0; nn < 4; ++nn) {
        foA[nn] = sw128_off(ta, 8 * (n0 + nn) + 2 * q);
        foB[nn] = sw128_off(ta + 8, 8 * (n0 + nn) + 2 * q);
    }

    const bool copy_thread = (tid == 32);
    if (copy_thread) {
        if (a.ckpt != nullptr) {  // state at the start of chunk 0, already in operand layout
            bulk_store(a.ckpt + (size_t)blockIdx.x * nchunks * 4096, sSB, kTile);
            bulk_commit();
        }
    }

    constexpr uint32_t idKK = umma_idesc_bf16(64, 64, false, false);
    constexpr uint32_t idKK96 = umma_idesc_bf16(64, 96, false, false);
    constexpr uint32_t idMM = umma_idesc_bf16(64, 64, true, true);
    constexpr uint32_t idKM = umma_idesc_bf16(64, 64, false, true);
    // operand descriptors of stage 0; a step of 16 along K is +2 (K-major, 32 bytes) or +128 (MN-major, 2048 bytes)
    // in the 16-byte units of the address field, the second stage is +kStage/16
    const uint64_t dR = umma_desc_sw128(smem_u32(smem)), dK = umma_desc_sw128(smem_u32(smem + kTile));
    const uint64_t dV = umma_desc_sw128(smem_u32(smem + 2 * kTile)), dW = umma_desc_sw128(smem_u32(smem + 3 * kTile));
    const uint64_t dKH = umma_desc_sw128(smem_u32(sKH)), dKD = umma_desc_sw128(smem_u32(sKD));
    const uint64_t dAM = umma_desc_sw128(smem_u32(sAM)), dSB = umma_desc_sw128(smem_u32(sSB));

    int err = 0;
    int loads_issued = (nchunks > 1) ? 2 : 1, loads_consumed = 0;  // chunks whose loads were issued / waited for
    // Pass 1 of a chunk: per-step log2 decays of this thread's 8 tokens x 2 channels and their running sums from the
    // first of them, block partial sums to shared memory.  It needs only the w tile, so it runs one chunk ahead, inside
    // the window in which the second MMA group of the chunk before executes.
    // Row t = 16*w4 + 8*half + tt has swizzle phase tt, so one per-thread base pointer plus a per-tt XOR term
    // addresses every tile (tile offsets are compile-time constants relative to the stage base).
    const uint32_t lane_chunk = (uint32_t)(lane >> 2);
    const uint32_t tofs = (uint32_t)((16 * w4 + 8 * half) * 128 + ((lane & 3) << 2));
    float2 x[8];
    auto pass1 = [&](int ic1) {
        const uint8_t *wt = smem + (ic1 & 1) * SM::kStage + 3 * kTile + tofs;
        const bool full_chunk = (ic1 + 1) * kChunk <= a.T;
        float2 cs = make_float2(0.f, 0.f);
#pragma unroll
        for (int tt = 0; tt < 8; ++tt) {
            const float2 w2 = ld_bf2(wt + tt * 128 + ((lane_chunk ^ tt) << 4));
            const float2 e2 = mul2(w2, make_float2(kLog2e, kLog2e));
            float2 l2 = mul2(make_float2(ex2f(e2.x), ex2f(e2.y)), make_float2(-kLog2e, -kLog2e));
            l2.x = fmaxf(l2.x, kMinLogDecay2);
            l2.y = fmaxf(l2.y, kMinLogDecay2);
            if (!full_chunk && ic1 * kChunk + 16 * w4 + 8 * half + tt >= a.T) l2 = make_float2(0.f, 0.f);
            cs = add2(cs, l2);
            x[tt] = cs;
        }
        *reinterpret_cast<float2 *>(&(half ? sTail : sHead)[w4 * 64 + 2 * lane]) = cs;
    };
    if (!cta_wait(&bar_full[0], 0, warp)) err = 1;
    if (err == 0) ++loads_consumed;
    WKV6_CSTAMP(4);
    pass1(0);
    if (!__syncthreads_and(err == 0)) err = err ? err : 10;

    WKV6_CSTAMP(5);
    for (int ic = 0; ic < nchunks && err == 0; ++ic) {
        const int c = ic;  // chunk processed in this iteration
        const int st = ic & 1;
        uint8_t *sR = smem + st * SM::kStage;  // this stage: r, k, v, w tiles at +0, +kTile, +2 kTile, +3 kTile
        const uint64_t so = (uint64_t)(st * (SM::kStage >> 4));
        uint8_t *const tbase = sR + tofs;
        bool wide;  // single reference point for this chunk (the same value in every warp)
        WKV6_TSTAMP(ic, 2);

        // ---- pass 2: scaled operands.  The block reference is the boundary between the two token halves, so the
        // running sums of the second half are already relative to it and those of the first half need only -head.
        // The scaling itself runs on packed bf16 pairs: r and k are exact bf16 inputs, factors are rounded to bf16.
        {
            float2 pre = make_float2(0.f, 0.f), head, tail, all;
            head = tail = all = make_float2(0.f, 0.f);
#pragma unroll
            for (int J = 0; J < 4; ++J) {
                const float2 hj = *reinterpret_cast<const float2 *>(&sHead[J * 64 + 2 * lane]);
                const float2 tl = *reinterpret_cast<const float2 *>(&sTail[J * 64 + 2 * lane]);
                const float2 tj = add2(hj, tl);
                if (J < w4) pre = add2(pre, tj);
                if (J == w4) { head = hj; tail = tl; }
                // log2 decay of the whole chunk, summed in the same order by every thread: the reference below is rounded
                // from it, and all warps must round the same bits
                all = add2(all, tj);
            }
            wide = !__any_sync(0xffffffffu, fminf(all.x, all.y) < kWideLimit2);  // a warp sees all 64 channels
            // reference relative to the chunk start: the block's 8th token, or half of the chunk's total decay (an integer)
            const float2 ref = wide ? make_float2(rintf(0.5f * all.x), rintf(0.5f * all.y)) : add2(pre, head);
            const float2 gstart = half ? add2(pre, head) : pre;  // running sum before this thread's first token
            const float2 nbase = make_float2(gstart.x - ref.x, gstart.y - ref.y);
            const __nv_bfloat162 fR = to_bf2(make_float2(ex2f(ref.x), ex2f(ref.y)));
            // factors of the k~ copies for block distances 1..3 (only those with w4 + delta <= 3 exist)
            // (a factor can lie below the bf16 range while its product with k~ <= 2^115 does not: it is applied in two parts)
            __nv_bfloat162 fD[3], fE[3];
            fD[0] = fD[1] = fD[2] = fE[0] = fE[1] = fE[2] = to_bf2(make_float2(0.f, 0.f));
            if (!wide) {
                float2 acc = tail;
#pragma unroll
                for (int dl = 1; dl <= 3; ++dl) {
                    const int Jt = w4 + dl;  // the row block this copy serves
                    if (Jt <= 3) {
                        const float2 hj = *reinterpret_cast<const float2 *>(&sHead[Jt * 64 + 2 * lane]);
                        const float2 tl = *reinterpret_cast<const float2 *>(&sTail[Jt * 64 + 2 * lane]);
                        const float2 n = add2(acc, hj), n1 = make_float2(fmaxf(n.x, -120.f), fmaxf(n.y, -120.f));
                        fD[dl - 1] = to_bf2(make_float2(ex2f(n1.x), ex2f(n1.y)));
                        fE[dl - 1] = to_bf2(make_float2(ex2f(fmaxf(n.x - n1.x, -120.f)), ex2f(fmaxf(n.y - n1.y, -120.f))));
                        acc = add2(acc, add2(hj, tl));
                    }
                }
            }
            if (warp == 0) *reinterpret_cast<float2 *>(&sDtot[2 * lane]) = make_float2(ex2f(all.x), ex2f(all.y));
            const float2 fK = make_float2(ex2f(all.x - ref.x), ex2f(all.y - ref.y));  // decay from the reference point to the chunk end
            if (warp == 4) *reinterpret_cast<float2 *>(&sFK[2 * lane]) = wide ? fK : make_float2(1.f, 1.f);
            const int kdo = (int)(sKD - sR), kho = (int)(sKH - sR);  // uniform offsets of the copy tiles from this stage
            // all loads first: shared-memory loads cannot be scheduled across the stores below
            __nv_bfloat162 rbv[8], kbv[8];
#pragma unroll
            for (int tt = 0; tt < 8; ++tt) {
                const uint8_t *pt = tbase + tt * 128 + ((lane_chunk ^ tt) << 4);
                rbv[tt] = *reinterpret_cast<const __nv_bfloat162 *>(pt);
                kbv[tt] = *reinterpret_cast<const __nv_bfloat162 *>(pt + kTile);
            }
            // One straight-line block for all eight tokens (no branch inside: the scheduler interleaves the eight
            // dependency chains exp -> round -> scale -> store); the copies of the rare per-block mode follow separately.
            // feb[tt] = e^{c_{t-1} - c_ref} for this thread's token tt; feb[tt + 1] is at the same time e^{c_t - c_ref},
            // the inverse of the factor of k~_t, which turns r_t u into the operand of the bonus product.
            __nv_bfloat162 ktv[8], rtv[8], feb[9];
            {
                float2 fe[9], fk2[8];
#pragma unroll
                for (int tt = 0; tt < 8; ++tt) {  // exponents, then all exponentials back to back
                    const float2 xp = (tt == 0) ? make_float2(0.f, 0.f) : x[tt - 1];
                    fe[tt] = add2(xp, nbase);                                              // c_{t-1} - c_ref
                    fk2[tt] = make_float2(-nbase.x - x[tt].x, -nbase.y - x[tt].y);         // c_ref - c_t
                }
                fe[8] = add2(x[7], nbase);
#pragma unroll
                for (int tt = 0; tt < 9; ++tt) feb[tt] = to_bf2(make_float2(ex2f(fe[tt].x), ex2f(fe[tt].y)));
#pragma unroll
                for (int tt = 0; tt < 8; ++tt) {
                    fk2[tt] = make_float2(ex2f(fk2[tt].x), ex2f(fk2[tt].y));
                    rtv[tt] = __hmul2(rbv[tt], feb[tt]);
                    ktv[tt] = __hmul2(kbv[tt], to_bf2(fk2[tt]));
                }
            }
#pragma unroll
            for (int tt = 0; tt < 8; ++tt) {
                uint8_t *pt = tbase + tt * 128 + ((lane_chunk ^ tt) << 4);
                *reinterpret_cast<__nv_bfloat162 *>(pt) = rtv[tt];                                  // r~
                *reinterpret_cast<__nv_bfloat162 *>(pt + 3 * kTile) = __hmul2(rtv[tt], fR);         // r^ (over w)
                *reinterpret_cast<__nv_bfloat162 *>(pt + kTile) = ktv[tt];                          // k~ distance 0
                if (wide) *reinterpret_cast<__nv_bfloat162 *>(pt + kho) = __hmul2(__hmul2(rbv[tt], ub), feb[tt + 1]);  // q
            }
            if (!wide) {
                const __nv_bfloat162 fKb = to_bf2(fK);
                float bon[8];
#pragma unroll
                for (int tt = 0; tt < 8; ++tt) {
                    uint8_t *pt = tbase + tt * 128 + ((lane_chunk ^ tt) << 4);
                    *reinterpret_cast<__nv_bfloat162 *>(pt + kho) = __hmul2(ktv[tt], fKb);  // k^
                    const float2 rk = mul2(__bfloat1622float2(rbv[tt]), __bfloat1622float2(kbv[tt]));
                    bon[tt] = fmaf(rk.x, u2.x, rk.y * u2.y);
                }
                // sum the bonus partials over the 32 channel pairs: 8 values across 32 lanes in 9 shuffles
                {
                    const bool up = (lane & 16) != 0;
#pragma unroll
                    for (int i2 = 0; i2 < 4; ++i2) {
                        const float send = up ? bon[i2] : bon[i2 + 4];
                        const float keep = up ? bon[i2 + 4] : bon[i2];
                        bon[i2] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
                    }
                }
                {
                    const bool up = (lane & 8) != 0;
#pragma unroll
                    for (int i2 = 0; i2 < 2; ++i2) {
                        const float send = up ? bon[i2] : bon[i2 + 2];
                        const float keep = up ? bon[i2 + 2] : bon[i2];
                        bon[i2] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
                    }
                }
                {
                    const bool up = (lane & 4) != 0;
                    const float send = up ? bon[0] : bon[1];
                    const float keep = up ? bon[1] : bon[0];
                    bon[0] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
                }
                bon[0] += __shfl_xor_sync(0xffffffffu, bon[0], 2);
                bon[0] += __shfl_xor_sync(0xffffffffu, bon[0], 1);
                if ((lane & 3) == 0) {
                    const int tok = ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
                    sBonus[16 * w4 + 8 * half + tok] = bon[0];
                }
#pragma unroll
                for (int tt = 0; tt < 8; ++tt) {
                    uint8_t *pt = tbase + tt * 128 + ((lane_chunk ^ tt) << 4);
                    const __nv_bfloat162 kt = ktv[tt];
                    if (w4 <= 2) *reinterpret_cast<__nv_bfloat162 *>(pt + kdo) = __hmul2(__hmul2(kt, fD[0]), fE[0]);              // rows [0,48)
                    if (w4 <= 1) *reinterpret_cast<__nv_bfloat162 *>(pt + kdo + 48 * 128) = __hmul2(__hmul2(kt, fD[1]), fE[1]);   // rows [48,80)
                    if (w4 == 0) *reinterpret_cast<__nv_bfloat162 *>(pt + kdo + 80 * 128) = __hmul2(__hmul2(kt, fD[2]), fE[2]);   // rows [80,96)
                }
            }
        }
        // the previous chunk's y tile and checkpoint copies must have left shared memory before the epilogues rewrite them
        if (copy_thread) bulk_wait_read<0>();
        fence_proxy_async_smem();
        tc_fence_before_sync();
        __syncthreads();
        WKV6_TSTAMP(ic, 3);

        if (tid == 0) {
            tc_fence_after_sync();
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)  // A (distance 0) = r~ k~^T
                umma_ss(tmA0, dR + so + 2 * kk, dK + so + 2 * kk, idKK, kk > 0);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)  // A (distances 1..3) = r~ [k~ copies]^T
                if (!wide) umma_ss(tmAD, dR + so + 2 * kk, dKD + 2 * kk, idKK96, kk > 0);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)  // q k~^T: its diagonal is the bonus sum_i r u k of every token
                if (wide) umma_ss(tmAU, dKH + 2 * kk, dK + so + 2 * kk, idKK, kk > 0);
            umma_commit(bar_mma1);
        } else if (tid == 64) {
            tc_fence_after_sync();
#pragma unroll
            // state increment = k~^T v with its rows scaled afterwards, or k^^T v
            const uint64_t dInc = wide ? dK + so : dKH;
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) umma_ss(tmS, dInc + 128 * kk, dV + so + 128 * kk, idMM, kk > 0);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)  // y = r^ S_in
                umma_ss(tmY, dW + so + 2 * kk, dSB + 128 * kk, idKM, kk > 0);
            umma_commit(bar_mma1);
        }
        WKV6_TSTAMP(ic, 4);
        if (!cta_wait(bar_mma1, ic & 1, warp)) err = 2;
        tc_fence_after_sync();
        WKV6_TSTAMP(ic, 5);

        // ---- epilogue of the intra-chunk matrix: pick, mask, round, store as the A operand of A v.
        // This warp covers column blocks J = 2*half and 2*half + 1 of row block I = w4.
        const float d0 = sDtot[ta], d1 = sDtot[ta + 8];
        const float g0 = sFK[ta], g1 = sFK[ta + 8];
        {
            const int I = w4;
#pragma unroll
            for (int jj = 0; jj < 2; ++jj) {
                const int J = 2 * half + jj;
                uint32_t o0 = 0, o1 = 0, o2 = 0, o3 = 0;  // (row ta: cols 2q,2q+1 | 8+2q,..) and the same for row ta+8
                if (J <= I) {
                    const int dl = I - J;
                    const uint32_t src = (dl == 0 || wide) ? (tmA0 + wl + 16 * J)
                                                           : (tmAD + wl + (dl == 1 ? 16 * J : dl == 2 ? 48 + 16 * J : 80));
                    uint32_t v8[8];
                    tmem_ld_16x256b_x2(src, v8);
                    tmem_wait_ld();
                    float f[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(v8[e]);
                    if (dl == 0) {
                        // diagonal block: rows r0 (e = 0, 1, 4, 5) and r0 + 8 (e = 2, 3, 6, 7), columns 2q + (e & 1) (+ 8 for
                        // e >= 4).  e = 2, 3 lie below the diagonal, e = 4, 5 above it; the other four need the test, and the
                        // diagonal element itself comes from the bonus product.
                        uint32_t b8[8];
                        if (wide) {
                            tmem_ld_16x256b_x2(tmAU + wl + 16 * J, b8);
                            tmem_wait_ld();
                        } else {
                            b8[0] = b8[1] = __float_as_uint(sBonus[ta]);
                            b8[6] = b8[7] = __float_as_uint(sBonus[ta + 8]);
                        }
                        const int c0 = 2 * q, c1 = 2 * q + 1;
                        f[0] = (c0 < r0) ? f[0] : (c0 == r0 ? __uint_as_float(b8[0]) : 0.f);
                        f[1] = (c1 < r0) ? f[1] : (c1 == r0 ? __uint_as_float(b8[1]) : 0.f);
                        f[6] = (c0 < r0) ? f[6] : (c0 == r0 ? __uint_as_float(b8[6]) : 0.f);
                        f[7] = (c1 < r0) ? f[7] : (c1 == r0 ? __uint_as_float(b8[7]) : 0.f);
                        f[4] = 0.f;
                        f[5] = 0.f;
                    }
                    o0 = pack_bf2(f[0], f[1]); o2 = pack_bf2(f[2], f[3]);
                    o1 = pack_bf2(f[4], f[5]); o3 = pack_bf2(f[6], f[7]);
                }
                *reinterpret_cast<uint32_t *>(sAM + foA[2 * jj]) = o0;      // columns 16J + 2q
                *reinterpret_cast<uint32_t *>(sAM + foA[2 * jj + 1]) = o1;  // columns 16J + 8 + 2q
                *reinterpret_cast<uint32_t *>(sAM + foB[2 * jj]) = o2;
                *reinterpret_cast<uint32_t *>(sAM + foB[2 * jj + 1]) = o3;
            }
        }
        // ---- state update in registers and its bf16 operand copy for the next chunk
        {
            uint32_t v16[16];
            tmem_ld_16x256b_x4(tmS + wl + cb, v16);
            tmem_wait_ld();
#pragma unroll
            for (int nn = 0; nn < 4; ++nn) {
                S[4 * nn + 0] = fmaf(S[4 * nn + 0], d0, g0 * __uint_as_float(v16[4 * nn + 0]));
                S[4 * nn + 1] = fmaf(S[4 * nn + 1], d0, g0 * __uint_as_float(v16[4 * nn + 1]));
                S[4 * nn + 2] = fmaf(S[4 * nn + 2], d1, g1 * __uint_as_float(v16[4 * nn + 2]));
                S[4 * nn + 3] = fmaf(S[4 * nn + 3], d1, g1 * __uint_as_float(v16[4 * nn + 3]));
                *reinterpret_cast<uint32_t *>(sSB + foA[nn]) = pack_bf2(S[4 * nn], S[4 * nn + 1]);
                *reinterpret_cast<uint32_t *>(sSB + foB[nn]) = pack_bf2(S[4 * nn + 2], S[4 * nn + 3]);
            }
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        if (!__syncthreads_and(err == 0)) { err = err ? err : 11; break; }
        WKV6_TSTAMP(ic, 6);

        if (tid == 0) {
            tc_fence_after_sync();
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)  // y += A v
                umma_ss(tmY, dAM + 2 * kk, dV + so + 128 * kk, idKM, true);
            umma_commit(bar_mma2);
        } else if (copy_thread) {
            // the state entering the next chunk is complete in shared memory: checkpoint it for the backward.
            // Its read is drained (bulk_wait_read) before the next chunk's first barrier, ahead of the rewrite.
            if (a.ckpt != nullptr && c + 1 < nchunks) {
                bulk_store(a.ckpt + ((size_t)blockIdx.x * nchunks + c + 1) * 4096, sSB, kTile);
                bulk_commit();
            }
        }
        WKV6_TSTAMP(ic, 7);
        if (ic + 1 < nchunks) {  // the next chunk's decays, while the tensor core works
            if (!cta_wait(&bar_full[st ^ 1], ((ic + 1) >> 1) & 1, warp)) err = 1;
            if (err == 0) ++loads_consumed;
            pass1(ic + 1);
        }
        if (!cta_wait(bar_mma2, ic & 1, warp)) err = err ? err : 3;
        tc_fence_after_sync();
        WKV6_TSTAMP(ic, 8);

        // ---- y epilogue: round to bf16 into the (now free) A tile, one TMA store per chunk
        {
            uint32_t v16[16];
            tmem_ld_16x256b_x4(tmY + wl + cb, v16);
            tmem_wait_ld();
#pragma unroll
            for (int nn = 0; nn < 4; ++nn) {
                *reinterpret_cast<uint32_t *>(sAM + foA[nn]) =
                    pack_bf2(__uint_as_float(v16[4 * nn]), __uint_as_float(v16[4 * nn + 1]));
                *reinterpret_cast<uint32_t *>(sAM + foB[nn]) =
                    pack_bf2(__uint_as_float(v16[4 * nn + 2]), __uint_as_float(v16[4 * nn + 3]));
            }
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        if (!__syncthreads_and(err == 0)) { err = err ? err : 12; break; }
        WKV6_TSTAMP(ic, 9);
        if (copy_thread && a.write_y) {
            tma_store_3d(&tm_y, sAM, h * 64, c * kChunk, b);
            bulk_commit();
        }
        if (ic + 2 < nchunks) { issue_loads(ic + 2); ++loads_issued; }
    }

    WKV6_CSTAMP(6);
    // ---- unwind: drain this CTA's copies, report, release tensor memory
    if (err != 0 && load_slot >= 0) {
        // loads still in flight target this CTA's shared memory: wait for them (bounded) before leaving
        for (int ic2 = loads_consumed; ic2 < loads_issued; ++ic2)
            if (ic2 != skip_chunk) mbar_wait(&bar_full[ic2 & 1], (ic2 >> 1) & 1);
    }
    if (copy_thread) {
        if (err != 0) atomicExch(&g_chunk_status, err);
        bulk_wait<0>();
    }
    if (err == 0 && a.s_out != nullptr) {
        const size_t so2 = (size_t)blockIdx.x * 4096;
#pragma unroll
        for (int nn = 0; nn < 4; ++nn)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int i = ta + (e >= 2 ? 8 : 0), j = 8 * (n0 + nn) + 2 * q + (e & 1);
                store_any(a.s_out, a.s_dtype, so2 + (size_t)i * 64 + j, S[4 * nn + e]);
            }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tb, 256);
    WKV6_CSTAMP(7);
}

}  // namespace wkv6
