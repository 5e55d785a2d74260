// Chunked WKV6 backward for sm_100a.  One CTA walks the 64-token chunks of one (batch, head) sequence in
// descending time; the reverse state Abar (N x N, fp32) and the running sum Z stay on chip across chunks, the
// forward state at each chunk start comes from the bf16 checkpoints the forward wrote.
//
// With c_t the inclusive running sum of log-decays inside the chunk, P[t][s] = gy_t . v_s (s < t; the diagonal
// vg_t = gy_t . v_t is kept aside), A the forward intra-chunk matrix (see wkv6_chunk_fwd.cuh):
//   gr_t[i] = e^{c_{t-1}[i]} ( sum_{s<t} P[t][s] k_s[i] e^{-c_s[i]}  +  sum_j S_in[i][j] gy_t[j] )  + u_i k_t[i] vg_t
//   gk_s[i] = e^{-c_s[i]}   ( sum_{t>s} P[t][s] r_t[i] e^{c_{t-1}[i]} + e^{c_63[i]} sum_j Abar[i][j] v_s[j] ) + u_i r_s[i] vg_s
//   gv_s[j] = sum_{t>=s} A[t][s] gy_t[j] + sum_i k_s[i] e^{c_63[i]-c_s[i]} Abar[i][j]
//   Abar'   = diag(e^{c_63}) Abar + sum_t (r_t e^{c_{t-1}}) (x) gy_t
//   gw_t[i] = -exp(w_t[i]) G_t[i],   G_t = e^{c_63} <S_in, Abar>_i + sum_{tau>t} (r_tau e^{c_{tau-1}}) GR2[tau]
//                                         + sum_{s<t} (k_s e^{c_63-c_s}) GK2[s] + sum_{s<t<tau} e^{c_{tau-1}-c_s} k_s r_tau P[tau][s]
//   where GR2 = gy S_in^T and GK2 = v Abar^T.  The last (rectangle) sum is obtained as
//   sum_{tau>t} r~_tau GR1[tau] - sum_{s>=t} k~_s GK1[s] from the intra-chunk parts GR1, GK1 of gr and gk: every product
//   e^{..} k_s r_tau P[tau][s] with s, tau > t occurs in both sums and cancels, and it cancels exactly because (1) the
//   block reference points are rounded to integers in the log2 domain, so the block-pair factor is a power of two
//   and commutes with bf16 rounding, and (2) the multipliers r~, k~ used here are the bf16-rounded operand values.
// The exponentials are split around per-16-token-block reference points exactly as in the forward, so every
// bf16 operand stays finite; block pairs (I, J) are separate MMAs whose output is restricted to the 16 rows of
// one block with the disable-output-lane mask of tcgen05.mma.  A chunk whose total decay is mild in every channel
// (kWideLimit2) uses one reference, half of the chunk's total log2 decay, for all four blocks: the block-pair factors are
// then 1, the copies are skipped and GR1 / GK1 are two plain MMAs.
//
// All element-wise work is done in the accumulator-fragment layout of tcgen05.ld.16x256b: a thread owns tokens
// {r0, r0+8} of block (warp & 3) and channels 8n+2q, 8n+2q+1 for four values of n ((warp >> 2) selects which
// four), so the per-element decay factors computed before the MMAs are still in registers when the
// accumulators come back.  Running sums along time are lane scans over the 8 lanes that share q.
//
// Tensor-memory map (256 columns): lanes 0-15: [0,64) P -> GR1 | [64,128) A (distance 0) -> GK1 | [128,192) GR2 | [192,256) GK2
//                                  lanes 16-31: [0,64) Abar increment | [64,128) gv | [128,224) A (distances 1..3)
//                                               | [224,256) per-thread stash of the bf16 log-decays until gw is formed
#pragma once

#include "wkv6_chunk_fwd.cuh"

namespace wkv6 {

struct ChunkBwdSmem {
    static constexpr int oR = 0;                    // r  -> r~ (in place)
    static constexpr int oK = oR + kTile;           // k  -> k~ (in place)
    static constexpr int oV = oK + kTile;
    static constexpr int oW = oV + kTile;           // w  -> r^ = r~ e^{c_rho - c_start} (in place)
    static constexpr int oG = oW + kTile;           // gy
    static constexpr int oS = oG + kTile;           // checkpointed state at the chunk start [i][j]
    static constexpr int oKH = oS + kTile;          // k^ = k~ e^{c_63 - c_rho}
    static constexpr int oKD = oKH + kTile;         // k~ copies for block distances 1..3 (96 rows); later the gv tile
    static constexpr int oRD = oKD + 96 * 128;      // r~ copies for block distances 1..3 (96 rows); later the gw tile
    static constexpr int oP = oRD + 96 * 128;       // masked P (bf16); later the gr tile
    static constexpr int oAM = oP + kTile;          // masked A (bf16); later the gk tile
    static constexpr int oAB = oAM + kTile;         // bf16 copy of Abar [i][j]
    static constexpr int oHead = oAB + kTile;       // float [4][64] log2-decay sum of the first 8 tokens of a block
    static constexpr int oTot = oHead + 1024;       // float [4][64] log2-decay sum of the block
    static constexpr int oOff = oTot + 1024;        // float [4][64] integer reference point of the block, relative to the block start
    static constexpr int oFRb = oOff + 1024;        // bf16  [4][64] 2^{ref(I)}            (reference relative to the chunk start)
    static constexpr int oFKb = oFRb + 512;         // bf16  [4][64] 2^{c_63 - ref(J)}
    static constexpr int oMKb = oFKb + 512;         // bf16  [6][64] 2^{ref(J+d) - ref(J)}: d=1: J=0..2, d=2: J=0..1, d=3: J=0
    static constexpr int oMK2 = oMKb + 768;         // bf16  [6][64] second part of the same factor when it is below 2^-120
    static constexpr int oU = oMK2 + 768;           // float [64]    u of this head
    static constexpr int oDtot = oU + 256;          // float [64]    2^{c_63}
    static constexpr int oBonus = oDtot + 256;      // float [2][64]
    static constexpr int oVG = oBonus + 512;        // float [64]
    static constexpr int oT1 = oVG + 256;           // float [2][64] <S_in, Abar>_i, one partial per column half
    static constexpr int oXtot = oTot;              // float [4][64] block sums for gw (sTot is dead by then)
    static constexpr int oBtot = oHead;             // float [4][64] block sums for gw (sHead is dead by then)
    static constexpr int oGU = oHead;               // float [4][64] final reduction of gu (after the last chunk)
    static constexpr int oBar = oT1 + 512;          // full, mma1, mma2
    static constexpr int oSlot = oBar + 32;
    static constexpr int kBytes = oSlot + 16;
    static constexpr int kAlloc = kBytes;
};

struct ChunkBwdArgs {
    const void *u; int u_dtype;
    void *gu; int gu_dtype;
    const __nv_bfloat16 *ckpt;
    const float *ab_in;  // optional [B*H][64][64]: reverse state entering at the end of the sequence (zero if NULL)
    bool zero_init;      // the forward started from a zero state: gw at t = 0 is exactly zero
    int B, T, H;
    // Hand-over between the two backward kernels, one word per (batch, head) sequence: chunk_bwd_wide_kernel writes
    // 1 for a sequence it abandoned (0 otherwise); chunk_bwd_kernel given the same array skips sequences marked 0.
    int *flags;
};

// D[tmem] (+)= A * B restricted to the TMEM lanes whose mask bit is 0.
__device__ __forceinline__ void umma_ss_masked(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                               bool accumulate, int enabled_block) {
    const uint32_t on = 0xFFFF0000u, off = 0xFFFFFFFFu;
    const uint32_t m0 = enabled_block == 0 ? on : off, m1 = enabled_block == 1 ? on : off;
    const uint32_t m2 = enabled_block == 2 ? on : off, m3 = enabled_block == 3 ? on : off;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"((uint32_t)accumulate), "r"(m0), "r"(m1), "r"(m2), "r"(m3)
        : "memory");
}

// one repetition: 8 columns, 4 values per thread (rows r0 / r0+8 x columns 2q, 2q+1); no wait
__device__ __forceinline__ void tmem_ld_16x256b_x1(uint32_t taddr, float (&f)[4]) {
    uint32_t v0, v1, v2, v3;
    asm volatile("tcgen05.ld.sync.aligned.16x256b.x1.b32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v0), "=r"(v1), "=r"(v2), "=r"(v3) : "r"(taddr));
    f[0] = __uint_as_float(v0); f[1] = __uint_as_float(v1); f[2] = __uint_as_float(v2); f[3] = __uint_as_float(v3);
}

__device__ __forceinline__ void tmem_ld_16x256b_x4(uint32_t taddr, float (&f)[16]) {
    uint32_t v[16];
    ptx::tmem_ld_16x256b_x4(taddr, v);
    ptx::tmem_wait_ld();
#pragma unroll
    for (int e = 0; e < 16; ++e) f[e] = __uint_as_float(v[e]);
}

// 2^n for an integer-valued float n (exact; flushes to zero below the normal range)
__device__ __forceinline__ float pow2i(float n) {
    const int e = (int)n + 127;
    return e <= 0 ? 0.f : __int_as_float((e > 254 ? 254 : e) << 23);
}

// inclusive prefix over the 16 tokens of a block: a = row r0, b = row r0 + 8, lanes sharing q hold consecutive r0
__device__ __forceinline__ void scan_prefix16(float &a, float &b, int r0, int lane) {
#pragma unroll
    for (int d = 1; d < 8; d <<= 1) {
        const float ta = __shfl_up_sync(0xffffffffu, a, 4 * d);
        const float tb = __shfl_up_sync(0xffffffffu, b, 4 * d);
        if (r0 >= d) { a += ta; b += tb; }
    }
    b += __shfl_sync(0xffffffffu, a, 28 + (lane & 3));
}
// inclusive suffix over the 16 tokens of a block
__device__ __forceinline__ void scan_suffix16(float &a, float &b, int r0, int lane) {
#pragma unroll
    for (int d = 1; d < 8; d <<= 1) {
        const float ta = __shfl_down_sync(0xffffffffu, a, 4 * d);
        const float tb = __shfl_down_sync(0xffffffffu, b, 4 * d);
        if (r0 + d < 8) { a += ta; b += tb; }
    }
    a += __shfl_sync(0xffffffffu, b, lane & 3);
}

// The same scans when a thread holds two ADJACENT tokens of the block (a = token 2 r0, b = token 2 r0 + 1; see the token
// order of chunk_bwd_wide_kernel): the pair is summed locally and only the pair sums travel, three shuffles per scan.
__device__ __forceinline__ void scan_prefix16_adj(float &a, float &b, int r0) {
    const float s = a + b;
    float t = s;
#pragma unroll
    for (int d = 1; d < 8; d <<= 1) {
        const float o = __shfl_up_sync(0xffffffffu, t, 4 * d);
        if (r0 >= d) t += o;
    }
    a += t - s;  // tokens before this pair, plus a
    b = t;       // ... plus a and b
}
__device__ __forceinline__ void scan_suffix16_adj(float &a, float &b, int r0) {
    const float s = a + b;
    float t = s;
#pragma unroll
    for (int d = 1; d < 8; d <<= 1) {
        const float o = __shfl_down_sync(0xffffffffu, t, 4 * d);
        if (r0 + d < 8) t += o;
    }
    b += t - s;  // tokens after this pair, plus b
    a = t;       // ... plus a and b
}

// MINB = CTAs per SM the kernel is compiled for.  With two, a thread has 128 registers and the kernel spills (its copies
// of k~ and r~ leave no shared or tensor memory to park state in); with one it has 224 and spills nothing: a launch with at
// most one CTA per SM anyway (B*H <= number of SMs) runs 30 % faster in that form, a full one 10 % slower.
template <int MINB>
__global__ void __launch_bounds__(256, MINB) chunk_bwd_kernel(const __grid_constant__ CUtensorMap tm_r,
                                                           const __grid_constant__ CUtensorMap tm_k,
                                                           const __grid_constant__ CUtensorMap tm_v,
                                                           const __grid_constant__ CUtensorMap tm_w,
                                                           const __grid_constant__ CUtensorMap tm_gy,
                                                           const __grid_constant__ CUtensorMap tm_gr,
                                                           const __grid_constant__ CUtensorMap tm_gk,
                                                           const __grid_constant__ CUtensorMap tm_gv,
                                                           const __grid_constant__ CUtensorMap tm_gw,
                                                           const ChunkBwdArgs a) {
    using namespace ptx;
    using SM = ChunkBwdSmem;
    // Declared with the alignment the swizzled tiles need, so that the compiler keeps every access in the shared
    // address space with 32-bit addresses; the base is verified once instead of being realigned by pointer math.
    extern __shared__ __align__(1024) uint8_t wkv6_chunk_smem[];
    uint8_t *const smem = wkv6_chunk_smem;
    if ((smem_u32(smem) & 1023u) != 0) {
        if (threadIdx.x == 0) atomicExch(&g_chunk_status, 50);
        return;
    }
    // Launched behind the fast kernel with programmatic serialization: its CTAs may already be resident while that
    // kernel runs; nothing it wrote (the flags first of all) is read before this wait returns.  (Without a kernel before
    // it in the stream, or without the launch attribute, the wait returns at once.)
    ptx::grid_dependency_wait();
    if (a.flags != nullptr && a.flags[blockIdx.x] == 0) return;  // the fast kernel has completed this sequence
    uint8_t *sR = smem + SM::oR, *sK = smem + SM::oK, *sV = smem + SM::oV, *sW = smem + SM::oW, *sG = smem + SM::oG;
    uint8_t *sS = smem + SM::oS, *sKH = smem + SM::oKH, *sKD = smem + SM::oKD, *sRD = smem + SM::oRD;
    uint8_t *sP = smem + SM::oP, *sAM = smem + SM::oAM, *sAB = smem + SM::oAB;
    float *sHead = reinterpret_cast<float *>(smem + SM::oHead), *sTot = reinterpret_cast<float *>(smem + SM::oTot);
    float *sOff = reinterpret_cast<float *>(smem + SM::oOff), *sDtot = reinterpret_cast<float *>(smem + SM::oDtot);
    __nv_bfloat16 *sFRb = reinterpret_cast<__nv_bfloat16 *>(smem + SM::oFRb);
    __nv_bfloat16 *sFKb = reinterpret_cast<__nv_bfloat16 *>(smem + SM::oFKb);
    __nv_bfloat16 *sMKb = reinterpret_cast<__nv_bfloat16 *>(smem + SM::oMKb);
    __nv_bfloat16 *sMK2 = reinterpret_cast<__nv_bfloat16 *>(smem + SM::oMK2);
    float *sU = reinterpret_cast<float *>(smem + SM::oU);
    float *sBonus = reinterpret_cast<float *>(smem + SM::oBonus), *sVG = reinterpret_cast<float *>(smem + SM::oVG);
    float *sXtot = reinterpret_cast<float *>(smem + SM::oXtot), *sBtot = reinterpret_cast<float *>(smem + SM::oBtot);
    float *sT1 = reinterpret_cast<float *>(smem + SM::oT1);
    float *sGU = reinterpret_cast<float *>(smem + SM::oGU);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + SM::oBar);
    // bar_full: w, r, k tiles (needed first); bar_late: v, gy and the checkpointed state (needed by the first MMA group)
    uint64_t *bar_full = bars, *bar_mma1 = bars + 1, *bar_mma2 = bars + 2, *bar_late = bars + 3;
    uint32_t *slot = reinterpret_cast<uint32_t *>(smem + SM::oSlot);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int w4 = warp & 3, half = warp >> 2, n0 = 4 * half;
    const int r0 = lane >> 2, q = lane & 3;
    const int ta = 16 * w4 + r0;  // this thread's rows: ta and ta + 8
    const int b = blockIdx.x / a.H, h = blockIdx.x % a.H;
    const int nchunks = (a.T + kChunk - 1) / kChunk;

    if (tid == 0) {
        mbar_init(bar_full, 1);
        mbar_init(bar_late, 1);
        mbar_init(bar_mma1, 4);  // four issuing threads
        mbar_init(bar_mma2, 3);  // three issuing threads
        fence_mbar_init();
        prefetch_tensormap(&tm_r); prefetch_tensormap(&tm_k); prefetch_tensormap(&tm_v); prefetch_tensormap(&tm_w);
        prefetch_tensormap(&tm_gy); prefetch_tensormap(&tm_gr); prefetch_tensormap(&tm_gk);
        prefetch_tensormap(&tm_gv); prefetch_tensormap(&tm_gw);
    }
    if (warp == 0) {
        tmem_alloc(slot, 256);
        tmem_relinquish();
    }
    // zero: the reverse state (registers + operand copy)
    float AB[16];
#pragma unroll
    for (int nn = 0; nn < 4; ++nn) {
        const int j0 = 8 * (n0 + nn) + 2 * q;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int i = ta + (e >= 2 ? 8 : 0);
            AB[4 * nn + e] = a.ab_in ? a.ab_in[(size_t)blockIdx.x * 4096 + (size_t)i * 64 + j0 + (e & 1)] : 0.f;
        }
        *reinterpret_cast<uint32_t *>(sAB + sw128_off(ta, j0)) = pack_bf2(AB[4 * nn], AB[4 * nn + 1]);
        *reinterpret_cast<uint32_t *>(sAB + sw128_off(ta + 8, j0)) = pack_bf2(AB[4 * nn + 2], AB[4 * nn + 3]);
    }
    float gu_acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) gu_acc[e] = 0.f;
    if (tid < 64) sU[tid] = load_any(a.u, a.u_dtype, (size_t)h * 64 + tid);
    // byte offsets of this thread's fragment elements in a swizzled tile: row ta, column pair 8(n0+nn)+2q; row ta+8 is
    // 1024 bytes further (same swizzle phase)
    uint32_t fo4[4];
#pragma unroll
    for (int nn = 0; nn < 4; ++nn) fo4[nn] = sw128_off(ta, 8 * (n0 + nn) + 2 * q);
#define FO(nn, hrow) (fo4[nn] + 1024u * (hrow))

    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tbase = *slot;
    const uint32_t lo = (uint32_t)(32 * w4) << 16;  // this warp's TMEM lane quarter
    const uint32_t tmP = tbase, tmA = tbase + 64, tmGR2 = tbase + 128, tmGK2 = tbase + 192;
    const uint32_t tmAN = tbase + (16u << 16), tmGV = tbase + (16u << 16) + 64, tmAD = tbase + (16u << 16) + 128;
    const uint32_t cb = 8 * n0;  // first accumulator column of this thread's fragment
    const uint32_t tmStash = tbase + (16u << 16) + lo + 224 + 16 * half;  // 16 columns x 16 lanes per warp: 8 registers per thread

    auto issue_loads = [&](int c) {
        mbar_expect_tx(bar_full, 3 * kTile);
        tma_load_3d(sW, &tm_w, bar_full, h * 64, c * kChunk, b);
        tma_load_3d(sR, &tm_r, bar_full, h * 64, c * kChunk, b);
        tma_load_3d(sK, &tm_k, bar_full, h * 64, c * kChunk, b);
        mbar_expect_tx(bar_late, 3 * kTile);
        tma_load_3d(sV, &tm_v, bar_late, h * 64, c * kChunk, b);
        tma_load_3d(sG, &tm_gy, bar_late, h * 64, c * kChunk, b);
        bulk_load(sS, a.ckpt + ((size_t)blockIdx.x * nchunks + c) * 4096, kTile, bar_late);
    };
    if (tid == 0) issue_loads(nchunks - 1);

    constexpr uint32_t idKK = umma_idesc_bf16(64, 64, false, false);
    constexpr uint32_t idKK96 = umma_idesc_bf16(64, 96, false, false);
    constexpr uint32_t idKM = umma_idesc_bf16(64, 64, false, true);
    constexpr uint32_t idMM = umma_idesc_bf16(64, 64, true, true);
    // first row of the distance-d copies inside sKD / sRD (a function, not an array: an array lands in local memory)
    auto goff = [](int d) { return d == 1 ? 0 : d == 2 ? 48 : 80; };
    // operand descriptors; a step of 16 along K is +2 (K-major operand) or +128 (MN-major operand)
    const uint64_t dR = umma_desc_sw128(smem_u32(sR)), dK = umma_desc_sw128(smem_u32(sK));
    const uint64_t dV = umma_desc_sw128(smem_u32(sV)), dW = umma_desc_sw128(smem_u32(sW));
    const uint64_t dG = umma_desc_sw128(smem_u32(sG)), dS = umma_desc_sw128(smem_u32(sS));
    const uint64_t dKH = umma_desc_sw128(smem_u32(sKH)), dKD = umma_desc_sw128(smem_u32(sKD));
    const uint64_t dRD = umma_desc_sw128(smem_u32(sRD)), dP = umma_desc_sw128(smem_u32(sP));
    const uint64_t dAM = umma_desc_sw128(smem_u32(sAM)), dAB = umma_desc_sw128(smem_u32(sAB));

    int err = 0;
    // thread 0: which of the two load barriers still has copies in flight, and the phase parity of their completion
    bool pend_full = true, pend_late = true;
    uint32_t pend_parity = 0;
    for (int it = 0; it < nchunks; ++it) {
        const int c = nchunks - 1 - it;
        WKV6_TSTAMP(it, 0);
        if (!cta_wait(bar_full, it & 1, warp)) err = 1;
        if (tid == 0) pend_full = false;
        WKV6_TSTAMP(it, 1);

        // ---- per-step log2 decays and their running sums inside the block (fragment layout)
        __nv_bfloat162 rp[8], kp[8];  // raw r, k pairs: index 2*nn + (row ta+8 ? 1 : 0)
        __nv_bfloat162 erb[8], ekb[8];  // e^{c_{t-1}-ref}, e^{ref-c_t}, rounded to bf16
        uint32_t lwst[8];               // log2-decays rounded to bf16, parked in tensor memory until gw is formed
        float cs[16], lw[16];
        const bool full_chunk = (c + 1) * kChunk <= a.T;
#pragma unroll
        for (int nn = 0; nn < 4; ++nn) {
#pragma unroll
            for (int hrow = 0; hrow < 2; ++hrow) {
                const uint32_t off = FO(nn, hrow);
                rp[2 * nn + hrow] = *reinterpret_cast<const __nv_bfloat162 *>(sR + off);
                kp[2 * nn + hrow] = *reinterpret_cast<const __nv_bfloat162 *>(sK + off);
                const float2 e2 = mul2(ld_bf2(sW + off), make_float2(kLog2e, kLog2e));
                float2 l2 = mul2(make_float2(ex2f(e2.x), ex2f(e2.y)), make_float2(-kLog2e, -kLog2e));
                l2.x = fmaxf(l2.x, kMinLogDecay2);
                l2.y = fmaxf(l2.y, kMinLogDecay2);
                if (!full_chunk && c * kChunk + ta + 8 * hrow >= a.T) l2 = make_float2(0.f, 0.f);
                lw[4 * nn + 2 * hrow] = l2.x;
                lw[4 * nn + 2 * hrow + 1] = l2.y;
                { const __nv_bfloat162 lb = to_bf2(l2); lwst[2 * nn + hrow] = *reinterpret_cast<const uint32_t *>(&lb); }
            }
        }
        tmem_st_16x256b_x2(tmStash, lwst);
#pragma unroll
        for (int nn = 0; nn < 4; ++nn)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                float pa = lw[4 * nn + e], pb = lw[4 * nn + 2 + e];
                scan_prefix16(pa, pb, r0, lane);
                cs[4 * nn + e] = pa;
                cs[4 * nn + 2 + e] = pb;
            }
        if (r0 == 7) {
#pragma unroll
            for (int nn = 0; nn < 4; ++nn) {
                const int col = 8 * (n0 + nn) + 2 * q;
                *reinterpret_cast<float2 *>(&sHead[w4 * 64 + col]) = make_float2(cs[4 * nn], cs[4 * nn + 1]);
                *reinterpret_cast<float2 *>(&sTot[w4 * 64 + col]) = make_float2(cs[4 * nn + 2], cs[4 * nn + 3]);
            }
        }
        tmem_wait_st();
        if (tid == 0) bulk_wait_read<0>();  // the previous chunk's output tiles have left shared memory
        if (!__syncthreads_and(err == 0)) { err = err ? err : 10; break; }
        WKV6_TSTAMP(it, 2);

        // ---- per (block, channel) factors, one pair per thread; the power-of-two ones are exact in bf16
        bool wide;  // one reference point for the whole chunk
        {
            const int J = tid >> 6, i = tid & 63;
            float base = 0.f, mybase = 0.f, ref[4], cmid = 0.f;
#pragma unroll
            for (int J2 = 0; J2 < 4; ++J2) {
                ref[J2] = rintf(base + sHead[J2 * 64 + i]);  // integer: block-pair factors become powers of two
                if (J2 == J) mybase = base;
                base += sTot[J2 * 64 + i];
            }
            cmid = rintf(0.5f * base);  // the single reference: half of the chunk's total log2 decay
            wide = !__syncthreads_or(base < kWideLimit2);
            float myref = ref[0];
#pragma unroll
            for (int J2 = 1; J2 < 4; ++J2) myref = (J2 == J) ? ref[J2] : myref;
            if (wide) myref = cmid;
            sOff[J * 64 + i] = myref - mybase;
            sFRb[J * 64 + i] = __float2bfloat16_rn(pow2i(myref));
            sFKb[J * 64 + i] = __float2bfloat16_rn(ex2f(base - myref));
            if (!wide) {
#pragma unroll
                for (int J2 = 1; J2 < 4; ++J2) {  // copy of block J serving row block J2 = J + d
                    const int d = J2 - J;
                    if (d >= 1) {
                        // 2^n, n = ref(J2) - ref(J) <= 0, can lie below the bf16 range while its product with an operand
                        // of up to 2^115 does not: it is applied as two factors 2^max(n,-120) * 2^max(n+120,-120)
                        const float n = ref[J2] - myref, n1 = fmaxf(n, -120.f);
                        const int slot = ((d == 1 ? 0 : d == 2 ? 3 : 5) + J) * 64 + i;
                        sMKb[slot] = __float2bfloat16_rn(pow2i(n1));
                        sMK2[slot] = __float2bfloat16_rn(pow2i(fmaxf(n - n1, -120.f)));
                    }
                }
            }
            if (J == 0) sDtot[i] = ex2f(base);
        }
        __syncthreads();
        WKV6_TSTAMP(it, 3);

        // ---- scaled operands, on packed bf16 pairs (r, k are exact bf16; the factors are rounded to bf16, the
        // block-pair and chunk-start factors are powers of two and stay exact)
        {
            float bon_a = 0.f, bon_b = 0.f;
#pragma unroll
            for (int nn = 0; nn < 4; ++nn) {
                const int col = 8 * (n0 + nn) + 2 * q;
                const float2 of = *reinterpret_cast<const float2 *>(&sOff[w4 * 64 + col]);
                const float2 uc = *reinterpret_cast<const float2 *>(&sU[col]);
                const __nv_bfloat162 fkb = *reinterpret_cast<const __nv_bfloat162 *>(&sFKb[w4 * 64 + col]);
                const __nv_bfloat162 frb = *reinterpret_cast<const __nv_bfloat162 *>(&sFRb[w4 * 64 + col]);
                __nv_bfloat162 mk[3], mr[3], mk2[3], mr2[3];  // power-of-two factors of the copies for block distances 1..3
#pragma unroll
                for (int d = 1; d <= 3; ++d) {
                    const int row0 = (d == 1 ? 0 : d == 2 ? 3 : 5);
                    mk[d - 1] = mr[d - 1] = mk2[d - 1] = mr2[d - 1] = frb;
                    if (wide) continue;
                    if (w4 + d <= 3) {
                        mk[d - 1] = *reinterpret_cast<const __nv_bfloat162 *>(&sMKb[(row0 + w4) * 64 + col]);
                        mk2[d - 1] = *reinterpret_cast<const __nv_bfloat162 *>(&sMK2[(row0 + w4) * 64 + col]);
                    }
                    if (w4 - d >= 0) {
                        mr[d - 1] = *reinterpret_cast<const __nv_bfloat162 *>(&sMKb[(row0 + w4 - d) * 64 + col]);
                        mr2[d - 1] = *reinterpret_cast<const __nv_bfloat162 *>(&sMK2[(row0 + w4 - d) * 64 + col]);
                    }
                }
#pragma unroll
                for (int hrow = 0; hrow < 2; ++hrow) {
                    const uint32_t off = FO(nn, hrow);
                    const int e0 = 4 * nn + 2 * hrow;
                    const float2 ea = make_float2(cs[e0] - lw[e0] - of.x, cs[e0 + 1] - lw[e0 + 1] - of.y);
                    const float2 eb = make_float2(of.x - cs[e0], of.y - cs[e0 + 1]);
                    const __nv_bfloat162 er = to_bf2(make_float2(ex2f(ea.x), ex2f(ea.y)));
                    const __nv_bfloat162 ek = to_bf2(make_float2(ex2f(eb.x), ex2f(eb.y)));
                    erb[2 * nn + hrow] = er;
                    ekb[2 * nn + hrow] = ek;
                    const __nv_bfloat162 rb = rp[2 * nn + hrow], kb = kp[2 * nn + hrow];
                    const float2 rk = mul2(__bfloat1622float2(rb), __bfloat1622float2(kb));
                    const float bon = fmaf(rk.x, uc.x, rk.y * uc.y);
                    if (hrow == 0) bon_a += bon; else bon_b += bon;
                    const __nv_bfloat162 rt = __hmul2(rb, er), kt = __hmul2(kb, ek);
                    *reinterpret_cast<__nv_bfloat162 *>(sR + off) = rt;
                    *reinterpret_cast<__nv_bfloat162 *>(sW + off) = __hmul2(rt, frb);
                    *reinterpret_cast<__nv_bfloat162 *>(sK + off) = kt;
                    *reinterpret_cast<__nv_bfloat162 *>(sKH + off) = __hmul2(kt, fkb);
#pragma unroll
                    for (int d = 1; d <= 3; ++d) {
                        if (wide) continue;
                        if (w4 + d <= 3)  // k~ copy serving row block w4 + d: row goff(d) + t
                            *reinterpret_cast<__nv_bfloat162 *>(sKD + goff(d) * 128 + off) = __hmul2(__hmul2(kt, mk[d - 1]), mk2[d - 1]);
                        if (w4 - d >= 0)  // r~ copy serving column block w4 - d: row goff(d) + t - 16 d
                            *reinterpret_cast<__nv_bfloat162 *>(sRD + (goff(d) - 16 * d) * 128 + off) = __hmul2(__hmul2(rt, mr[d - 1]), mr2[d - 1]);
                    }
                }
            }
            bon_a += __shfl_xor_sync(0xffffffffu, bon_a, 1); bon_a += __shfl_xor_sync(0xffffffffu, bon_a, 2);
            bon_b += __shfl_xor_sync(0xffffffffu, bon_b, 1); bon_b += __shfl_xor_sync(0xffffffffu, bon_b, 2);
            if (q == 0) { sBonus[half * 64 + ta] = bon_a; sBonus[half * 64 + ta + 8] = bon_b; }
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        {
            bool ok = true;
            if (warp == 0) ok = mbar_wait(bar_late, it & 1);  // v, gy, S_in have landed (long ago, normally)
            if (!__syncthreads_and(ok && err == 0)) { err = err ? err : 4; break; }
            if (tid == 0) pend_late = false;
        }
        WKV6_TSTAMP(it, 4);

        // ---- MMA group 1, four issuing threads (independent accumulators)
        if (lane == 0 && warp < 4) {
            tc_fence_after_sync();
            if (warp == 0) {
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)  // P = gy v^T
                    umma_ss(tmP, dG + 2 * kk, dV + 2 * kk, idKK, kk > 0);
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)  // GR2 = gy S_in^T
                    umma_ss(tmGR2, dG + 2 * kk, dS + 2 * kk, idKK, kk > 0);
            } else if (warp == 1) {
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)  // A, distance 0
                    umma_ss(tmA, dR + 2 * kk, dK + 2 * kk, idKK, kk > 0);
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)  // A, distances 1..3: r~ against the 96 rows of k~ copies
                    if (!wide) umma_ss(tmAD, dR + 2 * kk, dKD + 2 * kk, idKK96, kk > 0);
            } else if (warp == 2) {
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)  // GK2 = v Abar^T
                    umma_ss(tmGK2, dV + 2 * kk, dAB + 2 * kk, idKK, kk > 0);
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)  // gv = k^ Abar
                    umma_ss(tmGV, dKH + 2 * kk, dAB + 128 * kk, idKM, kk > 0);
            } else {
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)  // Abar increment = r^^T gy
                    umma_ss(tmAN, dW + 128 * kk, dG + 128 * kk, idMM, kk > 0);
            }
            umma_commit(bar_mma1);
        }
        WKV6_TSTAMP(it, 5);
        if (!cta_wait(bar_mma1, it & 1, warp)) err = 2;
        tc_fence_after_sync();
        WKV6_TSTAMP(it, 6);

        // ---- epilogue 1: masked P and A as bf16 operands, reverse-state update
        {
            float f[16];
            tmem_ld_16x256b_x4(tmP + lo + cb, f);
#pragma unroll
            for (int nn = 0; nn < 4; ++nn) {
                const int s0 = 8 * (n0 + nn) + 2 * q;  // columns s0, s0 + 1
#pragma unroll
                for (int hrow = 0; hrow < 2; ++hrow) {
                    const int t = ta + 8 * hrow;
                    float x0 = f[4 * nn + 2 * hrow], x1 = f[4 * nn + 2 * hrow + 1];
                    if (s0 == t) sVG[t] = x0;
                    if (s0 + 1 == t) sVG[t] = x1;
                    x0 = (s0 < t) ? x0 : 0.f;
                    x1 = (s0 + 1 < t) ? x1 : 0.f;
                    *reinterpret_cast<uint32_t *>(sP + FO(nn, hrow)) = pack_bf2(x0, x1);
                }
            }
            // A: this warp covers column blocks J = 2*half, 2*half+1 of row block I = w4; pick the copy per block pair
#pragma unroll
            for (int jj = 0; jj < 2; ++jj) {
                const int J = 2 * half + jj, I = w4;
                uint32_t o0 = 0, o1 = 0, o2 = 0, o3 = 0;
                if (J <= I) {
                    const int dl = I - J;
                    const uint32_t src = (dl == 0 || wide) ? (tmA + lo + 16 * J) : (tmAD + lo + goff(dl) + 16 * J);
                    uint32_t v8[8];
                    tmem_ld_16x256b_x2(src, v8);
                    tmem_wait_ld();
                    float g8[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) g8[e] = __uint_as_float(v8[e]);
                    if (dl == 0) {
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            const int row = r0 + ((e & 2) ? 8 : 0);
                            const int col = 8 * (e >> 2) + 2 * q + (e & 1);
                            g8[e] = (col < row) ? g8[e] : (col == row ? sBonus[16 * I + row] + sBonus[64 + 16 * I + row] : 0.f);
                        }
                    }
                    o0 = pack_bf2(g8[0], g8[1]); o2 = pack_bf2(g8[2], g8[3]);
                    o1 = pack_bf2(g8[4], g8[5]); o3 = pack_bf2(g8[6], g8[7]);
                }
                *reinterpret_cast<uint32_t *>(sAM + FO(2 * jj, 0)) = o0;
                *reinterpret_cast<uint32_t *>(sAM + FO(2 * jj + 1, 0)) = o1;
                *reinterpret_cast<uint32_t *>(sAM + FO(2 * jj, 1)) = o2;
                *reinterpret_cast<uint32_t *>(sAM + FO(2 * jj + 1, 1)) = o3;
            }
            // <S_in, Abar>_i with the reverse state at the chunk end (before its update), for gw
            float za = 0.f, zb = 0.f;
#pragma unroll
            for (int nn = 0; nn < 4; ++nn) {
                const float2 sa = ld_bf2(sS + FO(nn, 0)), sb = ld_bf2(sS + FO(nn, 1));
                za = fmaf(AB[4 * nn], sa.x, fmaf(AB[4 * nn + 1], sa.y, za));
                zb = fmaf(AB[4 * nn + 2], sb.x, fmaf(AB[4 * nn + 3], sb.y, zb));
            }
            za += __shfl_xor_sync(0xffffffffu, za, 1); za += __shfl_xor_sync(0xffffffffu, za, 2);
            zb += __shfl_xor_sync(0xffffffffu, zb, 1); zb += __shfl_xor_sync(0xffffffffu, zb, 2);
            if (q == 0) { sT1[half * 64 + ta] = za; sT1[half * 64 + ta + 8] = zb; }
            tmem_ld_16x256b_x4(tmAN + lo + cb, f);  // rows are key channels here
            const float d0 = sDtot[ta], d1 = sDtot[ta + 8];
#pragma unroll
            for (int nn = 0; nn < 4; ++nn) {
                AB[4 * nn + 0] = fmaf(AB[4 * nn + 0], d0, f[4 * nn + 0]);
                AB[4 * nn + 1] = fmaf(AB[4 * nn + 1], d0, f[4 * nn + 1]);
                AB[4 * nn + 2] = fmaf(AB[4 * nn + 2], d1, f[4 * nn + 2]);
                AB[4 * nn + 3] = fmaf(AB[4 * nn + 3], d1, f[4 * nn + 3]);
                *reinterpret_cast<uint32_t *>(sAB + FO(nn, 0)) = pack_bf2(AB[4 * nn], AB[4 * nn + 1]);
                *reinterpret_cast<uint32_t *>(sAB + FO(nn, 1)) = pack_bf2(AB[4 * nn + 2], AB[4 * nn + 3]);
            }
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        if (!__syncthreads_and(err == 0)) { err = err ? err : 11; break; }
        WKV6_TSTAMP(it, 7);

        // ---- MMA group 2, three issuing threads
        if (lane == 0 && warp < 3) {
            tc_fence_after_sync();
            if (wide && warp < 2) {
                if (warp == 0) {
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk)  // GR1 = P k~   (P is zero on and above the diagonal)
                        umma_ss(tmP, dP + 2 * kk, dK + 128 * kk, idKM, kk > 0);
                } else {
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk)  // GK1 = P^T r~
                        umma_ss(tmA, dP + 128 * kk, dR + 128 * kk, idMM, kk > 0);
                }
            } else if (warp == 0) {
#pragma unroll
                for (int I = 0; I < 4; ++I)
#pragma unroll
                    for (int J = 0; J <= I; ++J) {
                        // GR1 rows of block I += P[:, block J] k~copy(I-J)_J        (K = the 16 tokens of block J)
                        const uint64_t kb = (I == J) ? dK + 128 * J : dKD + 8 * (goff(I - J) + 16 * J);
                        umma_ss_masked(tmP, dP + 2 * J, kb, idKM, J > 0, I);
                    }
            } else if (warp == 1) {
#pragma unroll
                for (int J = 0; J < 4; ++J)
#pragma unroll
                    for (int I = J; I < 4; ++I) {
                        // GK1 rows of block J += P[block I, :]^T r~copy(I-J)_I      (K = the 16 tokens of block I)
                        const uint64_t rb2 = (I == J) ? dR + 128 * I : dRD + 8 * (goff(I - J) + 16 * J);
                        umma_ss_masked(tmA, dP + 128 * I, rb2, idMM, I > J, J);
                    }
            } else {
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)  // gv += A^T gy
                    umma_ss(tmGV, dAM + 128 * kk, dG + 128 * kk, idMM, true);
            }
            umma_commit(bar_mma2);
        }
        WKV6_TSTAMP(it, 8);
        if (!cta_wait(bar_mma2, it & 1, warp)) err = 3;
        tc_fence_after_sync();
        WKV6_TSTAMP(it, 9);
        // every input tile is dead once the second MMA group has completed: fetch the next chunk now
        if (tid == 0 && c > 0 && err == 0) {
            issue_loads(c - 1);
            pend_full = pend_late = true;
            pend_parity = (uint32_t)(it + 1) & 1u;
        }

        // ---- epilogue 2: gr, gk, gv, gw, one 8-column repetition at a time
        float loc[16];  // G minus its per-channel base (see below)
        {
            const float vga = sVG[ta], vgb = sVG[ta + 8];
#pragma unroll
            for (int nn = 0; nn < 4; ++nn) {
                const int col = 8 * (n0 + nn) + 2 * q;
                float g1[4], g2[4], h1[4], h2[4];
                tmem_ld_16x256b_x1(tmP + lo + cb + 8 * nn, g1);    // GR1
                tmem_ld_16x256b_x1(tmGR2 + lo + cb + 8 * nn, g2);  // GR2
                tmem_ld_16x256b_x1(tmA + lo + cb + 8 * nn, h1);    // GK1
                tmem_ld_16x256b_x1(tmGK2 + lo + cb + 8 * nn, h2);  // GK2
                tmem_wait_ld();
                const float2 fr = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&sFRb[w4 * 64 + col]));
                const float2 fk = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&sFKb[w4 * 64 + col]));
                const float2 uc = *reinterpret_cast<const float2 *>(&sU[col]);
                float qv[4], bsum0 = 0.f, bsum1 = 0.f;
#pragma unroll
                for (int hrow = 0; hrow < 2; ++hrow) {
                    const float vg = hrow ? vgb : vga;
                    const float2 r2 = __bfloat1622float2(rp[2 * nn + hrow]), k2 = __bfloat1622float2(kp[2 * nn + hrow]);
                    const float2 er = __bfloat1622float2(erb[2 * nn + hrow]), ek = __bfloat1622float2(ekb[2 * nn + hrow]);
                    // the bf16 operand values r~, k~ exactly as the MMAs saw them
                    const float2 rt = __bfloat1622float2(__hmul2(rp[2 * nn + hrow], erb[2 * nn + hrow]));
                    const float2 kt = __bfloat1622float2(__hmul2(kp[2 * nn + hrow], ekb[2 * nn + hrow]));
                    const float2 G1 = make_float2(g1[2 * hrow], g1[2 * hrow + 1]), G2 = make_float2(g2[2 * hrow], g2[2 * hrow + 1]);
                    const float2 H1 = make_float2(h1[2 * hrow], h1[2 * hrow + 1]), H2 = make_float2(h2[2 * hrow], h2[2 * hrow + 1]);
                    const float2 uvg = make_float2(uc.x * vg, uc.y * vg);
                    // gr = Er (GR1 + fR GR2) + u k vg ;  gk = Ek (GK1 + fK GK2) + u r vg
                    const float2 gr = fma2(er, fma2(fr, G2, G1), mul2(uvg, k2));
                    const float2 gk = fma2(ek, fma2(fk, H2, H1), mul2(uvg, r2));
                    *reinterpret_cast<__nv_bfloat162 *>(sP + FO(nn, hrow)) = to_bf2(gr);
                    *reinterpret_cast<__nv_bfloat162 *>(sAM + FO(nn, hrow)) = to_bf2(gk);
                    // gw pieces: a = r~ GR1 + r^ GR2, z = k~ GK1, b = k^ GK2
                    const float2 av = fma2(rt, G1, mul2(mul2(rt, fr), G2));
                    const float2 zv = mul2(kt, H1);
                    const float2 bv = mul2(mul2(kt, fk), H2);
                    const float2 zbv = add2(zv, bv);
                    qv[2 * hrow] = av.x - zbv.x;
                    qv[2 * hrow + 1] = av.y - zbv.y;
                    loc[4 * nn + 2 * hrow] = -av.x;      // becomes  suffix_incl(q) - q - (z + b) = suffix_incl(q) - a
                    loc[4 * nn + 2 * hrow + 1] = -av.y;
                    bsum0 += bv.x; bsum1 += bv.y;
                    const float2 rkv = mul2(mul2(r2, k2), make_float2(vg, vg));
                    gu_acc[2 * nn] += rkv.x;
                    gu_acc[2 * nn + 1] += rkv.y;
                }
                // sums over later tokens of the block by lane scans; block totals go through shared memory
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    float pa = qv[e], pb = qv[2 + e];
                    scan_suffix16(pa, pb, r0, lane);
                    loc[4 * nn + e] += pa;
                    loc[4 * nn + 2 + e] += pb;
                    if (r0 == 0) sXtot[w4 * 64 + col + e] = pa;
                }
                bsum0 += __shfl_xor_sync(0xffffffffu, bsum0, 4); bsum1 += __shfl_xor_sync(0xffffffffu, bsum1, 4);
                bsum0 += __shfl_xor_sync(0xffffffffu, bsum0, 8); bsum1 += __shfl_xor_sync(0xffffffffu, bsum1, 8);
                bsum0 += __shfl_xor_sync(0xffffffffu, bsum0, 16); bsum1 += __shfl_xor_sync(0xffffffffu, bsum1, 16);
                if (r0 == 0) *reinterpret_cast<float2 *>(&sBtot[w4 * 64 + col]) = make_float2(bsum0, bsum1);
            }
            float gv16[16];
            tmem_ld_16x256b_x4(tmGV + lo + cb, gv16);
#pragma unroll
            for (int nn = 0; nn < 4; ++nn) {
                *reinterpret_cast<uint32_t *>(sKD + FO(nn, 0)) = pack_bf2(gv16[4 * nn], gv16[4 * nn + 1]);
                *reinterpret_cast<uint32_t *>(sKD + FO(nn, 1)) = pack_bf2(gv16[4 * nn + 2], gv16[4 * nn + 3]);
            }
        }
        tc_fence_before_sync();
        __syncthreads();
        WKV6_TSTAMP(it, 10);
        // G_t = e^{c_63} <S_in, Abar> + sum_all b + sum_{later blocks} q + (suffix_incl(q) - a)_t ;  gw = -exp(w) G
        uint32_t lwst2[8];
        tmem_ld_16x256b_x2(tmStash, lwst2);
        tmem_wait_ld();
#pragma unroll
        for (int nn = 0; nn < 4; ++nn) {
            const int col = 8 * (n0 + nn) + 2 * q;
            const float2 t1 = add2(*reinterpret_cast<const float2 *>(&sT1[col]), *reinterpret_cast<const float2 *>(&sT1[64 + col]));
            const float2 dt = *reinterpret_cast<const float2 *>(&sDtot[col]);
            float2 base = mul2(t1, dt);
#pragma unroll
            for (int J2 = 0; J2 < 4; ++J2) {
                base = add2(base, *reinterpret_cast<const float2 *>(&sBtot[J2 * 64 + col]));
                if (J2 > w4) base = add2(base, *reinterpret_cast<const float2 *>(&sXtot[J2 * 64 + col]));
            }
#pragma unroll
            for (int hrow = 0; hrow < 2; ++hrow) {
                const int e0 = 4 * nn + 2 * hrow;
                const float2 lwf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&lwst2[2 * nn + hrow]));
                float2 gw = mul2(mul2(lwf, make_float2(1.0f / kLog2e, 1.0f / kLog2e)),
                                 make_float2(base.x + loc[e0], base.y + loc[e0 + 1]));  // -exp(w) = log-decay
                if (a.zero_init && c == 0 && ta + 8 * hrow == 0) gw = make_float2(0.f, 0.f);  // no dependence on w_0
                *reinterpret_cast<__nv_bfloat162 *>(sRD + FO(nn, hrow)) = to_bf2(gw);
            }
        }
        fence_proxy_async_smem();
        if (!__syncthreads_and(err == 0)) { err = err ? err : 12; break; }
        WKV6_TSTAMP(it, 11);
        if (tid == 0) {
            tma_store_3d(&tm_gr, sP, h * 64, c * kChunk, b);
            tma_store_3d(&tm_gk, sAM, h * 64, c * kChunk, b);
            tma_store_3d(&tm_gv, sKD, h * 64, c * kChunk, b);
            tma_store_3d(&tm_gw, sRD, h * 64, c * kChunk, b);
            bulk_commit();
        }
    }

    // ---- unwind
    if (tid == 0) {
        if (err != 0) {
            // copies still aimed at this CTA's shared memory: wait for them (bounded) before leaving
            if (pend_full) mbar_wait(bar_full, pend_parity);
            if (pend_late) mbar_wait(bar_late, pend_parity);
            atomicExch(&g_chunk_status, 100 + err);
        }
        bulk_wait<0>();
    }
    // gu[b][h][i]: sum this thread's channels over the 8 lanes sharing q, then over the four row blocks
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        float s2 = gu_acc[e];
        s2 += __shfl_xor_sync(0xffffffffu, s2, 4);
        s2 += __shfl_xor_sync(0xffffffffu, s2, 8);
        s2 += __shfl_xor_sync(0xffffffffu, s2, 16);
        gu_acc[e] = s2;
    }
    __syncthreads();
    if (r0 == 0) {
#pragma unroll
        for (int nn = 0; nn < 4; ++nn) {
            sGU[w4 * 64 + 8 * (n0 + nn) + 2 * q] = gu_acc[2 * nn];
            sGU[w4 * 64 + 8 * (n0 + nn) + 2 * q + 1] = gu_acc[2 * nn + 1];
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (tid < 64 && err == 0)
        store_any(a.gu, a.gu_dtype, (size_t)blockIdx.x * 64 + tid, sGU[tid] + sGU[64 + tid] + sGU[128 + tid] + sGU[192 + tid]);
    if (warp == 0) tmem_dealloc(tbase, 256);
}

}  // namespace wkv6
