// Chunked WKV6 backward, fast kernel: every chunk uses one reference (half of the chunk's total log2 decay) for the
// decay exponents, which is valid while the total log2 decay of a chunk stays above kWideLimit2 in every channel
// (see wkv6_chunk_fwd.cuh).  The mathematics and the thread <-> element mapping are those of chunk_bwd_kernel
// (wkv6_chunk_bwd.cuh); what differs is where per-element state lives between the phases of a chunk, because with
// two CTAs per SM a thread has 128 registers and next to no L1 behind them, so anything the compiler spills is
// served by L2:
//   * raw r, k stay in their input tiles (the scaled operands r~, k~ go to tiles of their own), and the factor
//     e^{c_{t-1}-ref} is parked in a shared-memory tile, so the second epilogue reloads them (and recomputes r~, k~
//     as the same bf16 products) instead of keeping them in registers across both MMA groups;
//   * the fp32 reverse state Abar and the running sum of gu are parked in tensor-memory columns that the per-block
//     reference points of the general kernel would need for the A copies.
// A sequence that contains a chunk beyond the limit is abandoned at that chunk: the kernel sets flag[b*H+h] = 1 and
// chunk_bwd_kernel, launched right after with the same flags, redoes exactly the flagged sequences.
//
// Tensor-memory map (256 columns): lanes 0-15: [0,64) P -> GR1 | [64,128) A -> GK1 | [128,192) GR2 | [192,256) GK2
//                                  lanes 16-31: [0,64) Abar increment | [64,128) gv | [128,192) Abar (fp32, parked)
//                                               | [192,224) gu partial sums (parked) | [224,256) bf16 log-decays
#pragma once

#include "wkv6_chunk_bwd.cuh"

namespace wkv6 {

struct WideBwdSmem {
    static constexpr int oR = 0;                    // r (raw, kept until the second epilogue has read it)
    static constexpr int oK = oR + kTile;           // k (raw)
    static constexpr int oV = oK + kTile;
    static constexpr int oW = oV + kTile;           // w  -> r^ = r~ 2^{ref} (in place)
    static constexpr int oG = oW + kTile;           // gy
    static constexpr int oS = oG + kTile;           // checkpointed state at the chunk start [i][j]
    static constexpr int oKH = oS + kTile;          // k^ = k~ 2^{c_63 - ref}
    static constexpr int oRT = oKH + kTile;         // r~ ; later the gw tile
    static constexpr int oKT = oRT + kTile;         // k~ ; later the gv tile
    static constexpr int oET = oKT + kTile;         // bf16 pairs of e^{c_{t-1} - ref}, at the element's tile position
    static constexpr int oP = oET + kTile;          // masked P (bf16); later the gr tile
    static constexpr int oAM = oP + kTile;          // masked A (bf16); later the gk tile
    static constexpr int oAB = oAM + kTile;         // bf16 copy of Abar [i][j]
    static constexpr int oHead = oAB + kTile;       // float [4][64] scratch of the gw phase and of the final gu reduction (below)
    static constexpr int oTot = oHead + 1024;       // float [4][64] log2-decay sum of the block
    static constexpr int oOff = oTot + 1024;        // float [4][64] reference point relative to the block start
    static constexpr int oFRb = oOff + 1024;        // bf16  [64] 2^{ref}   (ref relative to the chunk start, an integer)
    static constexpr int oFKb = oFRb + 128;         // bf16  [64] 2^{c_63 - ref}
    static constexpr int oU = oFKb + 128;           // float [64] u of this head
    static constexpr int oDtot = oU + 256;          // float [64] 2^{c_63}
    static constexpr int oBonus = oDtot + 256;      // float [2][64]
    static constexpr int oVG = oBonus + 512;        // float [64]
    static constexpr int oT1 = oVG + 256;           // float [2][64] <S_in, Abar>_i, one partial per column half
    static constexpr int oXtot = oTot;              // float [4][64] block sums for gw (sTot is dead by then)
    static constexpr int oBtot = oHead;             // float [4][64] block sums of b for gw
    static constexpr int oGU = oHead;               // float [4][64] final reduction of gu (after the last chunk)
    static constexpr int oBar = oT1 + 512;          // w, rk, late, mma1, mma2
    static constexpr int oSlot = oBar + 48;
    static constexpr int kBytes = oSlot + 16;
    static constexpr int kAlloc = kBytes;
};
static_assert(WideBwdSmem::kAlloc <= 115712, "two CTAs per SM");

__device__ __forceinline__ void tmem_st_16x256b_x4(uint32_t taddr, const float (&f)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.16x256b.x4.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "f"(f[0]), "f"(f[1]), "f"(f[2]), "f"(f[3]), "f"(f[4]), "f"(f[5]), "f"(f[6]), "f"(f[7]), "f"(f[8]),
          "f"(f[9]), "f"(f[10]), "f"(f[11]), "f"(f[12]), "f"(f[13]), "f"(f[14]), "f"(f[15])
        : "memory");
}
__device__ __forceinline__ void tmem_st_16x256b_x2(uint32_t taddr, const float (&f)[8]) {
    asm volatile("tcgen05.st.sync.aligned.16x256b.x2.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                 ::"r"(taddr), "f"(f[0]), "f"(f[1]), "f"(f[2]), "f"(f[3]), "f"(f[4]), "f"(f[5]), "f"(f[6]), "f"(f[7])
                 : "memory");
}
__device__ __forceinline__ void tmem_ld_16x256b_x2(uint32_t taddr, float (&f)[8]) {
    uint32_t v[8];
    ptx::tmem_ld_16x256b_x2(taddr, v);
    ptx::tmem_wait_ld();
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(v[e]);
}

// PERM: the tensor maps split the token axis as (j, p, I) with token = 16 I + 2 j + p and tile row = 16 I + 8 p + j, so
// that the two rows of a thread's fragment (r0 and r0 + 8 of block I) hold the ADJACENT tokens 2 r0 and 2 r0 + 1.  Every
// product of the kernel sums over tokens or is indexed by them row for row, so the order only shows in the causal masks
// and in the scans along the tokens, which then need three shuffles instead of seven.  Needs T % 16 == 0.
template <bool PERM>
__global__ void __launch_bounds__(256, 2) chunk_bwd_wide_kernel(const __grid_constant__ CUtensorMap tm_r,
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
    using SM = WideBwdSmem;
    extern __shared__ __align__(1024) uint8_t wkv6_chunk_smem[];
    uint8_t *const smem = wkv6_chunk_smem;
    // The general kernel behind this one is launched with programmatic serialization: it may be scheduled from now on
    // (its CTAs wait for this grid's completion before they read the flags).
    launch_dependents();
    if ((smem_u32(smem) & 1023u) != 0) {
        if (threadIdx.x == 0) { atomicExch(&g_chunk_status, 50); a.flags[blockIdx.x] = 0; }
        return;
    }
    uint8_t *sR = smem + SM::oR, *sK = smem + SM::oK, *sV = smem + SM::oV, *sW = smem + SM::oW, *sG = smem + SM::oG;
    uint8_t *sS = smem + SM::oS, *sKH = smem + SM::oKH, *sRT = smem + SM::oRT, *sKT = smem + SM::oKT;
    uint8_t *sET = smem + SM::oET, *sP = smem + SM::oP, *sAM = smem + SM::oAM, *sAB = smem + SM::oAB;
    float *sTot = reinterpret_cast<float *>(smem + SM::oTot);
    float *sOff = reinterpret_cast<float *>(smem + SM::oOff), *sDtot = reinterpret_cast<float *>(smem + SM::oDtot);
    __nv_bfloat16 *sFRb = reinterpret_cast<__nv_bfloat16 *>(smem + SM::oFRb);
    __nv_bfloat16 *sFKb = reinterpret_cast<__nv_bfloat16 *>(smem + SM::oFKb);
    float *sU = reinterpret_cast<float *>(smem + SM::oU);
    float *sBonus = reinterpret_cast<float *>(smem + SM::oBonus), *sVG = reinterpret_cast<float *>(smem + SM::oVG);
    float *sXtot = reinterpret_cast<float *>(smem + SM::oXtot), *sBtot = reinterpret_cast<float *>(smem + SM::oBtot);
    float *sT1 = reinterpret_cast<float *>(smem + SM::oT1);
    float *sGU = reinterpret_cast<float *>(smem + SM::oGU);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + SM::oBar);
    // bar_w: the w tile (needed first); bar_rk: r and k (needed by the operand pass; their tiles stay live until the
    // second epilogue, so they are fetched last); bar_late: v, gy and the checkpointed state (first MMA group)
    uint64_t *bar_w = bars, *bar_rk = bars + 1, *bar_late = bars + 2, *bar_mma1 = bars + 3, *bar_mma2 = bars + 4;
    uint32_t *slot = reinterpret_cast<uint32_t *>(smem + SM::oSlot);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int w4 = warp & 3, half = warp >> 2, n0 = 4 * half;
    const int r0 = lane >> 2, q = lane & 3;
    const int ta = 16 * w4 + r0;  // this thread's rows: ta and ta + 8
    const int b = blockIdx.x / a.H, h = blockIdx.x % a.H;
    const int nchunks = (a.T + kChunk - 1) / kChunk;
    WKV6_CSTAMP(0);

    if (tid == 0) {
        mbar_init(bar_w, 1);
        mbar_init(bar_rk, 1);
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
    if (tid < 64) sU[tid] = load_any(a.u, a.u_dtype, (size_t)h * 64 + tid);
    // byte offsets of this thread's fragment elements in a swizzled tile: row ta, column pair 8(n0+nn)+2q; row ta+8 is
    // 1024 bytes further (same swizzle phase)
    uint32_t fo4[4];
#pragma unroll
    for (int nn = 0; nn < 4; ++nn) fo4[nn] = sw128_off(ta, 8 * (n0 + nn) + 2 * q);

    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    WKV6_CSTAMP(1);
    const uint32_t tbase = *slot;
    const uint32_t lo = (uint32_t)(32 * w4) << 16;  // this warp's TMEM lane quarter
    const uint32_t tmP = tbase, tmA = tbase + 64, tmGR2 = tbase + 128, tmGK2 = tbase + 192;
    const uint32_t tmAN = tbase + (16u << 16), tmGV = tbase + (16u << 16) + 64;
    const uint32_t cb = 8 * n0;  // first accumulator column of this thread's fragment
    const uint32_t tmABp = tbase + (16u << 16) + 128 + lo + cb;              // this thread's 16 words of Abar
    const uint32_t tmGUp = tbase + (16u << 16) + lo + 192 + 16 * half;       // 8 words of gu partial sums
    const uint32_t tmStash = tbase + (16u << 16) + lo + 224 + 16 * half;     // 8 words of bf16 log-decays

    // the barriers are initialised: the last chunk's tiles are requested before the reverse state is read
    // copy thread: loads in flight per barrier and the phase parity their completion will have
    bool pend_w = false, pend_rk = false, pend_late = false;
    uint32_t par_early = 0, par_rk = 0;
    auto ld_tile = [&](void *dst, const CUtensorMap *m, uint64_t *bar, int c) {
        if (PERM) tma_load_5d(dst, m, bar, h * 64, 0, 0, 4 * c, b);
        else tma_load_3d(dst, m, bar, h * 64, c * kChunk, b);
    };
    auto st_tile = [&](const CUtensorMap *m, const void *src, int c) {
        if (PERM) tma_store_5d(m, src, h * 64, 0, 0, 4 * c, b);
        else tma_store_3d(m, src, h * 64, c * kChunk, b);
    };
    auto issue_early = [&](int c) {  // tiles that are dead once the second MMA group has completed
        par_early = (uint32_t)(nchunks - 1 - c) & 1u;
        mbar_expect_tx(bar_w, kTile);
        ld_tile(sW, &tm_w, bar_w, c);
        mbar_expect_tx(bar_late, 3 * kTile);
        ld_tile(sV, &tm_v, bar_late, c);
        ld_tile(sG, &tm_gy, bar_late, c);
        bulk_load(sS, a.ckpt + ((size_t)blockIdx.x * nchunks + c) * 4096, kTile, bar_late);
        pend_w = pend_late = true;
    };
    auto issue_rk = [&](int c) {  // tiles the second epilogue still reads
        par_rk = (uint32_t)(nchunks - 1 - c) & 1u;
        mbar_expect_tx(bar_rk, 2 * kTile);
        ld_tile(sR, &tm_r, bar_rk, c);
        ld_tile(sK, &tm_k, bar_rk, c);
        pend_rk = true;
    };
    // Copies are issued by one thread of warp 4, so that warps 0-3, whose first lanes issue the MMAs, never
    // queue behind them.
    const bool copy_thread = (tid == 128);
    if (copy_thread) { issue_early(nchunks - 1); issue_rk(nchunks - 1); }

    // the reverse state entering at the end of the sequence: fp32 copy in tensor memory, bf16 operand copy in shared memory
    {
        float AB[16];
#pragma unroll
        for (int nn = 0; nn < 4; ++nn) {
            const int j0 = 8 * (n0 + nn) + 2 * q;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int i = ta + (e >= 2 ? 8 : 0);
                AB[4 * nn + e] = a.ab_in ? a.ab_in[(size_t)blockIdx.x * 4096 + (size_t)i * 64 + j0 + (e & 1)] : 0.f;
            }
            *reinterpret_cast<uint32_t *>(sAB + FO(nn, 0)) = pack_bf2(AB[4 * nn], AB[4 * nn + 1]);
            *reinterpret_cast<uint32_t *>(sAB + FO(nn, 1)) = pack_bf2(AB[4 * nn + 2], AB[4 * nn + 3]);
        }
        tmem_st_16x256b_x4(tmABp, AB);
        float z8[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) z8[e] = 0.f;
        tmem_st_16x256b_x2(tmGUp, z8);
        tmem_wait_st();
    }
    WKV6_CSTAMP(2);
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    WKV6_CSTAMP(3);


    constexpr uint32_t idKK = umma_idesc_bf16(64, 64, false, false);
    constexpr uint32_t idKM = umma_idesc_bf16(64, 64, false, true);
    constexpr uint32_t idMM = umma_idesc_bf16(64, 64, true, true);
    // operand descriptors; a step of 16 along K is +2 (K-major operand) or +128 (MN-major operand)
    const uint64_t dV = umma_desc_sw128(smem_u32(sV)), dW = umma_desc_sw128(smem_u32(sW));
    const uint64_t dG = umma_desc_sw128(smem_u32(sG)), dS = umma_desc_sw128(smem_u32(sS));
    const uint64_t dKH = umma_desc_sw128(smem_u32(sKH)), dRT = umma_desc_sw128(smem_u32(sRT));
    const uint64_t dKT = umma_desc_sw128(smem_u32(sKT)), dP = umma_desc_sw128(smem_u32(sP));
    const uint64_t dAM = umma_desc_sw128(smem_u32(sAM)), dAB = umma_desc_sw128(smem_u32(sAB));

    int err = 0;
    bool bail = false;  // a chunk beyond the single-reference limit: leave this sequence to the general kernel
    for (int it = 0; it < nchunks; ++it) {
        const int c = nchunks - 1 - it;
        WKV6_TSTAMP(it, 0);
        if (!cta_wait(bar_w, it & 1, warp)) err = 1;
        if (copy_thread) pend_w = false;
        WKV6_TSTAMP(it, 1);
        if (it == 0) WKV6_CSTAMP(4);

        // ---- per-step log2 decays and their running sums inside the block (fragment layout)
        __nv_bfloat162 ekb[8];  // e^{ref-c_t} rounded to bf16: index 2*nn + (row ta+8 ? 1 : 0)
        float cs[16], lw[16];
        {
            uint32_t lwst[8];  // log2-decays rounded to bf16, parked in tensor memory until gw is formed
            const bool full_chunk = (c + 1) * kChunk <= a.T;
#pragma unroll
            for (int nn = 0; nn < 4; ++nn) {
#pragma unroll
                for (int hrow = 0; hrow < 2; ++hrow) {
                    const float2 e2 = mul2(ld_bf2(sW + FO(nn, hrow)), make_float2(kLog2e, kLog2e));
                    float2 l2 = mul2(make_float2(ex2f(e2.x), ex2f(e2.y)), make_float2(-kLog2e, -kLog2e));
                    l2.x = fmaxf(l2.x, kMinLogDecay2);
                    l2.y = fmaxf(l2.y, kMinLogDecay2);
                    if (!full_chunk && c * kChunk + (PERM ? 16 * w4 + 2 * r0 + hrow : ta + 8 * hrow) >= a.T) l2 = make_float2(0.f, 0.f);
                    lw[4 * nn + 2 * hrow] = l2.x;
                    lw[4 * nn + 2 * hrow + 1] = l2.y;
                    { const __nv_bfloat162 lb = to_bf2(l2); lwst[2 * nn + hrow] = *reinterpret_cast<const uint32_t *>(&lb); }
                }
            }
            tmem_st_16x256b_x2(tmStash, lwst);
        }
#pragma unroll
        for (int nn = 0; nn < 4; ++nn)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                float pa = lw[4 * nn + e], pb = lw[4 * nn + 2 + e];
                if (PERM) scan_prefix16_adj(pa, pb, r0); else scan_prefix16(pa, pb, r0, lane);
                cs[4 * nn + e] = pa;
                cs[4 * nn + 2 + e] = pb;
            }
        if (r0 == 7) {
#pragma unroll
            for (int nn = 0; nn < 4; ++nn) {
                const int col = 8 * (n0 + nn) + 2 * q;
                *reinterpret_cast<float2 *>(&sTot[w4 * 64 + col]) = make_float2(cs[4 * nn + 2], cs[4 * nn + 3]);
            }
        }
        tmem_wait_st();
        if (copy_thread) bulk_wait_read<0>();  // the previous chunk's output tiles have left shared memory
        if (!__syncthreads_and(err == 0)) { err = err ? err : 10; break; }
        WKV6_TSTAMP(it, 2);

        // ---- per channel: the reference (an integer in the log2 domain, half of the chunk's total decay) and the
        // factors that depend on it; one (block, channel) pair per thread
        {
            const int J = tid >> 6, i = tid & 63;
            float base = 0.f, mybase = 0.f, ref = 0.f;
#pragma unroll
            for (int J2 = 0; J2 < 4; ++J2) {
                if (J2 == J) mybase = base;
                base += sTot[J2 * 64 + i];
            }
            // The factors are written whether or not the chunk fits the single reference point; the test itself rides on
            // the barrier that publishes them (one CTA barrier fewer per chunk), with a second barrier only when it trips.
            ref = rintf(0.5f * base);  // half of the chunk's total log2 decay: both operands' largest factors are 2^{-base/2}
            const bool over = base < kWideLimit2;
            sOff[J * 64 + i] = ref - mybase;
            if (J == 0) {
                sFRb[i] = __float2bfloat16_rn(pow2i(ref));
                sFKb[i] = __float2bfloat16_rn(ex2f(base - ref));
                sDtot[i] = ex2f(base);
            }
            bool ok = true;
            if (warp == 0) ok = mbar_wait(bar_rk, it & 1);  // r, k have landed (long ago, normally)
            const bool bad = !ok || err != 0;
            if (__syncthreads_or(over || bad)) {
                if (__syncthreads_or(bad)) { err = err ? err : 5; break; }
                bail = true;  // r, k of this chunk have landed and are not read: the unwind's wait returns at once
                break;
            }
            if (copy_thread) pend_rk = false;
        }
        WKV6_TSTAMP(it, 3);

        // ---- scaled operands, on packed bf16 pairs (r, k are exact bf16; the factors are rounded to bf16, 2^{ref}
        // is a power of two and stays exact)
        {
            float bon_a = 0.f, bon_b = 0.f;
#pragma unroll
            for (int nn = 0; nn < 4; ++nn) {
                const int col = 8 * (n0 + nn) + 2 * q;
                const float2 of = *reinterpret_cast<const float2 *>(&sOff[w4 * 64 + col]);
                const float2 uc = *reinterpret_cast<const float2 *>(&sU[col]);
                const __nv_bfloat162 fkb = *reinterpret_cast<const __nv_bfloat162 *>(&sFKb[col]);
                const __nv_bfloat162 frb = *reinterpret_cast<const __nv_bfloat162 *>(&sFRb[col]);
#pragma unroll
                for (int hrow = 0; hrow < 2; ++hrow) {
                    const uint32_t off = FO(nn, hrow);
                    const int e0 = 4 * nn + 2 * hrow;
                    const __nv_bfloat162 rb = *reinterpret_cast<const __nv_bfloat162 *>(sR + off);
                    const __nv_bfloat162 kb = *reinterpret_cast<const __nv_bfloat162 *>(sK + off);
                    const float2 ea = make_float2(cs[e0] - lw[e0] - of.x, cs[e0 + 1] - lw[e0 + 1] - of.y);
                    const float2 eb = make_float2(of.x - cs[e0], of.y - cs[e0 + 1]);
                    const __nv_bfloat162 er = to_bf2(make_float2(ex2f(ea.x), ex2f(ea.y)));
                    const __nv_bfloat162 ek = to_bf2(make_float2(ex2f(eb.x), ex2f(eb.y)));
                    ekb[2 * nn + hrow] = ek;
                    const float2 rk = mul2(__bfloat1622float2(rb), __bfloat1622float2(kb));
                    const float bon = fmaf(rk.x, uc.x, rk.y * uc.y);
                    if (hrow == 0) bon_a += bon; else bon_b += bon;
                    const __nv_bfloat162 rt = __hmul2(rb, er), kt = __hmul2(kb, ek);
                    *reinterpret_cast<__nv_bfloat162 *>(sET + off) = er;
                    *reinterpret_cast<__nv_bfloat162 *>(sRT + off) = rt;
                    *reinterpret_cast<__nv_bfloat162 *>(sW + off) = __hmul2(rt, frb);
                    *reinterpret_cast<__nv_bfloat162 *>(sKT + off) = kt;
                    *reinterpret_cast<__nv_bfloat162 *>(sKH + off) = __hmul2(kt, fkb);
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
            if (copy_thread) pend_late = false;
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
                for (int kk = 0; kk < 4; ++kk)  // A = r~ k~^T (every block pair: one reference point)
                    umma_ss(tmA, dRT + 2 * kk, dKT + 2 * kk, idKK, kk > 0);
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
            // P is kept strictly below the diagonal; its diagonal vg_t = gy_t . v_t goes aside.  Column block J against this
            // warp's row block I = w4 decides per eight columns; only inside the diagonal block do single elements differ
            // (rows r0 / r0 + 8 against columns 2q, 2q + 1 of the first / second eight columns).
#pragma unroll
            for (int nn = 0; nn < 4; ++nn) {
                const int J = 2 * half + (nn >> 1);
                float x00 = f[4 * nn], x01 = f[4 * nn + 1], x10 = f[4 * nn + 2], x11 = f[4 * nn + 3];  // row ta: x0*, row ta+8: x1*
                if (J > w4) {
                    x00 = x01 = x10 = x11 = 0.f;
                } else if (J == w4) {
                    const int c0 = 2 * q, c1 = 2 * q + 1;
                    if ((nn & 1) == 0) {          // columns 0..7 of the block: row r0 + 8 lies below, row r0 needs the test
                        if (c0 == r0) sVG[ta] = x00;
                        if (c1 == r0) sVG[ta] = x01;
                        x00 = (c0 < r0) ? x00 : 0.f;
                        x01 = (c1 < r0) ? x01 : 0.f;
                        if (PERM) {               // columns are tokens 2 c, rows tokens 2 r0 and 2 r0 + 1
                            x10 = (c0 <= r0) ? x10 : 0.f;
                            x11 = (c1 <= r0) ? x11 : 0.f;
                        }
                    } else {                      // columns 8..15: row r0 lies above, row r0 + 8 needs the test
                        if (c0 == r0) sVG[ta + 8] = x10;
                        if (c1 == r0) sVG[ta + 8] = x11;
                        x10 = (c0 < r0) ? x10 : 0.f;
                        x11 = (c1 < r0) ? x11 : 0.f;
                        if (PERM) {               // columns are tokens 2 c + 1
                            x00 = (c0 < r0) ? x00 : 0.f;
                            x01 = (c1 < r0) ? x01 : 0.f;
                        } else {
                            x00 = x01 = 0.f;
                        }
                    }
                }
                *reinterpret_cast<uint32_t *>(sP + FO(nn, 0)) = pack_bf2(x00, x01);
                *reinterpret_cast<uint32_t *>(sP + FO(nn, 1)) = pack_bf2(x10, x11);
            }
            // A: this warp covers column blocks J = 2*half, 2*half+1 of row block I = w4
#pragma unroll
            for (int jj = 0; jj < 2; ++jj) {
                const int J = 2 * half + jj, I = w4;
                uint32_t o0 = 0, o1 = 0, o2 = 0, o3 = 0;
                if (J <= I) {
                    uint32_t v8[8];
                    tmem_ld_16x256b_x2(tmA + lo + 16 * J, v8);
                    tmem_wait_ld();
                    float g8[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) g8[e] = __uint_as_float(v8[e]);
                    if (J == I) {  // diagonal block: e = 2, 3 lie below the diagonal, e = 4, 5 above it, the others need the test
                        const float bonus_a = sBonus[ta] + sBonus[64 + ta], bonus_b = sBonus[ta + 8] + sBonus[72 + ta];
                        const int c0 = 2 * q, c1 = 2 * q + 1;
                        g8[0] = (c0 < r0) ? g8[0] : (c0 == r0 ? bonus_a : 0.f);
                        g8[1] = (c1 < r0) ? g8[1] : (c1 == r0 ? bonus_a : 0.f);
                        g8[6] = (c0 < r0) ? g8[6] : (c0 == r0 ? bonus_b : 0.f);
                        g8[7] = (c1 < r0) ? g8[7] : (c1 == r0 ? bonus_b : 0.f);
                        if (PERM) {
                            g8[2] = (c0 <= r0) ? g8[2] : 0.f;
                            g8[3] = (c1 <= r0) ? g8[3] : 0.f;
                            g8[4] = (c0 < r0) ? g8[4] : 0.f;
                            g8[5] = (c1 < r0) ? g8[5] : 0.f;
                        } else {
                            g8[4] = g8[5] = 0.f;
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
            float AB[16];
            tmem_ld_16x256b_x4(tmABp, AB);
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
            tmem_st_16x256b_x4(tmABp, AB);
            tmem_wait_st();
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        if (!__syncthreads_and(err == 0)) { err = err ? err : 11; break; }
        WKV6_TSTAMP(it, 7);

        // ---- MMA group 2, three issuing threads
        if (lane == 0 && warp < 3) {
            tc_fence_after_sync();
            if (warp == 0) {
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)  // GR1 = P k~   (P is zero on and above the diagonal)
                    umma_ss(tmP, dP + 2 * kk, dKT + 128 * kk, idKM, kk > 0);
            } else if (warp == 1) {
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)  // GK1 = P^T r~
                    umma_ss(tmA, dP + 128 * kk, dRT + 128 * kk, idMM, kk > 0);
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
        // w, v, gy and the state tile are dead once the second MMA group has completed: fetch the next chunk's now
        if (copy_thread && c > 0 && err == 0) issue_early(c - 1);

        // ---- epilogue 2: gr, gk, gv, gw, one 8-column repetition at a time
        float loc[16];  // G minus its per-channel base (see below)
        {
            const float vga = sVG[ta], vgb = sVG[ta + 8];
            float gu8[8], bs8[8];  // per-channel sums over this thread's two tokens: r k vg (for gu) and b (for gw)
#pragma unroll
            for (int e = 0; e < 8; ++e) gu8[e] = bs8[e] = 0.f;
            // [buffer][GR1, GR2, GK1, GK2][value]: the tensor-memory loads of the next repetition fly while this one is used
            float acc4[2][4][4];
            auto ld4 = [&](int buf, int nn) {
                tmem_ld_16x256b_x1(tmP + lo + cb + 8 * nn, acc4[buf][0]);
                tmem_ld_16x256b_x1(tmGR2 + lo + cb + 8 * nn, acc4[buf][1]);
                tmem_ld_16x256b_x1(tmA + lo + cb + 8 * nn, acc4[buf][2]);
                tmem_ld_16x256b_x1(tmGK2 + lo + cb + 8 * nn, acc4[buf][3]);
            };
            ld4(0, 0);
            tmem_wait_ld();
#pragma unroll
            for (int nn = 0; nn < 4; ++nn) {
                const int col = 8 * (n0 + nn) + 2 * q;
                if (nn < 3) ld4((nn + 1) & 1, nn + 1);  // not read before the wait at the end of this repetition
                float (&g1)[4] = acc4[nn & 1][0], (&g2)[4] = acc4[nn & 1][1], (&h1)[4] = acc4[nn & 1][2], (&h2)[4] = acc4[nn & 1][3];
                const float2 fr = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&sFRb[col]));
                const float2 fk = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&sFKb[col]));
                const float2 uc = *reinterpret_cast<const float2 *>(&sU[col]);
                float qv[4];
#pragma unroll
                for (int hrow = 0; hrow < 2; ++hrow) {
                    const uint32_t off = FO(nn, hrow);
                    const float vg = hrow ? vgb : vga;
                    const __nv_bfloat162 r2b = *reinterpret_cast<const __nv_bfloat162 *>(sR + off);
                    const __nv_bfloat162 k2b = *reinterpret_cast<const __nv_bfloat162 *>(sK + off);
                    const __nv_bfloat162 erb = *reinterpret_cast<const __nv_bfloat162 *>(sET + off);
                    const float2 r2 = __bfloat1622float2(r2b), k2 = __bfloat1622float2(k2b);
                    const float2 er = __bfloat1622float2(erb), ek = __bfloat1622float2(ekb[2 * nn + hrow]);
                    // the bf16 operand values r~, k~ exactly as the MMAs saw them (same products, same rounding)
                    const float2 rt = __bfloat1622float2(__hmul2(r2b, erb)), kt = __bfloat1622float2(__hmul2(k2b, ekb[2 * nn + hrow]));
                    const float2 G1 = make_float2(g1[2 * hrow], g1[2 * hrow + 1]), G2 = make_float2(g2[2 * hrow], g2[2 * hrow + 1]);
                    const float2 H1 = make_float2(h1[2 * hrow], h1[2 * hrow + 1]), H2 = make_float2(h2[2 * hrow], h2[2 * hrow + 1]);
                    const float2 uvg = make_float2(uc.x * vg, uc.y * vg);
                    // gr = Er (GR1 + fR GR2) + u k vg ;  gk = Ek (GK1 + fK GK2) + u r vg
                    const float2 MR = fma2(fr, G2, G1);
                    const float2 gr = fma2(er, MR, mul2(uvg, k2));
                    const float2 gk = fma2(ek, fma2(fk, H2, H1), mul2(uvg, r2));
                    *reinterpret_cast<__nv_bfloat162 *>(sP + off) = to_bf2(gr);
                    *reinterpret_cast<__nv_bfloat162 *>(sAM + off) = to_bf2(gk);
                    // gw pieces: a = r~ GR1 + r^ GR2 = r~ (GR1 + fR GR2) (fR is a power of two), z = k~ GK1, b = k^ GK2
                    const float2 av = mul2(rt, MR);
                    const float2 bv = mul2(mul2(kt, fk), H2);
                    const float2 zbv = fma2(kt, H1, bv);
                    qv[2 * hrow] = av.x - zbv.x;
                    qv[2 * hrow + 1] = av.y - zbv.y;
                    loc[4 * nn + 2 * hrow] = -av.x;      // becomes  suffix_incl(q) - q - (z + b) = suffix_incl(q) - a
                    loc[4 * nn + 2 * hrow + 1] = -av.y;
                    bs8[2 * nn] += bv.x; bs8[2 * nn + 1] += bv.y;
                    const float2 rkv = mul2(mul2(r2, k2), make_float2(vg, vg));
                    gu8[2 * nn] += rkv.x;
                    gu8[2 * nn + 1] += rkv.y;
                }
                // sums over later tokens of the block by lane scans; block totals go through shared memory
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    float pa = qv[e], pb = qv[2 + e];
                    if (PERM) scan_suffix16_adj(pa, pb, r0); else scan_suffix16(pa, pb, r0, lane);
                    loc[4 * nn + e] += pa;
                    loc[4 * nn + 2 + e] += pb;
                    if (r0 == 0) sXtot[w4 * 64 + col + e] = pa;
                }
                if (nn < 3) tmem_wait_ld();
            }
            {   // block totals of b: 8 channel sums over the 8 lanes that share q, in 7 shuffles; lane r0 ends with channel
                // value index e = 4*bit4 + 2*bit3 + bit2 of its lane number
                const bool u4 = (lane & 16) != 0, u3 = (lane & 8) != 0, u2 = (lane & 4) != 0;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float send = u4 ? bs8[e] : bs8[e + 4], keep = u4 ? bs8[e + 4] : bs8[e];
                    bs8[e] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
                }
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const float send = u3 ? bs8[e] : bs8[e + 2], keep = u3 ? bs8[e + 2] : bs8[e];
                    bs8[e] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
                }
                {
                    const float send = u2 ? bs8[0] : bs8[1], keep = u2 ? bs8[1] : bs8[0];
                    bs8[0] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
                }
                const int e = (u4 ? 4 : 0) + (u3 ? 2 : 0) + (u2 ? 1 : 0);  // value index: channel 8 (n0 + e/2) + 2 q + (e & 1)
                sBtot[w4 * 64 + 8 * (n0 + (e >> 1)) + 2 * q + (e & 1)] = bs8[0];
            }
            {   // running sums of gu live in tensor memory between chunks
                float acc[8];
                tmem_ld_16x256b_x2(tmGUp, acc);
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[e] += gu8[e];
                tmem_st_16x256b_x2(tmGUp, acc);
            }
            float gv16[16];
            tmem_ld_16x256b_x4(tmGV + lo + cb, gv16);
#pragma unroll
            for (int nn = 0; nn < 4; ++nn) {  // the k~ tile is free: its last reader was the second MMA group
                *reinterpret_cast<uint32_t *>(sKT + FO(nn, 0)) = pack_bf2(gv16[4 * nn], gv16[4 * nn + 1]);
                *reinterpret_cast<uint32_t *>(sKT + FO(nn, 1)) = pack_bf2(gv16[4 * nn + 2], gv16[4 * nn + 3]);
            }
            tmem_wait_st();
        }
        tc_fence_before_sync();
        __syncthreads();
        WKV6_TSTAMP(it, 10);
        // every thread has read its raw r, k: fetch the next chunk's
        if (copy_thread && c > 0 && err == 0) issue_rk(c - 1);
        // G_t = e^{c_63} <S_in, Abar> + sum_all b + sum_{later blocks} q + (suffix_incl(q) - a)_t ;  gw = -exp(w) G.
        // The part that is the same for all tokens of a block is formed once per (block, channel) by one thread.
        {
            const int J = tid >> 6, i = tid & 63;
            float base = (sT1[i] + sT1[64 + i]) * sDtot[i];
#pragma unroll
            for (int J2 = 0; J2 < 4; ++J2) {
                base += sBtot[J2 * 64 + i];
                if (J2 > J) base += sXtot[J2 * 64 + i];
            }
            sOff[J * 64 + i] = base;
        }
        uint32_t lwst2[8];
        tmem_ld_16x256b_x2(tmStash, lwst2);
        tmem_wait_ld();
        __syncthreads();
#pragma unroll
        for (int nn = 0; nn < 4; ++nn) {
            const int col = 8 * (n0 + nn) + 2 * q;
            const float2 base = *reinterpret_cast<const float2 *>(&sOff[w4 * 64 + col]);
#pragma unroll
            for (int hrow = 0; hrow < 2; ++hrow) {
                const int e0 = 4 * nn + 2 * hrow;
                const float2 lwf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&lwst2[2 * nn + hrow]));
                float2 gw = mul2(mul2(lwf, make_float2(1.0f / kLog2e, 1.0f / kLog2e)),
                                 make_float2(base.x + loc[e0], base.y + loc[e0 + 1]));  // -exp(w) = log-decay
                if (a.zero_init && c == 0 && ta + 8 * hrow == 0) gw = make_float2(0.f, 0.f);  // no dependence on w_0
                *reinterpret_cast<__nv_bfloat162 *>(sRT + FO(nn, hrow)) = to_bf2(gw);  // the r~ tile is free: its last reader was the second MMA group
            }
        }
        fence_proxy_async_smem();
        if (!__syncthreads_and(err == 0)) { err = err ? err : 12; break; }
        WKV6_TSTAMP(it, 11);
        if (copy_thread) {
            st_tile(&tm_gr, sP, c);
            st_tile(&tm_gk, sAM, c);
            st_tile(&tm_gv, sKT, c);
            st_tile(&tm_gw, sRT, c);
            bulk_commit();
        }
    }

    WKV6_CSTAMP(5);
    // ---- unwind: wait (bounded) for loads still aimed at this CTA's shared memory, drain the stores, report
    if (copy_thread) {
        if (err != 0 || bail) {
            if (pend_w) mbar_wait(bar_w, par_early);
            if (pend_late) mbar_wait(bar_late, par_early);
            if (pend_rk) mbar_wait(bar_rk, par_rk);
            if (err != 0) atomicExch(&g_chunk_status, 200 + err);
        }
        bulk_wait<0>();
        a.flags[blockIdx.x] = (bail && err == 0) ? 1 : 0;
    }
    __syncthreads();
    WKV6_CSTAMP(6);
    // gu[b][h][i]: sum this thread's channels over the 8 lanes sharing q, then over the four row blocks
    float gu_acc[8];
    tmem_ld_16x256b_x2(tmGUp, gu_acc);
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
    if (tid < 64 && err == 0 && !bail)
        store_any(a.gu, a.gu_dtype, (size_t)blockIdx.x * 64 + tid, sGU[tid] + sGU[64 + tid] + sGU[128 + tid] + sGU[192 + tid]);
    if (warp == 0) tmem_dealloc(tbase, 256);
    WKV6_CSTAMP(7);
}

}  // namespace wkv6
