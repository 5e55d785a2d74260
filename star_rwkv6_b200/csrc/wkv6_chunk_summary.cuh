// Segment summaries for sequence splitting: per (batch, head) sequence the state it builds from zero and the log2 of
// its total decay, without any of the output work of the forward kernel.
//
//   forward direction :  S = sum_t (k_t e^{c_end - c_t}) (x) v_t        (x1 = k, x2 = v)
//   reverse direction :  A = sum_t (r_t e^{c_{t-1} - c_start}) (x) gy_t  (x1 = r, x2 = gy; the reverse state of the backward)
// Both exponents are non-positive whatever the decays are, so no reference points are needed: per 64-token chunk the
// kernel scales x1 by one exponential (bf16 operand), takes x1^^T x2 on the tensor core (four tcgen05.mma of K = 16
// tokens, fp32 accumulator in tensor memory) and folds it into the fp32 state kept in registers,
//   forward:  S <- e^{c_63} S + chunk sum ,      reverse (chunks walked last to first):  A <- e^{c_63} A + chunk sum.
// One CTA of 256 threads per sequence, three input tiles per chunk (x1, x2, w) double-buffered through TMA.
#pragma once

#include "wkv6_chunk_fwd.cuh"

namespace wkv6 {

struct ChunkSumSmem {
    static constexpr int kStage = 3 * kTile;                 // x1, x2, w
    static constexpr int oHead = 2 * kStage;                 // float [4][64]: log2-decay sum of tokens 0..7 of a block
    static constexpr int oTail = oHead + 4 * 64 * 4;         // float [4][64]: log2-decay sum of tokens 8..15 of a block
    static constexpr int oDtot = oTail + 4 * 64 * 4;         // float [64]: decay over the whole chunk
    static constexpr int oBar = oDtot + 64 * 4;              // mbarriers: full[2], mma
    static constexpr int oSlot = oBar + 3 * 8;
    static constexpr int kBytes = oSlot + 16;
    static constexpr int kAlloc = kBytes;
};

__global__ void __launch_bounds__(256, 2) chunk_summary_kernel(const __grid_constant__ CUtensorMap tm_x1,
                                                               const __grid_constant__ CUtensorMap tm_x2,
                                                               const __grid_constant__ CUtensorMap tm_w,
                                                               const ChunkFwdArgs a) {
    using namespace ptx;
    using SM = ChunkSumSmem;
    extern __shared__ __align__(1024) uint8_t wkv6_chunk_smem[];
    uint8_t *const smem = wkv6_chunk_smem;
    if ((smem_u32(smem) & 1023u) != 0) {
        if (threadIdx.x == 0) atomicExch(&g_chunk_status, 50);
        return;
    }
    // a segment whose summary the caller's scan never reads (the last of a sequence going forward, the first in reverse)
    if (a.skip_mod > 0 && (int)(blockIdx.x / a.H) % a.skip_mod == a.skip_rem) return;
    float *sHead = reinterpret_cast<float *>(smem + SM::oHead);
    float *sTail = reinterpret_cast<float *>(smem + SM::oTail);
    float *sDtot = reinterpret_cast<float *>(smem + SM::oDtot);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + SM::oBar);
    uint64_t *bar_full = bars, *bar_mma = bars + 2;
    uint32_t *slot = reinterpret_cast<uint32_t *>(smem + SM::oSlot);

    // Operand pass: warp (w4, half) owns tokens 16*w4 + 8*half .. +7, lane = channel pair.  Accumulator pass: warp
    // (w4, half) owns rows 16*w4 + r0 (+8) and the 32 columns 32*half .. +31 (fragment layout of tcgen05.ld.16x256b).
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int w4 = warp & 3, half = warp >> 2, n0 = 4 * half;
    const int ta = 16 * w4 + (lane >> 2);
    const int b = blockIdx.x / a.H, h = blockIdx.x % a.H;
    const int nchunks = (a.T + kChunk - 1) / kChunk;

    if (tid == 0) {
        mbar_init(&bar_full[0], 3);  // one arrival per loading thread
        mbar_init(&bar_full[1], 3);
        mbar_init(bar_mma, 1);
        fence_mbar_init();
        prefetch_tensormap(&tm_x1); prefetch_tensormap(&tm_x2); prefetch_tensormap(&tm_w);
    }
    if (warp == 0) {
        tmem_alloc(slot, 64);
        tmem_relinquish();
    }
    float S[16];
#pragma unroll
    for (int e = 0; e < 16; ++e) S[e] = 0.f;
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tb = *slot;
    const uint32_t tmS = tb + ((uint32_t)(w4 * 32) << 16) + 8 * n0;  // this thread's fragment of the accumulator

    const int load_slot = (lane == 0 && warp >= 2 && warp <= 4) ? warp - 2 : -1;  // 0..2 = x1, x2, w
    auto issue_loads = [&](int ic2) {  // every thread calls it; the three loading threads act
        if (load_slot < 0) return;
        const int c = a.reverse_state ? nchunks - 1 - ic2 : ic2;
        const int st = ic2 & 1;
        uint8_t *dst = smem + st * SM::kStage + load_slot * kTile;
        const CUtensorMap *tm = load_slot == 0 ? &tm_x1 : load_slot == 1 ? &tm_x2 : &tm_w;
        mbar_expect_tx(&bar_full[st], kTile);
        tma_load_3d(dst, tm, &bar_full[st], h * 64, c * kChunk, b);
    };
    issue_loads(0);
    if (nchunks > 1) issue_loads(1);

    constexpr uint32_t idMM = umma_idesc_bf16(64, 64, true, true);
    const uint64_t dX1 = umma_desc_sw128(smem_u32(smem)), dX2 = umma_desc_sw128(smem_u32(smem + kTile));

    int err = 0;
    int loads_issued = (nchunks > 1) ? 2 : 1, loads_consumed = 0;
    float2 dsum = make_float2(0.f, 0.f);  // warp 0: log2 of the decay accumulated over all chunks, channels 2*lane, +1
    for (int ic = 0; ic < nchunks; ++ic) {
        const int c = a.reverse_state ? nchunks - 1 - ic : ic;
        const int st = ic & 1;
        uint8_t *sX = smem + st * SM::kStage;
        const uint64_t so = (uint64_t)(st * (SM::kStage >> 4));
        if (!cta_wait(&bar_full[st], (ic >> 1) & 1, warp)) err = 1;
        if (err == 0) ++loads_consumed;

        // ---- per-step log2 decays of this thread's 8 tokens x 2 channels, running sums from the first of them
        uint8_t *const tbase = sX + (16 * w4 + 8 * half) * 128 + ((lane & 3) << 2);
        const uint32_t lane_chunk = (uint32_t)(lane >> 2);
        const bool full_chunk = (c + 1) * kChunk <= a.T;
        float2 x[8];
        {
            float2 cs = make_float2(0.f, 0.f);
#pragma unroll
            for (int tt = 0; tt < 8; ++tt) {
                const uint8_t *pt = tbase + tt * 128 + ((lane_chunk ^ tt) << 4);
                const float2 e2 = mul2(ld_bf2(pt + 2 * kTile), make_float2(kLog2e, kLog2e));
                float2 l2 = mul2(make_float2(ex2f(e2.x), ex2f(e2.y)), make_float2(-kLog2e, -kLog2e));
                l2.x = fmaxf(l2.x, kMinLogDecay2);
                l2.y = fmaxf(l2.y, kMinLogDecay2);
                if (!full_chunk && c * kChunk + 16 * w4 + 8 * half + tt >= a.T) l2 = make_float2(0.f, 0.f);
                cs = add2(cs, l2);
                x[tt] = cs;
            }
            *reinterpret_cast<float2 *>(&(half ? sTail : sHead)[w4 * 64 + 2 * lane]) = cs;
        }
        if (!__syncthreads_and(err == 0)) { err = err ? err : 10; break; }

        // ---- x1 scaled by its exponential, in place
        {
            float2 pre = make_float2(0.f, 0.f), all = make_float2(0.f, 0.f), head = make_float2(0.f, 0.f);
#pragma unroll
            for (int J = 0; J < 4; ++J) {
                const float2 hj = *reinterpret_cast<const float2 *>(&sHead[J * 64 + 2 * lane]);
                const float2 tl = *reinterpret_cast<const float2 *>(&sTail[J * 64 + 2 * lane]);
                const float2 tj = add2(hj, tl);
                if (J < w4) pre = add2(pre, tj);
                if (J == w4) head = hj;
                all = add2(all, tj);
            }
            const float2 gstart = half ? add2(pre, head) : pre;  // running sum before this thread's first token
            if (warp == 0) {
                *reinterpret_cast<float2 *>(&sDtot[2 * lane]) = make_float2(ex2f(all.x), ex2f(all.y));
                dsum = add2(dsum, all);
            }
            // forward: c_63 - c_t = all - (gstart + x[tt]);  reverse: c_{t-1} - c_start = gstart + x[tt-1]
            const float2 base = a.reverse_state ? gstart : make_float2(all.x - gstart.x, all.y - gstart.y);
            __nv_bfloat162 xb[8];
#pragma unroll
            for (int tt = 0; tt < 8; ++tt)
                xb[tt] = *reinterpret_cast<const __nv_bfloat162 *>(tbase + tt * 128 + ((lane_chunk ^ tt) << 4));
#pragma unroll
            for (int tt = 0; tt < 8; ++tt) {
                float2 e;
                if (a.reverse_state) e = (tt == 0) ? base : add2(base, x[tt - 1]);
                else e = make_float2(base.x - x[tt].x, base.y - x[tt].y);
                xb[tt] = __hmul2(xb[tt], to_bf2(make_float2(ex2f(e.x), ex2f(e.y))));
            }
#pragma unroll
            for (int tt = 0; tt < 8; ++tt)
                *reinterpret_cast<__nv_bfloat162 *>(tbase + tt * 128 + ((lane_chunk ^ tt) << 4)) = xb[tt];
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        __syncthreads();

        if (tid == 0) {
            tc_fence_after_sync();
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)  // chunk sum = x1^^T x2
                umma_ss(tb, dX1 + so + 128 * kk, dX2 + so + 128 * kk, idMM, kk > 0);
            umma_commit(bar_mma);
        }
        if (!cta_wait(bar_mma, ic & 1, warp)) err = 2;
        tc_fence_after_sync();
        // the tiles of this stage are free again: fetch the chunk after next
        if (ic + 2 < nchunks && err == 0) { issue_loads(ic + 2); ++loads_issued; }

        {
            const float d0 = sDtot[ta], d1 = sDtot[ta + 8];
            uint32_t v16[16];
            tmem_ld_16x256b_x4(tmS, v16);
            tmem_wait_ld();
#pragma unroll
            for (int nn = 0; nn < 4; ++nn) {
                S[4 * nn + 0] = fmaf(S[4 * nn + 0], d0, __uint_as_float(v16[4 * nn + 0]));
                S[4 * nn + 1] = fmaf(S[4 * nn + 1], d0, __uint_as_float(v16[4 * nn + 1]));
                S[4 * nn + 2] = fmaf(S[4 * nn + 2], d1, __uint_as_float(v16[4 * nn + 2]));
                S[4 * nn + 3] = fmaf(S[4 * nn + 3], d1, __uint_as_float(v16[4 * nn + 3]));
            }
        }
        // The accumulator and the per-chunk arrays are rewritten only behind the next iteration's barriers, which no
        // thread passes before every thread has finished this update.
        tc_fence_before_sync();
    }

    // ---- unwind: drain this CTA's copies, report, release tensor memory
    if (err != 0 && load_slot >= 0) {
        for (int ic2 = loads_consumed; ic2 < loads_issued; ++ic2) mbar_wait(&bar_full[ic2 & 1], (ic2 >> 1) & 1);
    }
    if (tid == 32 && err != 0) atomicExch(&g_chunk_status, 300 + err);
    if (err == 0 && a.dec_out != nullptr && warp == 0)
        *reinterpret_cast<float2 *>(a.dec_out + (size_t)blockIdx.x * 64 + 2 * lane) = dsum;
    if (err == 0 && a.s_out != nullptr) {
        float *out = static_cast<float *>(a.s_out) + (size_t)blockIdx.x * 4096;
        const int q = lane & 3;
#pragma unroll
        for (int nn = 0; nn < 4; ++nn) {
            const int j = 8 * (n0 + nn) + 2 * q;
            *reinterpret_cast<float2 *>(out + (size_t)ta * 64 + j) = make_float2(S[4 * nn], S[4 * nn + 1]);
            *reinterpret_cast<float2 *>(out + (size_t)(ta + 8) * 64 + j) = make_float2(S[4 * nn + 2], S[4 * nn + 3]);
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tb, 64);
}

}  // namespace wkv6
