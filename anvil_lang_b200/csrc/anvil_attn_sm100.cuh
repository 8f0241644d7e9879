// anvil_attn_sm100.cuh — attention as ONE kernel per direction on sm_100a: product, row-wise softmax work and the
// second product without the T x T tensors making a round trip through HBM between them.
//
// The IR spells causal softmax attention as seven kernels (scores = q k^T, + mask, row max, exp, row sum, divide,
// o = p v) and its gradient as five (dp = do v^T, three softmax-gradient kernels, dq = ds k); each of them streams a
// [batch x heads, T, T] tensor through HBM. Here one CTA owns 128 query rows of one (batch, head) pair:
//
//   product 1   S[128 x T]  = A1[128 x DH] * B1[T x DH]^T       tcgen05.mma kind::tf32, 3xTF32, accumulator in TMEM
//   row phase   two warps per TMEM lane quarter, alternate 32-column chunks each; thread = row
//       forward   s = post(alpha1 * S, i, j);  m = max_j s;  e = exp(s - m);  sum = sum_j e;  p = e * (1 / sum)
//       backward  dp = S;  dt = sum_j dp * (-p / sum);  ds = (dp * (1 / sum) + dt) * e        (p, e, sum: from memory)
//     e, p and ds go to memory when a later kernel reads them; R = e (forward) or ds (backward) goes — split into
//     hi/lo, chunk by chunk as the last pass over the row produces it — straight back into TMEM as the A operand of
//   product 2   O[128 x DH] = R[128 x T] * B2[T x DH]          (A from tensor memory, B2 from shared memory; even and odd
//                                                               chunks of T into two accumulators, so two chains run)
//   epilogue    O = (even + odd) * scale, scale = 1 / sum of the row in the forward direction (product 2 ran on e, not
//               on p: it does not have to wait for the row sums), then the second product's own statements on O
//               (transposed through shared memory, coalesced).
//
// With a causal mask, query rows 0..127 cannot see keys 128..T-1: their CTA runs both products over 128 keys only
// and writes exact zeros for the rest (what exp(-1e9 - m) is in f32).
//
// Warps: 0-7 row phase + epilogue, 8-15 operand conversion (global -> hi/lo tiles in shared memory, the same split
// as anvil_gemm_sm100.cuh), 16 MMA issue. Every wait is an mbarrier wait bounded by a clock; a wait that runs out
// records TIMEOUT in the status word and the CTA leaves its loops, frees its tensor memory and returns.
#pragma once
#include "anvil_gemm_sm100.cuh"

namespace anvil {
namespace attn {

using namespace anvil::tc;

constexpr int QROWS = 128, ROW_WARPS = 8, CONV_WARPS = 8, MMA_W = ROW_WARPS + CONV_WARPS, THREADS_ATT = 32 * (MMA_W + 1);
constexpr int STAGE_FLOATS = 16 * 36;                                 // per row warp: 16 rows of 32 floats, rows 144 bytes apart
constexpr uint32_t COL_S = 0, COL_O = 256, COL_R = 384;            // TMEM columns: S (256), two O accumulators of 64, two R stages of 64 (hi 32 | lo 32)

__host__ __device__ constexpr uint32_t region_bytes(int t, int dh) {
    // phase 1: A1 and B1 for all of DH (hi + lo); phase 2 (overlaid): B2 for all of T (hi + lo)
    const uint32_t p1 = (uint32_t)(dh / BK) * 2u * (tile_bytes(QROWS) + tile_bytes(t));
    const uint32_t p2 = (uint32_t)(t / BK) * 2u * tile_bytes(dh);
    return p1 > p2 ? p1 : p2;
}
__host__ __device__ constexpr uint32_t smem_bytes_att(int t, int dh) { return region_bytes(t, dh) + ROW_WARPS * STAGE_FLOATS * 4 + 1024 + 256; }

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_st16_at(uint32_t taddr, const uint32_t *r) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
                 "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void row_bar() { asm volatile("bar.sync 1, 256;" ::: "memory"); }      // the eight row warps only

// A thread owns a row (the TMEM lane), but 32 lanes each moving 16 bytes of a different row cost the load/store unit 32
// lines per instruction. Chunks of W columns therefore pass through shared memory, 16 rows at a time: towards memory the
// owners write their rows, then W / 4 lanes move one row's 4 W bytes; from memory the other way round.
// stage = the warp's 16 x 36 floats, base = the chunk's first element in the warp's first row, rs = floats between rows.
template <int W>
__device__ __forceinline__ void tile_store(float *stage, int lane, float *base, int rs, const uint32_t *r) {
    constexpr int LPR = W / 4, RPI = 32 / LPR;
    const int srow = lane / LPR, scol = 4 * (lane % LPR);
#pragma unroll
    for (int half = 0; half < 2; half++) {
        if ((lane >> 4) == half) {
#pragma unroll
            for (int x = 0; x < W; x += 4)
                *reinterpret_cast<float4 *>(stage + (lane & 15) * 36 + x) = make_float4(__uint_as_float(r[x]), __uint_as_float(r[x + 1]),
                                                                                        __uint_as_float(r[x + 2]), __uint_as_float(r[x + 3]));
        }
        __syncwarp();
#pragma unroll
        for (int k = 0; k < 16 / RPI; k++)
            *reinterpret_cast<float4 *>(base + (16 * half + RPI * k + srow) * rs + scol) =
                *reinterpret_cast<const float4 *>(stage + (RPI * k + srow) * 36 + scol);
        __syncwarp();
    }
}
// From memory, 16 columns at a time, in two steps so that the loads of the next tile fly while this one is worked on:
// fetch (four 16-byte loads per lane: 4 lanes per row, 8 rows per instruction) and, later, the hand-over to the owners.
__device__ __forceinline__ void tile_fetch16(int lane, const float *base, int rs, float4 (&raw)[4]) {
    const int srow = lane >> 2, scol = 4 * (lane & 3);
#pragma unroll
    for (int k = 0; k < 4; k++) raw[k] = *reinterpret_cast<const float4 *>(base + (8 * k + srow) * rs + scol);
}
__device__ __forceinline__ void tile_hand_over16(float *stage, int lane, const float4 (&raw)[4], float *v) {
    const int srow = lane >> 2, scol = 4 * (lane & 3);
#pragma unroll
    for (int half = 0; half < 2; half++) {
#pragma unroll
        for (int k = 0; k < 2; k++) *reinterpret_cast<float4 *>(stage + (8 * k + srow) * 36 + scol) = raw[2 * half + k];
        __syncwarp();
        if ((lane >> 4) == half) {
#pragma unroll
            for (int x = 0; x < 16; x += 4) {
                const float4 t4 = *reinterpret_cast<const float4 *>(stage + (lane & 15) * 36 + x);
                v[x] = t4.x; v[x + 1] = t4.y; v[x + 2] = t4.z; v[x + 3] = t4.w;
            }
        }
        __syncwarp();
    }
}
__device__ __forceinline__ void tile_zero32(int lane, float *base, int rs) {
#pragma unroll
    for (int k = 0; k < 8; k++) *reinterpret_cast<float4 *>(base + (4 * k + (lane >> 3)) * rs + 4 * (lane & 7)) = make_float4(0.f, 0.f, 0.f, 0.f);
}

// F (generated):
//   T, DH, NBH, MODE (0 forward, 1 backward), CAUSAL, ALPHA1, ALPHA2, STORE_R, STORE_E, STORE_SUM, STORE_MAX
//   a1(i, k, bh, v[4]), b1(k, j, bh, v[4])      operands of product 1 (4 consecutive k)
//   b2(k, n, bh, v[4])                          B operand of product 2 (k runs over T, n over DH)
//   post(acc, i, j, bh)                         forward: the score from the scaled accumulator (mask)
//   r_row / e_row / p_row (i, bh) -> float *    row pointers (stride 1 along j) of the row result, exp values, probabilities
//   sum_at(i, bh) / max_at(i, bh) -> float *    per-row scalars
//   epi(i, n, bh, acc)                          statements of product 2
template <class F>
__device__ __forceinline__ void attn_fused(const F &f, uint32_t *status) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int T = F::T, DH = F::DH, NKB1 = DH / BK, NQT = T / QROWS;
    static_assert(T == 256 && DH == 64, "the template is laid out for T = 256, DH = 64");
    constexpr uint32_t TA1 = tile_bytes(QROWS), TB1 = tile_bytes(T), TB2 = tile_bytes(DH);
    constexpr uint32_t LBO_A1 = lbo_bytes(QROWS), LBO_B1 = lbo_bytes(T), LBO_B2 = lbo_bytes(DH);
    constexpr uint32_t REGION = region_bytes(T, DH), EPI_OFF = REGION, RED_OFF = EPI_OFF + ROW_WARPS * STAGE_FLOATS * 4, BAR_OFF = RED_OFF + 1024;
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const int WORK = F::NBH * NQT;

    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + BAR_OFF);
    const uint32_t bar0 = smem_u32(bars);
    const uint32_t qk_full = bar0, qk_free = bar0 + 8, s_full = bar0 + 16, s_free = bar0 + 24, v_full = bar0 + 32,
                   r_free = bar0 + 40, o_full = bar0 + 48;
    auto p_full = [&](int s) { return bar0 + 56u + 8u * s; };
    auto p_free = [&](int s) { return bar0 + 72u + 8u * s; };
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + BAR_OFF + 128);
    volatile uint32_t *failed = reinterpret_cast<volatile uint32_t *>(smem + BAR_OFF + 136);
    float *red = reinterpret_cast<float *>(smem + RED_OFF);                   // [2][128] row partials of the two column halves

    if (t == 0) {
        mbar_init(qk_full, CONV_WARPS); mbar_init(qk_free, 1); mbar_init(s_full, 1); mbar_init(s_free, ROW_WARPS);
        mbar_init(v_full, CONV_WARPS); mbar_init(r_free, 1); mbar_init(o_full, 1);
        for (int s = 0; s < 2; s++) { mbar_init(p_full(s), ROW_WARPS / 2); mbar_init(p_free(s), 1); }
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == MMA_W) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;

    // item w of a CTA's n-th round -> (batch x head, query tile); keys this tile can see. With a causal mask the later
    // query tile is about twice the work of the earlier one, and w % NQT alone would give a CTA the same tile every
    // round (the grid is a multiple of NQT wide): the tile index rotates with the round, so every CTA gets both kinds.
    const bool rotate = gridDim.x % NQT == 0;
    auto tile_of = [&](int w, int n) { return rotate ? (w % NQT + n) % NQT : w % NQT; };
    auto keys_of = [&](int qt) { return F::CAUSAL ? QROWS * (qt + 1) : T; };

    if (warp >= ROW_WARPS && warp < MMA_W) {
        // ---------------------------------------------------------------- operand conversion
        const int tc = t - 32 * ROW_WARPS;                                   // 0 .. 255
        int n = 0;
        for (int w = blockIdx.x; w < WORK && !*failed; w += gridDim.x, n++) {
            const int bh = w / NQT, qt = tile_of(w, n), i0 = qt * QROWS, NK = keys_of(qt);
            if (!mbar_wait(r_free, (uint32_t)(n & 1) ^ 1u)) { *failed = 1; break; }
            for (int kb = 0; kb < NKB1; kb++) {                                 // all loads of a block first, then the stores: the loads overlap
                uint8_t *a_hi = smem + kb * 2 * (TA1 + TB1), *a_lo = a_hi + TA1, *b_hi = a_lo + TA1, *b_lo = b_hi + TB1;
                const int row0 = tc / 8, kc = tc % 8;
                float va[QROWS / 32][4], vb[T / 32][4];
#pragma unroll
                for (int p = 0; p < QROWS / 32; p++) f.a1(i0 + row0 + 32 * p, kb * BK + kc * 4, bh, va[p]);
#pragma unroll
                for (int p = 0; p < T / 32; p++)
                    if (row0 + 32 * p < NK) f.b1(kb * BK + kc * 4, row0 + 32 * p, bh, vb[p]);
#pragma unroll
                for (int p = 0; p < QROWS / 32; p++) split_store(a_hi, a_lo, kc * LBO_A1 + (row0 + 32 * p) * 16, va[p]);
#pragma unroll
                for (int p = 0; p < T / 32; p++)
                    if (row0 + 32 * p < NK) split_store(b_hi, b_lo, kc * LBO_B1 + (row0 + 32 * p) * 16, vb[p]);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(qk_full);
            if (!mbar_wait(qk_free, (uint32_t)(n & 1))) { *failed = 1; break; }       // product 1 has read its tiles
            for (int kb = 0; kb < NK / BK; kb += 2) {                          // two blocks' loads in flight at a time
                const int row = tc % DH, kc0 = tc / DH;                         // lanes along n (contiguous in memory), 4 k each
                float vv[2][DH / 32][4];
#pragma unroll
                for (int u = 0; u < 2; u++)
#pragma unroll
                    for (int p = 0; p < DH / 32; p++) f.b2((kb + u) * BK + (kc0 + (256 / DH) * p) * 4, row, bh, vv[u][p]);
#pragma unroll
                for (int u = 0; u < 2; u++) {
                    uint8_t *b_hi = smem + (kb + u) * 2 * TB2, *b_lo = b_hi + TB2;
#pragma unroll
                    for (int p = 0; p < DH / 32; p++) split_store(b_hi, b_lo, (kc0 + (256 / DH) * p) * LBO_B2 + row * 16, vv[u][p]);
                }
            }
            if (w + (int)gridDim.x < WORK) {                                    // ask L2 for the next item's operands: one 128-byte line per call
                const int w2 = w + gridDim.x, bh2 = w2 / NQT, qt2 = tile_of(w2, n + 1), NK2 = keys_of(qt2);
                if (tc < QROWS * (DH / 32)) f.a1_touch(qt2 * QROWS + tc / (DH / 32), 32 * (tc % (DH / 32)), bh2);
                for (int x = tc; x < NK2 * (DH / 32); x += 256) f.b1_touch(32 * (x % (DH / 32)), x / (DH / 32), bh2);
                for (int x = tc; x < NK2 * (DH / 32); x += 256) f.b2_touch(x / (DH / 32), 32 * (x % (DH / 32)), bh2);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(v_full);
        }
    } else if (warp == MMA_W) {
        if (lane == 0) {
            // ------------------------------------------------------------ MMA issue
            const uint32_t base = smem_u32(smem);
            uint32_t pcount[2] = {0u, 0u};
            int n = 0;
            for (int w = blockIdx.x; w < WORK && !*failed; w += gridDim.x, n++) {
                const int qt = tile_of(w, n), NK = keys_of(qt);
                const uint32_t idesc1 = instr_desc(QROWS, NK), idesc2 = instr_desc(QROWS, DH);
                if (!mbar_wait(qk_full, (uint32_t)(n & 1))) { *failed = 1; break; }
                if (!mbar_wait(s_free, (uint32_t)(n & 1) ^ 1u)) { *failed = 1; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                for (int kb = 0; kb < NKB1; kb++) {
                    const uint32_t a_hi = base + kb * 2 * (TA1 + TB1), a_lo = a_hi + TA1, b_hi = a_lo + TA1, b_lo = b_hi + TB1;
#pragma unroll
                    for (int j = 0; j < BK / 8; j++) {
                        const uint64_t dah = smem_desc(a_hi + 2 * j * LBO_A1, LBO_A1), dal = smem_desc(a_lo + 2 * j * LBO_A1, LBO_A1);
                        const uint64_t dbh = smem_desc(b_hi + 2 * j * LBO_B1, LBO_B1), dbl = smem_desc(b_lo + 2 * j * LBO_B1, LBO_B1);
                        mma_tf32(tmem + COL_S, dah, dbl, idesc1, (kb | j) ? 1u : 0u);     // small terms first, then the large one
                        mma_tf32(tmem + COL_S, dal, dbh, idesc1, 1u);
                        mma_tf32(tmem + COL_S, dah, dbh, idesc1, 1u);
                    }
                }
                mma_commit(qk_free);
                mma_commit(s_full);
                if (!mbar_wait(v_full, (uint32_t)(n & 1))) { *failed = 1; break; }
                bool ok = true;
                for (int kb = 0; kb < NK / BK; kb++) {
                    const int s = kb & 1;
                    if (!mbar_wait(p_full(s), pcount[s] & 1u)) { ok = false; break; }
                    pcount[s]++;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t b_hi = base + kb * 2 * TB2, b_lo = b_hi + TB2;
                    const uint32_t a_hi = tmem + COL_R + 64u * s, a_lo = a_hi + 32u;
                    const uint32_t acc = tmem + COL_O + 64u * s;                     // even and odd chunks: accumulators of their own, two chains in flight
#pragma unroll
                    for (int j = 0; j < BK / 8; j++) {
                        const uint64_t dbh = smem_desc(b_hi + 2 * j * LBO_B2, LBO_B2), dbl = smem_desc(b_lo + 2 * j * LBO_B2, LBO_B2);
                        mma_tf32_ts(acc, a_hi + 8u * j, dbl, idesc2, ((kb >> 1) | j) ? 1u : 0u);
                        mma_tf32_ts(acc, a_lo + 8u * j, dbh, idesc2, 1u);
                        mma_tf32_ts(acc, a_hi + 8u * j, dbh, idesc2, 1u);
                    }
                    mma_commit(p_free(s));
                }
                if (!ok) { *failed = 1; break; }
                mma_commit(r_free);
                mma_commit(o_full);
            }
        }
    } else {
        // -------------------------------------------------------------------- row phase: thread = row; the two warps of a
        // lane quarter take alternate 32-column chunks (h = 0: chunks 0, 2, ..; h = 1: chunks 1, 3, ..), so a thread moves whole
        // 128-byte lines of its row and stage h of the A operand belongs to the warps with that h alone
        const int q = warp & 3, h = warp >> 2, row = 32 * q + lane;
        const uint32_t lane_addr = tmem + ((uint32_t)(32 * q) << 16);
        float *stage_f = reinterpret_cast<float *>(smem + EPI_OFF) + warp * STAGE_FLOATS;  // 16 rows of a 32-column chunk at a time
        uint32_t fcount = 0u;
        int n = 0;                                                                 // rounds of this CTA
        // The row warps meet at a named barrier, so they must all leave the loop at the same place: a wait that ran out
        // is recorded in a flag of their own and looked at by everybody right after the next barrier.
        volatile uint32_t *rfail = reinterpret_cast<volatile uint32_t *>(smem + BAR_OFF + 144);
        if (t == 0) *rfail = 0;
        row_bar();
        // one chunk of the second product's A operand: wait for stage h, split 16 columns at a time into hi / lo in tensor
        // memory, then tell the MMA warp
        auto feed_begin = [&]() -> bool {
            if (!__all_sync(0xFFFFFFFFu, mbar_wait(p_free(h), (fcount & 1u) ^ 1u))) return false;      // the warp stays together
            fcount++;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            return true;
        };
        auto feed_half = [&](int half, const uint32_t *r16) {
            uint32_t part[16];
#pragma unroll
            for (int x = 0; x < 16; x++) part[x] = r16[x] & 0xFFFFE000u;
            tmem_st16_at(lane_addr + COL_R + 64u * h + 16u * half, part);
#pragma unroll
            for (int x = 0; x < 16; x++) part[x] = __float_as_uint(__uint_as_float(r16[x]) - __uint_as_float(part[x]));
            tmem_st16_at(lane_addr + COL_R + 64u * h + 32u + 16u * half, part);
        };
        auto feed_end = [&]() {
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full(h));
        };
        for (int w = blockIdx.x; w < WORK; w += gridDim.x, n++) {
            const int bh = w / NQT, qt = tile_of(w, n), i = qt * QROWS + row, NK = keys_of(qt), NCH = NK / 32;
            // the warp's 32 rows of the row tensors: first row and the distance between rows (the tensors are affine in i)
            const int iw = qt * QROWS + 32 * q;
            float *r_base = F::STORE_R ? f.r_row(iw, bh) : nullptr;
            const int r_rs = F::STORE_R ? (int)(f.r_row(iw + 1, bh) - f.r_row(iw, bh)) : 0;
            float *e_base = (F::STORE_E || F::MODE == 1) ? f.e_row(iw, bh) : nullptr;
            const int e_rs = (F::STORE_E || F::MODE == 1) ? (int)(f.e_row(iw + 1, bh) - f.e_row(iw, bh)) : 0;
            const float *p_base = F::MODE == 1 ? f.p_row(iw, bh) : nullptr;
            const int p_rs = F::MODE == 1 ? (int)(f.p_row(iw + 1, bh) - f.p_row(iw, bh)) : 0;
            if (F::MODE == 1) {                                                   // this row's p and e lines: on their way while product 1 runs
                for (int c = h; c < NCH; c += 2) { anvil::prefetch_l2(p_base + lane * p_rs + 32 * c); anvil::prefetch_l2(e_base + lane * e_rs + 32 * c); }
            }
            // keys this tile cannot see: exp(-1e9 - m) = 0 exactly, so e, p and ds are zeros there; written while product 1 runs
            for (int c = NCH + h; c < T / 32; c += 2) {
                if (F::STORE_R) tile_zero32(lane, r_base + 32 * c, r_rs);
                if (F::STORE_E && F::MODE == 0) tile_zero32(lane, e_base + 32 * c, e_rs);
            }
            bool ok = mbar_wait(s_full, (uint32_t)(n & 1));
            if (!ok) *rfail = 1;
            row_bar();
            if (*rfail) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            float oscale = F::ALPHA2;                                              // what the epilogue multiplies this row of O by
            if (F::MODE == 0) {
                // ---- forward: max; then e = exp(s - max), its sum, and e straight into product 2 (which therefore sums
                // e * v; the division by the row sum is applied to its 64 results instead of to the T probabilities)
                float m4[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
                for (int c = h; c < NCH; c += 2) {
                    uint32_t r[32];
                    tmem_ld32(lane_addr + COL_S + 32 * c, r);
#pragma unroll
                    for (int x = 0; x < 32; x++) m4[x & 3] = anvil::fmax_nan(m4[x & 3], f.post(__uint_as_float(r[x]) * F::ALPHA1, i, 32 * c + x, bh));
                }
                red[h * 128 + row] = anvil::fmax_nan(anvil::fmax_nan(m4[0], m4[1]), anvil::fmax_nan(m4[2], m4[3]));
                row_bar();
                const float m = anvil::fmax_nan(red[row], red[128 + row]);
                row_bar();
                float sum = 0.0f;
                for (int c = h; c < NCH && ok; c += 2) {
                    uint32_t r[32];
                    tmem_ld32(lane_addr + COL_S + 32 * c, r);
#pragma unroll
                    for (int x = 0; x < 32; x++) {
                        const float e = expf(f.post(__uint_as_float(r[x]) * F::ALPHA1, i, 32 * c + x, bh) - m);
                        sum = sum + e;
                        r[x] = __float_as_uint(e);
                    }
                    if (F::STORE_R) {                                              // kept in place for the pass that writes p
                        tmem_st16_at(lane_addr + COL_S + 32 * c, r);
                        tmem_st16_at(lane_addr + COL_S + 32 * c + 16, r + 16);
                    }
                    if (F::STORE_E) tile_store<32>(stage_f, lane, e_base + 32 * c, e_rs, r);
                    ok = feed_begin();
                    if (ok) { feed_half(0, r); feed_half(1, r + 16); feed_end(); }
                }
                red[h * 128 + row] = sum;
                row_bar();
                const float rowsum = red[row] + red[128 + row];
                row_bar();
                const float rinv = 1.0f / rowsum;                                  // e / sum as e * (1 / sum)
                oscale = rinv * F::ALPHA2;
                if (h == 0) {
                    if (F::STORE_SUM) *f.sum_at(i, bh) = rowsum;
                    if (F::STORE_MAX) *f.max_at(i, bh) = m;
                }
                if (F::STORE_R) {                                                  // p = e / sum, for the kernels that read it later
                    for (int c = h; c < NCH; c += 2) {
                        uint32_t r[32];
                        tmem_ld32(lane_addr + COL_S + 32 * c, r);
#pragma unroll
                        for (int x = 0; x < 32; x++) r[x] = __float_as_uint(__uint_as_float(r[x]) * rinv);
                        tile_store<32>(stage_f, lane, r_base + 32 * c, r_rs, r);
                    }
                }
            } else {
                // ---- backward: dt = sum_j dp * (-p / sum); then ds = (dp / sum + dt) * e, to memory and into product 2
                const float tsum = *f.sum_at(i, bh);
                const float ninv = -1.0f / tsum;                                   // -p / sum as p * (-1 / sum): one rounding more, no division per element
                float dt = 0.0f;
                // 16 columns at a time (the registers hold two operands), the next tile's loads in flight during the work on this one
                auto next_of = [](int c2) { return c2 + ((c2 & 1) ? 3 : 1); };     // this warp's half chunks: 2h, 2h + 1, 2h + 4, 2h + 5, ..
                float4 raw[4];
                tile_fetch16(lane, p_base + 16 * (2 * h), p_rs, raw);
                for (int c2 = 2 * h; c2 < 2 * NCH; c2 = next_of(c2)) {
                    uint32_t r[16];
                    float pv[16];
                    tmem_ld16(lane_addr + COL_S + 16 * c2, r);
                    tile_hand_over16(stage_f, lane, raw, pv);
                    if (next_of(c2) < 2 * NCH) tile_fetch16(lane, p_base + 16 * next_of(c2), p_rs, raw);
                    else tile_fetch16(lane, e_base + 16 * (2 * h), e_rs, raw);   // the second pass's first tile
#pragma unroll
                    for (int x = 0; x < 16; x++) dt = dt + (__uint_as_float(r[x]) * F::ALPHA1) * (pv[x] * ninv);
                }
                red[h * 128 + row] = dt;
                row_bar();
                dt = red[row] + red[128 + row];
                row_bar();
                const float inv = 1.0f / tsum;
                for (int c2 = 2 * h; c2 < 2 * NCH; c2 = next_of(c2)) {
                    if (!(c2 & 1)) { ok = feed_begin(); if (!ok) break; }
                    uint32_t r[16];
                    float ev[16];
                    tmem_ld16(lane_addr + COL_S + 16 * c2, r);
                    tile_hand_over16(stage_f, lane, raw, ev);
                    if (next_of(c2) < 2 * NCH) tile_fetch16(lane, e_base + 16 * next_of(c2), e_rs, raw);
#pragma unroll
                    for (int x = 0; x < 16; x++) r[x] = __float_as_uint(((__uint_as_float(r[x]) * F::ALPHA1) * inv + dt) * ev[x]);
                    if (F::STORE_R) tile_store<16>(stage_f, lane, r_base + 16 * c2, r_rs, r);
                    feed_half(c2 & 1, r);
                    if (c2 & 1) feed_end();
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(s_free);                                    // the next tile's product 1 may overwrite S
            // ---- epilogue of product 2: warp (q, h) takes rows 32 q .. 32 q + 31, columns 32 h .. 32 h + 31 of O = the sum of
            // the two accumulators (even and odd key chunks), 16 rows at a time through shared memory for coalesced stores
            if (!ok || !mbar_wait(o_full, (uint32_t)(n & 1))) *rfail = 1;
            row_bar();
            if (*rfail) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            static_assert(DH / 32 == ROW_WARPS / 4, "one 32-column chunk of O per warp of a lane quarter");
            {
                float o[32];
#pragma unroll
                for (int hc = 0; hc < 2; hc++) {                                   // 16 columns at a time: fewer registers live
                    uint32_t ra[16], rb[16];
                    tmem_ld16(lane_addr + COL_O + 32 * h + 16 * hc, ra);
                    tmem_ld16(lane_addr + COL_O + 64 + 32 * h + 16 * hc, rb);
#pragma unroll
                    for (int x = 0; x < 16; x++) o[16 * hc + x] = (__uint_as_float(ra[x]) + __uint_as_float(rb[x])) * oscale;
                }
#pragma unroll
                for (int half = 0; half < 2; half++) {
                    if ((lane >> 4) == half) {
#pragma unroll
                        for (int x = 0; x < 32; x++)
                            stage_f[(lane & 15) * 36 + x] = o[x];
                    }
                    __syncwarp();
#pragma unroll 4
                    for (int rr = 0; rr < 16; rr++)
                        f.epi(qt * QROWS + 32 * q + 16 * half + rr, 32 * h + lane, bh, stage_f[rr * 36 + lane]);
                    __syncwarp();
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        }
        if (*rfail) *failed = 1;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == MMA_W) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
    if (t == 0 && *failed) atomicExch(status, TIMEOUT);
}

}  // namespace attn
}  // namespace anvil
