// anvil_gemm_sm100.cuh — tensor-core contraction template for sm_100a: tcgen05.mma (kind::tf32) with the
// accumulator in tensor memory, f32 accuracy recovered by the 3xTF32 split.
//
//   C[b, m, n] = epilogue(alpha * sum_k A[b, m, k] * B[b, k, n])        (same functor contract as
//                                                                        anvil_gemm_simt.cuh)
//
// Five templates share the operand conversion, the two-accumulator scheme and the bounded waits:
//   gemm_tc_tile             one CTA per 128 x BN tile, operands in shared memory, 32-wide k blocks (described next)
//   gemm_tc_ts_tile          the same with the A tiles kept in tensor memory
//   gemm_tc2_tile            16-wide k blocks, two CTAs per SM (short reductions on narrow outputs)
//   gemm_tc_pair_tile        two CTAs of a cluster on one 256-row tile, tcgen05.mma.cta_group::2
//   gemm_tc_pair_persistent  resident CTA pairs walking over the tiles with converter, MMA and epilogue warps
//                            overlapping across tiles — what every contraction with M >= 256 and N >= 64 takes
//
// gemm_tc_tile: one CTA computes a 128 x BN tile. Twenty-five warps:
//   warps 0-23 "converters" (three groups of eight; group g takes k blocks g, g + 3, ...): read operand values through the generated functor (so prologues such as
//              max(x, 0), scales and gathers cost nothing extra), split every f32 x into
//              hi = x with the low 13 mantissa bits cleared (exactly a TF32 value) and lo = x - hi
//              (exact in f32), and write both into shared memory in the tensor core's canonical
//              K-major no-swizzle layout: 16-byte chunk (row r, k-chunk c) at  c * LBO + r * 16.
//   warp 24    one thread issues, per 32-wide k block, 4 k-steps x 3 MMAs: hi*hi into the main TMEM
//              accumulator, hi*lo and lo*hi into a second one (the tensor core rounds its accumulator
//              toward zero at every accumulate, so the small terms are kept away from the large sum);
//              then it commits the stage's "empty" barrier.
//   warps 0-23 afterwards read the accumulator (tcgen05.ld, 32 lanes x 32 columns per warp), transpose
//              32 x 32 blocks through shared memory so that consecutive lanes hold consecutive n, and
//              run the kernel's statements (the epilogue functor) with coalesced stores.
// A 3-stage ring of {A hi, A lo, B hi, B lo} tiles (64.5 KB per stage at BN = 128) is handed back
// and forth with mbarriers: converters arrive on full[s] after a generic->async proxy fence, the MMA
// thread's tcgen05.commit arrives on empty[s].
//
// Every wait is bounded by a clock: a barrier that does not flip within about a second makes the
// waiting thread record ANVIL_TC_TIMEOUT in the arena header's status word and leave its loop; the
// CTA still meets at the final barrier and frees its tensor memory. Nothing here traps.
//
// Accumulation order is fixed by the tile shape alone: results are bit-reproducible.
#pragma once
#include <type_traits>
#include <cuda_runtime.h>
#include <stdint.h>

namespace anvil {
namespace tc {

constexpr int BM = 128, BK = 32, STAGES = 3;
constexpr int CONV_THREADS = 256, CONV_GROUPS = 3, MMA_WARP = 8 * CONV_GROUPS, THREADS = 32 * MMA_WARP + 32;
constexpr uint32_t TIMEOUT = 0x7C05u;

__host__ __device__ constexpr uint32_t lbo_bytes(int rows) { return (uint32_t)rows * 16u + 16u; }   // +16: no bank aliasing between k-chunks
__host__ __device__ constexpr uint32_t tile_bytes(int rows) { return (BK / 4) * lbo_bytes(rows); }
__host__ __device__ constexpr uint32_t stage_bytes(int bn) { return 2 * tile_bytes(BM) + 2 * tile_bytes(bn); }
__host__ __device__ constexpr int ss_stages(int bn) { return bn > 128 ? 2 : STAGES; }      // 227 KB of shared memory per CTA
__host__ __device__ constexpr uint32_t smem_bytes(int bn) { return ss_stages(bn) * stage_bytes(bn) + 256; }

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Bounded wait: false if the phase did not complete within `limit` clocks (by default ~2^31, about a second).
constexpr long long WAIT_CLOCKS = 1LL << 31;
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, long long limit = WAIT_CLOCKS) {
    const long long t0 = clock64();
    while (true) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if (clock64() - t0 > limit) return false;
    }
}

__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo) {
    // K-major, no swizzle: start >> 4 | LBO >> 4 at bit 16 | SBO >> 4 at bit 32 | version 1 at bit 46
    return (uint64_t)((addr >> 4) & 0x3FFFu) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(128u >> 4) << 32) | (1ull << 46);
}
__host__ __device__ constexpr uint32_t instr_desc(int m, int n) {
    // D = f32 (1 << 4), A and B = TF32 (2 << 7, 2 << 10), both K-major, N >> 3 at bit 17, M >> 4 at bit 24
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void mma_tf32(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// One operand tile of a k block, as the converter threads see it. ROWS x 32 values = ROWS/32 chunks
// of 4 per thread. KC (the operand is contiguous along k in memory): 8 consecutive lanes take the 8
// chunks of one row, so a warp reads 4 full 128-byte row segments. Otherwise consecutive lanes take
// consecutive rows. Either way a quarter warp's 16-byte shared stores fall into distinct banks.
template <bool KC, int ROWS>
struct TileMap {
    static constexpr int P = ROWS / 32;
    __device__ __forceinline__ static void at(int t, int p, int &row, int &kc) {
        if (KC) { kc = t % 8; row = t / 8 + 32 * p; }
        else { row = t % ROWS; kc = t / ROWS + (CONV_THREADS / ROWS) * p; }
    }
};

__device__ __forceinline__ void split_store(uint8_t *hi_tile, uint8_t *lo_tile, uint32_t off, const float (&v)[4]) {
    float4 hi, lo;
    hi.x = __uint_as_float(__float_as_uint(v[0]) & 0xFFFFE000u); lo.x = v[0] - hi.x;
    hi.y = __uint_as_float(__float_as_uint(v[1]) & 0xFFFFE000u); lo.y = v[1] - hi.y;
    hi.z = __uint_as_float(__float_as_uint(v[2]) & 0xFFFFE000u); lo.z = v[2] - hi.z;
    hi.w = __uint_as_float(__float_as_uint(v[3]) & 0xFFFFE000u); lo.w = v[3] - hi.w;
    *reinterpret_cast<float4 *>(hi_tile + off) = hi;
    *reinterpret_cast<float4 *>(lo_tile + off) = lo;
}

// F: M, N, K, NB, ALPHA; a4(m, k, b, v[4]) / b4(k, n, b, v[4]) give 4 consecutive k; epi(m, n, b, acc).
// AK / BKC: operand is contiguous along k. SPLIT > 1: blockIdx.y % SPLIT picks a k range and the raw
// tile goes to `partial`. Requires F::K % 4 == 0.
template <class F, bool AK, bool BKC, int BN, int SPLIT>
__device__ __forceinline__ void gemm_tc_tile(const F &f, float *__restrict__ partial, uint32_t *status) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int M = F::M, N = F::N, K = F::K;
    constexpr int TILES_N = (N + BN - 1) / BN;
    constexpr uint32_t LBO_A = lbo_bytes(BM), LBO_B = lbo_bytes(BN);
    constexpr uint32_t TA = tile_bytes(BM), TB = tile_bytes(BN), STAGE = stage_bytes(BN);
    constexpr int KCH = ((K + SPLIT - 1) / SPLIT + BK - 1) / BK * BK;          // k range of one split
    constexpr int NST = ss_stages(BN);
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const int tile_m = blockIdx.x / TILES_N, tile_n = blockIdx.x % TILES_N;
    const int bt = SPLIT > 1 ? blockIdx.y / SPLIT : blockIdx.y;
    const int sp = SPLIT > 1 ? blockIdx.y % SPLIT : 0;
    const int m0 = tile_m * BM, n0 = tile_n * BN;
    const int k_begin = sp * KCH, k_end = min(K, k_begin + KCH);
    const int nkb = k_end > k_begin ? (k_end - k_begin + BK - 1) / BK : 0;

    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + NST * STAGE);         // full[3], empty[3], accum
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + NST * STAGE + 64);
    volatile uint32_t *failed = reinterpret_cast<volatile uint32_t *>(smem + NST * STAGE + 72);
    const uint32_t bar0 = smem_u32(bars);
    auto full = [&](int s) { return bar0 + 8u * s; };
    auto empty = [&](int s) { return bar0 + 8u * (NST + s); };
    const uint32_t accum = bar0 + 8u * (2 * NST);

    if (t == 0) {
        for (int s = 0; s < NST; s++) { mbar_init(full(s), CONV_THREADS); mbar_init(empty(s), 1); }
        mbar_init(accum, 1);
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == MMA_WARP) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)(2 * BN)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;

    if (warp < MMA_WARP) {
        // ---------------------------------------------------------------- converters
        // Groups of 8 warps take k blocks in turn, so one group's global loads are in flight while
        // the others convert and store.
        const int grp = warp >> 3;
        const int t = threadIdx.x & (CONV_THREADS - 1);
        float va[BM / 32][4], vb[BN / 32][4];
        auto fetch = [&](int k0) {
#pragma unroll
            for (int p = 0; p < BM / 32; p++) {
                int row, kc;
                TileMap<AK, BM>::at(t, p, row, kc);
                const int m = m0 + row, k = k0 + kc * 4;
                if (m < M && k < k_end) f.a4(m, k, bt, va[p]);
                else { va[p][0] = va[p][1] = va[p][2] = va[p][3] = 0.0f; }
            }
#pragma unroll
            for (int p = 0; p < BN / 32; p++) {
                int row, kc;
                TileMap<BKC, BN>::at(t, p, row, kc);
                const int n = n0 + row, k = k0 + kc * 4;
                if (n < N && k < k_end) f.b4(k, n, bt, vb[p]);
                else { vb[p][0] = vb[p][1] = vb[p][2] = vb[p][3] = 0.0f; }
            }
        };
        if (grp < nkb) fetch(k_begin + grp * BK);
        for (int kb = grp; kb < nkb; kb += CONV_GROUPS) {
            const int s = kb % NST;
            const uint32_t ph = (kb / NST) & 1;
            if (!mbar_wait(empty(s), ph ^ 1)) { *failed = 1; break; }
            uint8_t *st = smem + s * STAGE;
#pragma unroll
            for (int p = 0; p < BM / 32; p++) {
                int row, kc;
                TileMap<AK, BM>::at(t, p, row, kc);
                split_store(st, st + TA, kc * LBO_A + row * 16, va[p]);
            }
#pragma unroll
            for (int p = 0; p < BN / 32; p++) {
                int row, kc;
                TileMap<BKC, BN>::at(t, p, row, kc);
                split_store(st + 2 * TA, st + 2 * TA + TB, kc * LBO_B + row * 16, vb[p]);
            }
            if (kb + CONV_GROUPS < nkb) fetch(k_begin + (kb + CONV_GROUPS) * BK);   // this group's next block: loads fly during the wait
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(full(s));
        }
    } else if (lane == 0) {
        // ---------------------------------------------------------------- MMA issuer
        constexpr uint32_t IDESC = instr_desc(BM, BN);
        const uint32_t base = smem_u32(smem);
        for (int kb = 0; kb < nkb; kb++) {
            const int s = kb % NST;
            const uint32_t ph = (kb / NST) & 1;
            if (!mbar_wait(full(s), ph)) { *failed = 1; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a_hi = base + s * STAGE, a_lo = a_hi + TA, b_hi = a_hi + 2 * TA, b_lo = b_hi + TB;
#pragma unroll
            for (int j = 0; j < BK / 8; j++) {
                const uint64_t dah = smem_desc(a_hi + 2 * j * LBO_A, LBO_A), dal = smem_desc(a_lo + 2 * j * LBO_A, LBO_A);
                const uint64_t dbh = smem_desc(b_hi + 2 * j * LBO_B, LBO_B), dbl = smem_desc(b_lo + 2 * j * LBO_B, LBO_B);
                // The accumulator rounds toward zero on every accumulate, at the ulp of the running sum.
                // The two correction products are ~2^-11 of the main one: they get an accumulator of
                // their own (columns BN .. 2BN-1), so the main sum is rounded once per k-step, not thrice.
                mma_tf32(tmem + BN, dah, dbl, IDESC, (kb | j) ? 1u : 0u);
                mma_tf32(tmem + BN, dal, dbh, IDESC, 1u);
                mma_tf32(tmem, dah, dbh, IDESC, (kb | j) ? 1u : 0u);
            }
            mma_commit(empty(s));
        }
        mma_commit(accum);
    }

    // ---------------------------------------------------------------- epilogue
    if (warp < MMA_WARP) {
        const bool ok = nkb == 0 || (!*failed && mbar_wait(accum, 0));
        if (!ok) *failed = 1;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        float *stage_f = reinterpret_cast<float *>(smem) + warp * (32 * 33);    // this warp's 32 x 32 transpose block
        const int q = warp & 3;                                                  // TMEM lanes 32q .. 32q + 31
        constexpr int CHUNKS = BN / 32;
        for (int c = warp >> 2; c < CHUNKS; c += MMA_WARP / 4) {
            uint32_t r[32], r2[32];
            if (ok && nkb > 0) {
                tmem_ld32(tmem + ((uint32_t)(32 * q) << 16) + (uint32_t)(32 * c), r);
                tmem_ld32(tmem + ((uint32_t)(32 * q) << 16) + (uint32_t)(BN + 32 * c), r2);
            } else {
#pragma unroll
                for (int i = 0; i < 32; i++) r[i] = r2[i] = 0u;
            }
#pragma unroll
            for (int i = 0; i < 32; i++) stage_f[lane * 33 + i] = __uint_as_float(r[i]) + __uint_as_float(r2[i]);
            __syncwarp();
            const int n = n0 + 32 * c + lane;
#pragma unroll 4
            for (int rr = 0; rr < 32; rr++) {
                const int m = m0 + 32 * q + rr;
                const float v = stage_f[rr * 33 + lane];
                if (m < M && n < N) {
                    if (SPLIT > 1) partial[(((long)bt * SPLIT + sp) * M + m) * N + n] = v;
                    else f.epi(m, n, bt, v * F::ALPHA);
                }
            }
            __syncwarp();
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == MMA_WARP) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)(2 * BN)) : "memory");
    }
    if (t == 0 && *failed) atomicExch(status, TIMEOUT);
}


// ---------------------------------------------------------------------------- A operand in tensor memory
// The same product with the A tiles kept in TMEM instead of shared memory. A kind::tf32 MMA of
// 128 x 128 x 8 reads 4 KB of A and 4 KB of B; with both in shared memory the three MMAs per k-step
// plus the converters' own stores ask for more than the 128 B/clk a shared memory delivers, and the
// tensor pipe waits. Converter threads hold A values in registers anyway (lane = row), so they write
// hi and lo straight into TMEM with tcgen05.st (lane = row, column = k) and the MMA takes A from
// there; shared memory then carries B only.
//
// TMEM columns (512 allocated): [0, BN) main accumulator, [BN, 2BN) correction accumulator,
// then per stage 64 columns: A hi (32 k) and A lo (32 k).
constexpr int TS_STAGES = 4;
__host__ __device__ constexpr uint32_t ts_stage_bytes(int bn) { return 2 * tile_bytes(bn); }
// At least 116 KB, so that two CTAs never share an SM: each allocates all 512 TMEM columns.
__host__ __device__ constexpr uint32_t ts_smem_bytes(int bn) {
    return (TS_STAGES * ts_stage_bytes(bn) > 116u * 1024u ? TS_STAGES * ts_stage_bytes(bn) : 116u * 1024u) + 256;
}

__device__ __forceinline__ void mma_tf32_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "r"(a_tmem), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
                 "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}

template <class F, bool BKC, int BN, int SPLIT>
__device__ __forceinline__ void gemm_tc_ts_tile(const F &f, float *__restrict__ partial, uint32_t *status) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int M = F::M, N = F::N, K = F::K;
    constexpr int TILES_N = (N + BN - 1) / BN;
    constexpr uint32_t LBO_B = lbo_bytes(BN), TB = tile_bytes(BN), STAGE = ts_stage_bytes(BN);
    constexpr uint32_t BAR_OFF = ts_smem_bytes(BN) - 256;
    constexpr int KCH = ((K + SPLIT - 1) / SPLIT + BK - 1) / BK * BK;
    constexpr uint32_t A_COLS = 2 * BN;                       // first TMEM column of the A stages
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tile_m = blockIdx.x / TILES_N, tile_n = blockIdx.x % TILES_N;
    const int bt = SPLIT > 1 ? blockIdx.y / SPLIT : blockIdx.y;
    const int sp = SPLIT > 1 ? blockIdx.y % SPLIT : 0;
    const int m0 = tile_m * BM, n0 = tile_n * BN;
    const int k_begin = sp * KCH, k_end = min(K, k_begin + KCH);
    const int nkb = k_end > k_begin ? (k_end - k_begin + BK - 1) / BK : 0;

    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + BAR_OFF);               // full[4], empty[4], accum
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + BAR_OFF + 96);
    volatile uint32_t *failed = reinterpret_cast<volatile uint32_t *>(smem + BAR_OFF + 104);
    const uint32_t bar0 = smem_u32(bars);
    auto full = [&](int s) { return bar0 + 8u * s; };
    auto empty = [&](int s) { return bar0 + 8u * (TS_STAGES + s); };
    const uint32_t accum = bar0 + 8u * (2 * TS_STAGES);

    if (tid == 0) {
        for (int s = 0; s < TS_STAGES; s++) { mbar_init(full(s), CONV_THREADS); mbar_init(empty(s), 1); }
        mbar_init(accum, 1);
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == MMA_WARP) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;

    if (warp < MMA_WARP) {
        // ---------------------------------------------------------------- converters
        const int grp = warp >> 3, wi = warp & 7;
        const int t = tid & (CONV_THREADS - 1);
        const int q = wi & 3, half = wi >> 2;                 // A: TMEM lanes 32q.., k 16*half .. 16*half + 15
        const int am = m0 + 32 * q + lane;
        float va[4][4], vb[BN / 32][4];
        auto fetch = [&](int k0) {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int k = k0 + 16 * half + 4 * i;
                if (am < M && k < k_end) f.a4(am, k, bt, va[i]);
                else { va[i][0] = va[i][1] = va[i][2] = va[i][3] = 0.0f; }
            }
#pragma unroll
            for (int p = 0; p < BN / 32; p++) {
                int row, kc;
                TileMap<BKC, BN>::at(t, p, row, kc);
                const int n = n0 + row, k = k0 + kc * 4;
                if (n < N && k < k_end) f.b4(k, n, bt, vb[p]);
                else { vb[p][0] = vb[p][1] = vb[p][2] = vb[p][3] = 0.0f; }
            }
        };
        if (grp < nkb) fetch(k_begin + grp * BK);
        for (int kb = grp; kb < nkb; kb += CONV_GROUPS) {
            const int s = kb % TS_STAGES;
            const uint32_t ph = (kb / TS_STAGES) & 1;
            if (!mbar_wait(empty(s), ph ^ 1)) { *failed = 1; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t hi[16], lo[16];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const uint32_t h = __float_as_uint(va[i][e]) & 0xFFFFE000u;
                    hi[4 * i + e] = h;
                    lo[4 * i + e] = __float_as_uint(va[i][e] - __uint_as_float(h));
                }
            const uint32_t a_base = tmem + ((uint32_t)(32 * q) << 16) + A_COLS + 64u * s + 16u * half;
            tmem_st16(a_base, hi);
            tmem_st16(a_base + 32u, lo);
            uint8_t *st = smem + s * STAGE;
#pragma unroll
            for (int p = 0; p < BN / 32; p++) {
                int row, kc;
                TileMap<BKC, BN>::at(t, p, row, kc);
                split_store(st, st + TB, kc * LBO_B + row * 16, vb[p]);
            }
            if (kb + CONV_GROUPS < nkb) fetch(k_begin + (kb + CONV_GROUPS) * BK);
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(full(s));
        }
    } else if (lane == 0) {
        // ---------------------------------------------------------------- MMA issuer
        constexpr uint32_t IDESC = instr_desc(BM, BN);
        const uint32_t base = smem_u32(smem);
        for (int kb = 0; kb < nkb; kb++) {
            const int s = kb % TS_STAGES;
            const uint32_t ph = (kb / TS_STAGES) & 1;
            if (!mbar_wait(full(s), ph)) { *failed = 1; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t b_hi = base + s * STAGE, b_lo = b_hi + TB;
            const uint32_t a_hi = tmem + A_COLS + 64u * s, a_lo = a_hi + 32u;
#pragma unroll
            for (int j = 0; j < BK / 8; j++) {
                const uint64_t dbh = smem_desc(b_hi + 2 * j * LBO_B, LBO_B), dbl = smem_desc(b_lo + 2 * j * LBO_B, LBO_B);
                mma_tf32_ts(tmem + BN, a_hi + 8u * j, dbl, IDESC, (kb | j) ? 1u : 0u);
                mma_tf32_ts(tmem + BN, a_lo + 8u * j, dbh, IDESC, 1u);
                mma_tf32_ts(tmem, a_hi + 8u * j, dbh, IDESC, (kb | j) ? 1u : 0u);
            }
            mma_commit(empty(s));
        }
        mma_commit(accum);
    }

    // ---------------------------------------------------------------- epilogue
    if (warp < MMA_WARP) {
        const bool ok = nkb == 0 || (!*failed && mbar_wait(accum, 0));
        if (!ok) *failed = 1;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        float *stage_f = reinterpret_cast<float *>(smem) + warp * (32 * 33);
        const int q = warp & 3;
        constexpr int CHUNKS = BN / 32;
        for (int c = warp >> 2; c < CHUNKS; c += MMA_WARP / 4) {
            uint32_t r[32], r2[32];
            if (ok && nkb > 0) {
                tmem_ld32(tmem + ((uint32_t)(32 * q) << 16) + (uint32_t)(32 * c), r);
                tmem_ld32(tmem + ((uint32_t)(32 * q) << 16) + (uint32_t)(BN + 32 * c), r2);
            } else {
#pragma unroll
                for (int i = 0; i < 32; i++) r[i] = r2[i] = 0u;
            }
#pragma unroll
            for (int i = 0; i < 32; i++) stage_f[lane * 33 + i] = __uint_as_float(r[i]) + __uint_as_float(r2[i]);
            __syncwarp();
            const int n = n0 + 32 * c + lane;
#pragma unroll 4
            for (int rr = 0; rr < 32; rr++) {
                const int m = m0 + 32 * q + rr;
                const float v = stage_f[rr * 33 + lane];
                if (m < M && n < N) {
                    if (SPLIT > 1) partial[(((long)bt * SPLIT + sp) * M + m) * N + n] = v;
                    else f.epi(m, n, bt, v * F::ALPHA);
                }
            }
            __syncwarp();
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == MMA_WARP) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
    if (tid == 0 && *failed) atomicExch(status, TIMEOUT);
}


// ---------------------------------------------------------------------------- two CTAs per SM
// The shared-memory variant again, sized so that TWO CTAs fit on an SM (16-wide k blocks, three stages
// of 32.5 KB, 2 x 128 TMEM columns, 288 threads): while one CTA runs its epilogue, or waits for its
// first loads, the other one keeps the tensor pipe busy. With one CTA per SM nothing overlaps a
// tile's prologue and epilogue, which costs a fifth of the time of a K = 512 product and most of the
// time of the K = 64 attention products.
constexpr int BK2 = 16, ST2 = 3, MMA_WARP2 = 8, THREADS2 = 288;
__host__ __device__ constexpr uint32_t lbo2_bytes(int rows) { return (uint32_t)rows * 16u + 32u; }   // +32: 4 k-chunks x 2 rows per quarter warp
__host__ __device__ constexpr uint32_t tile2_bytes(int rows) { return (BK2 / 4) * lbo2_bytes(rows); }
__host__ __device__ constexpr uint32_t stage2_bytes(int bn) { return 2 * tile2_bytes(BM) + 2 * tile2_bytes(bn); }
__host__ __device__ constexpr uint32_t smem2_bytes(int bn) {
    return (ST2 * stage2_bytes(bn) > 8u * 32u * 33u * 4u ? ST2 * stage2_bytes(bn) : 8u * 32u * 33u * 4u) + 256;
}

template <bool KC, int ROWS>
struct TileMap2 {                                   // ROWS x 16 values = ROWS / 64 chunks of 4 per thread
    __device__ __forceinline__ static void at(int t, int p, int &row, int &kc) {
        if (KC) { kc = t % 4; row = t / 4 + 64 * p; }
        else { row = t % ROWS; kc = t / ROWS + (CONV_THREADS / ROWS) * p; }
    }
};

template <class F, bool AK, bool BKC, int BN, int SPLIT>
__device__ __forceinline__ void gemm_tc2_tile(const F &f, float *__restrict__ partial, uint32_t *status) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int M = F::M, N = F::N, K = F::K;
    constexpr int TILES_N = (N + BN - 1) / BN;
    constexpr uint32_t LBO_A = lbo2_bytes(BM), LBO_B = lbo2_bytes(BN);
    constexpr uint32_t TA = tile2_bytes(BM), TB = tile2_bytes(BN), STAGE = stage2_bytes(BN);
    constexpr uint32_t BAR_OFF = smem2_bytes(BN) - 256;
    constexpr int KCH = ((K + SPLIT - 1) / SPLIT + BK2 - 1) / BK2 * BK2;
    constexpr int PA = BM / 64, PB = BN / 64;
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const int tile_m = blockIdx.x / TILES_N, tile_n = blockIdx.x % TILES_N;
    const int bt = SPLIT > 1 ? blockIdx.y / SPLIT : blockIdx.y;
    const int sp = SPLIT > 1 ? blockIdx.y % SPLIT : 0;
    const int m0 = tile_m * BM, n0 = tile_n * BN;
    const int k_begin = sp * KCH, k_end = min(K, k_begin + KCH);
    const int nkb = k_end > k_begin ? (k_end - k_begin + BK2 - 1) / BK2 : 0;

    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + BAR_OFF);                // full[3], empty[3], accum
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + BAR_OFF + 64);
    volatile uint32_t *failed = reinterpret_cast<volatile uint32_t *>(smem + BAR_OFF + 72);
    const uint32_t bar0 = smem_u32(bars);
    auto full = [&](int s) { return bar0 + 8u * s; };
    auto empty = [&](int s) { return bar0 + 8u * (ST2 + s); };
    const uint32_t accum = bar0 + 8u * (2 * ST2);

    if (t == 0) {
        for (int s = 0; s < ST2; s++) { mbar_init(full(s), CONV_THREADS); mbar_init(empty(s), 1); }
        mbar_init(accum, 1);
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == MMA_WARP2) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)(2 * BN)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;

    if (warp < MMA_WARP2) {
        // ---------------------------------------------------------------- converters (one group, prefetch one block ahead)
        float va[PA][4], vb[PB][4];
        auto fetch = [&](int k0) {
#pragma unroll
            for (int p = 0; p < PA; p++) {
                int row, kc;
                TileMap2<AK, BM>::at(t, p, row, kc);
                const int m = m0 + row, k = k0 + kc * 4;
                if (m < M && k < k_end) f.a4(m, k, bt, va[p]);
                else { va[p][0] = va[p][1] = va[p][2] = va[p][3] = 0.0f; }
            }
#pragma unroll
            for (int p = 0; p < PB; p++) {
                int row, kc;
                TileMap2<BKC, BN>::at(t, p, row, kc);
                const int n = n0 + row, k = k0 + kc * 4;
                if (n < N && k < k_end) f.b4(k, n, bt, vb[p]);
                else { vb[p][0] = vb[p][1] = vb[p][2] = vb[p][3] = 0.0f; }
            }
        };
        if (nkb > 0) fetch(k_begin);
        for (int kb = 0; kb < nkb; kb++) {
            const int s = kb % ST2;
            const uint32_t ph = (kb / ST2) & 1;
            if (!mbar_wait(empty(s), ph ^ 1)) { *failed = 1; break; }
            uint8_t *st = smem + s * STAGE;
#pragma unroll
            for (int p = 0; p < PA; p++) {
                int row, kc;
                TileMap2<AK, BM>::at(t, p, row, kc);
                split_store(st, st + TA, kc * LBO_A + row * 16, va[p]);
            }
#pragma unroll
            for (int p = 0; p < PB; p++) {
                int row, kc;
                TileMap2<BKC, BN>::at(t, p, row, kc);
                split_store(st + 2 * TA, st + 2 * TA + TB, kc * LBO_B + row * 16, vb[p]);
            }
            if (kb + 1 < nkb) fetch(k_begin + (kb + 1) * BK2);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(full(s));
        }
    } else if (lane == 0) {
        // ---------------------------------------------------------------- MMA issuer
        constexpr uint32_t IDESC = instr_desc(BM, BN);
        const uint32_t base = smem_u32(smem);
        for (int kb = 0; kb < nkb; kb++) {
            const int s = kb % ST2;
            const uint32_t ph = (kb / ST2) & 1;
            if (!mbar_wait(full(s), ph)) { *failed = 1; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a_hi = base + s * STAGE, a_lo = a_hi + TA, b_hi = a_hi + 2 * TA, b_lo = b_hi + TB;
#pragma unroll
            for (int j = 0; j < BK2 / 8; j++) {
                const uint64_t dah = smem_desc(a_hi + 2 * j * LBO_A, LBO_A), dal = smem_desc(a_lo + 2 * j * LBO_A, LBO_A);
                const uint64_t dbh = smem_desc(b_hi + 2 * j * LBO_B, LBO_B), dbl = smem_desc(b_lo + 2 * j * LBO_B, LBO_B);
                mma_tf32(tmem + BN, dah, dbl, IDESC, (kb | j) ? 1u : 0u);
                mma_tf32(tmem + BN, dal, dbh, IDESC, 1u);
                mma_tf32(tmem, dah, dbh, IDESC, (kb | j) ? 1u : 0u);
            }
            mma_commit(empty(s));
        }
        mma_commit(accum);
    }

    // ---------------------------------------------------------------- epilogue
    if (warp < MMA_WARP2) {
        const bool ok = nkb == 0 || (!*failed && mbar_wait(accum, 0));
        if (!ok) *failed = 1;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        float *stage_f = reinterpret_cast<float *>(smem) + warp * (32 * 33);
        const int q = warp & 3;
        constexpr int CHUNKS = BN / 32;
        for (int c = warp >> 2; c < CHUNKS; c += MMA_WARP2 / 4) {
            uint32_t r[32], r2[32];
            if (ok && nkb > 0) {
                tmem_ld32(tmem + ((uint32_t)(32 * q) << 16) + (uint32_t)(32 * c), r);
                tmem_ld32(tmem + ((uint32_t)(32 * q) << 16) + (uint32_t)(BN + 32 * c), r2);
            } else {
#pragma unroll
                for (int i = 0; i < 32; i++) r[i] = r2[i] = 0u;
            }
#pragma unroll
            for (int i = 0; i < 32; i++) stage_f[lane * 33 + i] = __uint_as_float(r[i]) + __uint_as_float(r2[i]);
            __syncwarp();
            const int n = n0 + 32 * c + lane;
#pragma unroll 4
            for (int rr = 0; rr < 32; rr++) {
                const int m = m0 + 32 * q + rr;
                const float v = stage_f[rr * 33 + lane];
                if (m < M && n < N) {
                    if (SPLIT > 1) partial[(((long)bt * SPLIT + sp) * M + m) * N + n] = v;
                    else f.epi(m, n, bt, v * F::ALPHA);
                }
            }
            __syncwarp();
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == MMA_WARP2) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)(2 * BN)) : "memory");
    }
    if (t == 0 && *failed) atomicExch(status, TIMEOUT);
}


// ---------------------------------------------------------------------------- CTA pairs (cta_group::2)
// A 128 x 128 x 8 kind::tf32 MMA takes ~39 ns and reads 8 KB of shared memory: with the converters'
// own stores a single CTA asks its shared memory for more than 128 B/clk, and the tensor pipe idles
// half of the time. Two CTAs of a cluster therefore share one 256 x BN tile: CTA r converts A rows
// 128 r .. 128 r + 127 and B rows (n) r BN/2 .. r BN/2 + BN/2 - 1 into its own shared memory, and ONE thread of
// CTA 0 issues tcgen05.mma.cta_group::2 (M = 256, N = BN): both tensor cores run, each reads its
// own A and both halves of B, and each keeps its 128 accumulator rows in its own TMEM. Per flop
// the shared-memory traffic is half that of the single-CTA tile.
//   full[s]   lives in CTA 0; one arrival per converter warp of BOTH CTAs (the peer's arrive through
//             the cluster window, release.cluster after the generic->async proxy fence)
//   empty[s], accum: one copy per CTA, flipped by tcgen05.commit.cta_group::2 multicast to both.
// Each CTA allocates its tensor memory itself (cta_group::1, same column count, one CTA per SM, so
// both get the same base; the kernel checks that and reports TIMEOUT status if not).
// Every mbarrier wait is clock-bounded as above; the two cluster barriers are reached by all
// threads because no loop before them is unbounded.
__host__ __device__ constexpr uint32_t pair_stage_bytes(int bn) { return 2 * tile_bytes(BM) + 2 * tile_bytes(bn / 2); }
__host__ __device__ constexpr uint32_t pair_smem_bytes(int bn) {
    return (STAGES * pair_stage_bytes(bn) > 116u * 1024u ? STAGES * pair_stage_bytes(bn) : 116u * 1024u) + 256;
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity) {
    const long long t0 = clock64();
    while (true) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if (clock64() - t0 > (1LL << 31)) return false;
    }
}
__device__ __forceinline__ void mma_tf32_pair(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives on the mbarrier at this shared-memory offset in both CTAs of the pair once all MMAs issued so far are done.
__device__ __forceinline__ void mma_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((uint16_t)3) : "memory");
}

// ---- TMA (cp.async.bulk.tensor) for operands that are plain row-major matrices read along k
// A 2-d tensor map {k, rows} with a box of {4 floats, R rows} brings one 16-byte column of R rows — exactly one k-chunk
// of the K-major no-swizzle operand layout, rows 16 bytes apart. Eight such copies fill a 32-wide k block. The raw f32
// words ARE the hi operand: a kind::tf32 MMA reads the upper 19 bits of each word and ignores the low 13 mantissa bits,
// which is the truncation the converters otherwise do by hand; they then only read the tile back and write lo = x - hi.
// No cluster multicast: each CTA of a pair loads its own rows into its own shared memory.
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void *tmap, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(tmap), "r"(x), "r"(y), "r"(bar) : "memory");
}
// lo = x - trunc_tf32(x) for a ROWS x 32 tile the TMA wrote densely (k-chunk c at c * ROWS * 16); lo goes to the padded layout
template <int ROWS>
__device__ __forceinline__ void lo_from_raw_tile(const uint8_t *hi_tile, uint8_t *lo_tile, uint32_t lbo, int t) {
#pragma unroll
    for (int p = 0; p < ROWS / 32; p++) {
        const int row = t % ROWS, kc = t / ROWS + (CONV_THREADS / ROWS) * p;        // consecutive lanes on consecutive rows: no bank conflicts
        const float4 x = *reinterpret_cast<const float4 *>(hi_tile + kc * (ROWS * 16) + row * 16);
        float4 lo;
        lo.x = x.x - __uint_as_float(__float_as_uint(x.x) & 0xFFFFE000u);
        lo.y = x.y - __uint_as_float(__float_as_uint(x.y) & 0xFFFFE000u);
        lo.z = x.z - __uint_as_float(__float_as_uint(x.z) & 0xFFFFE000u);
        lo.w = x.w - __uint_as_float(__float_as_uint(x.w) & 0xFFFFE000u);
        *reinterpret_cast<float4 *>(lo_tile + kc * lbo + row * 16) = lo;
    }
}

// Launched with cluster dimensions (2, 1, 1): blockIdx.x >> 1 is the tile, %cluster_ctarank the half.
template <class F, bool AK, bool BKC, int BN, int SPLIT>
__device__ __forceinline__ void gemm_tc_pair_tile(const F &f, float *__restrict__ partial, uint32_t *status) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int M = F::M, N = F::N, K = F::K;
    constexpr int BH = BN / 2;                                                   // B rows converted by one CTA
    constexpr int TILES_N = (N + BN - 1) / BN;
    constexpr uint32_t LBO_A = lbo_bytes(BM), LBO_B = lbo_bytes(BH);
    constexpr uint32_t TA = tile_bytes(BM), TB = tile_bytes(BH), STAGE = pair_stage_bytes(BN);
    constexpr uint32_t BAR_OFF = pair_smem_bytes(BN) - 256;
    constexpr int KCH = ((K + SPLIT - 1) / SPLIT + BK - 1) / BK * BK;
    constexpr int NST = STAGES;
    constexpr uint32_t FULL_ARRIVALS = 2 * (CONV_THREADS / 32);
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const uint32_t rank = cluster_ctarank();
    const int cid = blockIdx.x >> 1;
    const int tile_m = cid / TILES_N, tile_n = cid % TILES_N;
    const int bt = SPLIT > 1 ? blockIdx.y / SPLIT : blockIdx.y;
    const int sp = SPLIT > 1 ? blockIdx.y % SPLIT : 0;
    const int m0 = tile_m * (2 * BM) + (int)rank * BM;                           // this CTA's accumulator rows
    const int n0 = tile_n * BN;
    const int nb0 = n0 + (int)rank * BH;                                         // this CTA's B rows
    const int k_begin = sp * KCH, k_end = min(K, k_begin + KCH);
    const int nkb = k_end > k_begin ? (k_end - k_begin + BK - 1) / BK : 0;

    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + BAR_OFF);               // full[3], empty[3], accum
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + BAR_OFF + 64);
    volatile uint32_t *failed = reinterpret_cast<volatile uint32_t *>(smem + BAR_OFF + 72);
    const uint32_t bar0 = smem_u32(bars);
    auto full = [&](int s) { return bar0 + 8u * s; };
    auto empty = [&](int s) { return bar0 + 8u * (NST + s); };
    const uint32_t accum = bar0 + 8u * (2 * NST);

    if (t == 0) {
        for (int s = 0; s < NST; s++) { mbar_init(full(s), FULL_ARRIVALS); mbar_init(empty(s), 1); }
        mbar_init(accum, 1);
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == MMA_WARP) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)(2 * BN)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync();                                                              // both CTAs' barriers and TMEM exist
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;

    if (warp < MMA_WARP) {
        // ---------------------------------------------------------------- converters
        const int grp = warp >> 3;
        const int tc = threadIdx.x & (CONV_THREADS - 1);
        float va[BM / 32][4], vb[BH / 32][4];
        auto fetch = [&](int k0) {
#pragma unroll
            for (int p = 0; p < BM / 32; p++) {
                int row, kc;
                TileMap<AK, BM>::at(tc, p, row, kc);
                const int m = m0 + row, k = k0 + kc * 4;
                if (m < M && k < k_end) f.a4(m, k, bt, va[p]);
                else { va[p][0] = va[p][1] = va[p][2] = va[p][3] = 0.0f; }
            }
#pragma unroll
            for (int p = 0; p < BH / 32; p++) {
                int row, kc;
                TileMap<BKC, BH>::at(tc, p, row, kc);
                const int n = nb0 + row, k = k0 + kc * 4;
                if (n < N && k < k_end) f.b4(k, n, bt, vb[p]);
                else { vb[p][0] = vb[p][1] = vb[p][2] = vb[p][3] = 0.0f; }
            }
        };
        const uint32_t full_leader0 = map_to_cta(full(0), 0);
        if (grp < nkb) fetch(k_begin + grp * BK);
        for (int kb = grp; kb < nkb; kb += CONV_GROUPS) {
            const int s = kb % NST;
            const uint32_t ph = (kb / NST) & 1;
            if (!mbar_wait(empty(s), ph ^ 1)) { *failed = 1; break; }
            uint8_t *st = smem + s * STAGE;
#pragma unroll
            for (int p = 0; p < BM / 32; p++) {
                int row, kc;
                TileMap<AK, BM>::at(tc, p, row, kc);
                split_store(st, st + TA, kc * LBO_A + row * 16, va[p]);
            }
#pragma unroll
            for (int p = 0; p < BH / 32; p++) {
                int row, kc;
                TileMap<BKC, BH>::at(tc, p, row, kc);
                split_store(st + 2 * TA, st + 2 * TA + TB, kc * LBO_B + row * 16, vb[p]);
            }
            if (kb + CONV_GROUPS < nkb) fetch(k_begin + (kb + CONV_GROUPS) * BK);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(full_leader0 + 8u * s);
        }
    } else if (lane == 0 && rank == 0) {
        // ---------------------------------------------------------------- MMA issuer (CTA 0 of the pair only)
        constexpr uint32_t IDESC = instr_desc(2 * BM, BN);
        const uint32_t base = smem_u32(smem);
        uint32_t peer_tmem;
        asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(peer_tmem) : "r"(map_to_cta(smem_u32(tmem_slot), 1)) : "memory");
        if (peer_tmem != tmem) *failed = 1;
        for (int kb = 0; kb < nkb && !*failed; kb++) {
            const int s = kb % NST;
            const uint32_t ph = (kb / NST) & 1;
            if (!mbar_wait_cluster(full(s), ph)) { *failed = 1; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a_hi = base + s * STAGE, a_lo = a_hi + TA, b_hi = a_hi + 2 * TA, b_lo = b_hi + TB;
#pragma unroll
            for (int j = 0; j < BK / 8; j++) {
                const uint64_t dah = smem_desc(a_hi + 2 * j * LBO_A, LBO_A), dal = smem_desc(a_lo + 2 * j * LBO_A, LBO_A);
                const uint64_t dbh = smem_desc(b_hi + 2 * j * LBO_B, LBO_B), dbl = smem_desc(b_lo + 2 * j * LBO_B, LBO_B);
                mma_tf32_pair(tmem + BN, dah, dbl, IDESC, (kb | j) ? 1u : 0u);
                mma_tf32_pair(tmem + BN, dal, dbh, IDESC, 1u);
                mma_tf32_pair(tmem, dah, dbh, IDESC, (kb | j) ? 1u : 0u);
            }
            mma_commit_pair(empty(s));
        }
        mma_commit_pair(accum);
    }

    // ---------------------------------------------------------------- epilogue: 128 rows x BN columns per CTA
    if (warp < MMA_WARP) {
        const bool ok = nkb == 0 || (!*failed && mbar_wait(accum, 0));
        if (!ok) *failed = 1;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        float *stage_f = reinterpret_cast<float *>(smem) + warp * (32 * 33);
        const int q = warp & 3;
        constexpr int CHUNKS = BN / 32;
        for (int c = warp >> 2; c < CHUNKS; c += MMA_WARP / 4) {
            uint32_t r[32], r2[32];
            if (ok && nkb > 0) {
                tmem_ld32(tmem + ((uint32_t)(32 * q) << 16) + (uint32_t)(32 * c), r);
                tmem_ld32(tmem + ((uint32_t)(32 * q) << 16) + (uint32_t)(BN + 32 * c), r2);
            } else {
#pragma unroll
                for (int i = 0; i < 32; i++) r[i] = r2[i] = 0u;
            }
#pragma unroll
            for (int i = 0; i < 32; i++) stage_f[lane * 33 + i] = __uint_as_float(r[i]) + __uint_as_float(r2[i]);
            __syncwarp();
            const int n = n0 + 32 * c + lane;
#pragma unroll 4
            for (int rr = 0; rr < 32; rr++) {
                const int m = m0 + 32 * q + rr;
                const float v = stage_f[rr * 33 + lane];
                if (m < M && n < N) {
                    if (SPLIT > 1) partial[(((long)bt * SPLIT + sp) * M + m) * N + n] = v;
                    else f.epi(m, n, bt, v * F::ALPHA);
                }
            }
            __syncwarp();
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync();                                                              // nobody leaves while the peer may still touch this CTA's shared memory
    if (warp == MMA_WARP) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)(2 * BN)) : "memory");
    }
    if (t == 0 && *failed) atomicExch(status, TIMEOUT);
}


// ---------------------------------------------------------------------------- persistent CTA pairs
// Timeline of one 256 x 256 x 512 tile of the kernel above (globaltimer stamps, B200): 0.9 us set-up,
// 3.1 us until the first stage is full, 13.1 us main loop (the tensor pipe's own rate), 1.2 us until
// the accumulator is seen, 3.6 us epilogue (14.8 us when the epilogue reads what it adds to),
// 0.7 us exit — the tensor pipe works during 58 % of a tile's life. Here one cluster per SM pair stays
// resident and walks over the work items (tile, batch, k split) in a fixed round-robin order, with
// the three jobs on different warps so that they overlap across tiles:
//   warps 0-15  converters, two groups of eight, stage ring and block counter running on across tiles
//               (the next tile's first stages are filled while the current one is still being stored);
//   warps 16-23 epilogue: (TMEM lane quarter, column half) each, transposes in their own shared memory;
//   warp 24     MMA issuer (CTA 0) as above.
// ACCS = 2 keeps the correction accumulator (one TMEM buffer of 512 columns: the next tile's MMAs wait
// for the epilogue's loads, the converters do not). ACCS = 1 adds all three products into one accumulator,
// which costs three roundings toward zero per k-step instead of one (relative error ~7e-9 per unit of
// chain length) and is used for chains of at most 512; the 512 columns then hold two buffers and
// the epilogue of a tile runs under the main loop of the next.
//   tfull[b]  per CTA, flipped by the multicast commit after a tile's last MMA
//   tempty[b] in CTA 0, one arrival per epilogue warp of both CTAs once its tcgen05.ld are done.
constexpr int PP_CONV_GROUPS = 2, PP_EPI_WARPS = 8;
constexpr int PP_MMA_WARP = 8 * PP_CONV_GROUPS + PP_EPI_WARPS, PP_THREADS = 32 * PP_MMA_WARP + 32;
// A functor of several members side by side (products that share an operand or an output fused into one launch) names
// its member count as SEGS and offers every method as a template on the member index (a4s<S>, b4s<S>, ...). Which member
// a whole k block, a whole tile belongs to is looked up once (op_seg, epi_seg) and the loops below are instantiated per
// member: a run-time branch inside every operand fetch costs a quarter of the kernel's speed (measured: 208 -> 167
// TFLOP/s on 16384 x 512 x 1536 with three members).
template <class F, class = void> struct seg_count { static constexpr int value = 1; };
template <class F> struct seg_count<F, std::void_t<decltype(F::SEGS)>> { static constexpr int value = F::SEGS; };
template <int V> struct SegC { static constexpr int value = V; };
template <class F, class Fn> __device__ __forceinline__ void with_seg(int seg, Fn &&fn) {
    constexpr int NS = seg_count<F>::value;
    static_assert(NS >= 1 && NS <= 4, "one to four members");
    if constexpr (NS == 1) fn(SegC<0>{});
    else if constexpr (NS == 2) { if (seg == 0) fn(SegC<0>{}); else fn(SegC<1>{}); }
    else if constexpr (NS == 3) { if (seg == 0) fn(SegC<0>{}); else if (seg == 1) fn(SegC<1>{}); else fn(SegC<2>{}); }
    else { if (seg == 0) fn(SegC<0>{}); else if (seg == 1) fn(SegC<1>{}); else if (seg == 2) fn(SegC<2>{}); else fn(SegC<3>{}); }
}
template <class F> __device__ __forceinline__ int op_seg_of(const F &f, int k0, int n0) {
    if constexpr (seg_count<F>::value > 1) return f.op_seg(k0, n0); else return 0;
}
template <class F> __device__ __forceinline__ int epi_seg_of(const F &f, int n0) {
    if constexpr (seg_count<F>::value > 1) return f.epi_seg(n0); else return 0;
}
#define ANVIL_SEG_CALL(NAME, SIG, ARGS)                                                                              \
    template <int S, class F> __device__ __forceinline__ void f_##NAME SIG {                                          \
        if constexpr (seg_count<F>::value > 1) f.template NAME##s<S> ARGS; else f.NAME ARGS;                          \
    }
ANVIL_SEG_CALL(a4, (const F &f, int m, int k, int bt, float (&v)[4]), (m, k, bt, v))
ANVIL_SEG_CALL(b4, (const F &f, int k, int n, int bt, float (&v)[4]), (k, n, bt, v))
ANVIL_SEG_CALL(a_touch, (const F &f, int m, int k, int bt), (m, k, bt))
ANVIL_SEG_CALL(b_touch, (const F &f, int k, int n, int bt), (k, n, bt))
ANVIL_SEG_CALL(epi_touch, (const F &f, int m, int n, int bt), (m, n, bt))
ANVIL_SEG_CALL(epi_near, (const F &f, int m, int n, int bt), (m, n, bt))
template <int S, class F, int L> __device__ __forceinline__ void f_epi_loads(const F &f, int m, int n, int bt, float (&ld)[L]) {
    if constexpr (seg_count<F>::value > 1) f.template epi_loadss<S>(m, n, bt, ld); else f.epi_loads(m, n, bt, ld);
}
template <int S, class F, int L> __device__ __forceinline__ void f_epi2(const F &f, int m, int n, int bt, float acc, const float (&ld)[L]) {
    if constexpr (seg_count<F>::value > 1) f.template epi2s<S>(m, n, bt, acc, ld); else f.epi2(m, n, bt, acc, ld);
}
#undef ANVIL_SEG_CALL

constexpr int PP_AHEAD = 4;                                       // operand prefetch distance, in blocks of one converter group
constexpr int PP_SLOTS = 74;                                      // clusters resident at once: one per SM pair
__host__ __device__ constexpr uint32_t pp_smem_bytes(int bn = 256) {
    return (STAGES * pair_stage_bytes(bn) > 82u * 1024u ? STAGES * pair_stage_bytes(bn) : 82u * 1024u)   // one CTA per SM: each takes all of TMEM
           + PP_EPI_WARPS * 32 * 33 * 4 + 256;
}

// BN = 256, 128 or 64 columns per tile (narrow outputs: the attention products with a 64-wide head). With BN <= 128
// two accumulator pairs fit, so ACCS = 2 is double-buffered as well.
// TMA: bit 0 — the A operand comes by TMA through the tensor map `tma` ({K, M} f32, box {4, 128}); bit 1 — B through `tmb`
// ({K, N}, box {4, BN / 2}). Both need the operand to be a plain row-major matrix read along k with 16-byte aligned rows.
template <class F, bool AK, bool BKC, int SPLIT, int ACCS, int BN = 256, int TMA = 0>
__device__ __forceinline__ void gemm_tc_pair_persistent(const F &f, float *__restrict__ partial, uint32_t *status,
                                                        const void *tma = nullptr, const void *tmb = nullptr) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int M = F::M, N = F::N, K = F::K;
    constexpr int BH = BN / 2;
    static_assert(BN == 256 || BN == 128 || BN == 64, "tile width");
    constexpr int TILES_N = (N + BN - 1) / BN, TILES = ((M + 2 * BM - 1) / (2 * BM)) * TILES_N;
    constexpr int WORK = TILES * F::NB * SPLIT;
    constexpr int NBUF = ACCS * BN <= 256 ? 2 : 1;
    constexpr uint32_t BUF_COLS = ACCS * BN;
    constexpr uint32_t LBO_A = lbo_bytes(BM), LBO_B = lbo_bytes(BH);
    constexpr uint32_t TA = tile_bytes(BM), TB = tile_bytes(BH), STAGE = pair_stage_bytes(BN);
    constexpr uint32_t BAR_OFF = pp_smem_bytes(BN) - 256, EPI_OFF = BAR_OFF - PP_EPI_WARPS * 32 * 33 * 4;
    constexpr int KCH = ((K + SPLIT - 1) / SPLIT + BK - 1) / BK * BK;
    constexpr int NST = STAGES, G = PP_CONV_GROUPS;
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const uint32_t rank = cluster_ctarank();
    const int cid = blockIdx.x >> 1, ncl = gridDim.x >> 1;

    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + BAR_OFF);               // full[3], empty[3], tfull[2], tempty[2]
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + BAR_OFF + 96);
    volatile uint32_t *failed = reinterpret_cast<volatile uint32_t *>(smem + BAR_OFF + 104);
    const uint32_t bar0 = smem_u32(bars);
    auto full = [&](int s) { return bar0 + 8u * s; };
    auto empty = [&](int s) { return bar0 + 8u * (NST + s); };
    auto tfull = [&](int b) { return bar0 + 8u * (2 * NST + b); };
    auto tempty = [&](int b) { return bar0 + 8u * (2 * NST + 2 + b); };
    const uint32_t alldone = smem_u32(smem + BAR_OFF + 112);                     // every MMA of this cluster has completed
    auto raw_full = [&](int s) { return smem_u32(smem + BAR_OFF + 120) + 8u * s; };   // this CTA's TMA copies of stage s have landed
    constexpr bool TMA_A = (TMA & 1) != 0, TMA_B = (TMA & 2) != 0;
    constexpr uint32_t LBO_AH = TMA_A ? (uint32_t)BM * 16u : LBO_A, LBO_BH = TMA_B ? (uint32_t)BH * 16u : LBO_B;   // hi tiles from TMA are dense
    static_assert(!TMA || F::NB == 1, "tensor maps describe one matrix");

    // One work item: which rows / columns / k range. All roles walk the same sequence w = cid, cid + ncl, ...
    struct Item { int m0, n0, nb0, bt, sp, k_begin, k_end, nkb; };
    auto item = [&](int w) {
        Item it;
        const int tile = w % TILES, y = w / TILES;
        it.bt = y / SPLIT; it.sp = y % SPLIT;
        it.m0 = (tile / TILES_N) * (2 * BM) + (int)rank * BM;
        it.n0 = (tile % TILES_N) * BN;
        it.nb0 = it.n0 + (int)rank * BH;
        it.k_begin = it.sp * KCH; it.k_end = min(K, it.k_begin + KCH);
        it.nkb = max(1, (it.k_end - it.k_begin + BK - 1) / BK);                 // an empty k range still runs one block of zeros
        return it;
    };

    if (t == 0) {
        for (int s = 0; s < NST; s++) { mbar_init(full(s), 2 * 8); mbar_init(empty(s), 1); }
        for (int b = 0; b < 2; b++) { mbar_init(tfull(b), 1); mbar_init(tempty(b), 2 * PP_EPI_WARPS); }
        mbar_init(alldone, 1);
        for (int s = 0; s < NST; s++) mbar_init(raw_full(s), 1);
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == PP_MMA_WARP) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;

    // One 32-row x 32-column piece of an accumulator buffer: tensor memory -> registers -> transposed through
    // `stage_f` (32 x 33 floats of this warp) -> the statements, eight rows at a time: first everything the
    // statements read, then the statements. release >= 0: hand tensor-memory buffer `release` back after the loads.
    auto drain = [&](const Item &it, uint32_t acc, int c, float *stage_f, int release, uint32_t tempty_leader0) {
        const int q = warp & 3;
        // What the statements read at this piece (32 rows of one 128-byte line each) is asked into L1 first: the loads
        // below go out eight rows at a time, and every batch that has to go to L2 costs its full latency — with long k
        // loops (two accumulators, no second tensor-memory buffer) nothing hides the epilogue.
        const int eseg = epi_seg_of(f, it.n0);
        if (SPLIT == 1 && F::NLD > 0 && it.m0 + 32 * q + lane < M && it.n0 + 32 * c < N)
            with_seg<F>(eseg, [&](auto S_) { f_epi_near<decltype(S_)::value>(f, it.m0 + 32 * q + lane, it.n0 + 32 * c, it.bt); });
        uint32_t r[32];
        tmem_ld32(acc + (uint32_t)(32 * c), r);
        if (ACCS == 2) {
            uint32_t r2[32];
            tmem_ld32(acc + (uint32_t)(BN + 32 * c), r2);
#pragma unroll
            for (int x = 0; x < 32; x++) r[x] = __float_as_uint(__uint_as_float(r[x]) + __uint_as_float(r2[x]));
        }
        if (release >= 0) {
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(tempty_leader0 + 8u * release);
        }
#pragma unroll
        for (int x = 0; x < 32; x++) stage_f[lane * 33 + x] = __uint_as_float(r[x]);
        __syncwarp();
        const int n = it.n0 + 32 * c + lane;
        constexpr int NLD = F::NLD > 0 ? F::NLD : 1, RB = 8;
        with_seg<F>(eseg, [&](auto S_) {
            constexpr int SG = decltype(S_)::value;
            for (int r0 = 0; r0 < 32; r0 += RB) {
                const int mb = it.m0 + 32 * q + r0;
                float ld[RB][NLD];
                if (SPLIT == 1 && F::NLD > 0) {
#pragma unroll
                    for (int rr = 0; rr < RB; rr++)
                        if (mb + rr < M && n < N) f_epi_loads<SG>(f, mb + rr, n, it.bt, ld[rr]);
                }
#pragma unroll
                for (int rr = 0; rr < RB; rr++) {
                    const int m = mb + rr;
                    const float v = stage_f[(r0 + rr) * 33 + lane];
                    if (m < M && n < N) {
                        if (SPLIT > 1) partial[(((long)it.bt * SPLIT + it.sp) * M + m) * N + n] = v;
                        else f_epi2<SG>(f, m, n, it.bt, v * F::ALPHA, ld[rr]);
                    }
                }
            }
        });
        __syncwarp();
    };
    // The cluster's last item has no main loop after it to hide its epilogue, and the converter warps are idle
    // by then: its column chunks are dealt round-robin to the six warps of each lane quarter (two epilogue
    // warps, four converter warps) instead of the two epilogue warps alone.
    constexpr int NCH = BN / 32, LAST_WORKERS = 2 + 2 * G;
    const int n_items = cid < WORK ? (WORK - cid + ncl - 1) / ncl : 0;

    if (warp < 8 * G) {
        // ---------------------------------------------------------------- converters
        const int grp = warp >> 3;
        const int tc = t & (CONV_THREADS - 1);
        float va[BM / 32][4], vb[BH / 32][4];
        auto fetch = [&](const Item &it, int kb) {
            const int k0 = it.k_begin + kb * BK;
            with_seg<F>(op_seg_of(f, k0, it.n0), [&](auto S_) {
                constexpr int SG = decltype(S_)::value;
                if (!TMA_A) {
#pragma unroll
                    for (int p = 0; p < BM / 32; p++) {
                        int row, kc;
                        TileMap<AK, BM>::at(tc, p, row, kc);
                        const int m = it.m0 + row, k = k0 + kc * 4;
                        if (m < M && k < it.k_end) f_a4<SG>(f, m, k, it.bt, va[p]);
                        else { va[p][0] = va[p][1] = va[p][2] = va[p][3] = 0.0f; }
                    }
                }
                if (!TMA_B) {
#pragma unroll
                    for (int p = 0; p < BH / 32; p++) {
                        int row, kc;
                        TileMap<BKC, BH>::at(tc, p, row, kc);
                        const int n = it.nb0 + row, k = k0 + kc * 4;
                        if (n < N && k < it.k_end) f_b4<SG>(f, k, n, it.bt, vb[p]);
                        else { vb[p][0] = vb[p][1] = vb[p][2] = vb[p][3] = 0.0f; }
                    }
                }
            });
        };
        // The TMA copies of block (it, kb) into stage s: eight 16-byte columns per operand; rows or k beyond the matrix read as zeros
        auto tma_issue = [&](const Item &it, int kb, int s) {
            const int k0 = it.k_begin + kb * BK;
            const uint32_t st = smem_u32(smem + s * STAGE);
            mbar_expect_tx(raw_full(s), (TMA_A ? BM * 128u : 0u) + (TMA_B ? BH * 128u : 0u));
#pragma unroll
            for (int c = 0; c < BK / 4; c++) {
                if (TMA_A) tma_load_2d(st + c * (BM * 16), tma, k0 + 4 * c, it.m0, raw_full(s));
                if (TMA_B) tma_load_2d(st + 2 * TA + c * (BH * 16), tmb, k0 + 4 * c, it.nb0, raw_full(s));
            }
        };
        // L2 prefetch of a later block of the same item: one 128-byte line per 32 k of a row (operand contiguous
        // along k), or per 32 rows at one k (operand contiguous along its rows); one lane per line asks.
        auto touch = [&](const Item &it, int kb) {
            if (kb >= it.nkb) return;
            const int k0 = it.k_begin + kb * BK;
            with_seg<F>(op_seg_of(f, k0, it.n0), [&](auto S_) {
            constexpr int SG = decltype(S_)::value;
#pragma unroll
            for (int p = 0; p < BM / 32; p++) {
                int row, kc;
                TileMap<AK, BM>::at(tc, p, row, kc);
                const int m = it.m0 + row, k = k0 + kc * 4;
                if (m < M && k < it.k_end) {
                    if (AK) { if (kc == 0) f_a_touch<SG>(f, m, k, it.bt); }
                    else if (lane == 0) { f_a_touch<SG>(f, m, k, it.bt); f_a_touch<SG>(f, m, k + 1, it.bt); f_a_touch<SG>(f, m, k + 2, it.bt); f_a_touch<SG>(f, m, k + 3, it.bt); }
                }
            }
#pragma unroll
            for (int p = 0; p < BH / 32; p++) {
                int row, kc;
                TileMap<BKC, BH>::at(tc, p, row, kc);
                const int n = it.nb0 + row, k = k0 + kc * 4;
                if (n < N && k < it.k_end) {
                    if (BKC) { if (kc == 0) f_b_touch<SG>(f, k, n, it.bt); }
                    else if (lane == 0) { f_b_touch<SG>(f, k, n, it.bt); f_b_touch<SG>(f, k + 1, n, it.bt); f_b_touch<SG>(f, k + 2, n, it.bt); f_b_touch<SG>(f, k + 3, n, it.bt); }
                }
            }
            });
        };
        // (w, kb) of this group's current block; `advance` moves it G blocks on
        int w = cid, kb = grp;
        Item it = item(w < WORK ? w : 0);
        auto settle = [&]() { while (w < WORK && kb >= it.nkb) { kb -= it.nkb; w += ncl; if (w < WORK) it = item(w); } };
        settle();
        const uint32_t full_leader0 = map_to_cta(full(0), 0);
        // a second cursor runs PP_AHEAD group turns in front of the first, across item boundaries, and asks L2 for its block
        int tw = w, tkb = kb;
        Item tit = it;
        auto touch_next = [&]() {
            tkb += G;
            while (tw < WORK && tkb >= tit.nkb) { tkb -= tit.nkb; tw += ncl; if (tw < WORK) tit = item(tw); }
            if (tw < WORK) touch(tit, tkb);
        };
        if (w < WORK) {
            fetch(it, kb);
#pragma unroll 1
            for (int a = 0; a < PP_AHEAD; a++) touch_next();
        }
        for (long n = grp; w < WORK; n += G) {
            const int s = (int)(n % NST);
            const uint32_t ph = (uint32_t)(n / NST) & 1u;
            if (!mbar_wait(empty(s), ph ^ 1)) { *failed = 1; break; }
            uint8_t *st = smem + s * STAGE;
            if (TMA && (warp & 7) == 0 && lane == 0) tma_issue(it, kb, s);       // one thread of the group starts this block's copies
            if (!TMA_A) {
#pragma unroll
                for (int p = 0; p < BM / 32; p++) {
                    int row, kc;
                    TileMap<AK, BM>::at(tc, p, row, kc);
                    split_store(st, st + TA, kc * LBO_A + row * 16, va[p]);
                }
            }
            if (!TMA_B) {
#pragma unroll
                for (int p = 0; p < BH / 32; p++) {
                    int row, kc;
                    TileMap<BKC, BH>::at(tc, p, row, kc);
                    split_store(st + 2 * TA, st + 2 * TA + TB, kc * LBO_B + row * 16, vb[p]);
                }
            }
            kb += G;
            settle();
            if (w < WORK) { fetch(it, kb); touch_next(); }
            if (TMA) {                                                           // the raw tiles have landed: they are the hi operand; make lo
                if (!mbar_wait(raw_full(s), ph)) { *failed = 1; break; }
                if (TMA_A) lo_from_raw_tile<BM>(st, st + TA, LBO_A, tc);
                if (TMA_B) lo_from_raw_tile<BH>(st + 2 * TA, st + 2 * TA + TB, LBO_B, tc);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(full_leader0 + 8u * s);
        }
        if (n_items > 0 && !*failed) {
            const int il = n_items - 1, buf = il % NBUF;
            if (mbar_wait(alldone, 0)) {                                     // every MMA is done: the stages are free
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const Item itl = item(cid + il * ncl);
                const uint32_t acc = tmem + (uint32_t)buf * BUF_COLS + ((uint32_t)(32 * (warp & 3)) << 16);
                float *stage_f = reinterpret_cast<float *>(smem) + warp * (32 * 33);
                for (int c = 2 + (warp >> 2); c < NCH; c += LAST_WORKERS) drain(itl, acc, c, stage_f, -1, 0u);
            } else {
                *failed = 1;
            }
        }
    } else if (warp == PP_MMA_WARP) {
        if (lane == 0 && rank == 0) {
            // ------------------------------------------------------------ MMA issuer (CTA 0 of the pair only)
            constexpr uint32_t IDESC = instr_desc(2 * BM, BN);
            const uint32_t base = smem_u32(smem);
            uint32_t peer_tmem;
            asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(peer_tmem) : "r"(map_to_cta(smem_u32(tmem_slot), 1)) : "memory");
            if (peer_tmem != tmem) *failed = 1;
            long n = 0;
            int i = 0;
            for (int w = cid; w < WORK && !*failed; w += ncl, i++) {
                const Item it = item(w);
                const int buf = i % NBUF;
                if (!mbar_wait_cluster(tempty(buf), (((uint32_t)(i / NBUF)) & 1u) ^ 1u)) { *failed = 1; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t acc = tmem + (uint32_t)buf * BUF_COLS;
                for (int kb = 0; kb < it.nkb; kb++, n++) {
                    const int s = (int)(n % NST);
                    if (!mbar_wait_cluster(full(s), (uint32_t)(n / NST) & 1u)) { *failed = 1; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_hi = base + s * STAGE, a_lo = a_hi + TA, b_hi = a_hi + 2 * TA, b_lo = b_hi + TB;
#pragma unroll
                    for (int j = 0; j < BK / 8; j++) {
                        const uint64_t dah = smem_desc(a_hi + 2 * j * LBO_AH, LBO_AH), dal = smem_desc(a_lo + 2 * j * LBO_A, LBO_A);
                        const uint64_t dbh = smem_desc(b_hi + 2 * j * LBO_BH, LBO_BH), dbl = smem_desc(b_lo + 2 * j * LBO_B, LBO_B);
                        if (ACCS == 2) {
                            mma_tf32_pair(acc + BN, dah, dbl, IDESC, (kb | j) ? 1u : 0u);
                            mma_tf32_pair(acc + BN, dal, dbh, IDESC, 1u);
                            mma_tf32_pair(acc, dah, dbh, IDESC, (kb | j) ? 1u : 0u);
                        } else {                                     // small terms first, then the large one
                            mma_tf32_pair(acc, dah, dbl, IDESC, (kb | j) ? 1u : 0u);
                            mma_tf32_pair(acc, dal, dbh, IDESC, 1u);
                            mma_tf32_pair(acc, dah, dbh, IDESC, 1u);
                        }
                    }
                    mma_commit_pair(empty(s));
                }
                mma_commit_pair(tfull(buf));
            }
            mma_commit_pair(alldone);                            // a barrier of its own: tfull's parity alone cannot tell the last use from an earlier one
        }
    } else {
        // ---------------------------------------------------------------- epilogue warps
        const int e = warp - 8 * G, q = warp & 3, half = e >> 2;
        float *stage_f = reinterpret_cast<float *>(smem + EPI_OFF) + e * (32 * 33);
        const uint32_t tempty_leader0 = map_to_cta(tempty(0), 0);
        constexpr int CPW = (BN / 32) / (PP_EPI_WARPS / 4);                       // column chunks per warp (4, 2 or 1)
        // What the statements read besides the accumulator (a residual, the old value of a `+=`) is
        // asked into L2 one item ahead: lane = row, one 128-byte line per column chunk.
        auto touch = [&](const Item &it) {
            if (SPLIT > 1) return;
            const int m = it.m0 + 32 * q + lane;
#pragma unroll
            for (int cc = 0; cc < CPW; cc++) {
                const int n = it.n0 + 32 * (half * CPW + cc);
                if (m < M && n < N) with_seg<F>(epi_seg_of(f, it.n0), [&](auto S_) { f_epi_touch<decltype(S_)::value>(f, m, n, it.bt); });
            }
        };
        if (cid < WORK) touch(item(cid));
        int i = 0;
        for (int w = cid; w < WORK; w += ncl, i++) {
            const Item it = item(w);
            const int buf = i % NBUF;
            const bool ok = !*failed && mbar_wait(tfull(buf), ((uint32_t)(i / NBUF)) & 1u);
            if (!ok) { *failed = 1; break; }
            if (w + ncl < WORK) touch(item(w + ncl));
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t acc = tmem + (uint32_t)buf * BUF_COLS + ((uint32_t)(32 * q) << 16);
            if (i == n_items - 1) {
                for (int c = half; c < NCH; c += LAST_WORKERS) drain(it, acc, c, stage_f, -1, 0u);
            } else {
                for (int cc = 0; cc < CPW; cc++)                 // after the last chunk's loads the buffer goes back to the MMA warp
                    drain(it, acc, half * CPW + cc, stage_f, cc == CPW - 1 ? buf : -1, tempty_leader0);
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync();
    if (warp == PP_MMA_WARP) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
    if (t == 0 && *failed) atomicExch(status, TIMEOUT);
}

}  // namespace tc
}  // namespace anvil
