// Short-K variant of the tcgen05 kind::i8 kernel: the whole K extent fits one 128-byte k block
// (K <= 128; the attention scores Q K^T with K = 64 are the case it was written for).
//
// With so little K the tensor pipe is idle most of the time and a tile's cost is its epilogue:
// 2S-1 TMEM reads, the INT64 recombination, one rounding and four bytes of C per output.  The
// general kernel cannot overlap that work with the next tile's MMAs at S = 3 (its 128 x 64 tile fills
// 320 of the 512 TMEM columns), so this one is organised around the epilogue instead:
//   * 128 x 48 tiles: the (2S-1) * 48 accumulator columns fit TMEM twice.  Two groups of eight
//     epilogue warps own one accumulator set each and alternate tiles, so sixteen warps drain, round
//     and store while the MMA warp is already one or two tiles ahead.
//   * issue cost: a thread needs on the order of a hundred cycles to issue an MMA whatever its size (a chain
//     of dependent instructions on a scheduler it shares with epilogue warps), far more than these small MMAs
//     keep the tensor pipe busy.  So a tile's first k step takes 2S-1 MMAs (see issue_first_k_step) instead of
//     S^2, descriptors are formed with one addition (umma_i8_lo), the 48-column tile spreads the cost over half
//     as many more outputs than a 32-column one would, and two threads on two schedulers issue alternate tiles.
//   * A-stationary: a CTA takes half rows of tiles round-robin and walks each with the column tile running
//     fastest, so the 128-row A tile (all S planes, the whole K) is loaded once per half row into one of two
//     buffers; only the small B tiles stream through a ring of stages (see TileWalk).
//   * k steps beyond K (zero padding of the 128-byte block) are not issued.
// The arithmetic (level accumulators, exact INT64 sums, single rounding) is that of the general
// kernel; see rgb200_mma.cuh.  Reference counterpart: gemm_wmma_i8<S> (repro_gemm_cuda/repro_gemm.cu:280-364);
// the batched attention products it serves are listed as pending at gpt2_ops_suite/gpt2_ops_suite.cu:543-548.
#pragma once
#include "rgb200_mma.cuh"

namespace rgb200 {

constexpr int SK_NT = 48;                     // columns of C per tile
constexpr int SK_B_STAGES = 5;
constexpr int SK_EPI_GROUPS = 2;              // one per accumulator set
constexpr int SK_GROUP_WARPS = 8;
constexpr int SK_GROUP_THREADS = SK_GROUP_WARPS * 32;
// warp 0: TMA producer; warp 1 and the last warp: the MMA issuers of accumulator set 0 and 1; between them the
// sixteen epilogue warps
constexpr int SK_THREADS = 64 + SK_EPI_GROUPS * SK_GROUP_THREADS + 32;    // 608
constexpr int SK_SECOND_ISSUER_WARP = SK_THREADS / 32 - 1;

// 32 lanes x 8 consecutive 32-bit columns: thread i of the warp receives row (lane base + i).
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, int (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr) : "memory");
}

// Bounded wait for the many-thread roles (epilogue, converters): like mbar_wait, but a waiting thread sleeps a little
// between polls, so that the issue slots of its scheduler go to the single thread that feeds the tensor pipe.
__device__ __forceinline__ bool mbar_wait_relaxed(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    long long t0 = clock64();
    for (uint32_t spins = 1;; ++spins) {
        __nanosleep(40);
        if (mbar_try_wait(bar, parity)) return true;
        if ((spins & 63u) == 0) {
            if (*abort_flag) return false;
            if (clock64() - t0 > WAIT_LIMIT_CLOCKS) {
                atomicCAS(status, 0, code);
                *abort_flag = 1;
                __threadfence_block();
                return false;
            }
        }
    }
}

// The order in which a CTA visits tiles.  A "unit" is half a row of tiles (one A tile, half of the column tiles); the
// CTAs take units round-robin, so the CTAs running together work on neighbouring rows of a few batches and their B
// planes are shared in L2 (a contiguous range per CTA spreads the 148 CTAs over all batches at once, and with the
// output stream passing through L2 the B tiles then keep coming from HBM).  Within a unit the column tile runs
// fastest, so the A tile is loaded once per unit.  No 64-bit divisions: the roles that walk this order are single
// threads on the critical path.
struct TileWalk {
    int unit, stride, total_units, halves, split;     // split: first column tile of the second half
    int n_tiles, m_tiles;
    int n_blk, n_end, m_blk, batch;
    __device__ __forceinline__ void place() {
        const int row = unit / halves, half = unit - row * halves;
        batch = row / m_tiles;
        m_blk = row - batch * m_tiles;
        n_blk = half ? split : 0;
        n_end = (half || halves == 1) ? n_tiles : split;
    }
    __device__ __forceinline__ void init(int first_unit, int stride_, int n_tiles_, int m_tiles_, int batches) {
        n_tiles = n_tiles_; m_tiles = m_tiles_;
        halves = n_tiles >= 2 ? 2 : 1;
        split = (n_tiles + 1) / 2;
        total_units = batches * m_tiles * halves;
        unit = first_unit; stride = stride_;
        if (valid()) place();
    }
    __device__ __forceinline__ bool valid() const { return unit < total_units; }
    // Moves one tile on; true when that left the current unit (the next tile, if any, needs another A tile).
    __device__ __forceinline__ bool advance() {
        if (++n_blk < n_end) return false;
        unit += stride;
        if (valid()) place();
        return true;
    }
};

// Exact sum T = sum_L level_L * 128^(2S-2-L) for level sums over at most 128 values of k.  Each level is then
// below 128 * 20352 < 2^22, so neighbouring levels combine in 32-bit arithmetic (level * 128 stays below 2^29)
// and only the last steps need 64 bits.
__device__ __forceinline__ long long mad_wide(int a, int b, long long c) {      // a * b + c with a 32 x 32 -> 64 bit product
    long long d;
    asm("mad.wide.s32 %0, %1, %2, %3;" : "=l"(d) : "r"(a), "r"(b), "l"(c));
    return d;
}
template <int S>
__device__ __forceinline__ typename std::conditional<S == 1, int, long long>::type
combine_levels_short_k(const int (&lv)[2 * S - 1][8], int j) {
    if constexpr (S == 1) {
        return lv[0][j];
    } else if constexpr (S == 2) {
        return mad_wide(lv[0][j], 1 << 14, (long long)(lv[2][j] + lv[1][j] * 128));
    } else {
        const int low = lv[4][j] + lv[3][j] * 128;
        const int mid = lv[2][j] + lv[1][j] * 128;
        return mad_wide(lv[0][j], 1 << 28, mad_wide(mid, 1 << 14, (long long)low));
    }
}

template <int S>
struct SmallKTraits {
    static constexpr int LEVELS = 2 * S - 1;
    static constexpr int A_PLANE_BYTES = BLOCK_M * BLOCK_K;
    static constexpr int A_BYTES = S * A_PLANE_BYTES;
    static constexpr int B_PLANE_BYTES = SK_NT * BLOCK_K;
    static constexpr int B_STAGE_BYTES = S * B_PLANE_BYTES;
    static constexpr int ACC_COLS = LEVELS * SK_NT;
    static constexpr int TMEM_COLS = 2 * ACC_COLS <= 64 ? 64 : 2 * ACC_COLS <= 128 ? 128 : 2 * ACC_COLS <= 256 ? 256 : 512;
    static constexpr int CPT = SK_NT / 2;                    // columns per epilogue thread
    static constexpr int BAR_BYTES = 256;
    static constexpr int SMEM_BYTES = 2 * A_BYTES + SK_B_STAGES * B_STAGE_BYTES + 1024 + BAR_BYTES +
                                      SK_EPI_GROUPS * SK_GROUP_WARPS * CPT * 4;
    static_assert(2 * ACC_COLS <= 512, "two accumulator sets must fit TMEM");
    static_assert(CPT % 8 == 0, "the epilogue reads eight TMEM columns at a time");
};

struct SmallKParams {
    const int* expo_a;       // [batch][M]
    const int* expo_b;       // [batch][N]
    float* C;
    int* status;
    int M, N, batch;
    long long stride_c;
    int m_tiles, n_tiles;
    int k_steps;             // ceil(K / 32): MMAs beyond it would multiply the zero padding
    int e0;
};

template <int S>
__global__ void __launch_bounds__(SK_THREADS, 1)
gemm_i8_smallk_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                      const SmallKParams P) {
    using Tr = SmallKTraits<S>;
    constexpr int NT = SK_NT, CPT = Tr::CPT;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t a_base = smem_base;
    const uint32_t b_base = smem_base + 2 * Tr::A_BYTES;
    const uint32_t bar_base = b_base + SK_B_STAGES * Tr::B_STAGE_BYTES;
    auto a_full = [&](int i) { return bar_base + 8u * i; };
    auto a_empty = [&](int i) { return bar_base + 8u * (2 + i); };
    auto b_full = [&](int s) { return bar_base + 8u * (4 + s); };
    auto b_empty = [&](int s) { return bar_base + 8u * (4 + SK_B_STAGES + s); };
    auto tmem_full = [&](int g) { return bar_base + 8u * (4 + 2 * SK_B_STAGES + g); };
    auto tmem_empty = [&](int g) { return bar_base + 8u * (6 + 2 * SK_B_STAGES + g); };
    const uint32_t tmem_slot = bar_base + 8u * (8 + 2 * SK_B_STAGES);
    uint8_t* gen_base = smem_raw + (smem_base - smem_u32(smem_raw));
    uint8_t* gen_bar = gen_base + 2 * Tr::A_BYTES + SK_B_STAGES * Tr::B_STAGE_BYTES;
    volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(gen_bar + 8 * (8 + 2 * SK_B_STAGES));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_bar + 8 * (9 + 2 * SK_B_STAGES));
    int* eb_slots = reinterpret_cast<int*>(gen_bar + Tr::BAR_BYTES);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int i = 0; i < 2; ++i) { mbar_init(a_full(i), 1); mbar_init(a_empty(i), SK_EPI_GROUPS); }
        for (int s = 0; s < SK_B_STAGES; ++s) { mbar_init(b_full(s), 1); mbar_init(b_empty(s), 1); }
        for (int g = 0; g < SK_EPI_GROUPS; ++g) { mbar_init(tmem_full(g), 1); mbar_init(tmem_empty(g), SK_GROUP_THREADS); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(tmem_slot, Tr::TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_ptr;

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            uint32_t a_it = 0, b_it = 0;
            bool ok = true, new_row = true;
            TileWalk w;
            w.init(blockIdx.x, gridDim.x, P.n_tiles, P.m_tiles, P.batch);
            for (; w.valid(); ++b_it) {
                if (new_row) {
                    const int ab = a_it & 1;
                    if (!(ok = mbar_wait(a_empty(ab), ((a_it >> 1) & 1u) ^ 1u, abort_flag, P.status, STATUS_WAIT_EMPTY))) break;
                    mbar_arrive_expect_tx(a_full(ab), Tr::A_BYTES);
                    tma_load_4d(a_base + ab * Tr::A_BYTES, &tmap_a, a_full(ab), 0, w.m_blk * BLOCK_M, 0, w.batch);
                    ++a_it;
                }
                const int s = b_it % SK_B_STAGES;
                if (!(ok = mbar_wait(b_empty(s), ((b_it / SK_B_STAGES) & 1u) ^ 1u, abort_flag, P.status, STATUS_WAIT_EMPTY))) break;
                mbar_arrive_expect_tx(b_full(s), Tr::B_STAGE_BYTES);
                tma_load_4d(b_base + s * Tr::B_STAGE_BYTES, &tmap_b, b_full(s), 0, w.n_blk * NT, 0, w.batch);
                new_row = w.advance();
            }
            if (!ok) {
                // abort: let copies that are still in flight land before the CTA gives up its shared memory
                auto drain = [&](uint32_t bar, uint32_t parity) {
                    long long c0 = clock64();
                    while (!mbar_try_wait(bar, parity))
                        if (clock64() - c0 > WAIT_LIMIT_CLOCKS) { atomicCAS(P.status, 0, STATUS_WAIT_DRAIN); break; }
                };
                for (uint32_t j = 0; j < (b_it < (uint32_t)SK_B_STAGES ? b_it : (uint32_t)SK_B_STAGES); ++j) {
                    const uint32_t i2 = b_it - 1 - j;
                    drain(b_full(i2 % SK_B_STAGES), (i2 / SK_B_STAGES) & 1u);
                }
                for (uint32_t j = 0; j < (a_it < 2u ? a_it : 2u); ++j) {
                    const uint32_t i2 = a_it - 1 - j;
                    drain(a_full(i2 & 1), (i2 >> 1) & 1u);
                }
            }
        }
    } else if (warp == 1 || warp == SK_SECOND_ISSUER_WARP) {
        // ---------------------------------------------------------------- MMA issuers
        // One thread per accumulator set: issuer g takes the tiles of parity g.  A tile's MMAs cost the issuing thread
        // far more time than they cost the tensor pipe, so two threads on two schedulers issue alternate tiles.
        // Both follow the rows of tiles: each waits for a row's A tile and, after its last tile of the row, commits
        // to the A buffer's "empty" barrier (two arrivals: tcgen05.commit covers the committing thread's MMAs only).
        if (lane == 0) {
            constexpr uint32_t IDESC_WIDE = idesc_i8(BLOCK_M, S * NT);
            const int g = warp == 1 ? 0 : 1;
            uint32_t a_it = 0, use = 0;
            uint32_t sa = 0, cur_ab = 0;
            bool ok = true, new_row = true;
            TileWalk w;
            w.init(blockIdx.x, gridDim.x, P.n_tiles, P.m_tiles, P.batch);
            for (int i = 0; ok && w.valid(); ++i) {
                if (new_row) {
                    cur_ab = a_it & 1;
                    if (!(ok = mbar_wait(a_full(cur_ab), (a_it >> 1) & 1u, abort_flag, P.status, STATUS_WAIT_FULL))) break;
                    sa = a_base + cur_ab * Tr::A_BYTES;
                    ++a_it;
                }
                if ((i & 1) == g) {
                    const int s = i % SK_B_STAGES;
                    if (!(ok = mbar_wait(b_full(s), (i / SK_B_STAGES) & 1u, abort_flag, P.status, STATUS_WAIT_FULL))) break;
                    if (!(ok = mbar_wait(tmem_empty(g), (use & 1u) ^ 1u, abort_flag, P.status, STATUS_WAIT_TMEM_EMPTY))) break;
                    ++use;
                    tc_fence_after();
                    const uint32_t sb = b_base + s * Tr::B_STAGE_BYTES;
                    const uint32_t acc = tmem_base + g * Tr::ACC_COLS;
                    issue_first_k_step<S, NT>(acc, sa, sb, Tr::A_PLANE_BYTES, Tr::B_PLANE_BYTES);
                    const uint32_t a_lo = sw128_desc_lo(sa), b_lo = sw128_desc_lo(sb);
                    for (int k = 1; k < P.k_steps; ++k)
#pragma unroll
                        for (int p = 0; p < S; ++p)
                            umma_i8_lo<true>(acc + p * NT, a_lo + p * (Tr::A_PLANE_BYTES >> 4) + k * (UMMA_K >> 4),
                                             b_lo + k * (UMMA_K >> 4), IDESC_WIDE);
                    umma_commit(b_empty(s));
                    umma_commit(tmem_full(g));
                }
                // last tile of this unit: this issuer is done with the A buffer
                new_row = w.advance();
                if (new_row) umma_commit(a_empty(cur_ab));
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue (two groups of eight warps)
        using TAcc = typename std::conditional<S == 1, int, long long>::type;
        const int ew = warp - 2;
        const int g = ew / SK_GROUP_WARPS;             // accumulator set of this group
        const int quarter = warp & 3;                  // TMEM lanes this warp may read
        const int half = (ew % SK_GROUP_WARPS) >> 2;   // which half of the tile's columns
        const int row_in_tile = quarter * 32 + lane;
        int* eb_s = eb_slots + ew * CPT;
        bool ok = true;
        uint32_t use = 0;                              // how often this group's accumulator set has been used
        TileWalk w;
        w.init(blockIdx.x, gridDim.x, P.n_tiles, P.m_tiles, P.batch);
        for (int i = 0; ok && w.valid(); ++i, w.advance()) {
            if ((i & 1) != g) continue;                 // the other group's tile
            const int n_blk = w.n_blk, m_blk = w.m_blk, batch = w.batch;
            const uint32_t use_now = use++;
            const int row = m_blk * BLOCK_M + row_in_tile;
            const bool row_ok = row < P.M;
            const int ea = row_ok ? __ldg(P.expo_a + (size_t)batch * P.M + row) : 0;
            const int col0 = n_blk * NT + half * CPT;
            // The slot holds the column exponents already shifted into the exponent field of a float, and the warp
            // learns their range: when every exponent this row can meet keeps any non-zero sum a normal number
            // (the float of a non-zero sum has a biased exponent of 127..190, so E in [-126, 64] is safe), the
            // rounding below needs no range check per output.
            __syncwarp();
            int eb_lo = 0x7FFFFFFF, eb_hi = -0x7FFFFFFF;
            if (lane < CPT && col0 + lane < P.N) {
                const int eb = __ldg(P.expo_b + (size_t)batch * P.N + col0 + lane);
                eb_s[lane] = eb << 23;
                eb_lo = eb_hi = eb;
            } else if (lane < CPT) {
                eb_s[lane] = 0;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                eb_lo = min(eb_lo, __shfl_xor_sync(0xFFFFFFFFu, eb_lo, o));
                eb_hi = max(eb_hi, __shfl_xor_sync(0xFFFFFFFFu, eb_hi, o));
            }
            ok = mbar_wait_relaxed(tmem_full(g), use_now & 1u, abort_flag, P.status, STATUS_WAIT_TMEM_FULL);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (!ok) break;
            tc_fence_after();
            // accumulators -> exact sums in registers, then hand the set back to the MMA warp
            const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + g * Tr::ACC_COLS + half * CPT;
            TAcc T[CPT];
#pragma unroll
            for (int c0 = 0; c0 < CPT; c0 += 8) {       // eight columns at a time keeps the register count low
                int lv[Tr::LEVELS][8];
#pragma unroll
                for (int L = 0; L < Tr::LEVELS; ++L) tmem_ld8(t_row + L * NT + c0, lv[L]);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 8; ++j) T[c0 + j] = combine_levels_short_k<S>(lv, j);
            }
            tc_fence_before();
            mbar_arrive(tmem_empty(g));
            if (!row_ok || col0 >= P.N) continue;
            // one rounding per output
            uint32_t* dst = reinterpret_cast<uint32_t*>(P.C + (size_t)batch * P.stride_c + (size_t)row * P.N + col0);
            const int ebase = ea + P.e0;
            const bool safe = ebase + eb_lo >= -126 && ebase + eb_hi <= 64;
            const uint32_t ebase23 = (uint32_t)ebase << 23;
            auto round4 = [&](int j, uint32_t (&r)[4]) {
                if (safe) {
                    // one hardware conversion (round to nearest even, sign included), then the exponent is added in
                    // place; a zero sum converts to +0 and stays +0
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const uint32_t fb = f32_bits(__ll2float_rn((long long)T[j + q]));
                        r[q] = fb ? fb + ebase23 + (uint32_t)eb_s[j + q] : 0u;
                    }
                } else {                                // subnormal or overflowing results are possible: exact path
#pragma unroll
                    for (int q = 0; q < 4; ++q) r[q] = round_to_f32_bits(T[j + q], ebase + (eb_s[j + q] >> 23));
                }
            };
            const bool whole = col0 + CPT <= P.N;
            if (whole && (reinterpret_cast<uintptr_t>(dst) & 31) == 0) {
#pragma unroll
                for (int j = 0; j < CPT; j += 8) {
                    uint32_t r[4], q[4];
                    round4(j, r);
                    round4(j + 4, q);
                    st_global_256(dst + j, r[0], r[1], r[2], r[3], q[0], q[1], q[2], q[3]);
                }
            } else if (whole && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
                for (int j = 0; j < CPT; j += 4) {
                    uint32_t r[4];
                    round4(j, r);
                    *reinterpret_cast<uint4*>(dst + j) = make_uint4(r[0], r[1], r[2], r[3]);
                }
            } else {
#pragma unroll
                for (int j = 0; j < CPT; j += 4) {
                    uint32_t r[4];
                    round4(j, r);
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        if (col0 + j + q < P.N) dst[j + q] = r[q];
                }
            }
        }
    }

    // common exit: every thread arrives, then the allocating warp returns the TMEM columns
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, Tr::TMEM_COLS);
    }
}

}  // namespace rgb200
