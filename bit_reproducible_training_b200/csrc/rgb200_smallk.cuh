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
//   * output: a thread owns one row of the tile (TMEM lane = row), so a warp-wide store of its results would touch
//     32 different 128-byte lines per instruction, and the L1 store path, not HBM, bounded the kernel.  When C allows
//     it (16-byte aligned base, rows and batches a multiple of four floats apart) the rounded tile goes into a
//     swizzled shared-memory staging buffer instead (conflict-free 16-byte writes) and a dedicated thread sends it
//     to C with TMA tensor stores, which also clip the ragged edges; otherwise the threads store their rows directly.
// The arithmetic (level accumulators, exact INT64 sums, single rounding) is that of the general
// kernel; see rgb200_mma.cuh.  Reference counterpart: gemm_wmma_i8<S> (repro_gemm_cuda/repro_gemm.cu:280-364);
// the batched attention products it serves are listed as pending at gpt2_ops_suite/gpt2_ops_suite.cu:543-548.
#pragma once
#include "rgb200_mma.cuh"

namespace rgb200 {

constexpr int SK_NT = 48;                     // columns of C per tile
constexpr int SK_B_STAGES = 4;
constexpr int SK_EPI_GROUPS = 2;              // one per accumulator set
constexpr int SK_GROUP_WARPS = 8;
constexpr int SK_GROUP_THREADS = SK_GROUP_WARPS * 32;
// warp 0: TMA producer; warp 1 and warp 18: the MMA issuers of accumulator set 0 and 1; between them the sixteen
// epilogue warps; warp 19: issues the TMA stores of the staged output tiles
constexpr int SK_THREADS = 64 + SK_EPI_GROUPS * SK_GROUP_THREADS + 64;    // 640
constexpr int SK_SECOND_ISSUER_WARP = SK_THREADS / 32 - 2;
constexpr int SK_STORE_WARP = SK_THREADS / 32 - 1;
// staged output tile: columns 0..31 as 128 rows of 128 bytes (128-byte swizzle), columns 32..47 as 128 rows of 64
// bytes (64-byte swizzle); one TMA tensor store each
constexpr int SK_STAGE_X_COLS = 32;
constexpr int SK_STAGE_X_BYTES = BLOCK_M * SK_STAGE_X_COLS * 4;
constexpr int SK_STAGE_Y_BYTES = BLOCK_M * (SK_NT - SK_STAGE_X_COLS) * 4;
constexpr int SK_STAGE_BYTES = SK_STAGE_X_BYTES + SK_STAGE_Y_BYTES;
enum : int { STATUS_WAIT_STAGE = 6 };         // a role gave up waiting for the output staging buffer

// 32 lanes x 8 consecutive 32-bit columns: thread i of the warp receives row (lane base + i).
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                 :: "l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void st_shared_128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    // no memory clobber: the staging buffer is read by the copy engine only, after the proxy fence (a volatile asm,
    // so it stays behind these stores), and ordinary loads may be scheduled across the store
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" :: "r"(addr), "r"(a), "r"(b), "r"(c), "r"(d));
}

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
    static constexpr int SMEM_BYTES = 2 * A_BYTES + SK_EPI_GROUPS * SK_STAGE_BYTES + SK_B_STAGES * B_STAGE_BYTES + 1024 +
                                      BAR_BYTES + SK_EPI_GROUPS * SK_GROUP_WARPS * CPT * 4;
    static_assert(SMEM_BYTES <= 232448, "shared memory of one CTA");
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

// The exact rounding of four sums, kept out of line: the hot loops use it only for rows whose results may be
// subnormal or overflow.
__device__ __noinline__ uint4 round4_exact(long long t0, long long t1, long long t2, long long t3, int e0, int e1, int e2, int e3) {
    return make_uint4(round_to_f32_bits(t0, e0), round_to_f32_bits(t1, e1), round_to_f32_bits(t2, e2), round_to_f32_bits(t3, e3));
}

// STAGED: C takes TMA tensor stores (tmap_cx / tmap_cy are valid); otherwise the threads store their rows.
template <int S, bool STAGED>
__global__ void __launch_bounds__(SK_THREADS, 1)
gemm_i8_smallk_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                      const __grid_constant__ CUtensorMap tmap_cx, const __grid_constant__ CUtensorMap tmap_cy,
                      const SmallKParams P) {
    using Tr = SmallKTraits<S>;
    constexpr int NT = SK_NT, CPT = Tr::CPT;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t a_base = smem_base;
    const uint32_t c_base = smem_base + 2 * Tr::A_BYTES;
    const uint32_t b_base = c_base + SK_EPI_GROUPS * SK_STAGE_BYTES;
    const uint32_t bar_base = b_base + SK_B_STAGES * Tr::B_STAGE_BYTES;
    auto a_full = [&](int i) { return bar_base + 8u * i; };
    auto a_empty = [&](int i) { return bar_base + 8u * (2 + i); };
    auto b_full = [&](int s) { return bar_base + 8u * (4 + s); };
    auto b_empty = [&](int s) { return bar_base + 8u * (4 + SK_B_STAGES + s); };
    auto tmem_full = [&](int g) { return bar_base + 8u * (4 + 2 * SK_B_STAGES + g); };
    auto tmem_empty = [&](int g) { return bar_base + 8u * (6 + 2 * SK_B_STAGES + g); };
    const uint32_t tmem_slot = bar_base + 8u * (8 + 2 * SK_B_STAGES);
    auto stage_free = [&](int g) { return bar_base + 8u * (10 + 2 * SK_B_STAGES + g); };
    auto stage_full = [&](int g) { return bar_base + 8u * (12 + 2 * SK_B_STAGES + g); };
    static_assert(8 * (14 + 2 * SK_B_STAGES) <= Tr::BAR_BYTES, "barrier area");
    uint8_t* gen_base = smem_raw + (smem_base - smem_u32(smem_raw));
    uint8_t* gen_bar = gen_base + 2 * Tr::A_BYTES + SK_EPI_GROUPS * SK_STAGE_BYTES + SK_B_STAGES * Tr::B_STAGE_BYTES;
    volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(gen_bar + 8 * (8 + 2 * SK_B_STAGES));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_bar + 8 * (9 + 2 * SK_B_STAGES));
    int* eb_slots = reinterpret_cast<int*>(gen_bar + Tr::BAR_BYTES);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int i = 0; i < 2; ++i) { mbar_init(a_full(i), 1); mbar_init(a_empty(i), SK_EPI_GROUPS); }
        for (int s = 0; s < SK_B_STAGES; ++s) { mbar_init(b_full(s), 1); mbar_init(b_empty(s), 1); }
        for (int g = 0; g < SK_EPI_GROUPS; ++g) { mbar_init(tmem_full(g), 1); mbar_init(tmem_empty(g), SK_GROUP_THREADS); }
        for (int g = 0; g < SK_EPI_GROUPS; ++g) { mbar_init(stage_free(g), 1); mbar_init(stage_full(g), SK_GROUP_THREADS); }
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
            uint32_t a_it = 0, b_it = 0, units = 0;      // A tiles requested, B tiles requested, units entered
            bool ok = true, new_row = true;
            int in_unit = 0;
            TileWalk w, wa;                               // wa: the unit whose A tile is requested next
            w.init(blockIdx.x, gridDim.x, P.n_tiles, P.m_tiles, P.batch);
            wa = w;
            auto load_a = [&]() {
                const int ab = a_it & 1;
                if (!mbar_wait(a_empty(ab), ((a_it >> 1) & 1u) ^ 1u, abort_flag, P.status, STATUS_WAIT_EMPTY)) return false;
                mbar_arrive_expect_tx(a_full(ab), Tr::A_BYTES);
                tma_load_4d(a_base + ab * Tr::A_BYTES, &tmap_a, a_full(ab), 0, wa.m_blk * BLOCK_M, 0, wa.batch);
                ++a_it;
                wa.unit += wa.stride;
                if (wa.valid()) wa.place();
                return true;
            };
            for (; w.valid(); ++b_it) {
                if (new_row) {
                    if (a_it == units && !(ok = load_a())) break;      // not requested ahead (the first unit)
                    ++units;
                    in_unit = 0;
                }
                // The next unit's A tile is requested well before the MMA issuers get there: once this unit is as
                // many tiles old as there are B stages, the unit before it is over and its buffer is free (a short
                // unit asks at its last tile and may have to wait for that).
                if (a_it == units && wa.valid() && (in_unit >= SK_B_STAGES || w.n_blk + 1 >= w.n_end) && !(ok = load_a())) break;
                const int s = b_it % SK_B_STAGES;
                if (!(ok = mbar_wait(b_empty(s), ((b_it / SK_B_STAGES) & 1u) ^ 1u, abort_flag, P.status, STATUS_WAIT_EMPTY))) break;
                mbar_arrive_expect_tx(b_full(s), Tr::B_STAGE_BYTES);
                tma_load_4d(b_base + s * Tr::B_STAGE_BYTES, &tmap_b, b_full(s), 0, w.n_blk * NT, 0, w.batch);
                ++in_unit;
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
    } else if (warp == SK_STORE_WARP) {
        // ---------------------------------------------------------------- TMA stores of the staged tiles
        // One thread follows the tile order: when all threads of the tile's group have written their rows it sends
        // the two parts of the staging buffer to C and, once the copy engine has read them, hands the buffer back.
        if (lane == 0 && STAGED) {
            bool ok = true;
            TileWalk w;
            w.init(blockIdx.x, gridDim.x, P.n_tiles, P.m_tiles, P.batch);
            for (uint32_t i = 0; w.valid(); ++i, w.advance()) {
                const int g = i & 1;
                if (!(ok = mbar_wait_relaxed(stage_full(g), (i >> 1) & 1u, abort_flag, P.status, STATUS_WAIT_STAGE))) break;
                const uint32_t src = c_base + g * SK_STAGE_BYTES;
                const int col = w.n_blk * NT;
                tma_store_3d(&tmap_cx, src, col, w.m_blk * BLOCK_M, w.batch);
                if (col + SK_STAGE_X_COLS < P.N) tma_store_3d(&tmap_cy, src + SK_STAGE_X_BYTES, col + SK_STAGE_X_COLS, w.m_blk * BLOCK_M, w.batch);
                bulk_commit();
                bulk_wait_read_all();
                mbar_arrive(stage_free(g));
            }
            bulk_wait_all();
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
        // where this thread's six 16-byte pieces go in the staging buffer: piece c of a row of the 32-column part at
        // chunk c ^ (row % 8) of the row's 128 bytes, of the 16-column part at chunk c ^ ((row / 2) % 4) of its 64
        // bytes - the images TMA's 128-byte and 64-byte swizzles expect, and free of bank conflicts for a warp's rows
        uint32_t stage_off[CPT / 4];
#pragma unroll
        for (int j = 0; j < CPT / 4; ++j) {
            const int c = half * (CPT / 4) + j;
            stage_off[j] = c_base + g * SK_STAGE_BYTES +
                           (c < SK_STAGE_X_COLS / 4
                                ? row_in_tile * 128 + ((c ^ (row_in_tile & 7)) << 4)
                                : SK_STAGE_X_BYTES + row_in_tile * 64 + (((c - SK_STAGE_X_COLS / 4) ^ ((row_in_tile >> 1) & 3)) << 4));
        }
        bool ok = true;
        TileWalk w;
        w.init(blockIdx.x, gridDim.x, P.n_tiles, P.m_tiles, P.batch);
        if (g == 1 && w.valid()) w.advance();          // this group's first tile
        // The exponents of a tile are requested one tile of this group ahead of their use.
        int ea_next = 0, eb_next = 0;
        bool col_ok_next = false;
        auto request_exponents = [&]() {
            const int row = w.m_blk * BLOCK_M + row_in_tile;
            const int col = w.n_blk * NT + half * CPT + lane;
            ea_next = row < P.M ? __ldg(P.expo_a + (size_t)w.batch * P.M + row) : 0;
            col_ok_next = lane < CPT && col < P.N;
            eb_next = col_ok_next ? __ldg(P.expo_b + (size_t)w.batch * P.N + col) : 0;
        };
        if (w.valid()) request_exponents();
        for (uint32_t use = 0; ok && w.valid(); ++use) {   // use: how often this group's accumulator set has been used
            const int n_blk = w.n_blk, m_blk = w.m_blk, batch = w.batch;
            const int ea = ea_next, eb = eb_next;
            const bool col_ok = col_ok_next;
            w.advance();                                // the other group's tile
            if (w.valid()) w.advance();
            if (w.valid()) request_exponents();
            const int row = m_blk * BLOCK_M + row_in_tile;
            const bool row_ok = row < P.M;
            const int col0 = n_blk * NT + half * CPT;
            // The slot holds the column exponents already shifted into the exponent field of a float, and the warp
            // learns their range: when every exponent its rows can meet keeps any non-zero sum a normal number
            // (the float of a non-zero sum has a biased exponent of 127..190, so E in [-126, 64] is safe), a sum is
            // converted as soon as it is drained and only the exponent is added afterwards.
            __syncwarp();                               // the previous tile's reads of the slot are over
            if (lane < CPT) eb_s[lane] = eb << 23;
            int eb_lo = __reduce_min_sync(0xFFFFFFFFu, col_ok ? eb : 0x7FFFFFFF);
            int eb_hi = __reduce_max_sync(0xFFFFFFFFu, col_ok ? eb : -0x7FFFFFFF);
            if (eb_lo > eb_hi) eb_lo = eb_hi = 0;       // no column of this half lies inside the matrix
            const int ebase = ea + P.e0;
            const bool fast = __all_sync(0xFFFFFFFFu, ebase + eb_lo >= -126 && ebase + eb_hi <= 64);
            __syncwarp();
            const uint32_t ebase23 = (uint32_t)ebase << 23;
            const int4* eb4 = reinterpret_cast<const int4*>(eb_s);
            ok = mbar_wait_relaxed(tmem_full(g), use & 1u, abort_flag, P.status, STATUS_WAIT_TMEM_FULL);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (!ok) break;
            tc_fence_after();
            const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + g * Tr::ACC_COLS + half * CPT;
            // where four results go: the staging buffer, or (no tensor map for C) the thread's row of C
            uint32_t* dst = reinterpret_cast<uint32_t*>(P.C + (size_t)batch * P.stride_c + (size_t)row * P.N + col0);
            const bool inside = row_ok && col0 < P.N;
            const bool vec = inside && col0 + CPT <= P.N && (reinterpret_cast<uintptr_t>(dst) & 15) == 0;
            auto emit = [&](int j, const uint32_t (&r)[4]) {
                if constexpr (STAGED) {
                    st_shared_128(stage_off[j / 4], r[0], r[1], r[2], r[3]);
                } else if (vec) {
                    *reinterpret_cast<uint4*>(dst + j) = make_uint4(r[0], r[1], r[2], r[3]);
                } else if (inside) {
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        if (col0 + j + q < P.N) dst[j + q] = r[q];
                }
            };
            // rows and columns beyond the matrix hold zero sums (their operand rows were filled with zeros) and are
            // clipped by the tensor store; every thread of the group takes part in the hand-over of the staging buffer
            auto wait_stage = [&]() {
                if constexpr (STAGED) {
                    ok = mbar_wait_relaxed(stage_free(g), (use & 1u) ^ 1u, abort_flag, P.status, STATUS_WAIT_STAGE);
                    ok = __all_sync(0xFFFFFFFFu, ok);
                }
            };
            if (fast) {
                // accumulators -> exact sums -> one hardware conversion each (round to nearest even, sign included),
                // eight columns at a time, then the set goes back to its MMA issuer
                uint32_t fb[CPT];
#pragma unroll
                for (int c0 = 0; c0 < CPT; c0 += 8) {
                    int lv[Tr::LEVELS][8];
#pragma unroll
                    for (int L = 0; L < Tr::LEVELS; ++L) tmem_ld8(t_row + L * NT + c0, lv[L]);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 8; ++j) fb[c0 + j] = f32_bits(__ll2float_rn((long long)combine_levels_short_k<S>(lv, j)));
                }
                tc_fence_before();
                mbar_arrive(tmem_empty(g));
                wait_stage();
                if (!ok) break;
                // the exponent is added in place; a zero sum converted to +0 and stays +0
#pragma unroll
                for (int j = 0; j < CPT; j += 4) {
                    const int4 e4 = eb4[j >> 2];
                    const uint32_t r[4] = {fb[j] ? fb[j] + ebase23 + (uint32_t)e4.x : 0u, fb[j + 1] ? fb[j + 1] + ebase23 + (uint32_t)e4.y : 0u,
                                           fb[j + 2] ? fb[j + 2] + ebase23 + (uint32_t)e4.z : 0u, fb[j + 3] ? fb[j + 3] + ebase23 + (uint32_t)e4.w : 0u};
                    emit(j, r);
                }
            } else {
                // some result of this warp's rows may be subnormal or overflow: exact sums are kept and rounded by the
                // exact routine (out of line: it is rare and large)
                TAcc T[CPT];
#pragma unroll
                for (int c0 = 0; c0 < CPT; c0 += 8) {
                    int lv[Tr::LEVELS][8];
#pragma unroll
                    for (int L = 0; L < Tr::LEVELS; ++L) tmem_ld8(t_row + L * NT + c0, lv[L]);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 8; ++j) T[c0 + j] = combine_levels_short_k<S>(lv, j);
                }
                tc_fence_before();
                mbar_arrive(tmem_empty(g));
                wait_stage();
                if (!ok) break;
#pragma unroll 1
                for (int j = 0; j < CPT; j += 4) {
                    const int4 e4 = eb4[j >> 2];
                    const uint4 x = round4_exact(T[j], T[j + 1], T[j + 2], T[j + 3], ebase + (e4.x >> 23), ebase + (e4.y >> 23),
                                                 ebase + (e4.z >> 23), ebase + (e4.w >> 23));
                    const uint32_t r[4] = {x.x, x.y, x.z, x.w};
                    emit(j, r);
                }
            }
            if constexpr (STAGED) {
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_arrive(stage_full(g));
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
