// Skinny-output variant of the tcgen05 kind::i8 kernel with the split of A fused into the producer
// (N <= 64, A stored k-contiguous; the attention product P V with P [1024 x 1024] and V [1024 x 64] is
// the case it was written for).
//
// For such a product A is nearly all of the traffic: staging its S digit planes in HBM, as the general
// path does, writes and re-reads S bytes per element on top of the four that must be read.  Here a CTA
// owns a 128-row block of A and never stores its planes:
//   producer one thread streams the block's rows through a ring of shared-memory stages with TMA, as FP32
//           chunks of 128 rows x 64 k (zero-filled beyond M and K), twice: once for pass 1, once for pass 2
//           (the block was just read, so the second time most of it comes from L2), and, during pass 2, B's
//           digit planes (small, staged in HBM by the usual pre-pass) one k block at a time;
//   pass 1  sixteen warps take the row maxima of the chunks as they land; the rows' scale exponents follow;
//   pass 2  the same warps round every value to its fixed-point integer, split it into S digits and store
//           them straight into the 128-byte-swizzled shared-memory image the MMA reads - the layout TMA
//           would have produced - one k block (two chunks) per MMA stage;
//   MMA     one thread issues the same level-accumulating MMAs as the general kernel;
//   finish  the sixteen warps drain TMEM, rebuild the exact sums, round once and store C.
// Shared memory holds only two 32 KiB FP32 landing stages beside the MMA stages, too few bytes in flight to keep
// HBM busy; so (a) the producer also issues TMA prefetches into L2 a few chunks ahead of its loads, across pass
// and tile boundaries, and the loads themselves find their data in L2, and (b) during pass 1, when the int8 stages
// of A hold nothing (the previous block's MMAs are over, this block's digits do not exist yet), their memory
// serves as S more landing stages: pass 1 keeps 2 + S chunks in flight.
// The arithmetic is that of the general kernel (rgb200_mma.cuh) and of the split pre-pass
// (rgb200_prepass.cuh); only where the digits of A live differs.  Reference counterparts:
// quantize_kmajor + gemm_wmma_i8 (repro_gemm_cuda/repro_gemm.cu:54-79, 280-364).
#pragma once
#include "rgb200_mma.cuh"
#include "rgb200_prepass.cuh"
#include "rgb200_smallk.cuh"

namespace rgb200 {

constexpr int RF_NT = 64;                     // columns of C per tile (one tile covers all of N)
constexpr int RF_A_STAGES = 2;                // int8 stages the MMA reads (one k block each)
constexpr int RF_B_STAGES = 2;                // (one stage would stall the producer, which issues B's loads in chunk order)
constexpr int RF_F_STAGES = 2;                // FP32 landing stages
constexpr int RF_CHUNK_K = 64;                // k per FP32 chunk: 128 rows x 256 bytes
constexpr int RF_CHUNKS_PER_BLOCK = BLOCK_K / RF_CHUNK_K;
constexpr int RF_LANES_PER_ROW = RF_CHUNK_K / 4;          // one 16-byte load per lane
constexpr int RF_ROWS_PER_LOAD = 32 / RF_LANES_PER_ROW;   // rows a warp-wide load covers
constexpr int RF_ROW_ITERS = 8 / RF_ROWS_PER_LOAD;        // loads per warp and chunk (a warp owns eight rows)
constexpr int RF_PREFETCH = 4;                // chunks requested into L2 ahead of the loads (more than a few evict the block that pass 2 re-reads)
constexpr int RF_F_STAGE_BYTES = BLOCK_M * RF_CHUNK_K * 4;
constexpr int RF_WORK_WARPS = 16;             // converter + epilogue warps
constexpr int RF_WORK_THREADS = RF_WORK_WARPS * 32;
constexpr int RF_THREADS = 64 + RF_WORK_THREADS;      // 576

template <int S>
struct RowFusedTraits {
    static constexpr int LEVELS = 2 * S - 1;
    static constexpr int A_PLANE_BYTES = BLOCK_M * BLOCK_K;
    static constexpr int A_STAGE_BYTES = S * A_PLANE_BYTES;
    static constexpr int B_PLANE_BYTES = RF_NT * BLOCK_K;
    static constexpr int B_STAGE_BYTES = S * B_PLANE_BYTES;
    static constexpr int ACC_COLS = LEVELS * RF_NT;
    static constexpr int TMEM_COLS = ACC_COLS <= 64 ? 64 : ACC_COLS <= 128 ? 128 : ACC_COLS <= 256 ? 256 : 512;
    static constexpr int CPT = RF_NT / 4;     // sixteen columns per epilogue thread
    // FP32 landing stages that pass 1 borrows from the int8 stages of A, and the length of its chunk cycle
    static constexpr int X_STAGES = RF_A_STAGES * A_STAGE_BYTES / RF_F_STAGE_BYTES;
    static constexpr int P1_CYCLE = RF_F_STAGES + X_STAGES;
    static constexpr int BAR_BYTES = 256;
    static constexpr int SMEM_BYTES = RF_F_STAGES * RF_F_STAGE_BYTES + RF_A_STAGES * A_STAGE_BYTES + RF_B_STAGES * B_STAGE_BYTES + 1024 + BAR_BYTES +
                                      RF_WORK_WARPS * CPT * 4 /* column exponents */ + BLOCK_M * 4 /* row exponents */;
    static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
    static_assert(RF_CHUNK_K == 32 || RF_CHUNK_K == 64, "a chunk row is one or two 128-byte lines");
};

struct RowFusedParams {
    const int* expo_b;       // [batch][N]
    float* C;
    int* status;
    int M, N, K, batch;
    long long stride_c;
    int m_tiles, k_blocks;
    int e0;
};

template <int S>
__global__ void __launch_bounds__(RF_THREADS, 1)
gemm_i8_rowfused_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                        const RowFusedParams P) {
    using Tr = RowFusedTraits<S>;
    constexpr int NT = RF_NT, CPT = Tr::CPT;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t a_base = smem_base;
    const uint32_t b_base = smem_base + RF_A_STAGES * Tr::A_STAGE_BYTES;
    const uint32_t f_base = b_base + RF_B_STAGES * Tr::B_STAGE_BYTES;
    const uint32_t bar_base = f_base + RF_F_STAGES * RF_F_STAGE_BYTES;
    auto a_full = [&](int s) { return bar_base + 8u * s; };
    auto a_empty = [&](int s) { return bar_base + 8u * (RF_A_STAGES + s); };
    auto b_full = [&](int s) { return bar_base + 8u * (2 * RF_A_STAGES + s); };
    auto b_empty = [&](int s) { return bar_base + 8u * (2 * RF_A_STAGES + RF_B_STAGES + s); };
    auto f_full = [&](int s) { return bar_base + 8u * (2 * RF_A_STAGES + 2 * RF_B_STAGES + s); };
    auto f_empty = [&](int s) { return bar_base + 8u * (2 * RF_A_STAGES + 2 * RF_B_STAGES + RF_F_STAGES + s); };
    constexpr int NBAR = 2 * RF_A_STAGES + 2 * RF_B_STAGES + 2 * RF_F_STAGES;
    const uint32_t tmem_full_bar = bar_base + 8u * NBAR;
    const uint32_t tmem_empty_bar = bar_base + 8u * (NBAR + 1);
    // two barriers among the sixteen work warps (one arrival per warp); waits on them are bounded like all others
    const uint32_t rows_bar = bar_base + 8u * (NBAR + 2);       // every warp has published its rows' exponents
    const uint32_t done_bar = bar_base + 8u * (NBAR + 3);       // every warp has finished the tile's epilogue
    const uint32_t tmem_slot = bar_base + 8u * (NBAR + 4);
    auto x_full = [&](int s) { return bar_base + 8u * (NBAR + 6 + s); };
    auto x_empty = [&](int s) { return bar_base + 8u * (NBAR + 6 + Tr::X_STAGES + s); };
    static_assert(8 * (NBAR + 6 + 2 * Tr::X_STAGES) <= Tr::BAR_BYTES, "barrier area");
    uint8_t* gen_base = smem_raw + (smem_base - smem_u32(smem_raw));
    uint8_t* gen_a = gen_base;
    const uint8_t* gen_f = gen_base + RF_A_STAGES * Tr::A_STAGE_BYTES + RF_B_STAGES * Tr::B_STAGE_BYTES;
    uint8_t* gen_bar = gen_base + RF_A_STAGES * Tr::A_STAGE_BYTES + RF_B_STAGES * Tr::B_STAGE_BYTES + RF_F_STAGES * RF_F_STAGE_BYTES;
    volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(gen_bar + 8 * (NBAR + 4));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_bar + 8 * (NBAR + 5));
    int* eb_slots = reinterpret_cast<int*>(gen_bar + Tr::BAR_BYTES);
    int* ea_rows = eb_slots + RF_WORK_WARPS * CPT;        // scale exponents of the tile's 128 rows

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_tiles = P.batch * P.m_tiles;          // one tile per (batch, row block)

    if (threadIdx.x == 0) {
        for (int s = 0; s < RF_A_STAGES; ++s) { mbar_init(a_full(s), RF_WORK_WARPS); mbar_init(a_empty(s), 1); }
        for (int s = 0; s < RF_B_STAGES; ++s) { mbar_init(b_full(s), 1); mbar_init(b_empty(s), 1); }
        for (int s = 0; s < RF_F_STAGES; ++s) { mbar_init(f_full(s), 1); mbar_init(f_empty(s), RF_WORK_WARPS); }
        for (int s = 0; s < Tr::X_STAGES; ++s) { mbar_init(x_full(s), 1); mbar_init(x_empty(s), RF_WORK_WARPS); }
        mbar_init(tmem_full_bar, 1);
        mbar_init(tmem_empty_bar, RF_WORK_THREADS);
        mbar_init(rows_bar, RF_WORK_WARPS);
        mbar_init(done_bar, RF_WORK_WARPS);
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
        // ---------------------------------------------------------------- TMA producer (FP32 chunks of A, planes of B)
        if (lane == 0) {
            uint32_t f_it = 0, b_it = 0, x_it = 0;
            bool ok = true;
            // pass 1 only: a chunk into one of the stages borrowed from A's int8 stages
            auto load_chunk_x = [&](int c, int m_blk, int batch) {
                const int s = x_it % Tr::X_STAGES;
                if (!mbar_wait(x_empty(s), ((x_it / Tr::X_STAGES) & 1u) ^ 1u, abort_flag, P.status, STATUS_WAIT_EMPTY)) return false;
                mbar_arrive_expect_tx(x_full(s), RF_F_STAGE_BYTES);
                tma_load_3d(a_base + s * RF_F_STAGE_BYTES, &tmap_a, x_full(s), c * RF_CHUNK_K, m_blk * BLOCK_M, batch);
                ++x_it;
                return true;
            };
            auto load_chunk = [&](int c, int m_blk, int batch) {
                const int s = f_it % RF_F_STAGES;
                if (!mbar_wait(f_empty(s), ((f_it / RF_F_STAGES) & 1u) ^ 1u, abort_flag, P.status, STATUS_WAIT_EMPTY)) return false;
                mbar_arrive_expect_tx(f_full(s), RF_F_STAGE_BYTES);
                tma_load_3d(f_base + s * RF_F_STAGE_BYTES, &tmap_a, f_full(s), c * RF_CHUNK_K, m_blk * BLOCK_M, batch);
                ++f_it;
                return true;
            };
            // Chunk order (the work warps consume in the same order): per tile all chunks for pass 1 - chunk c into a
            // landing stage when c modulo (2 + S) is below two, else into a borrowed stage - then all chunks again
            // for pass 2, landing stages only, with B's planes of a k block in front of that block's chunks.  The
            // borrowed stages are free once the previous tile's MMAs are over (its tmem_full commit).  A second cursor
            // runs RF_PREFETCH chunks ahead of the loads and only asks for the chunk to be brought into L2, so that
            // enough bytes are on their way from HBM although just RF_F_STAGES chunks fit shared memory.
            struct Cursor { int tile, pass, c, batch, m_blk; };
            const int chunks = RF_CHUNKS_PER_BLOCK * P.k_blocks;
            auto place = [&](Cursor& x) { x.batch = x.tile / P.m_tiles; x.m_blk = x.tile - x.batch * P.m_tiles; };
            auto step = [&](Cursor& x) {
                if (++x.c == chunks) { x.c = 0; if (++x.pass == 2) { x.pass = 0; x.tile += gridDim.x; place(x); } }
            };
            auto prefetch = [&](const Cursor& x) {
                if (x.tile >= total_tiles) return;
                asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];"
                             ::"l"(&tmap_a), "r"(x.c * RF_CHUNK_K), "r"(x.m_blk * BLOCK_M), "r"(x.batch) : "memory");
            };
            uint32_t tile_it = 0;                 // tiles whose first pass has been started
            bool x_open = true;                   // the borrowed stages may be written for the current tile's first pass
            Cursor cur{(int)blockIdx.x, 0, 0, 0, 0}, ahead{(int)blockIdx.x, 0, 0, 0, 0};
            place(cur);
            place(ahead);
            for (int i = 0; i < RF_PREFETCH; ++i) { prefetch(ahead); step(ahead); }
            while (ok && cur.tile < total_tiles) {
                if (cur.pass == 1 && cur.c % RF_CHUNKS_PER_BLOCK == 0) {         // B's planes of this k block
                    const int s = b_it % RF_B_STAGES;
                    if (!(ok = mbar_wait(b_empty(s), ((b_it / RF_B_STAGES) & 1u) ^ 1u, abort_flag, P.status, STATUS_WAIT_EMPTY))) break;
                    mbar_arrive_expect_tx(b_full(s), Tr::B_STAGE_BYTES);
                    tma_load_4d(b_base + s * Tr::B_STAGE_BYTES, &tmap_b, b_full(s), (cur.c / RF_CHUNKS_PER_BLOCK) * BLOCK_K, 0, 0, cur.batch);
                    ++b_it;
                }
                if (cur.pass == 0 && cur.c % Tr::P1_CYCLE >= RF_F_STAGES) {
                    if (!x_open) {
                        // the previous tile's MMAs still read the int8 stages until its last commit has arrived
                        if (!(ok = mbar_wait(tmem_full_bar, (tile_it - 1) & 1u, abort_flag, P.status, STATUS_WAIT_FULL))) break;
                        x_open = true;
                    }
                    if (!(ok = load_chunk_x(cur.c, cur.m_blk, cur.batch))) break;
                } else {
                    if (!(ok = load_chunk(cur.c, cur.m_blk, cur.batch))) break;
                }
                prefetch(ahead);
                step(ahead);
                const int tile_before = cur.tile;
                step(cur);
                if (cur.tile != tile_before) { ++tile_it; x_open = false; }
            }
            if (!ok) {
                // abort: let copies that are still in flight land before the CTA gives up its shared memory
                auto drain = [&](uint32_t bar, uint32_t parity) {
                    long long c0 = clock64();
                    while (!mbar_try_wait(bar, parity))
                        if (clock64() - c0 > WAIT_LIMIT_CLOCKS) { atomicCAS(P.status, 0, STATUS_WAIT_DRAIN); break; }
                };
                for (uint32_t j = 0; j < (b_it < (uint32_t)RF_B_STAGES ? b_it : (uint32_t)RF_B_STAGES); ++j) {
                    const uint32_t i2 = b_it - 1 - j;
                    drain(b_full(i2 % RF_B_STAGES), (i2 / RF_B_STAGES) & 1u);
                }
                for (uint32_t j = 0; j < (f_it < (uint32_t)RF_F_STAGES ? f_it : (uint32_t)RF_F_STAGES); ++j) {
                    const uint32_t i2 = f_it - 1 - j;
                    drain(f_full(i2 % RF_F_STAGES), (i2 / RF_F_STAGES) & 1u);
                }
                for (uint32_t j = 0; j < (x_it < (uint32_t)Tr::X_STAGES ? x_it : (uint32_t)Tr::X_STAGES); ++j) {
                    const uint32_t i2 = x_it - 1 - j;
                    drain(x_full(i2 % Tr::X_STAGES), (i2 / Tr::X_STAGES) & 1u);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t IDESC_WIDE = idesc_i8(BLOCK_M, S * NT);
            uint32_t it = 0, tile_it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++tile_it) {
                if (!(ok = mbar_wait(tmem_empty_bar, (tile_it & 1u) ^ 1u, abort_flag, P.status, STATUS_WAIT_TMEM_EMPTY))) break;
                tc_fence_after();
                for (int kb = 0; kb < P.k_blocks; ++kb, ++it) {
                    const int sa_i = it % RF_A_STAGES, sb_i = it % RF_B_STAGES;
                    if (!(ok = mbar_wait(a_full(sa_i), (it / RF_A_STAGES) & 1u, abort_flag, P.status, STATUS_WAIT_FULL))) break;
                    if (!(ok = mbar_wait(b_full(sb_i), (it / RF_B_STAGES) & 1u, abort_flag, P.status, STATUS_WAIT_FULL))) break;
                    tc_fence_after();
                    const uint32_t sa = a_base + sa_i * Tr::A_STAGE_BYTES;
                    const uint32_t sb = b_base + sb_i * Tr::B_STAGE_BYTES;
#pragma unroll
                    for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
                        if (kb == 0 && k == 0) {
                            issue_first_k_step<S, NT>(tmem_base, sa, sb, Tr::A_PLANE_BYTES, Tr::B_PLANE_BYTES);
                        } else {
#pragma unroll
                            for (int p = 0; p < S; ++p)
                                umma_i8(tmem_base + p * NT, smem_desc_sw128(sa + p * Tr::A_PLANE_BYTES + k * UMMA_K),
                                        smem_desc_sw128(sb + k * UMMA_K), IDESC_WIDE, 1u);
                        }
                    }
                    umma_commit(a_empty(sa_i));
                    umma_commit(b_empty(sb_i));
                }
                if (ok) umma_commit(tmem_full_bar);
            }
        }
    } else {
        // ---------------------------------------------------------------- converters, then epilogue (warps 2..17)
        using TAcc = typename std::conditional<S == 1, int, long long>::type;
        const int cw = warp - 2;
        const int quarter = warp & 3;                  // TMEM lanes this warp may read
        const int cgroup = cw >> 2;                    // which sixteen columns of the tile
        int* eb_s = eb_slots + cw * CPT;
        // Chunk layout in shared memory: [128 rows][RF_CHUNK_K] FP32.  A warp owns eight rows; one 16-byte load per
        // lane covers RF_ROWS_PER_LOAD rows at a time: rows rsel * RF_ROW_ITERS + i of the eight, which makes the
        // swizzled digit stores of the lane groups fall into different bank groups.
        const int cl = lane % RF_LANES_PER_ROW;        // which four k of the chunk
        const int rsel = lane / RF_LANES_PER_ROW;
        uint32_t f_it = 0, a_it = 0, tile_it = 0, x_it = 0;
        bool ok = true;
        // one FP32 chunk into the running row maxima; chunk c of the pass sits in a landing stage or in a borrowed one
        auto max_chunk = [&](int c, float (&m)[RF_ROW_ITERS]) {
            const bool borrowed = c % Tr::P1_CYCLE >= RF_F_STAGES;
            const int s = borrowed ? x_it % Tr::X_STAGES : f_it % RF_F_STAGES;
            const uint32_t full = borrowed ? x_full(s) : f_full(s), empty = borrowed ? x_empty(s) : f_empty(s);
            const uint32_t parity = borrowed ? (x_it / Tr::X_STAGES) & 1u : (f_it / RF_F_STAGES) & 1u;
            bool got = mbar_wait_relaxed(full, parity, abort_flag, P.status, STATUS_WAIT_FULL);
            got = __all_sync(0xFFFFFFFFu, got);
            if (!got) return false;
            const uint8_t* chunk = borrowed ? gen_a + s * RF_F_STAGE_BYTES : gen_f + s * RF_F_STAGE_BYTES;
#pragma unroll
            for (int i = 0; i < RF_ROW_ITERS; ++i) {
                const int r = cw * 8 + rsel * RF_ROW_ITERS + i;
                m[i] = abs4max(m[i], *reinterpret_cast<const float4*>(chunk + r * (RF_CHUNK_K * 4) + cl * 16));
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty);
            if (borrowed) ++x_it; else ++f_it;
            return true;
        };
        for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++tile_it) {
            const int batch = tile / P.m_tiles, m_blk = tile - batch * P.m_tiles;
            // pass 1: row maxima
            float m[RF_ROW_ITERS];
#pragma unroll
            for (int i = 0; i < RF_ROW_ITERS; ++i) m[i] = 0.0f;
            for (int c = 0; ok && c < RF_CHUNKS_PER_BLOCK * P.k_blocks; ++c) ok = max_chunk(c, m);
            if (!ok) break;
            int e[RF_ROW_ITERS];
            float f1[RF_ROW_ITERS];
            bool all_plain = true;
#pragma unroll
            for (int i = 0; i < RF_ROW_ITERS; ++i) {
#pragma unroll
                for (int o = RF_LANES_PER_ROW / 2; o > 0; o >>= 1) m[i] = fmaxf(m[i], __shfl_xor_sync(0xFFFFFFFFu, m[i], o));   // over the row's lanes
                e[i] = scale_exponent(m[i]);
                f1[i] = quant_scale(e[i], S).f1;
                all_plain = all_plain && plain_row(e[i]);
                if (cl == 0) ea_rows[cw * 8 + rsel * RF_ROW_ITERS + i] = e[i];    // the previous tile's epilogue has finished reading (done_bar)
            }
            all_plain = __all_sync(0xFFFFFFFFu, all_plain);
            // every warp has left pass 1 - the borrowed stages are about to be overwritten with digits - and every
            // warp's row exponents are in ea_rows before any warp's epilogue reads them
            __syncwarp();
            if (lane == 0) mbar_arrive(rows_bar);
            ok = mbar_wait_relaxed(rows_bar, tile_it & 1u, abort_flag, P.status, STATUS_WAIT_FULL);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (!ok) break;
            // pass 2: digits into the swizzled stages
            for (int kb = 0; kb < P.k_blocks; ++kb, ++a_it) {
                const int sa_i = a_it % RF_A_STAGES;
                ok = mbar_wait_relaxed(a_empty(sa_i), ((a_it / RF_A_STAGES) & 1u) ^ 1u, abort_flag, P.status, STATUS_WAIT_EMPTY);
                ok = __all_sync(0xFFFFFFFFu, ok);
                if (!ok) break;
                uint8_t* stage = gen_a + sa_i * Tr::A_STAGE_BYTES;
#pragma unroll
                for (int h = 0; h < RF_CHUNKS_PER_BLOCK; ++h) {
                    const int s = f_it % RF_F_STAGES;
                    ok = mbar_wait_relaxed(f_full(s), (f_it / RF_F_STAGES) & 1u, abort_flag, P.status, STATUS_WAIT_FULL);
                    ok = __all_sync(0xFFFFFFFFu, ok);
                    if (!ok) break;
                    const uint8_t* chunk = gen_f + s * RF_F_STAGE_BYTES;
#pragma unroll
                    for (int i = 0; i < RF_ROW_ITERS; ++i) {
                        const int r = cw * 8 + rsel * RF_ROW_ITERS + i;           // row inside the tile
                        const float4 v = *reinterpret_cast<const float4*>(chunk + r * (RF_CHUNK_K * 4) + cl * 16);
                        // 128-byte rows of int8, 16-byte pieces XOR-ed with the row index modulo 8 (the 128-byte swizzle);
                        // this chunk's k are bytes RF_CHUNK_K * h .. of the row
                        const size_t off = (size_t)r * 128 + (size_t)((((h * (RF_CHUNK_K / 16) + (cl >> 2)) ^ (r & 7))) << 4) + ((cl & 3) << 2);
                        if (all_plain) {
                            QuantScale q; q.f1 = f1[i]; q.f2 = 1.0f; q.lim = 0;
                            store_quad_impl<S, true>(v, q, reinterpret_cast<int8_t*>(stage), Tr::A_PLANE_BYTES, off);
                        } else {
                            store_quad<S>(v, quant_scale(e[i], S), plain_row(e[i]), reinterpret_cast<int8_t*>(stage), Tr::A_PLANE_BYTES, off);
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(f_empty(s));
                    ++f_it;
                }
                if (!ok) break;
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");    // generic-proxy stores -> visible to the MMA's reads
                __syncwarp();
                if (lane == 0) mbar_arrive(a_full(sa_i));
            }
            if (!ok) break;
            // epilogue: 32 rows x 16 columns per warp
            const int row_in_tile = quarter * 32 + lane;
            const int row = m_blk * BLOCK_M + row_in_tile;
            const bool row_ok = row < P.M;
            const int col0 = cgroup * CPT;
            if (lane < CPT) eb_s[lane] = col0 + lane < P.N ? __ldg(P.expo_b + (size_t)batch * P.N + col0 + lane) : 0;
            __syncwarp();
            const int ea = ea_rows[row_in_tile];
            ok = mbar_wait_relaxed(tmem_full_bar, tile_it & 1u, abort_flag, P.status, STATUS_WAIT_TMEM_FULL);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (!ok) break;
            tc_fence_after();
            const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + col0;
            TAcc T[CPT];
#pragma unroll
            for (int c0 = 0; c0 < CPT; c0 += 8) {
                int lv[Tr::LEVELS][8];
#pragma unroll
                for (int L = 0; L < Tr::LEVELS; ++L) tmem_ld8(t_row + L * NT + c0, lv[L]);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    long long t = lv[Tr::LEVELS - 1][j];
#pragma unroll
                    for (int L = Tr::LEVELS - 2; L >= 0; --L)
                        t += (long long)lv[L][j] * (long long)(1 << (7 * (Tr::LEVELS - 1 - L)));
                    T[c0 + j] = (TAcc)t;
                }
            }
            tc_fence_before();
            mbar_arrive(tmem_empty_bar);
            if (row_ok && col0 < P.N) {
                uint32_t* dst = reinterpret_cast<uint32_t*>(P.C + (size_t)batch * P.stride_c + (size_t)row * P.N + col0);
                const int ebase = ea + P.e0;
                const bool whole = col0 + CPT <= P.N && (reinterpret_cast<uintptr_t>(dst) & 15) == 0;
#pragma unroll
                for (int j = 0; j < CPT; j += 4) {
                    uint32_t r[4];
                    bool k0, k1, k2, k3;
                    r[0] = round_to_f32_bits_signed(T[j + 0], ebase + eb_s[j + 0], &k0);
                    r[1] = round_to_f32_bits_signed(T[j + 1], ebase + eb_s[j + 1], &k1);
                    r[2] = round_to_f32_bits_signed(T[j + 2], ebase + eb_s[j + 2], &k2);
                    r[3] = round_to_f32_bits_signed(T[j + 3], ebase + eb_s[j + 3], &k3);
                    if (!(k0 && k1 && k2 && k3)) {
                        r[0] = round_to_f32_bits(T[j + 0], ebase + eb_s[j + 0]);
                        r[1] = round_to_f32_bits(T[j + 1], ebase + eb_s[j + 1]);
                        r[2] = round_to_f32_bits(T[j + 2], ebase + eb_s[j + 2]);
                        r[3] = round_to_f32_bits(T[j + 3], ebase + eb_s[j + 3]);
                    }
                    if (whole) {
                        *reinterpret_cast<uint4*>(dst + j) = make_uint4(r[0], r[1], r[2], r[3]);
                    } else {
#pragma unroll
                        for (int q = 0; q < 4; ++q)
                            if (col0 + j + q < P.N) dst[j + q] = r[q];
                    }
                }
            }
            // ea_rows is rewritten by the next tile's first pass
            __syncwarp();
            if (lane == 0) mbar_arrive(done_bar);
            ok = mbar_wait_relaxed(done_bar, tile_it & 1u, abort_flag, P.status, STATUS_WAIT_TMEM_FULL);
            ok = __all_sync(0xFFFFFFFFu, ok);
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
