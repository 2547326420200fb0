// tcgen05 kind::i8 mainloop with TMA-fed operands, TMEM level accumulators and the fused
// exact-recombine-and-round epilogue (sm_100a only).
//
// Work decomposition.  A CTA owns one 128 x NT tile of C at a time (persistent, static round-robin
// over tiles).  The S digit planes of an operand tile are fetched by ONE 4-D TMA box
// (k = 128 bytes, rows, S planes, 1 batch) into 128-byte-swizzled shared memory, so the S planes of
// the B tile sit back to back as a single K-major matrix of S*NT rows.  For every 32-wide k step the
// issuing thread then launches S MMAs, one per A plane p:
//        D[128 x S*NT] += A_p[128 x 32] * [B_0; B_1; ...; B_{S-1}]^T
// with D placed at TMEM column p*NT.  Column block L of TMEM therefore accumulates every digit-plane
// product with p + q = L ("level" L, weight 128^(2S-2-L)): S MMAs per k step cover all S^2 products
// and A_p is read from shared memory once per step.  Only the very first k step of a tile is issued
// as S^2 separate NT-wide MMAs, because there the "overwrite" flag differs between column blocks.
// Level sums are exact in INT32 for max_k_per_pass(S) values of k; the host never gives one pass more.
//
// Epilogue: eight warps read the 2S-1 level accumulators with tcgen05.ld and rebuild
// T = sum_L level_L * 128^(2S-2-L) in INT64 registers (one 32x32->64 multiply-add per level), then
// hand TMEM back to the MMA warp at once, so the next tile's mainloop runs while the epilogue rounds
// once to FP32 (fused; the reference's write_output, repro_gemm_cuda/repro_gemm.cu:124-132, and
// round_to_float) or stores T for a later integer reduction (K ranges, K-sharded multi-GPU).
//
// Reference counterpart of the whole kernel: gemm_wmma_i8<S> (repro_gemm_cuda/repro_gemm.cu:280-364).
//
// Every wait on an mbarrier is bounded: after about two seconds the waiting role records a code in
// the status word, raises a CTA-wide abort flag, and all roles drain and leave through the common
// exit, which frees the CTA's TMEM.
#pragma once
#include <cuda.h>
#include <type_traits>
#include "rgb200_math.cuh"

// Build-time option.  RGB200_TILE_GROUP_M: row tiles per schedule group.
#ifndef RGB200_TILE_GROUP_M
#define RGB200_TILE_GROUP_M 8
#endif

namespace rgb200 {

constexpr int BLOCK_M = 128;
constexpr int BLOCK_K = 128;         // bytes = int8 elements per pipeline stage and per swizzled row
constexpr int UMMA_K = 32;           // k extent of one kind::i8 MMA
constexpr int EPI_WARPS = 8;         // two warps per TMEM lane quarter, each taking half of the tile's columns
constexpr int EPI_THREADS = EPI_WARPS * 32;
constexpr int GEMM_THREADS = 64 + EPI_THREADS;   // warp 0: TMA producer, warp 1: MMA issuer + TMEM owner, then the epilogue
constexpr long long WAIT_LIMIT_CLOCKS = 4000000000ll;   // about two seconds

enum : int {
    STATUS_OK = 0,
    STATUS_WAIT_EMPTY = 1,      // producer gave up waiting for a free pipeline stage
    STATUS_WAIT_FULL = 2,       // MMA issuer gave up waiting for operand bytes
    STATUS_WAIT_TMEM_EMPTY = 3, // MMA issuer gave up waiting for the epilogue to drain TMEM
    STATUS_WAIT_TMEM_FULL = 4,  // epilogue gave up waiting for the accumulators
    STATUS_WAIT_DRAIN = 5       // producer gave up waiting for its own copies during an abort
};

template <int S, int NT>
struct GemmTraits {
    static constexpr int LEVELS = 2 * S - 1;
    static constexpr int A_PLANE_BYTES = BLOCK_M * BLOCK_K;
    static constexpr int B_PLANE_BYTES = NT * BLOCK_K;
    static constexpr int A_STAGE_BYTES = S * A_PLANE_BYTES;
    static constexpr int B_STAGE_BYTES = S * B_PLANE_BYTES;
    static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
    static constexpr int SMEM_BUDGET = 220 * 1024;
    static constexpr int STAGES_RAW = SMEM_BUDGET / STAGE_BYTES;
    static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
    static constexpr int TMEM_COLS_USED = LEVELS * NT;
    static constexpr int TMEM_COLS = TMEM_COLS_USED <= 32 ? 32 : TMEM_COLS_USED <= 64 ? 64 :
                                     TMEM_COLS_USED <= 128 ? 128 : TMEM_COLS_USED <= 256 ? 256 : 512;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */ +
                                      EPI_WARPS * (NT / 2) * 4 /* column exponents, one slot per epilogue warp */;
    static_assert(TMEM_COLS_USED <= 512, "level accumulators do not fit TMEM");
    static_assert(S * NT <= 256 && (S * NT) % 16 == 0 && NT % 16 == 0, "invalid UMMA N");
    static_assert(STAGES >= 2, "pipeline needs two stages");
};

struct GemmParams {
    const int* expo_a;       // [batch][M]
    const int* expo_b;       // [batch][N]
    float* C;                // fused-rounding output, or null
    long long* partial;      // INT64 output [split][batch][M][N], or null
    int* status;             // one word, zero on entry
    int M, N;
    int batch;
    long long stride_c;      // elements between consecutive batches of C
    int k_blocks;            // total number of 128-wide k blocks
    int split;               // number of K ranges
    int m_tiles, n_tiles;
    int e0;                  // -14 (S - 1)
    // Row-block scatter of the INT64 output (K-sharded multi-GPU): rows [o * scatter_rows, (o+1) * scatter_rows)
    // go to scatter[o], the buffer of the rank that owns them (its own or a peer's memory over NVLink), into
    // slot `scatter_slot`.  A slot is stored tile by tile in the order the epilogue produces it (see
    // scatter_offset), so every store instruction of a warp covers one contiguous kilobyte.
    // scatter_rows == 0: off; otherwise a multiple of 128.
    long long* scatter[8];
    int scatter_rows, scatter_slot;
    // Row tiles are visited starting at tile scatter_rot (and wrapping around): every rank starts with the rows of the
    // owner after itself and ends with its own, so that at any moment the ranks send to different owners and no
    // owner's NVLink ingress has to take all of them at once.
    int scatter_rot;
    // Image-major C (kernels built with IMAGE_MAJOR_C): row r = image * c_image_rows + place, and element
    // (r, col) is stored at C[(image * N + col) * c_image_rows + place], the [N, F, OH, OW] / [N, C, H, W]
    // layouts of a convolution's results.  A warp's 32 rows are consecutive places, so each column is one
    // 128-byte store.  0 in the row-major kernels.
    int c_image_rows;
};

// ------------------------------------------------------------------------------------------
// PTX wrappers
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    return done;
}

// Bounded wait.  Returns false after the limit or once another role has raised the abort flag.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code,
                                          long long limit = WAIT_LIMIT_CLOCKS) {
    if (mbar_try_wait(bar, parity)) return true;
    long long t0 = clock64();
    for (uint32_t spins = 1;; ++spins) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spins & 63u) == 0) {
            if (*abort_flag) return false;
            if (clock64() - t0 > limit) {
                atomicCAS(status, 0, code);
                *abort_flag = 1;
                __threadfence_block();
                return false;
            }
        }
    }
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem]^T, int8 x int8 -> int32, issued by one thread.
__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrive on an mbarrier once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 32 lanes x 16 consecutive 32-bit columns: thread i of the warp receives row (lane base + i).
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, int (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor: K-major, 128-byte swizzle, rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4)      // start address
         | (1ull << 16)                              // leading byte offset (unused with swizzled K-major)
         | ((uint64_t)(1024 >> 4) << 32)             // stride byte offset between 8-row groups
         | (1ull << 46)                              // descriptor version of this architecture
         | (2ull << 61);                             // 128-byte swizzle
}
// Instruction descriptor: int8 x int8 -> int32, both operands K-major, dense, no saturation.
__host__ __device__ constexpr uint32_t idesc_i8(int m, int n) {
    return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// The 64-bit shared-memory matrix descriptor of smem_desc_sw128 in two halves: the upper word is a constant, and
// the lower word of an operand at a byte offset (a multiple of 16) is the base's lower word plus offset / 16, so
// the issuing thread - a single thread whose instruction latency competes with the tensor pipe's time per MMA - spends one
// addition per operand.
constexpr uint32_t SW128_DESC_HI = (uint32_t)(1024 >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t sw128_desc_lo(uint32_t saddr) { return ((saddr & 0x3FFFFu) >> 4) | (1u << 16); }
template <bool ACCUMULATE>
__device__ __forceinline__ void umma_i8_lo(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "mov.b64 da, {%1, %5};\n\t"
        "mov.b64 db, {%2, %5};\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], da, db, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "n"(ACCUMULATE ? 1 : 0), "r"(SW128_DESC_HI) : "memory");
}

// First k step of a tile: level L = p + q is written for the first time by (p = 0, q = L) or, for L >= S, by
// (p = L - S + 1, q = S - 1), and accumulated into by every other pair.  So A plane 0 takes one MMA over all S
// planes of B that overwrites levels 0..S-1, and every further A plane p one MMA over B planes 0..S-2 that
// accumulates into levels p..p+S-2 plus one over B plane S-1 that overwrites the new level p+S-1:
// 2S-1 MMAs.  sa / sb: shared-memory addresses of the operands' plane 0 at this k step.
template <int S, int NT>
__device__ __forceinline__ void issue_first_k_step(uint32_t acc, uint32_t sa, uint32_t sb, uint32_t a_plane_bytes,
                                                   uint32_t b_plane_bytes) {
    const uint32_t a_lo = sw128_desc_lo(sa), b_lo = sw128_desc_lo(sb);
    umma_i8_lo<false>(acc, a_lo, b_lo, idesc_i8(BLOCK_M, S * NT));
#pragma unroll
    for (int p = 1; p < S; ++p) {
        umma_i8_lo<true>(acc + p * NT, a_lo + p * (a_plane_bytes >> 4), b_lo, idesc_i8(BLOCK_M, (S - 1) * NT));
        umma_i8_lo<false>(acc + (p + S - 1) * NT, a_lo + p * (a_plane_bytes >> 4), b_lo + (S - 1) * (b_plane_bytes >> 4),
                          idesc_i8(BLOCK_M, NT));
    }
}

// ------------------------------------------------------------------------------------------
// Tile schedule shared by the three roles.  Order: batch-major, then K range, then groups of 16
// row tiles swept column tile by column tile, so CTAs running together share operand panels in L2.
// ------------------------------------------------------------------------------------------
struct TileCoord { int batch, z, m_blk, n_blk, kb_begin, kb_end; };

__device__ __forceinline__ TileCoord tile_coord(const GemmParams& P, long long tile) {
    const int GROUP = RGB200_TILE_GROUP_M;
    long long per_mat = (long long)P.m_tiles * P.n_tiles;
    long long bz = tile / per_mat;
    int t = (int)(tile - bz * per_mat);
    TileCoord c;
    c.batch = (int)(bz / P.split);
    c.z = (int)(bz - (long long)c.batch * P.split);
    int group_size = GROUP * P.n_tiles;
    int g = t / group_size, in_g = t - g * group_size;
    int rows_here = min(GROUP, P.m_tiles - g * GROUP);
    c.n_blk = in_g / rows_here;
    c.m_blk = g * GROUP + (in_g - c.n_blk * rows_here);
    if (P.scatter_rot) {
        c.m_blk += P.scatter_rot;
        if (c.m_blk >= P.m_tiles) c.m_blk -= P.m_tiles;
    }
    c.kb_begin = (int)((long long)P.k_blocks * c.z / P.split);
    c.kb_end = (int)((long long)P.k_blocks * (c.z + 1) / P.split);
    return c;
}

// 32-byte global stores (one full sector per lane and instruction); the address must be 32-byte aligned.
__device__ __forceinline__ void st_global_256(uint32_t* p, uint32_t a, uint32_t b, uint32_t c, uint32_t d,
                                              uint32_t e, uint32_t f, uint32_t g, uint32_t h) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"l"(p), "r"(a), "r"(b), "r"(c), "r"(d), "r"(e), "r"(f), "r"(g), "r"(h) : "memory");
}
__device__ __forceinline__ void st_global_256(long long* p, long long a, long long b, long long c, long long d) {
    asm volatile("st.global.v4.b64 [%0], {%1, %2, %3, %4};" ::"l"(p), "l"(a), "l"(b), "l"(c), "l"(d) : "memory");
}

// Stores CPT consecutive values of one row whose start is HEAD elements before a 16-byte boundary:
// HEAD scalar stores, then 16-byte stores, then the scalar rest.  Rows of C are 16-byte aligned only
// when N % 4 == 0 (and the base pointer is); for ragged N the alignment changes from row to row.
template <int CPT, int HEAD>
__device__ __forceinline__ void store_row_u32(uint32_t* dst, const uint32_t (&o)[CPT]) {
#pragma unroll
    for (int j = 0; j < HEAD; ++j) dst[j] = o[j];
    constexpr int BODY = (CPT - HEAD) / 4;
#pragma unroll
    for (int i = 0; i < BODY; ++i)
        *reinterpret_cast<uint4*>(dst + HEAD + 4 * i) = make_uint4(o[HEAD + 4 * i], o[HEAD + 4 * i + 1], o[HEAD + 4 * i + 2], o[HEAD + 4 * i + 3]);
#pragma unroll
    for (int j = HEAD + 4 * BODY; j < CPT; ++j) dst[j] = o[j];
}
template <int CPT, int HEAD, class TAcc>
__device__ __forceinline__ void store_row_i64(long long* dst, const TAcc (&t)[CPT]) {
    if (HEAD) dst[0] = t[0];
    constexpr int BODY = (CPT - HEAD) / 2;
#pragma unroll
    for (int i = 0; i < BODY; ++i)
        *reinterpret_cast<longlong2*>(dst + HEAD + 2 * i) = make_longlong2((long long)t[HEAD + 2 * i], (long long)t[HEAD + 2 * i + 1]);
    if (HEAD) dst[CPT - 1] = t[CPT - 1];
}

// Tile-native layout of one slot of a scatter buffer.  A slot holds the owner's rows as
// [row tile][column tile][w = 0..7][store j][lane 0..31][4] INT64, where w = 4 * (column half) + (TMEM lane
// quarter), i.e. block w covers quarter w % 4 (rows 32 (w % 4) .. +31 of the tile) and column half w / 4, and store j covers columns
// 4 j .. 4 j + 3 of that half.  Returns the element offset of (tile, warp, j, lane) inside the slot.
template <int NT>
__host__ __device__ __forceinline__ size_t scatter_offset(int m_local, int n_blk, int n_tiles, int w, int j, int lane) {
    constexpr int CPT = NT / 2;
    return ((((size_t)m_local * n_tiles + n_blk) * 8 + w) * (CPT / 4) + j) * 128 + (size_t)lane * 4;
}

// Position in the flattened (tile, k block) sequence a CTA works through.
struct KCursor { long long tile; TileCoord tc; int kb; bool valid; };

__device__ __forceinline__ void cursor_start(KCursor& c, const GemmParams& P, long long first, long long total) {
    c.tile = first;
    c.valid = first < total;
    if (c.valid) { c.tc = tile_coord(P, first); c.kb = c.tc.kb_begin; }
}
__device__ __forceinline__ void cursor_next(KCursor& c, const GemmParams& P, long long stride, long long total) {
    if (++c.kb < c.tc.kb_end) return;
    c.tile += stride;
    c.valid = c.tile < total;
    if (c.valid) { c.tc = tile_coord(P, c.tile); c.kb = c.tc.kb_begin; }
}

// IMAGE_MAJOR_C (the convolutions): the rows of the product are (image, place) pairs and C is stored
// [image][column][place], see GemmParams::c_image_rows; only the FP32 store of the epilogue differs.
template <int S, int NT, bool IMAGE_MAJOR_C = false>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_i8_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                       const GemmParams P) {
    using Tr = GemmTraits<S, NT>;
    constexpr int STAGES = Tr::STAGES;
    extern __shared__ uint8_t smem_raw[];
    // operand stages need 1024-byte alignment for the 128-byte swizzle pattern
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar_base = smem_base + STAGES * Tr::STAGE_BYTES;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    const uint32_t tmem_full_bar = bar_base + 8u * (2 * STAGES);
    const uint32_t tmem_empty_bar = bar_base + 8u * (2 * STAGES + 1);
    const uint32_t tmem_slot = bar_base + 8u * (2 * STAGES + 2);
    uint8_t* gen_base = smem_raw + (smem_base - smem_u32(smem_raw));
    volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(gen_base + STAGES * Tr::STAGE_BYTES + 8 * (2 * STAGES + 2));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + STAGES * Tr::STAGE_BYTES + 8 * (2 * STAGES + 3));
    int* eb_slots = reinterpret_cast<int*>(gen_base + STAGES * Tr::STAGE_BYTES + 256);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long total_tiles = (long long)P.batch * P.split * P.m_tiles * P.n_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        mbar_init(tmem_full_bar, 1);
        mbar_init(tmem_empty_bar, EPI_THREADS);
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
            uint32_t it = 0;
            bool ok = true;
            KCursor ld;
            cursor_start(ld, P, blockIdx.x, total_tiles);
            for (; ld.valid; ++it) {
                const int s = it % STAGES;
                const uint32_t ph = (it / STAGES) & 1u;
                if (!(ok = mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, P.status, STATUS_WAIT_EMPTY))) break;
                const uint32_t sa = smem_base + s * Tr::STAGE_BYTES;
                mbar_arrive_expect_tx(full_bar(s), Tr::STAGE_BYTES);
                tma_load_4d(sa, &tmap_a, full_bar(s), ld.kb * BLOCK_K, ld.tc.m_blk * BLOCK_M, 0, ld.tc.batch);
                tma_load_4d(sa + Tr::A_STAGE_BYTES, &tmap_b, full_bar(s), ld.kb * BLOCK_K, ld.tc.n_blk * NT, 0, ld.tc.batch);
                cursor_next(ld, P, gridDim.x, total_tiles);
            }
            if (!ok) {
                // abort: let copies that are still in flight land before the CTA gives up its shared memory
                const uint32_t issued = it < (uint32_t)STAGES ? it : (uint32_t)STAGES;
                for (uint32_t j = 0; j < issued; ++j) {
                    const uint32_t i2 = it - 1 - j;
                    long long t0 = clock64();
                    while (!mbar_try_wait(full_bar(i2 % STAGES), (i2 / STAGES) & 1u)) {
                        if (clock64() - t0 > WAIT_LIMIT_CLOCKS) { atomicCAS(P.status, 0, STATUS_WAIT_DRAIN); break; }
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t IDESC_WIDE = idesc_i8(BLOCK_M, S * NT);
            uint32_t it = 0, tile_it = 0;
            bool ok = true;
            for (long long tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++tile_it) {
                const TileCoord tc = tile_coord(P, tile);
                if (!(ok = mbar_wait(tmem_empty_bar, (tile_it & 1u) ^ 1u, abort_flag, P.status, STATUS_WAIT_TMEM_EMPTY))) break;
                tc_fence_after();
                for (int kb = tc.kb_begin; kb < tc.kb_end; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1u;
                    if (!(ok = mbar_wait(full_bar(s), ph, abort_flag, P.status, STATUS_WAIT_FULL))) break;
                    tc_fence_after();
                    const uint32_t sa = smem_base + s * Tr::STAGE_BYTES;
                    const uint32_t sb = sa + Tr::A_STAGE_BYTES;
                    const uint32_t a_lo = sw128_desc_lo(sa), b_lo = sw128_desc_lo(sb);
#pragma unroll
                    for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
                        if (kb == tc.kb_begin && k == 0) {
                            // first k step of the tile: 2S-1 MMAs that overwrite each level where it is first written
                            issue_first_k_step<S, NT>(tmem_base, sa, sb, Tr::A_PLANE_BYTES, Tr::B_PLANE_BYTES);
                        } else {
#pragma unroll
                            for (int p = 0; p < S; ++p)
                                umma_i8_lo<true>(tmem_base + p * NT, a_lo + p * (Tr::A_PLANE_BYTES >> 4) + k * (UMMA_K >> 4),
                                                 b_lo + k * (UMMA_K >> 4), IDESC_WIDE);
                        }
                    }
                    umma_commit(empty_bar(s));          // frees the stage once these MMAs have read it
                }
                if (ok) umma_commit(tmem_full_bar);     // accumulators complete
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue (warps 2..9)
        constexpr int CPT = NT / 2;                    // columns per thread
        static_assert(CPT % 16 == 0, "epilogue reads TMEM sixteen columns at a time");
        // exact sums kept in registers between the TMEM drain and the rounding: one level (S = 1) fits INT32
        using TAcc = typename std::conditional<S == 1, int, long long>::type;
        static_assert(CPT * (S == 1 ? 1 : 2) <= 128, "the tile's sums must fit the register file");
        const int quarter = warp & 3;                  // TMEM lanes this warp may read: 32*quarter .. +31
        const int half = (warp - 2) >> 2;              // which half of the tile's columns
        const int row_in_tile = quarter * 32 + lane;
        uint32_t tile_it = 0;
        bool ok = true;
        for (long long tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++tile_it) {
            const TileCoord tc = tile_coord(P, tile);
            const int row = tc.m_blk * BLOCK_M + row_in_tile;
            const bool row_ok = row < P.M;
            const int ea = row_ok ? __ldg(P.expo_a + (size_t)tc.batch * P.M + row) : 0;
            const int col0 = tc.n_blk * NT + half * CPT;
            // this warp's column exponents go through its own shared-memory slot: one coalesced load here,
            // issued before the wait below, instead of a dependent global load per output in phase 2
            int* eb_s = eb_slots + (warp - 2) * CPT;
            __syncwarp();
            if (!P.partial)
                for (int c = lane; c < CPT; c += 32)
                    eb_s[c] = col0 + c < P.N ? __ldg(P.expo_b + (size_t)tc.batch * P.N + col0 + c) : 0;
            __syncwarp();
            ok = mbar_wait(tmem_full_bar, tile_it & 1u, abort_flag, P.status, STATUS_WAIT_TMEM_FULL);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (!ok) break;
            tc_fence_after();
            // phase 1: accumulators -> exact INT64 sums in registers, then release TMEM
            const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + half * CPT;
            TAcc T[CPT];
#pragma unroll
            for (int c0 = 0; c0 < CPT; c0 += 16) {
                int lv[Tr::LEVELS][16];
#pragma unroll
                for (int L = 0; L < Tr::LEVELS; ++L) tmem_ld16(t_row + L * NT + c0, lv[L]);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    long long t = lv[Tr::LEVELS - 1][j];
#pragma unroll
                    for (int L = Tr::LEVELS - 2; L >= 0; --L)
                        t += (long long)lv[L][j] * (long long)(1 << (7 * (Tr::LEVELS - 1 - L)));
                    T[c0 + j] = (TAcc)t;
                }
            }
            tc_fence_before();
            mbar_arrive(tmem_empty_bar);
            // phase 2: one rounding per output (or the raw sums), overlapped with the next tile's MMAs
            if (!P.scatter_rows && (!row_ok || col0 >= P.N)) continue;
            if (P.partial) {
                long long* dst = P.partial + (((size_t)tc.z * P.batch + tc.batch) * P.M + row) * P.N + col0;
                if (P.scatter_rows) {          // ordinary global stores into the owner's memory (its own or a peer's)
                    const int owner = row / P.scatter_rows;
                    const int m_local = tc.m_blk - owner * (P.scatter_rows / BLOCK_M);
                    const size_t slot_elems = (size_t)P.scatter_rows * P.n_tiles * NT;
                    long long* base = P.scatter[owner] + (size_t)P.scatter_slot * slot_elems;
#pragma unroll
                    for (int j = 0; j < CPT / 4; ++j)
                        st_global_256(base + scatter_offset<NT>(m_local, tc.n_blk, P.n_tiles, (half << 2) | quarter, j, lane),
                                      (long long)T[4 * j], (long long)T[4 * j + 1], (long long)T[4 * j + 2], (long long)T[4 * j + 3]);
                    continue;
                }
                if (col0 + CPT <= P.N) {
                    if ((reinterpret_cast<uintptr_t>(dst) & 31) == 0) {
#pragma unroll
                        for (int j = 0; j < CPT; j += 4)
                            st_global_256(dst + j, (long long)T[j], (long long)T[j + 1], (long long)T[j + 2], (long long)T[j + 3]);
                    } else if ((reinterpret_cast<uintptr_t>(dst) & 8) == 0) store_row_i64<CPT, 0>(dst, T);
                    else store_row_i64<CPT, 1>(dst, T);
                } else {
#pragma unroll
                    for (int j = 0; j < CPT; ++j) if (col0 + j < P.N) dst[j] = T[j];
                }
            } else {
                uint32_t* dst = reinterpret_cast<uint32_t*>(P.C + (size_t)tc.batch * P.stride_c + (size_t)row * P.N + col0);
                const int ebase = ea + P.e0;
                auto round4 = [&](int j, uint32_t (&r)[4]) {
                    bool k0, k1, k2, k3;
                    r[0] = round_to_f32_bits_signed(T[j + 0], ebase + eb_s[j + 0], &k0);
                    r[1] = round_to_f32_bits_signed(T[j + 1], ebase + eb_s[j + 1], &k1);
                    r[2] = round_to_f32_bits_signed(T[j + 2], ebase + eb_s[j + 2], &k2);
                    r[3] = round_to_f32_bits_signed(T[j + 3], ebase + eb_s[j + 3], &k3);
                    if (!(k0 && k1 && k2 && k3)) {          // zero, subnormal or overflowing results: exact path
                        r[0] = round_to_f32_bits(T[j + 0], ebase + eb_s[j + 0]);
                        r[1] = round_to_f32_bits(T[j + 1], ebase + eb_s[j + 1]);
                        r[2] = round_to_f32_bits(T[j + 2], ebase + eb_s[j + 2]);
                        r[3] = round_to_f32_bits(T[j + 3], ebase + eb_s[j + 3]);
                    }
                };
                if (IMAGE_MAJOR_C) {
                    // lanes are consecutive places of an image: every column is one contiguous 128-byte store per warp
                    const int image = row / P.c_image_rows, place = row - image * P.c_image_rows;
                    dst = reinterpret_cast<uint32_t*>(P.C) + ((size_t)image * P.N + col0) * P.c_image_rows + place;
#pragma unroll
                    for (int j = 0; j < CPT; j += 4) {
                        uint32_t r[4];
                        round4(j, r);
#pragma unroll
                        for (int q = 0; q < 4; ++q)
                            if (col0 + j + q < P.N) dst[(size_t)(j + q) * P.c_image_rows] = r[q];
                    }
                    continue;
                }
                const int past = (int)((reinterpret_cast<uintptr_t>(dst) >> 2) & 3);    // elements past a 16-byte boundary
                if ((reinterpret_cast<uintptr_t>(dst) & 31) == 0 && col0 + CPT <= P.N) {
                    // sector-aligned row segment: round eight, store one full 32-byte sector
#pragma unroll
                    for (int j = 0; j < CPT; j += 8) {
                        uint32_t r[4], q[4];
                        round4(j, r);
                        round4(j + 4, q);
                        st_global_256(dst + j, r[0], r[1], r[2], r[3], q[0], q[1], q[2], q[3]);
                    }
                } else if (past == 0 && col0 + CPT <= P.N) {
                    // aligned row segment: round four, store sixteen bytes, so stores overlap the next roundings
#pragma unroll
                    for (int j = 0; j < CPT; j += 4) {
                        uint32_t r[4];
                        round4(j, r);
                        *reinterpret_cast<uint4*>(dst + j) = make_uint4(r[0], r[1], r[2], r[3]);
                    }
                } else {
                    uint32_t o[CPT];
#pragma unroll
                    for (int j = 0; j < CPT; j += 4) {
                        uint32_t r[4];
                        round4(j, r);
                        o[j] = r[0]; o[j + 1] = r[1]; o[j + 2] = r[2]; o[j + 3] = r[3];
                    }
                    if (col0 + CPT <= P.N) {
                        if (past == 1) store_row_u32<CPT, 3>(dst, o);
                        else if (past == 2) store_row_u32<CPT, 2>(dst, o);
                        else store_row_u32<CPT, 1>(dst, o);
                    } else {
#pragma unroll
                        for (int j = 0; j < CPT; ++j) if (col0 + j < P.N) dst[j] = o[j];
                    }
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

// Self-test of the bounded wait: one warp waits on a barrier that nothing will ever complete, with a
// short limit.  Lane 0 must give up after `limit` clocks, store `code` in *status and raise the abort
// flag; lane 1, waiting with the full limit, must leave early because it sees that flag.
// out[0] = lane 0 returned false, out[1] = lane 1 returned false, out[2] = clocks lane 0 waited.
__global__ void bounded_wait_probe_kernel(int* status, long long limit, long long* out) {
    __shared__ __align__(8) unsigned long long bar;
    __shared__ int abort_flag;
    const uint32_t b = smem_u32(&bar);
    if (threadIdx.x == 0) {
        mbar_init(b, 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        long long t0 = clock64();
        bool ok = mbar_wait(b, 0, &abort_flag, status, STATUS_WAIT_FULL, limit);
        out[0] = ok ? 0 : 1;
        out[2] = clock64() - t0;
    } else if (threadIdx.x == 32) {
        bool ok = mbar_wait(b, 0, &abort_flag, status, STATUS_WAIT_EMPTY);
        out[1] = ok ? 0 : 1;
    }
}

// ------------------------------------------------------------------------------------------
// Verification path (RGB200_ALGO_REFERENCE): the definition on CUDA cores, one thread per output,
// digits re-assembled to the fixed-point integers and multiplied in INT64.
// Reference counterpart: gemm_reference (repro_gemm_cuda/repro_gemm.cu:139-153).
// grid = (ceil(N/16), ceil(M/16), batch)
// ------------------------------------------------------------------------------------------
template <int S>
__global__ void gemm_int64_check_kernel(const int8_t* __restrict__ qa, const int8_t* __restrict__ qb,
                                        const int* __restrict__ ea, const int* __restrict__ eb, float* __restrict__ C,
                                        int M, int N, int Kp, long long stride_c, int e0) {
    const int col = blockIdx.x * 16 + threadIdx.x, row = blockIdx.y * 16 + threadIdx.y, b = blockIdx.z;
    if (row >= M || col >= N) return;
    const size_t pa = (size_t)M * Kp, pb = (size_t)N * Kp;
    const int8_t* x = qa + (size_t)b * S * pa + (size_t)row * Kp;
    const int8_t* y = qb + (size_t)b * S * pb + (size_t)col * Kp;
    long long t = 0;
    for (int k = 0; k < Kp; ++k) {
        int X = 0, Y = 0;
#pragma unroll
        for (int p = 0; p < S; ++p) { X = X * 128 + x[p * pa + k]; Y = Y * 128 + y[p * pb + k]; }
        t += (long long)X * Y;
    }
    C[(size_t)b * stride_c + (size_t)row * N + col] =
        bits_f32(round_to_f32_bits(t, ea[(size_t)b * M + row] + eb[(size_t)b * N + col] + e0));
}

// C = round(sum over `parts` INT64 partials); the reference's reduce_round (repro_gemm.cu:156-165).
// partial is [parts][batch*M*N]; exponents either precomputed (ea/eb) or derived from maxima.
// VEC: four consecutive columns per thread with 32-byte loads and 16-byte stores (N % 4 == 0, aligned
// buffers, dense C); otherwise one element per thread.  Grid-stride loop.
template <bool VEC>
__global__ void __launch_bounds__(256)
round_partial_kernel(const long long* __restrict__ partial, int parts, size_t part_stride,
                     const int* __restrict__ ea, const int* __restrict__ eb,
                     const float* __restrict__ max_a, const float* __restrict__ max_b,
                     float* __restrict__ C, int M, int N, int batch, long long stride_c, int e0) {
    constexpr int W = VEC ? 4 : 1;
    const size_t per_mat = (size_t)M * N;
    const size_t total = (size_t)batch * per_mat / W;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t idx = i * W;
        long long t[W];
#pragma unroll
        for (int j = 0; j < W; ++j) t[j] = 0;
        for (int p = 0; p < parts; ++p) {
            const long long* src = partial + (size_t)p * part_stride + idx;
            if (VEC) {
                longlong4 v = *reinterpret_cast<const longlong4*>(src);
                t[0] += v.x; t[W > 1 ? 1 : 0] += v.y; t[W > 2 ? 2 : 0] += v.z; t[W > 3 ? 3 : 0] += v.w;
            } else {
                t[0] += src[0];
            }
        }
        const size_t b = idx / per_mat, rc = idx - b * per_mat;
        const int r = (int)(rc / N), c = (int)(rc - (size_t)r * N);
        const int e_r = (ea ? ea[b * M + r] : scale_exponent(max_a[b * M + r])) + e0;
        uint32_t o[W];
#pragma unroll
        for (int j = 0; j < W; ++j) {
            const int e_c = eb ? eb[b * N + c + j] : scale_exponent(max_b[b * N + c + j]);
            o[j] = round_to_f32_bits(t[j], e_r + e_c);
        }
        float* dst = C + b * (size_t)stride_c + (size_t)r * N + c;
        if (VEC) *reinterpret_cast<uint4*>(dst) = make_uint4(o[0], o[W > 1 ? 1 : 0], o[W > 2 ? 2 : 0], o[W > 3 ? 3 : 0]);
        else dst[0] = bits_f32(o[0]);
    }
}

// Owner-side finish of the scattered K-shard reduction: adds the `world` slots of a tile-native scatter
// buffer (see scatter_offset), rounds once and writes the owner's rows of C densely ([rows][N]).
// A warp reads one contiguous kilobyte per slot (lane = row within a 32-row group, four columns each).
template <int NT>
__global__ void __launch_bounds__(256)
round_scattered_kernel(const long long* __restrict__ buffer, int world, const float* __restrict__ max_a,
                       const float* __restrict__ max_b, float* __restrict__ C, int rows, int N, int n_tiles, int e0) {
    constexpr int CPT = NT / 2;
    const size_t slot_elems = (size_t)rows * n_tiles * NT;
    const size_t chunks = slot_elems / 4;                       // 32-byte chunks per slot
    for (size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x; t < chunks; t += (size_t)gridDim.x * blockDim.x) {
        const int lane = (int)(t & 31);
        size_t u = t >> 5;
        const int j = (int)(u % (CPT / 4)); u /= (CPT / 4);
        const int w = (int)(u & 7); u >>= 3;
        const int n_blk = (int)(u % n_tiles);
        const int m_local = (int)(u / n_tiles);
        const int row = m_local * BLOCK_M + (w & 3) * 32 + lane;
        const int col = n_blk * NT + (w >> 2) * CPT + 4 * j;
        if (col >= N) continue;
        long long s0 = 0, s1 = 0, s2 = 0, s3 = 0;
        for (int p = 0; p < world; ++p) {
            const longlong4 v = *reinterpret_cast<const longlong4*>(buffer + (size_t)p * slot_elems + t * 4);
            s0 += v.x; s1 += v.y; s2 += v.z; s3 += v.w;
        }
        const int e_r = scale_exponent(max_a[row]) + e0;
        float* dst = C + (size_t)row * N + col;
        const long long sum[4] = {s0, s1, s2, s3};
#pragma unroll
        for (int q = 0; q < 4; ++q)
            if (col + q < N) dst[q] = bits_f32(round_to_f32_bits(sum[q], e_r + scale_exponent(max_b[col + q])));
    }
}

}  // namespace rgb200
