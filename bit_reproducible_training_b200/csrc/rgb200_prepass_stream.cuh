// One-kernel split of a k-strided operand (element (r, k) at src[k * R + r]: B without trans_b, A with
// trans_a) that crosses HBM once.
//
// The column maxima over the whole K must be known before the first element can be scaled.  A thread-block
// cluster of eight CTAs owns a panel of 32 columns, CTA c the k range [c * KC, (c + 1) * KC):
//   phase 1  every warp streams k rows of the slab (one 128-byte segment per warp-wide load, eight in flight per
//            lane) and keeps a running maximum per column; the CTA's 32 maxima go to shared memory;
//   exchange the eight CTAs read each other's maxima through distributed shared memory (two cluster barriers);
//   phase 2  the CTA reads its slab again - it was read microseconds ago by the same SM, so it comes from L2 -
//            with the lanes along r: a thread gathers 32 consecutive k of one column (32 independent loads),
//            rounds and splits them, and writes one 32-byte store per digit plane.  No shared-memory staging and
//            no transposing pass: a warp's 32 loads are whole 128-byte lines, its stores whole 32-byte sectors.
// Nothing but the 32 maxima lives in shared memory, so eight CTAs share an SM and their phases overlap.
// Any R, K and alignment; (4 + S) bytes of HBM traffic per element as long as a CTA's slab survives in L2
// between the phases (KC * 128 bytes per CTA).
// Reference counterpart: quantize_kstrided (repro_gemm_cuda/repro_gemm.cu:84-121), which reads the operand twice.
#pragma once
#include <cooperative_groups.h>
#include "rgb200_mma.cuh"
#include "rgb200_prepass.cuh"

namespace rgb200 {

constexpr int KSS_CLUSTER = 8;               // CTAs per cluster (the portable maximum)
constexpr int KSS_W = 32;                    // columns per cluster

// Four consecutive k of one column -> one packed word per digit plane (most significant plane first).
template <int S, bool PLAIN>
__device__ __forceinline__ void quad_words(float a, float b, float c, float d, const QuantScale& q, float limf, uint32_t (&w)[S]) {
    int y0 = biased_fixed_point<S, PLAIN>(a, q, limf), y1 = biased_fixed_point<S, PLAIN>(b, q, limf);
    int y2 = biased_fixed_point<S, PLAIN>(c, q, limf), y3 = biased_fixed_point<S, PLAIN>(d, q, limf);
#pragma unroll
    for (int p = S - 1; p >= 0; --p) {
        uint32_t x = pack_low_bytes(y0, y1, y2, y3);
        if (p > 0) { x = unbias_bytes(x); y0 >>= 7; y1 >>= 7; y2 >>= 7; y3 >>= 7; }
        w[p] = x;
    }
}

// grid = (KSS_CLUSTER * ceil(R / 32), batch), cluster = (KSS_CLUSTER, 1, 1), block = 256 threads.
// KC: k values per CTA, a multiple of 32; Kp: K rounded up to 128 (planes are zero beyond K).
// given_max: externally reduced maxima [batch][R] (K-sharded operation) or null.
template <int S>
__global__ void __cluster_dims__(KSS_CLUSTER, 1, 1) __launch_bounds__(PREPASS_THREADS)
split_kstrided_stream_kernel(const float* __restrict__ src, const float* __restrict__ given_max, int8_t* __restrict__ planes,
                             int* __restrict__ expo, int R, int K, int Kp, int KC, long long src_batch_stride) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    __shared__ float red[PREPASS_THREADS / 32][KSS_W];
    __shared__ float cmax[KSS_W];                          // this CTA's column maxima, read by the whole cluster
    __shared__ int e_sh[KSS_W];
    constexpr int WARPS = PREPASS_THREADS / 32;
    const int rank = (int)cluster.block_rank();
    const int panel = blockIdx.x / KSS_CLUSTER;
    const int b = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r = panel * KSS_W + lane;
    const bool live = r < R;
    const int k0 = rank * KC;
    const int k1 = min(k0 + KC, Kp);                       // planes are written up to Kp
    const int k1_data = min(k1, K);                        // values exist up to K
    const float* col = src + (size_t)b * src_batch_stride + (live ? r : 0);

    // phase 1: column maxima of the slab (rows k0 + warp, k0 + warp + 8, ...)
    float m = 0.0f;
    if (!given_max && live) {
        int k = k0 + warp;
        for (; k + 7 * WARPS < k1_data; k += 8 * WARPS) {
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = __ldg(col + (size_t)(k + i * WARPS) * R);
#pragma unroll
            for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(v[i]));
        }
        for (; k < k1_data; k += WARPS) m = fmaxf(m, fabsf(__ldg(col + (size_t)k * R)));
    }
    red[warp][lane] = m;
    __syncthreads();
    if (threadIdx.x < KSS_W) {
        float mm = red[0][threadIdx.x];
#pragma unroll
        for (int i = 1; i < WARPS; ++i) mm = fmaxf(mm, red[i][threadIdx.x]);
        cmax[threadIdx.x] = mm;
    }
    cluster.sync();                                          // every CTA's maxima are in place
    if (threadIdx.x < KSS_W) {
        float mm = 0.0f;
        if (given_max) {
            mm = live ? given_max[(size_t)b * R + r] : 0.0f;
        } else {
#pragma unroll
            for (int c = 0; c < KSS_CLUSTER; ++c) mm = fmaxf(mm, cluster.map_shared_rank(cmax, c)[threadIdx.x]);
        }
        const int e = scale_exponent(mm);
        e_sh[threadIdx.x] = e;
        if (rank == 0 && live) expo[(size_t)b * R + r] = e;
    }
    cluster.sync();                                          // nobody reads remote shared memory after this point

    // phase 2: thread (column r, warp) turns 32 consecutive k into one 32-byte store per plane
    const int e = e_sh[lane];                                // 0 for columns beyond R
    const QuantScale q = quant_scale(e, S);
    const float limf = (float)q.lim;
    const bool plain = __all_sync(0xFFFFFFFFu, plain_row(e));
    if (!live) return;
    const size_t plane_stride = (size_t)R * Kp;
    int8_t* out = planes + (size_t)b * S * plane_stride + (size_t)r * Kp;
    for (int kk = k0 + warp * 32; kk < k1; kk += WARPS * 32) {
        float v[32];
        if (kk + 32 <= k1_data) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __ldg(col + (size_t)(kk + j) * R);
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = kk + j < k1_data ? __ldg(col + (size_t)(kk + j) * R) : 0.0f;
        }
        uint32_t w[S][8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            uint32_t x[S];
            if (plain) quad_words<S, true>(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3], q, limf, x);
            else quad_words<S, false>(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3], q, limf, x);
#pragma unroll
            for (int p = 0; p < S; ++p) w[p][j] = x[p];
        }
#pragma unroll
        for (int p = 0; p < S; ++p)
            st_global_256(reinterpret_cast<uint32_t*>(out + p * plane_stride + kk),
                          w[p][0], w[p][1], w[p][2], w[p][3], w[p][4], w[p][5], w[p][6], w[p][7]);
    }
}

}  // namespace rgb200
