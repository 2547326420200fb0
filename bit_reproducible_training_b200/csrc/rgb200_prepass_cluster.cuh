// Single-read split of a k-strided operand (element (r, k) at src[k * R + r]: B without trans_b, A with
// trans_a) by thread-block clusters.
//
// The column maxima over the whole K must be known before the first element can be scaled, which made the
// plain form read the operand twice (maxima kernel, then split kernel).  Here a cluster of eight CTAs owns a
// panel of W columns: CTA c of the cluster fetches the k range [c * KC, (c + 1) * KC) of the panel into its
// shared memory with TMA (2-D boxes of W floats x 64 k, zero-filled beyond K and R), takes the column maxima of
// its slab, the eight CTAs exchange their W maxima through distributed shared memory, and every CTA then
// splits its slab from shared memory: the operand crosses HBM once, (4 + S) bytes per element.
// The slab is read along r by the lanes (conflict-free) and every thread turns 32 consecutive k of one column
// into one 32-byte store per digit plane, so no transposing staging pass is needed either.
// Reference counterpart: quantize_kstrided (repro_gemm_cuda/repro_gemm.cu:84-121).
#pragma once
#include <cooperative_groups.h>
#include <cuda.h>
#include "rgb200_mma.cuh"
#include "rgb200_prepass.cuh"

namespace rgb200 {

constexpr int KSC_CLUSTER = 8;               // CTAs per cluster (the portable maximum)
constexpr int KSC_BOX_K = 64;                // k rows per TMA box
constexpr int KSC_MAX_SLAB_BYTES = 192 * 1024;

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

// grid = (KSC_CLUSTER * ceil(R / W), batch), cluster = (KSC_CLUSTER, 1, 1), block = 256 threads,
// dynamic shared memory = KC * W * 4 bytes.  KC is a multiple of 64; Kp a multiple of 128.
// tmap: 3-D FP32 map (r, k, batch) with box (W, 64, 1), no swizzle, zero fill.
// given_max: externally reduced maxima [batch][R] (K-sharded operation) or null.
// status: word that receives STATUS_WAIT_FULL if the slab never arrives (the cluster still leaves in step).
template <int S, int W>
__global__ void __cluster_dims__(KSC_CLUSTER, 1, 1) __launch_bounds__(PREPASS_THREADS)
split_kstrided_cluster_kernel(const __grid_constant__ CUtensorMap tmap, const float* __restrict__ given_max,
                              int8_t* __restrict__ planes, int* __restrict__ expo, int R, int K, int Kp, int KC, int* status) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    extern __shared__ uint8_t slab_raw[];
    // [KC][W] floats, 128-byte aligned for the TMA boxes (the launch reserves 128 bytes of slack)
    float* slab = reinterpret_cast<float*>(slab_raw + ((128u - (smem_u32(slab_raw) & 127u)) & 127u));
    __shared__ __align__(8) unsigned long long bar_mem;
    __shared__ float red[PREPASS_THREADS];
    __shared__ float cmax[W];                               // this CTA's column maxima, read by the whole cluster
    __shared__ int e_sh[W];
    constexpr int G = PREPASS_THREADS / W;                  // k groups working side by side
    const int rank = (int)cluster.block_rank();
    const int panel = blockIdx.x / KSC_CLUSTER;
    const int b = blockIdx.y;
    const int r = threadIdx.x % W, g = threadIdx.x / W;
    const int r_glob = panel * W + r;
    const int k0 = rank * KC;
    const int k1 = min(k0 + KC, Kp);
    const int nk = max(k1 - k0, 0);                         // multiple of 64
    const uint32_t bar = smem_u32(&bar_mem);
    // a split of the other operand launched behind this one with programmatic serialization may start now
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (threadIdx.x == 0) {
        mbar_init(bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    bool arrived = true;
    if (nk > 0) {
        if (threadIdx.x == 0) {
            mbar_arrive_expect_tx(bar, (uint32_t)nk * W * 4u);
            for (int kk = 0; kk < nk; kk += KSC_BOX_K)
                tma_load_3d(smem_u32(slab + (size_t)kk * W), &tmap, bar, panel * W, k0 + kk, b);
        }
        // bounded wait for the slab; on expiry the CTA records it and goes on to the cluster barriers without data
        long long c0 = clock64();
        while (!mbar_try_wait(bar, 0)) {
            if (clock64() - c0 > WAIT_LIMIT_CLOCKS) { arrived = false; break; }
        }
        if (!arrived && threadIdx.x == 0 && status) atomicCAS(status, 0, STATUS_WAIT_FULL);
    }
    arrived = __syncthreads_and(arrived);

    // column maxima of this slab
    float m = 0.0f;
    if (!given_max && arrived)
        for (int k = g; k < nk; k += G) m = fmaxf(m, fabsf(slab[(size_t)k * W + r]));
    red[threadIdx.x] = m;
    __syncthreads();
    if (threadIdx.x < W) {
        float mm = red[threadIdx.x];
#pragma unroll
        for (int i = 1; i < G; ++i) mm = fmaxf(mm, red[i * W + threadIdx.x]);
        cmax[threadIdx.x] = mm;
    }
    cluster.sync();                                          // every CTA's maxima are in place
    if (threadIdx.x < W) {
        float mm = 0.0f;
        if (given_max) {
            mm = r_glob < R ? given_max[(size_t)b * R + r_glob] : 0.0f;
        } else {
#pragma unroll
            for (int c = 0; c < KSC_CLUSTER; ++c) mm = fmaxf(mm, cluster.map_shared_rank(cmax, c)[threadIdx.x]);
        }
        const int e = scale_exponent(mm);
        e_sh[threadIdx.x] = e;
        if (rank == 0 && r_glob < R) expo[(size_t)b * R + r_glob] = e;
    }
    cluster.sync();                                          // nobody reads remote shared memory after this point

    // split: thread (r, g) turns 32 consecutive k of column r into one 32-byte store per plane
    const int e = e_sh[r];                                   // 0 for columns beyond R (their maxima read as zero)
    const QuantScale q = quant_scale(e, S);
    const float limf = (float)q.lim;
    const bool plain = __all_sync(0xFFFFFFFFu, plain_row(e));
    const size_t plane_stride = (size_t)R * Kp;
    int8_t* out = planes + (size_t)b * S * plane_stride + (size_t)r_glob * Kp + k0;
    for (int kk = g * 32; arrived && r_glob < R && kk < nk; kk += G * 32) {
        const float* col = slab + (size_t)kk * W + r;
        uint32_t w[S][8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float a = col[(4 * j + 0) * W], bb = col[(4 * j + 1) * W], c = col[(4 * j + 2) * W], d = col[(4 * j + 3) * W];
            uint32_t x[S];
            if (plain) quad_words<S, true>(a, bb, c, d, q, limf, x);
            else quad_words<S, false>(a, bb, c, d, q, limf, x);
#pragma unroll
            for (int p = 0; p < S; ++p) w[p][j] = x[p];
        }
#pragma unroll
        for (int p = 0; p < S; ++p)
            st_global_256(reinterpret_cast<uint32_t*>(out + p * plane_stride + kk),
                          w[p][0], w[p][1], w[p][2], w[p][3], w[p][4], w[p][5], w[p][6], w[p][7]);
    }
    // launched behind the other operand's split with programmatic serialization, this grid must not complete before
    // that one has (the MMA kernel is launched behind this grid); nothing to wait for in an ordinary launch
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

}  // namespace rgb200
