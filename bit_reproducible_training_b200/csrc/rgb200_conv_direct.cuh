// Direct CUDA-core path for the smallest convolutions (a LeNet-style first layer: one input channel, six
// filters, 25 values per window).  For such a layer the implicit-GEMM path moves more padding than data: a
// window's 25 values occupy a 128-byte row in each of S digit planes and the 6 filters a 64-column MMA tile.
// Here one thread owns one output place and evaluates the definition as it stands - scale exponent from the
// maximum, one rounding to the 7S-bit fixed-point integer per input, exact INT64 dot products, one rounding
// per output - which for these sizes is a few hundred instructions per thread and two launches per call.
//   forward      Y[n, f, oy, ox] = round(sum_k X[w, k] W[f, k],  e_window(w) + e_filter(f) + e0)
//   input grad   dX[n, c, y, x]  = round(sum D[w, f] W[f, k],    e_image(dY, n) + e_all_weights + e0)
// (reference: repro_conv_cuda/repro_conv_math.cuh:10-17; its own kernels forward_kernel / input_grad_kernel,
// repro_conv_cuda/repro_conv.cu:19-150, are direct kernels of the same kind).  The weight gradient keeps the
// tensor-core path: its sum runs over all windows and is long enough.
#pragma once
#include "rgb200_conv.cuh"

namespace rgb200 {

constexpr int CONV_DIRECT_MAX_F = 16;        // filters the forward kernel keeps accumulators for
constexpr int CONV_DIRECT_MAX_K = 64;        // values per window (forward)
constexpr int CONV_DIRECT_MAX_WEIGHTS = 4096; // quantised weights held in shared memory (input gradient)
constexpr int CONV_DIRECT_THREADS = 128;

// Forward, step 1: one warp per filter -> scale exponent and fixed-point weights wq[f][k].  grid = 1, block = 32 * F.
template <int S>
__global__ void conv_direct_filters_kernel(const float* __restrict__ w, int* __restrict__ wq, int* __restrict__ ef, int F, int K) {
    const int f = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (f >= F) return;
    float m = 0.0f;
    for (int k = lane; k < K; k += 32) m = fmaxf(m, fabsf(w[(size_t)f * K + k]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    const int e = scale_exponent(m);
    if (lane == 0) ef[f] = e;
    const QuantScale q = quant_scale(e, S);
    for (int k = lane; k < K; k += 32) wq[f * K + k] = fixed_point(w[(size_t)f * K + k], q);
}

// Forward, step 2: one thread per window.  The window is read twice (maximum, then values; the second read
// hits L1), so no per-thread array of values is needed.  grid = ceil(windows / 128).
template <int S>
__global__ void __launch_bounds__(CONV_DIRECT_THREADS)
conv_direct_forward_kernel(const float* __restrict__ x, const int* __restrict__ wq, const int* __restrict__ ef,
                           float* __restrict__ out, const ConvGeom g) {
    __shared__ int wq_s[CONV_DIRECT_MAX_F * CONV_DIRECT_MAX_K];
    __shared__ int ef_s[CONV_DIRECT_MAX_F];
    for (int i = threadIdx.x; i < g.F * g.K; i += CONV_DIRECT_THREADS) wq_s[i] = wq[i];
    if (threadIdx.x < g.F) ef_s[threadIdx.x] = ef[threadIdx.x];
    __syncthreads();
    const int win = blockIdx.x * CONV_DIRECT_THREADS + threadIdx.x;
    const int per = g.OH * g.OW;
    if (win >= g.N * per) return;
    const int n = g.by_per.div(win), place = win - n * per;
    const int oy = g.by_ow.div(place), ox = place - oy * g.OW;
    const int y0 = oy * g.SY - g.PY, x0 = ox * g.SX - g.PX;
    const float* img = x + (size_t)n * g.C * g.H * g.W;
    float m = 0.0f;
    for (int c = 0; c < g.C; ++c)
        for (int ky = 0; ky < g.KH; ++ky) {
            const int iy = y0 + ky;
            if (iy < 0 || iy >= g.H) continue;
            for (int kx = 0; kx < g.KW; ++kx) {
                const int ix = x0 + kx;
                if (ix >= 0 && ix < g.W) m = fmaxf(m, fabsf(__ldg(img + ((size_t)c * g.H + iy) * g.W + ix)));
            }
        }
    const int ew = scale_exponent(m);
    const QuantScale q = quant_scale(ew, S);
    long long acc[CONV_DIRECT_MAX_F];
#pragma unroll
    for (int f = 0; f < CONV_DIRECT_MAX_F; ++f) acc[f] = 0;
    int k = 0;
    for (int c = 0; c < g.C; ++c)
        for (int ky = 0; ky < g.KH; ++ky) {
            const int iy = y0 + ky;
            if (iy < 0 || iy >= g.H) { k += g.KW; continue; }
            for (int kx = 0; kx < g.KW; ++kx, ++k) {
                const int ix = x0 + kx;
                if (ix < 0 || ix >= g.W) continue;
                const int X = fixed_point(__ldg(img + ((size_t)c * g.H + iy) * g.W + ix), q);
#pragma unroll
                for (int f = 0; f < CONV_DIRECT_MAX_F; ++f)
                    if (f < g.F) acc[f] += (long long)X * wq_s[f * g.K + k];
            }
        }
    const int e0 = -14 * (S - 1);
#pragma unroll
    for (int f = 0; f < CONV_DIRECT_MAX_F; ++f)
        if (f < g.F) out[((size_t)n * g.F + f) * per + place] = bits_f32(round_to_f32_bits(acc[f], ew + ef_s[f] + e0));
}

// Input gradient, step 1: blocks 0..N-1 take the maximum of one image of dY -> e_img[n]; block N takes the
// maximum of all weights -> e_img[N] and the fixed-point weights wq.  grid = N + 1, block = 256.
template <int S>
__global__ void __launch_bounds__(256)
conv_direct_grad_input_scales_kernel(const float* __restrict__ dy, const float* __restrict__ w, int* __restrict__ e_img,
                                     int* __restrict__ wq, int N, int per_image, int weights) {
    __shared__ float red[8];
    __shared__ int e_s;
    const bool is_w = (int)blockIdx.x == N;
    const float* src = is_w ? w : dy + (size_t)blockIdx.x * per_image;
    const int count = is_w ? weights : per_image;
    float m = 0.0f;
    for (int i = threadIdx.x; i < count; i += 256) m = fmaxf(m, fabsf(__ldg(src + i)));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        float mm = red[0];
#pragma unroll
        for (int i = 1; i < 8; ++i) mm = fmaxf(mm, red[i]);
        const int e = scale_exponent(mm);
        e_s = e;
        e_img[blockIdx.x] = e;
    }
    __syncthreads();
    if (is_w) {
        const QuantScale q = quant_scale(e_s, S);
        for (int i = threadIdx.x; i < weights; i += 256) wq[i] = fixed_point(__ldg(w + i), q);
    }
}

// Input gradient, step 2: one thread per input pixel (n, c, y, x); the sum runs over (f, ky, kx) with the output
// place (oy, ox) that tap reaches, where it exists.  grid = ceil(N*C*H*W / 128).
template <int S>
__global__ void __launch_bounds__(CONV_DIRECT_THREADS)
conv_direct_grad_input_kernel(const float* __restrict__ dy, const int* __restrict__ wq, const int* __restrict__ e_img,
                              float* __restrict__ dx, const ConvGeom g) {
    __shared__ int wq_s[CONV_DIRECT_MAX_WEIGHTS];
    const int weights = g.F * g.C * g.KH * g.KW;
    for (int i = threadIdx.x; i < weights; i += CONV_DIRECT_THREADS) wq_s[i] = wq[i];
    __syncthreads();
    const int idx = blockIdx.x * CONV_DIRECT_THREADS + threadIdx.x;
    const int hw = g.H * g.W;
    if (idx >= g.N * g.C * hw) return;
    const int nc = g.by_hw.div(idx), pix = idx - nc * hw;
    const int n = g.by_c.div(nc), c = nc - n * g.C;
    const int y = g.by_w.div(pix), xx = pix - y * g.W;
    const int e_n = e_img[n], e_w = e_img[g.N];
    const QuantScale q = quant_scale(e_n, S);
    const int per = g.OH * g.OW;
    const float* dimg = dy + (size_t)n * g.F * per;
    long long acc = 0;
    for (int ky = 0; ky < g.KH; ++ky) {
        const int ty = y + g.PY - ky;
        if (ty < 0) continue;
        const int oy = g.by_sy.div(ty);
        if (oy * g.SY != ty || oy >= g.OH) continue;
        for (int kx = 0; kx < g.KW; ++kx) {
            const int tx = xx + g.PX - kx;
            if (tx < 0) continue;
            const int ox = g.by_sx.div(tx);
            if (ox * g.SX != tx || ox >= g.OW) continue;
            for (int f = 0; f < g.F; ++f) {
                const int D = fixed_point(__ldg(dimg + (size_t)f * per + oy * g.OW + ox), q);
                acc += (long long)D * wq_s[((f * g.C + c) * g.KH + ky) * g.KW + kx];
            }
        }
    }
    dx[idx] = bits_f32(round_to_f32_bits(acc, e_n + e_w - 14 * (S - 1)));
}

}  // namespace rgb200
