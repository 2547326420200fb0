// Direct CUDA-core path for the smallest convolutions (a LeNet-style first layer: one input channel, six
// filters, 25 values per window).  For such a layer the implicit-GEMM path moves more padding than data: a
// window's 25 values occupy a 128-byte row in each of S digit planes and the 6 filters a 64-column MMA tile.
// Here one thread owns one output place and evaluates the definition as it stands - scale exponent from the
// maximum, one rounding to the 7S-bit fixed-point integer per input, exact INT64 dot products, one rounding
// per output - which for these sizes is a few hundred instructions per thread and one launch per call.
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

// Forward: one thread per window.  Every CTA first quantises the (few) weights itself - a warp per filter: maximum,
// scale exponent, fixed-point values into shared memory - which is cheaper than a second launch.  The window is
// read twice (maximum, then values; the second read hits L1), so no per-thread array of values is needed.
// grid = ceil(windows / 128).
template <int S>
__global__ void __launch_bounds__(CONV_DIRECT_THREADS)
conv_direct_forward_kernel(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ out, const ConvGeom g) {
    __shared__ int wq_s[CONV_DIRECT_MAX_F * CONV_DIRECT_MAX_K];
    __shared__ int ef_s[CONV_DIRECT_MAX_F];
    {
        const int lane = threadIdx.x & 31;
        for (int f = threadIdx.x >> 5; f < g.F; f += CONV_DIRECT_THREADS / 32) {
            float m = 0.0f;
            for (int k = lane; k < g.K; k += 32) m = fmaxf(m, fabsf(__ldg(w + (size_t)f * g.K + k)));
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
            const int e = scale_exponent(m);
            if (lane == 0) ef_s[f] = e;
            const QuantScale q = quant_scale(e, S);
            for (int k = lane; k < g.K; k += 32) wq_s[f * g.K + k] = fixed_point(__ldg(w + (size_t)f * g.K + k), q);
        }
    }
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

// Input gradient: one thread per input pixel (c, y, x) of image n = blockIdx.y; the sum runs over (f, ky, kx) with the
// output place (oy, ox) that tap reaches, where it exists.  Every CTA first takes the maximum of its image of dY and
// of all weights itself (both are small and come from L2) and quantises the weights into shared memory.
// grid = (ceil(C*H*W / 128), N).
template <int S>
__global__ void __launch_bounds__(CONV_DIRECT_THREADS)
conv_direct_grad_input_kernel(const float* __restrict__ dy, const float* __restrict__ w, float* __restrict__ dx, const ConvGeom g) {
    __shared__ int wq_s[CONV_DIRECT_MAX_WEIGHTS];
    __shared__ float red[2][CONV_DIRECT_THREADS / 32];
    __shared__ int e_s[2];
    const int weights = g.F * g.C * g.KH * g.KW;
    const int per = g.OH * g.OW, per_image = g.F * per;
    const int n = blockIdx.y;
    const float* dimg = dy + (size_t)n * per_image;
    {
        float md = 0.0f, mw = 0.0f;
        for (int i = threadIdx.x; i < per_image; i += CONV_DIRECT_THREADS) md = fmaxf(md, fabsf(__ldg(dimg + i)));
        for (int i = threadIdx.x; i < weights; i += CONV_DIRECT_THREADS) mw = fmaxf(mw, fabsf(__ldg(w + i)));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            md = fmaxf(md, __shfl_xor_sync(0xFFFFFFFFu, md, o));
            mw = fmaxf(mw, __shfl_xor_sync(0xFFFFFFFFu, mw, o));
        }
        if ((threadIdx.x & 31) == 0) { red[0][threadIdx.x >> 5] = md; red[1][threadIdx.x >> 5] = mw; }
        __syncthreads();
        if (threadIdx.x < 2) {
            float mm = red[threadIdx.x][0];
#pragma unroll
            for (int i = 1; i < CONV_DIRECT_THREADS / 32; ++i) mm = fmaxf(mm, red[threadIdx.x][i]);
            e_s[threadIdx.x] = scale_exponent(mm);
        }
        __syncthreads();
        const QuantScale qw = quant_scale(e_s[1], S);
        for (int i = threadIdx.x; i < weights; i += CONV_DIRECT_THREADS) wq_s[i] = fixed_point(__ldg(w + i), qw);
        __syncthreads();
    }
    const int idx = blockIdx.x * CONV_DIRECT_THREADS + threadIdx.x;
    const int hw = g.H * g.W;
    if (idx >= g.C * hw) return;
    const int c = g.by_hw.div(idx), pix = idx - c * hw;
    const int y = g.by_w.div(pix), xx = pix - y * g.W;
    const int e_n = e_s[0], e_w = e_s[1];
    const QuantScale q = quant_scale(e_n, S);
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
    dx[(size_t)n * g.C * hw + idx] = bits_f32(round_to_f32_bits(acc, e_n + e_w - 14 * (S - 1)));
}

}  // namespace rgb200
