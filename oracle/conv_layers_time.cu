// TEST INFRASTRUCTURE, NOT PRODUCT CODE.
//
// Times the convolution forward, weight gradient and input gradient (S = 3) on a few layer shapes
// through the reference's C++ interface (repro_conv_cuda/repro_conv.cuh:22-32).  oracle/Makefile
// links it twice: against the reference's own CUDA sources (the time to beat on this GPU) and against
// librgb200.so.  Inputs follow the reference's benchmark (repro_conv_cuda/bench_repro_conv.cu:70-73):
// x ~ N(0,1), weights ~ 0.1 N(0,1), dY ~ 1e-3 N(0,1).  Median of ten runs after three warm-ups.
#include "repro_conv.cuh"
#include <algorithm>
#include <cstdio>
#include <random>
#include <vector>

using namespace repro_conv;

#define CK(call)                                                                                  \
    do {                                                                                          \
        cudaError_t err_ = (call);                                                                \
        if (err_ != cudaSuccess) { std::printf("%s (line %d)\n", cudaGetErrorString(err_), __LINE__); return 1; } \
    } while (0)

template <class F>
static float median_ms(F run) {
    std::vector<float> t;
    cudaEvent_t a, b;
    cudaEventCreate(&a);
    cudaEventCreate(&b);
    for (int i = 0; i < 13; ++i) {
        cudaEventRecord(a);
        run();
        cudaEventRecord(b);
        cudaEventSynchronize(b);
        float ms;
        cudaEventElapsedTime(&ms, a, b);
        if (i >= 3) t.push_back(ms);
    }
    std::sort(t.begin(), t.end());
    return t[t.size() / 2];
}

int main() {
    const int shapes[][11] = {{32, 64, 56, 56, 64, 3, 3, 1, 1, 1, 1},      // 64 -> 64 channels, 3 x 3, 56 x 56
                              {32, 16, 32, 32, 32, 3, 3, 1, 1, 1, 1},      // 16 -> 32 channels, 3 x 3, 32 x 32
                              {64, 32, 28, 28, 64, 5, 5, 1, 1, 2, 2}};     // 32 -> 64 channels, 5 x 5, 28 x 28
    for (const auto& s : shapes) {
        ConvShape g;
        g.N = s[0]; g.C = s[1]; g.H = s[2]; g.W = s[3]; g.F = s[4]; g.KH = s[5]; g.KW = s[6];
        g.SY = s[7]; g.SX = s[8]; g.PY = s[9]; g.PX = s[10];
        std::mt19937_64 rng(5);
        std::normal_distribution<float> nd(0.0f, 1.0f);
        std::vector<float> x(g.input_size()), w(g.weight_size()), dy(g.output_size());
        for (auto& v : x) v = nd(rng);
        for (auto& v : w) v = 0.1f * nd(rng);
        for (auto& v : dy) v = 1e-3f * nd(rng);
        float *dx, *dw, *ddy, *out, *gw, *gi;
        CK(cudaMalloc(&dx, x.size() * 4)); CK(cudaMalloc(&dw, w.size() * 4)); CK(cudaMalloc(&ddy, dy.size() * 4));
        CK(cudaMalloc(&out, dy.size() * 4)); CK(cudaMalloc(&gw, w.size() * 4)); CK(cudaMalloc(&gi, x.size() * 4));
        CK(cudaMemcpy(dx, x.data(), x.size() * 4, cudaMemcpyHostToDevice));
        CK(cudaMemcpy(dw, w.data(), w.size() * 4, cudaMemcpyHostToDevice));
        CK(cudaMemcpy(ddy, dy.data(), dy.size() * 4, cudaMemcpyHostToDevice));
        size_t b0, b1, b2;
        CK(conv2d_workspace(g, 3, &b0)); CK(conv2d_grad_weight_workspace(g, 3, &b1)); CK(conv2d_grad_input_workspace(g, 3, &b2));
        void *w0, *w1, *w2;
        CK(cudaMalloc(&w0, b0)); CK(cudaMalloc(&w1, b1)); CK(cudaMalloc(&w2, b2));
        std::printf("x[%d,%d,%d,%d] -> %d filters %dx%d (%d values per window, %d windows): ", g.N, g.C, g.H, g.W, g.F, g.KH, g.KW,
                    g.K(), g.windows());
        std::printf("forward %.3f ms, ", median_ms([&] { repro_conv2d_ws(dx, dw, out, g, 3, w0, b0); }));
        std::printf("weight grad %.3f ms, ", median_ms([&] { repro_conv2d_grad_weight_ws(ddy, dx, gw, g, 3, w1, b1); }));
        std::printf("input grad %.3f ms\n", median_ms([&] { repro_conv2d_grad_input_ws(ddy, dw, gi, g, 3, w2, b2); }));
        CK(cudaDeviceSynchronize());
        cudaFree(dx); cudaFree(dw); cudaFree(ddy); cudaFree(out); cudaFree(gw); cudaFree(gi);
        cudaFree(w0); cudaFree(w1); cudaFree(w2);
    }
    return 0;
}
