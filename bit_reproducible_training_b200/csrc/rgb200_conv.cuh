// Convolution as an implicit GEMM: the scale-and-split pre-pass reads the image (or the output
// gradient) through an index map instead of a stored im2col matrix, writes the same int8 digit
// planes the matrix pre-pass writes, and the tcgen05 kernel runs unchanged on them.
//
// Definition (reference: repro_conv_cuda/repro_conv_math.cuh:1-22, repro_conv_cpu.h:25-90), with
// a "window" one (n, oy, ox), position k = (c, ky, kx), K = C*KH*KW and e0 = -14 (S - 1):
//   forward      Y[n, f, oy, ox] = round(sum_k X[w, k] W[f, k],  e_window(w) + e_filter(f) + e0)
//   weight grad  dW[f, k]        = round(sum_w D[w, f] X[w, k],  e_filter(dY, f) + e_position(k) + e0)
//   input grad   dX[n, c, y, x]  = round(sum D[w, f] W[f, k],    e_image(dY, n) + e_all_weights + e0)
// The first two are the GEMM definition applied to the im2col matrix; the third is a GEMM over
// k = (f, ky, kx) whose operands use one scale per image and one for all weights.
//
// As products on the digit planes (rows of op(A) x rows of op(B)^T, k contiguous in both):
//   forward      [windows x K] window values       times  [F x K] weights        -> out[n][f][place]
//   weight grad  [F x windows] dY                   times  [K x windows] windows  -> dW[f][k]
//   input grad   [pixels x F*KH*KW] dY taps         times  [C x F*KH*KW] weights  -> dX[n][c][place]
// The many-row operand sits on the 128-row side of the MMA tile; forward and input gradient use the
// image-major store of the MMA kernel, so every result lands directly in the PyTorch layout of its
// tensor.  (When K is too long for one INT32 accumulation pass, forward and input gradient fall back
// to one product per image with the weights on the row side, which needs no special store.)
//
// The order of k inside a product is free (the sum is exact) as long as both operands use the same
// one.  Forward (with at least four channels) and input gradient run k "tap-major": k = tap * I + i
// with tap = ky * KW + kx and the inner index i the channel (forward) or the filter (input
// gradient).  Sixteen consecutive k are then usually sixteen inner indices at one tap: one bounds
// check and address computation, sixteen loads a whole plane apart, one 16-byte store per digit plane.
#pragma once
#include "rgb200_prepass.cuh"

namespace rgb200 {

// Division of a non-negative 32-bit integer (below 2^31) by a fixed divisor as one multiply-high and a
// shift: with p = 31 + ceil(log2 d) and mul = ceil(2^p / d), floor(n / d) = (n * mul) >> p for all such n.
// The index maps divide by kernel and image extents for every group of elements they fetch.
struct FastDiv {
    unsigned d, mul, shr;
    FastDiv() : d(1), mul(0), shr(0) {}
    explicit FastDiv(int divisor) : d((unsigned)divisor), mul(0), shr(0) {
        if (d > 1) {
            unsigned lg = 0;
            while ((1ull << lg) < d) ++lg;
            const unsigned p = 31 + lg;
            mul = (unsigned)(((1ull << p) + d - 1) / d);
            shr = p - 32;
        }
    }
    __host__ __device__ __forceinline__ int div(int n) const {
#ifdef __CUDA_ARCH__
        return d == 1 ? n : (int)(__umulhi((unsigned)n, mul) >> shr);
#else
        return d == 1 ? n : (int)((((unsigned long long)(unsigned)n * mul) >> 32) >> shr);
#endif
    }
};

struct ConvGeom {
    int N, C, H, W, F, KH, KW, SY, SX, PY, PX;
    int OH, OW, K;            // output height and width, values per window
    FastDiv by_khw, by_kw, by_ow, by_per, by_w, by_hw, by_sy, by_sx, by_f, by_c;   // KH*KW, KW, OW, OH*OW, W, H*W, SY, SX, F, C
    void prepare() {
        by_khw = FastDiv(KH * KW); by_kw = FastDiv(KW); by_ow = FastDiv(OW); by_per = FastDiv(OH * OW);
        by_w = FastDiv(W); by_hw = FastDiv(H * W); by_sy = FastDiv(SY); by_sx = FastDiv(SX);
        by_f = FastDiv(F); by_c = FastDiv(C);
    }
};

// ---------------------------------------------------------------------------------------------
// Index maps.  at(b, r, k) is element (row r, index k) of operand matrix number b; quad and hex
// fetch 4 and 16 consecutive k with zeros from index K on (the padding of the digit planes).
// ---------------------------------------------------------------------------------------------
template <class Source>
__device__ __forceinline__ float4 quad_by_elements(const Source& s, int b, int r, int k, int K) {
    float4 v;
    v.x = k + 0 < K ? s.at(b, r, k + 0) : 0.0f;
    v.y = k + 1 < K ? s.at(b, r, k + 1) : 0.0f;
    v.z = k + 2 < K ? s.at(b, r, k + 2) : 0.0f;
    v.w = k + 3 < K ? s.at(b, r, k + 3) : 0.0f;
    return v;
}
template <class Source>
__device__ __forceinline__ void hex_by_quads(const Source& s, int b, int r, int k, int K, float (&v)[16]) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float4 q = s.quad(b, r, k + 4 * j, K);
        v[4 * j] = q.x; v[4 * j + 1] = q.y; v[4 * j + 2] = q.z; v[4 * j + 3] = q.w;
    }
}
#define RGB_QUAD_BY_ELEMENTS \
    __device__ __forceinline__ float4 quad(int b, int r, int k, int K) const { return quad_by_elements(*this, b, r, k, K); }
#define RGB_HEX_BY_QUADS \
    __device__ __forceinline__ void hex(int b, int r, int k, int K, float (&v)[16]) const { hex_by_quads(*this, b, r, k, K, v); }

// Tap-major gathers: k = tap * I + i.  lookup(tap) returns the address of inner index 0 at that tap
// (inner indices are `stride` floats apart) or null where the tap reads zero (padding, no such window).
template <class Lookup>
__device__ __forceinline__ float tap_major_at(const Lookup& lookup, int I, FastDiv by_I, size_t stride, int k) {
    const int tap = by_I.div(k), i = k - tap * I;
    const float* p = lookup(tap);
    return p ? __ldg(p + i * stride) : 0.0f;
}
template <class Lookup>
__device__ __forceinline__ float4 tap_major_quad(const Lookup& lookup, int I, FastDiv by_I, size_t stride, int taps, int k, int K) {
    if (k >= K) return make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    float e[4];
    if (I < 4) {                                  // a quad could span three taps
#pragma unroll
        for (int j = 0; j < 4; ++j) e[j] = k + j < K ? tap_major_at(lookup, I, by_I, stride, k + j) : 0.0f;
        return make_float4(e[0], e[1], e[2], e[3]);
    }
    // elements 0 .. first-1 are inner indices i .. of this tap, the rest 0 .. of the next tap (none after the last)
    const int tap = by_I.div(k), i = k - tap * I;
    const int first = min(4, I - i);
    const float* p0 = lookup(tap);
    const float* p1 = (first < 4 && tap + 1 < taps) ? lookup(tap + 1) : nullptr;
    if (p0) p0 += i * stride;
    if (p1) p1 -= first * stride;                 // so that element j reads p1 + j * stride
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float* p = j < first ? p0 : p1;
        e[j] = p ? __ldg(p + j * stride) : 0.0f;
    }
    return make_float4(e[0], e[1], e[2], e[3]);
}
template <class Lookup>
__device__ __forceinline__ void tap_major_hex(const Lookup& lookup, int I, FastDiv by_I, size_t stride, int taps, int k, int K,
                                              float (&v)[16]) {
    const int tap = by_I.div(k), i = k - tap * I;
    if (k + 15 < K && i + 15 < I) {               // sixteen inner indices at one tap
        const float* p = lookup(tap);
        if (p) p += i * stride;
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = p ? __ldg(p + j * stride) : 0.0f;
        return;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float4 q = tap_major_quad(lookup, I, by_I, stride, taps, k + 4 * j, K);
        v[4 * j] = q.x; v[4 * j + 1] = q.y; v[4 * j + 2] = q.z; v[4 * j + 3] = q.w;
    }
}
// kSixteenPerLane: whether the long-row kernels fetch sixteen consecutive k per lane (sources whose consecutive
// k lie a plane apart: nothing to coalesce, fewer index computations) or four (sources whose consecutive k are
// consecutive in memory: a warp's loads then cover contiguous 512 bytes).
#define RGB_TAP_MAJOR(I_, BY_I_, STRIDE_, LOOKUP_)                                                                   \
    static constexpr bool kSixteenPerLane = true;                                                                    \
    __device__ __forceinline__ float at(int b, int r, int k) const {                                                 \
        return tap_major_at(LOOKUP_, I_, BY_I_, STRIDE_, k);                                                         \
    }                                                                                                                \
    __device__ __forceinline__ float4 quad(int b, int r, int k, int K) const {                                       \
        return tap_major_quad(LOOKUP_, I_, BY_I_, STRIDE_, g.KH * g.KW, k, K);                                       \
    }                                                                                                                \
    __device__ __forceinline__ void hex(int b, int r, int k, int K, float (&v)[16]) const {                          \
        tap_major_hex(LOOKUP_, I_, BY_I_, STRIDE_, g.KH * g.KW, k, K, v);                                            \
    }

// x[n, 0, y, x] under tap (ky, kx) of window (oy, ox), or null in the padding.
__device__ __forceinline__ const float* conv_pixel_under_tap(const float* __restrict__ x, const ConvGeom& g, int n, int oy, int ox, int tap) {
    const int ky = g.by_kw.div(tap), kx = tap - ky * g.KW;
    const int y = oy * g.SY - g.PY + ky, xx = ox * g.SX - g.PX + kx;
    if ((unsigned)y >= (unsigned)g.H || (unsigned)xx >= (unsigned)g.W) return nullptr;
    return x + ((size_t)n * g.C * g.H + y) * g.W + xx;
}
// dY[n, 0, oy, ox] of the window whose tap (ky, kx) lies on pixel (y, x), or null when the strides and edges allow none.
__device__ __forceinline__ const float* conv_window_over_pixel(const float* __restrict__ dy, const ConvGeom& g, int n, int pixel, int tap) {
    const int ky = g.by_kw.div(tap), kx = tap - ky * g.KW;
    const int y = g.by_w.div(pixel), xx = pixel - y * g.W;
    const int ry = y + g.PY - ky, rx = xx + g.PX - kx;
    if (ry < 0 || rx < 0) return nullptr;
    const int oy = g.by_sy.div(ry), ox = g.by_sx.div(rx);
    if (oy * g.SY != ry || ox * g.SX != rx || oy >= g.OH || ox >= g.OW) return nullptr;
    return dy + ((size_t)n * g.F * g.OH + oy) * g.OW + ox;
}

// ---- forward, k = (tap, channel): used when C >= 4 ----
struct WindowTapsOfImage {      // b = image, r = window (oy, ox) of that image
    const float* x; ConvGeom g;
    RGB_TAP_MAJOR(g.C, g.by_c, (size_t)g.H * g.W,
                  ([&](int tap) { const int oy = g.by_ow.div(r); return conv_pixel_under_tap(x, g, b, oy, r - oy * g.OW, tap); }))
};
struct AllWindowTaps {          // r = window (n, oy, ox) over all images
    const float* x; ConvGeom g;
    RGB_TAP_MAJOR(g.C, g.by_c, (size_t)g.H * g.W, ([&](int tap) {
                      const int n = g.by_per.div(r), j = r - n * (g.OH * g.OW);
                      const int oy = g.by_ow.div(j);
                      return conv_pixel_under_tap(x, g, n, oy, j - oy * g.OW, tap);
                  }))
};
// Weights [F][C][KH][KW] as rows over k = (tap, inner): row r and inner index i at w[r * row_stride + i * inner_stride + tap].
// Forward: rows are filters, inner the channel.  Input gradient: rows are channels, inner the filter.
struct TapMajorWeights {
    const float* w; ConvGeom g; int I; FastDiv by_I; size_t row_stride, inner_stride;
    RGB_TAP_MAJOR(I, by_I, inner_stride, ([&](int tap) { return w + (size_t)r * row_stride + tap; }))
};

// ---- forward, k = (c, ky, kx) as the weights are stored: used for fewer than four channels ----
__device__ __forceinline__ float conv_window_value(const float* __restrict__ x, const ConvGeom& g, int n, int oy, int ox, int k) {
    const int c = g.by_khw.div(k), rem = k - c * (g.KH * g.KW);
    const int ky = g.by_kw.div(rem), kx = rem - ky * g.KW;
    const int y = oy * g.SY - g.PY + ky, xx = ox * g.SX - g.PX + kx;
    if ((unsigned)y >= (unsigned)g.H || (unsigned)xx >= (unsigned)g.W) return 0.0f;   // zero padding
    return __ldg(x + (((size_t)n * g.C + c) * g.H + y) * g.W + xx);
}
// Positions k .. k+3 of one window: (c, ky, kx) is found once and stepped with carries.
__device__ __forceinline__ float4 conv_window_quad(const float* __restrict__ x, const ConvGeom& g, int n, int oy, int ox, int k, int K) {
    int c = g.by_khw.div(k);
    const int rem = k - c * (g.KH * g.KW);
    int ky = g.by_kw.div(rem), kx = rem - ky * g.KW;
    const int y0 = oy * g.SY - g.PY, x0 = ox * g.SX - g.PX;
    float e[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int y = y0 + ky, xx = x0 + kx;
        const bool inside = k + i < K && (unsigned)y < (unsigned)g.H && (unsigned)xx < (unsigned)g.W;
        e[i] = inside ? __ldg(x + (((size_t)n * g.C + c) * g.H + y) * g.W + xx) : 0.0f;
        if (++kx == g.KW) { kx = 0; if (++ky == g.KH) { ky = 0; ++c; } }
    }
    return make_float4(e[0], e[1], e[2], e[3]);
}
struct WindowsOfImage {         // b = image, r = window (oy, ox) of that image, k = position
    static constexpr bool kSixteenPerLane = false;
    const float* x; ConvGeom g;
    __device__ __forceinline__ float at(int b, int r, int k) const {
        const int oy = g.by_ow.div(r);
        return conv_window_value(x, g, b, oy, r - oy * g.OW, k);
    }
    __device__ __forceinline__ float4 quad(int b, int r, int k, int K) const {
        const int oy = g.by_ow.div(r);
        return conv_window_quad(x, g, b, oy, r - oy * g.OW, k, K);
    }
    RGB_HEX_BY_QUADS
};
struct AllWindows {             // r = window (n, oy, ox) over all images, k = position
    static constexpr bool kSixteenPerLane = false;
    const float* x; ConvGeom g;
    __device__ __forceinline__ float at(int, int r, int k) const {
        const int n = g.by_per.div(r), j = r - n * (g.OH * g.OW);
        const int oy = g.by_ow.div(j);
        return conv_window_value(x, g, n, oy, j - oy * g.OW, k);
    }
    __device__ __forceinline__ float4 quad(int, int r, int k, int K) const {
        const int n = g.by_per.div(r), j = r - n * (g.OH * g.OW);
        const int oy = g.by_ow.div(j);
        return conv_window_quad(x, g, n, oy, j - oy * g.OW, k, K);
    }
    RGB_HEX_BY_QUADS
};

// ---- weight gradient: k = window (n, oy, ox) ----
struct PositionsOverWindows {   // r = position (c, ky, kx)
    static constexpr bool kSixteenPerLane = false;
    const float* x; ConvGeom g;
    __device__ __forceinline__ float at(int, int r, int k) const {
        const int n = g.by_per.div(k), j = k - n * (g.OH * g.OW);
        const int oy = g.by_ow.div(j);
        return conv_window_value(x, g, n, oy, j - oy * g.OW, r);
    }
    // COUNT consecutive windows of one position; (n, oy, ox) is found once and stepped with carries
    template <int COUNT>
    __device__ __forceinline__ void run(int r, int k, int K, float* e) const {
        const int c = g.by_khw.div(r), rem = r - c * (g.KH * g.KW);
        const int ky = g.by_kw.div(rem), kx = rem - ky * g.KW;
        int n = g.by_per.div(k);
        const int j = k - n * (g.OH * g.OW);
        int oy = g.by_ow.div(j), ox = j - oy * g.OW;
        if (k + COUNT <= K && ox + COUNT <= g.OW) {       // one output row: one image row, consecutive (strided) pixels
            const int y = oy * g.SY - g.PY + ky;
            const bool row_inside = (unsigned)y < (unsigned)g.H;
            const float* row = x + (((size_t)n * g.C + c) * g.H + (row_inside ? y : 0)) * g.W;
            int xx = ox * g.SX - g.PX + kx;
#pragma unroll
            for (int i = 0; i < COUNT; ++i, xx += g.SX) e[i] = (row_inside && (unsigned)xx < (unsigned)g.W) ? __ldg(row + xx) : 0.0f;
            return;
        }
#pragma unroll
        for (int i = 0; i < COUNT; ++i) {
            const int y = oy * g.SY - g.PY + ky, xx = ox * g.SX - g.PX + kx;
            const bool inside = k + i < K && (unsigned)y < (unsigned)g.H && (unsigned)xx < (unsigned)g.W;
            e[i] = inside ? __ldg(x + (((size_t)n * g.C + c) * g.H + y) * g.W + xx) : 0.0f;
            if (++ox == g.OW) { ox = 0; if (++oy == g.OH) { oy = 0; ++n; } }
        }
    }
    __device__ __forceinline__ float4 quad(int, int r, int k, int K) const {
        float e[4];
        run<4>(r, k, K, e);
        return make_float4(e[0], e[1], e[2], e[3]);
    }
    __device__ __forceinline__ void hex(int, int r, int k, int K, float (&v)[16]) const { run<16>(r, k, K, v); }
};
struct FiltersOverWindows {     // r = filter; dY is [N][F][OH*OW]: contiguous within an image
    static constexpr bool kSixteenPerLane = false;
    const float* dy; ConvGeom g;
    __device__ __forceinline__ float at(int, int r, int k) const {
        const int per = g.OH * g.OW;
        const int n = g.by_per.div(k), j = k - n * per;
        return __ldg(dy + ((size_t)n * g.F + r) * per + j);
    }
    template <int COUNT>
    __device__ __forceinline__ bool run(int r, int k, int K, float* e) const {
        const int per = g.OH * g.OW;
        const int n = g.by_per.div(k), j = k - n * per;
        if (k + COUNT > K || j + COUNT > per) return false;
        const float* p = dy + ((size_t)n * g.F + r) * per + j;
#pragma unroll
        for (int i = 0; i < COUNT; ++i) e[i] = __ldg(p + i);
        return true;
    }
    __device__ __forceinline__ float4 quad(int b, int r, int k, int K) const {
        float e[4];
        if (!run<4>(r, k, K, e)) return quad_by_elements(*this, b, r, k, K);
        return make_float4(e[0], e[1], e[2], e[3]);
    }
    __device__ __forceinline__ void hex(int b, int r, int k, int K, float (&v)[16]) const {
        if (!run<16>(r, k, K, v)) hex_by_quads(*this, b, r, k, K, v);
    }
};

// ---- input gradient, k = (tap, filter) ----
struct PixelTapsOfImage {       // b = image, r = pixel (y, x) of that image
    const float* dy; ConvGeom g;
    RGB_TAP_MAJOR(g.F, g.by_f, (size_t)g.OH * g.OW, ([&](int tap) { return conv_window_over_pixel(dy, g, b, r, tap); }))
};
struct AllPixelTaps {           // r = pixel (n, y, x) over all images
    const float* dy; ConvGeom g;
    RGB_TAP_MAJOR(g.F, g.by_f, (size_t)g.OH * g.OW, ([&](int tap) {
                      const int n = g.by_hw.div(r);
                      return conv_window_over_pixel(dy, g, n, r - n * (g.H * g.W), tap);
                  }))
};

struct StoredRows {             // a stored matrix [R][K] (the weights as they are; whole tensors for their maxima)
    static constexpr bool kSixteenPerLane = false;
    const float* src; long long row_len;
    __device__ __forceinline__ float at(int, int r, int k) const { return __ldg(src + (size_t)r * row_len + k); }
    RGB_QUAD_BY_ELEMENTS
    __device__ __forceinline__ void hex(int b, int r, int k, int K, float (&v)[16]) const {
        if (k + 15 < K) {
            const float* p = src + (size_t)r * row_len + k;
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = __ldg(p + i);
        } else {
            hex_by_quads(*this, b, r, k, K, v);
        }
    }
};

// ---------------------------------------------------------------------------------------------
// Weight gradient: the maxima of the position rows without gathering.  What position (c, ky, kx) sees
// over all windows is a (strided) rectangle of channel c's plane in every image.  So: the maximum over
// the images of every pixel of every channel (one pass over x), then per position the maximum over
// its rectangle of that small map.  Both exact (maxima of magnitudes, compared as bit patterns).
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(PREPASS_THREADS)
pixel_max_over_images_kernel(const float* __restrict__ x, uint32_t* __restrict__ pixmax, int N, int C, int HW) {
    const int p = blockIdx.x * PREPASS_THREADS + threadIdx.x;       // grid = (ceil(HW / 256), min(C, 65535))
    if (p >= HW) return;
    for (int c = blockIdx.y; c < C; c += gridDim.y) {
        float m = 0.0f;
        for (int n = 0; n < N; ++n) m = fmaxf(m, fabsf(__ldg(x + ((size_t)n * C + c) * HW + p)));
        pixmax[(size_t)c * HW + p] = f32_bits(m);
    }
}

__global__ void __launch_bounds__(PREPASS_THREADS)
position_max_kernel(const uint32_t* __restrict__ pixmax, uint32_t* __restrict__ maxbits, const ConvGeom g) {
    const int pos = blockIdx.x;                                     // grid = K, one CTA per position; maxbits zero on entry
    const int c = g.by_khw.div(pos), rem = pos - c * (g.KH * g.KW);
    const int ky = g.by_kw.div(rem), kx = rem - ky * g.KW;
    uint32_t m = 0u;
    for (int j = threadIdx.x; j < g.OH * g.OW; j += PREPASS_THREADS) {
        const int oy = g.by_ow.div(j), ox = j - oy * g.OW;
        const int y = oy * g.SY - g.PY + ky, xx = ox * g.SX - g.PX + kx;
        if ((unsigned)y < (unsigned)g.H && (unsigned)xx < (unsigned)g.W) m = max(m, pixmax[((size_t)c * g.H + y) * g.W + xx]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    if ((threadIdx.x & 31) == 0 && m) atomicMax(maxbits + pos, m);
}

// ---------------------------------------------------------------------------------------------
// Digit split of sixteen consecutive k: one 16-byte store per plane (idx a multiple of 16).
// ---------------------------------------------------------------------------------------------
template <int S, bool PLAIN>
__device__ __forceinline__ void store_hex_impl(const float (&v)[16], const QuantScale& q, int8_t* plane0, size_t plane_stride, size_t idx) {
    const float limf = (float)q.lim;
    int y[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) y[i] = biased_fixed_point<S, PLAIN>(v[i], q, limf);
#pragma unroll
    for (int p = S - 1; p >= 0; --p) {
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            w[j] = pack_low_bytes(y[4 * j], y[4 * j + 1], y[4 * j + 2], y[4 * j + 3]);
            if (p > 0) w[j] = unbias_bytes(w[j]);
        }
        if (p > 0) {
#pragma unroll
            for (int i = 0; i < 16; ++i) y[i] >>= 7;
        }
        *reinterpret_cast<uint4*>(plane0 + p * plane_stride + idx) = make_uint4(w[0], w[1], w[2], w[3]);
    }
}
template <int S>
__device__ __forceinline__ void store_hex(const float (&v)[16], const QuantScale& q, bool plain, int8_t* plane0, size_t plane_stride, size_t idx) {
    if (plain) store_hex_impl<S, true>(v, q, plane0, plane_stride, idx);
    else store_hex_impl<S, false>(v, q, plane0, plane_stride, idx);
}
__device__ __forceinline__ float abs16max(float m, const float (&v)[16]) {
#pragma unroll
    for (int i = 0; i < 16; ++i) m = fmaxf(m, fabsf(v[i]));
    return m;
}

// ---------------------------------------------------------------------------------------------
// Long rows, two launches of the same shape: maxima (integer atomicMax on the bit patterns, exact and
// order-free; the slots must be zero on entry), then scale and split.  One warp works on one row and
// one chunk of GATHER_CHUNK indices, sixteen per lane and step.
// A row's maximum lives in maxbits[b * slot_batch_mul + (r / slot_div) * slot_row_mul]: (R, 1) with
// slot_div 1 gives one scale per row, (1, 0) one per operand matrix, (0, 0) one for everything, and
// (0, 1) with slot_div = rows per image one per image when all images share one operand matrix.
// grid = (ceil(R / 8), ceil(K or Kp / GATHER_CHUNK), batch), 256 threads
// ---------------------------------------------------------------------------------------------
constexpr int GATHER_CHUNK = 1024;

template <class Source>
__global__ void __launch_bounds__(PREPASS_THREADS)
gather_max_kernel(const Source src, uint32_t* __restrict__ maxbits, int R, int K, int slot_batch_mul, int slot_row_mul) {
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * (PREPASS_THREADS / 32) + (threadIdx.x >> 5);
    const int b = blockIdx.z;
    if (row >= R) return;
    const int k_lo = blockIdx.y * GATHER_CHUNK, k_hi = min(K, k_lo + GATHER_CHUNK);
    float m = 0.0f;
    if (Source::kSixteenPerLane) {
        for (int k = k_lo + lane * 16; k < k_hi; k += 512) {
            float v[16];
            src.hex(b, row, k, K, v);
            m = abs16max(m, v);
        }
    } else {
        for (int k = k_lo + lane * 4; k < k_hi; k += 128) m = abs4max(m, src.quad(b, row, k, K));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    if (lane == 0 && m > 0.0f) atomicMax(maxbits + (size_t)b * slot_batch_mul + (size_t)row * slot_row_mul, f32_bits(m));
}

template <int S, class Source>
__global__ void __launch_bounds__(PREPASS_THREADS)
gather_split_kernel(const Source src, const uint32_t* __restrict__ maxbits, int8_t* __restrict__ planes,
                    int* __restrict__ expo, int R, int K, int Kp, int slot_batch_mul, int slot_row_mul, FastDiv slot_div) {
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * (PREPASS_THREADS / 32) + (threadIdx.x >> 5);
    const int b = blockIdx.z;
    if (row >= R) return;
    const int e = scale_exponent(bits_f32(maxbits[(size_t)b * slot_batch_mul + (size_t)slot_div.div(row) * slot_row_mul]));
    if (blockIdx.y == 0 && lane == 0) expo[(size_t)b * R + row] = e;
    const QuantScale q = quant_scale(e, S);
    const bool plain = plain_row(e);
    const size_t plane_stride = (size_t)R * Kp;
    int8_t* out = planes + (size_t)b * S * plane_stride + (size_t)row * Kp;
    const int k_lo = blockIdx.y * GATHER_CHUNK, k_hi = min(Kp, k_lo + GATHER_CHUNK);
    if (Source::kSixteenPerLane) {
        for (int k = k_lo + lane * 16; k < k_hi; k += 512) {     // a warp writes 512 contiguous bytes per plane
            float v[16];
            src.hex(b, row, k, K, v);                            // zeros from K up to Kp
            store_hex<S>(v, q, plain, out, plane_stride, (size_t)k);
        }
    } else {
        for (int k = k_lo + lane * 4; k < k_hi; k += 128)        // a warp writes 128 contiguous bytes per plane
            store_quad<S>(src.quad(b, row, k, K), q, plain, out, plane_stride, (size_t)k);
    }
}

// ---------------------------------------------------------------------------------------------
// Short rows: a group of lanes keeps a whole row in registers between the maximum and the split, so
// the index map is evaluated once per element and one launch does both steps.  With OWN_MAX = false
// the scale comes from a maximum reduced beforehand (shared by several rows).
//   gather_rows_kernel      four k per lane; rows of at most 32 or 64 values take 8 or 16 lanes (4 or 2 rows
//                           per warp) and fill the rest of the 128-byte plane row with 16-byte zero stores
//   gather_rows16_kernel    sixteen k per lane and step (HEXES steps), 8, 16 or 32 lanes per row
// grid = (ceil(R / (8 * 32 / LANES)), 1, batch), 256 threads
// ---------------------------------------------------------------------------------------------
template <int S, class Source, int LANES, bool OWN_MAX>
__global__ void __launch_bounds__(PREPASS_THREADS)
gather_rows_kernel(const Source src, const uint32_t* __restrict__ maxbits, int8_t* __restrict__ planes,
                   int* __restrict__ expo, int R, int K, int Kp, int slot_batch_mul, int slot_row_mul, FastDiv slot_div) {
    constexpr int ROWS_PER_WARP = 32 / LANES;
    const int lane = threadIdx.x & 31, sub = lane % LANES;
    const int row = (blockIdx.x * (PREPASS_THREADS / 32) + (threadIdx.x >> 5)) * ROWS_PER_WARP + lane / LANES;
    const int b = blockIdx.z;
    const bool live = row < R;
    const int r = live ? row : R - 1;               // idle groups of the last warp redo the last row and store nothing
    const float4 v = src.quad(b, r, sub * 4, K);
    float m = 0.0f;
    if (OWN_MAX) {
        m = abs4max(m, v);
#pragma unroll
        for (int o = LANES / 2; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    } else {
        m = bits_f32(maxbits[(size_t)b * slot_batch_mul + (size_t)slot_div.div(r) * slot_row_mul]);
    }
    if (!live) return;
    const int e = scale_exponent(m);
    if (sub == 0) expo[(size_t)b * R + row] = e;
    const QuantScale q = quant_scale(e, S);
    const size_t plane_stride = (size_t)R * Kp;
    int8_t* out = planes + (size_t)b * S * plane_stride + (size_t)row * Kp;
    store_quad<S>(v, q, plain_row(e), out, plane_stride, (size_t)sub * 4);
    for (int c = sub; c < (Kp - 4 * LANES) / 16; c += LANES)          // bytes [4 * LANES, Kp) of every plane row are padding
#pragma unroll
        for (int p = 0; p < S; ++p)
            *reinterpret_cast<uint4*>(out + p * plane_stride + 4 * LANES + 16 * c) = make_uint4(0u, 0u, 0u, 0u);
}

template <int S, class Source, int HEXES, int LANES, bool OWN_MAX>
__global__ void __launch_bounds__(PREPASS_THREADS)
gather_rows16_kernel(const Source src, const uint32_t* __restrict__ maxbits, int8_t* __restrict__ planes,
                     int* __restrict__ expo, int R, int K, int Kp, int slot_batch_mul, int slot_row_mul, FastDiv slot_div) {
    constexpr int ROWS_PER_WARP = 32 / LANES;
    const int lane = threadIdx.x & 31, sub = lane % LANES;
    const int row = (blockIdx.x * (PREPASS_THREADS / 32) + (threadIdx.x >> 5)) * ROWS_PER_WARP + lane / LANES;
    const int b = blockIdx.z;
    const bool live = row < R;
    const int r = live ? row : R - 1;
    float v[HEXES][16];
    float m = 0.0f;
#pragma unroll
    for (int i = 0; i < HEXES; ++i) {
        src.hex(b, r, (sub + LANES * i) * 16, K, v[i]);
        if (OWN_MAX) m = abs16max(m, v[i]);
    }
    if (OWN_MAX) {
#pragma unroll
        for (int o = LANES / 2; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    } else {
        m = bits_f32(maxbits[(size_t)b * slot_batch_mul + (size_t)slot_div.div(r) * slot_row_mul]);
    }
    if (!live) return;
    const int e = scale_exponent(m);
    if (sub == 0) expo[(size_t)b * R + row] = e;
    const QuantScale q = quant_scale(e, S);
    const bool plain = plain_row(e);
    const size_t plane_stride = (size_t)R * Kp;
    int8_t* out = planes + (size_t)b * S * plane_stride + (size_t)row * Kp;
#pragma unroll
    for (int i = 0; i < HEXES; ++i) {
        const int k = (sub + LANES * i) * 16;
        if (k < Kp) store_hex<S>(v[i], q, plain, out, plane_stride, (size_t)k);
    }
}

constexpr int GATHER_ROWS_MAX_KP = 1024;       // longest padded row the one-launch forms keep in registers

template <int S, class Source, bool OWN_MAX>
void launch_gather_rows_s(const Source& src, const uint32_t* maxbits, int8_t* planes, int* expo, int R, int K, int Kp,
                          int batch, int slot_batch_mul, int slot_row_mul, FastDiv slot_div, cudaStream_t st) {
#define RGB_GRID(LN) dim3((R + 8 * (32 / LN) - 1) / (8 * (32 / LN)), 1, batch), PREPASS_THREADS, 0, st
#define RGB_ARGS src, maxbits, planes, expo, R, K, Kp, slot_batch_mul, slot_row_mul, slot_div
    if (K <= 32) gather_rows_kernel<S, Source, 8, OWN_MAX><<<RGB_GRID(8)>>>(RGB_ARGS);
    else if (K <= 64) gather_rows_kernel<S, Source, 16, OWN_MAX><<<RGB_GRID(16)>>>(RGB_ARGS);
    // lanes per row x steps chosen so that few lanes idle: 8, 16, 24, 32, 48 and 64 sixteens per row fit exactly
    else if (Kp <= 128) gather_rows16_kernel<S, Source, 1, 8, OWN_MAX><<<RGB_GRID(8)>>>(RGB_ARGS);
    else if (Kp <= 256) gather_rows16_kernel<S, Source, 1, 16, OWN_MAX><<<RGB_GRID(16)>>>(RGB_ARGS);
    else if (Kp <= 384) gather_rows16_kernel<S, Source, 3, 8, OWN_MAX><<<RGB_GRID(8)>>>(RGB_ARGS);
    else if (Kp <= 512) gather_rows16_kernel<S, Source, 1, 32, OWN_MAX><<<RGB_GRID(32)>>>(RGB_ARGS);
    else if (Kp <= 768) gather_rows16_kernel<S, Source, 3, 16, OWN_MAX><<<RGB_GRID(16)>>>(RGB_ARGS);
    else gather_rows16_kernel<S, Source, 2, 32, OWN_MAX><<<RGB_GRID(32)>>>(RGB_ARGS);
#undef RGB_GRID
#undef RGB_ARGS
}

template <class Source>
void launch_gather_max(const Source& src, uint32_t* maxbits, int R, int K, int batch, int slot_batch_mul, int slot_row_mul,
                       cudaStream_t st) {
    const dim3 grid((R + 7) / 8, (K + GATHER_CHUNK - 1) / GATHER_CHUNK, batch);
    gather_max_kernel<Source><<<grid, PREPASS_THREADS, 0, st>>>(src, maxbits, R, K, slot_batch_mul, slot_row_mul);
}

template <class Source>
void launch_gather_split(int S, const Source& src, const uint32_t* maxbits, int8_t* planes, int* expo, int R, int K, int Kp,
                         int batch, int slot_batch_mul, int slot_row_mul, FastDiv slot_div, cudaStream_t st) {
    const dim3 grid((R + 7) / 8, (Kp + GATHER_CHUNK - 1) / GATHER_CHUNK, batch);
    switch (S) {
        case 1: gather_split_kernel<1, Source><<<grid, PREPASS_THREADS, 0, st>>>(src, maxbits, planes, expo, R, K, Kp, slot_batch_mul, slot_row_mul, slot_div); break;
        case 2: gather_split_kernel<2, Source><<<grid, PREPASS_THREADS, 0, st>>>(src, maxbits, planes, expo, R, K, Kp, slot_batch_mul, slot_row_mul, slot_div); break;
        default: gather_split_kernel<3, Source><<<grid, PREPASS_THREADS, 0, st>>>(src, maxbits, planes, expo, R, K, Kp, slot_batch_mul, slot_row_mul, slot_div); break;
    }
}

// One operand through the gather pre-pass.  OWN_MAX: every row has its own scale (its slot is
// b * R + r); otherwise the maxima were reduced beforehand into the given slots.
template <bool OWN_MAX, class Source>
void launch_gather_operand(int S, const Source& src, uint32_t* maxbits, int8_t* planes, int* expo, int R, int K, int Kp,
                           int batch, int slot_batch_mul, int slot_row_mul, FastDiv slot_div, cudaStream_t st) {
    if (OWN_MAX) { slot_batch_mul = R; slot_row_mul = 1; slot_div = FastDiv(); }
    if (Kp > GATHER_ROWS_MAX_KP) {             // long rows: maxima by atomics over chunks, then the split
        if (OWN_MAX) launch_gather_max(src, maxbits, R, K, batch, slot_batch_mul, slot_row_mul, st);
        launch_gather_split(S, src, maxbits, planes, expo, R, K, Kp, batch, slot_batch_mul, slot_row_mul, slot_div, st);
        return;
    }
    switch (S) {
        case 1: launch_gather_rows_s<1, Source, OWN_MAX>(src, maxbits, planes, expo, R, K, Kp, batch, slot_batch_mul, slot_row_mul, slot_div, st); break;
        case 2: launch_gather_rows_s<2, Source, OWN_MAX>(src, maxbits, planes, expo, R, K, Kp, batch, slot_batch_mul, slot_row_mul, slot_div, st); break;
        default: launch_gather_rows_s<3, Source, OWN_MAX>(src, maxbits, planes, expo, R, K, Kp, batch, slot_batch_mul, slot_row_mul, slot_div, st); break;
    }
}

}  // namespace rgb200
