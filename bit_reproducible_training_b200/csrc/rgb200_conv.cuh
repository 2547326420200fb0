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
#pragma once
#include "rgb200_prepass.cuh"

namespace rgb200 {

// Division of a non-negative 32-bit integer (below 2^31) by a fixed divisor as one multiply-high and a
// shift: with p = 31 + ceil(log2 d) and mul = ceil(2^p / d), floor(n / d) = (n * mul) >> p for all such n.
// The index maps divide by kernel and image extents for every element they fetch.
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
    FastDiv by_khw, by_kw, by_ow, by_per, by_w, by_sy, by_sx, by_f;   // KH*KW, KW, OW, OH*OW, W, SY, SX, F
    void prepare() {
        by_khw = FastDiv(KH * KW); by_kw = FastDiv(KW); by_ow = FastDiv(OW); by_per = FastDiv(OH * OW);
        by_w = FastDiv(W); by_sy = FastDiv(SY); by_sx = FastDiv(SX); by_f = FastDiv(F);
    }
};

// ---------------------------------------------------------------------------------------------
// Index maps: at(b, r, k) is element (row r, index k) of operand matrix number b; quad(b, r, k, K)
// is the four elements k .. k+3 with zeros from index K on (the padding of the digit planes).
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
#define RGB_QUAD_BY_ELEMENTS \
    __device__ __forceinline__ float4 quad(int b, int r, int k, int K) const { return quad_by_elements(*this, b, r, k, K); }

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

struct WindowsOfImage {      // forward: b = image, r = window (oy, ox) of that image, k = position
    const float* x; ConvGeom g;
    __device__ __forceinline__ float at(int b, int r, int k) const {
        const int oy = g.by_ow.div(r);
        return conv_window_value(x, g, b, oy, r - oy * g.OW, k);
    }
    __device__ __forceinline__ float4 quad(int b, int r, int k, int K) const {
        const int oy = g.by_ow.div(r);
        return conv_window_quad(x, g, b, oy, r - oy * g.OW, k, K);
    }
};

struct AllWindows {          // forward: r = window (n, oy, ox) over all images, k = position
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
};

struct PositionsOverWindows {   // weight gradient: r = position, k = window (n, oy, ox)
    const float* x; ConvGeom g;
    __device__ __forceinline__ float at(int, int r, int k) const {
        const int n = g.by_per.div(k), j = k - n * (g.OH * g.OW);
        const int oy = g.by_ow.div(j);
        return conv_window_value(x, g, n, oy, j - oy * g.OW, r);
    }
    __device__ __forceinline__ float4 quad(int, int r, int k, int K) const {   // four consecutive windows, one position
        const int c = g.by_khw.div(r), rem = r - c * (g.KH * g.KW);
        const int ky = g.by_kw.div(rem), kx = rem - ky * g.KW;
        int n = g.by_per.div(k);
        const int j = k - n * (g.OH * g.OW);
        int oy = g.by_ow.div(j), ox = j - oy * g.OW;
        float e[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int y = oy * g.SY - g.PY + ky, xx = ox * g.SX - g.PX + kx;
            const bool inside = k + i < K && (unsigned)y < (unsigned)g.H && (unsigned)xx < (unsigned)g.W;
            e[i] = inside ? __ldg(x + (((size_t)n * g.C + c) * g.H + y) * g.W + xx) : 0.0f;
            if (++ox == g.OW) { ox = 0; if (++oy == g.OH) { oy = 0; ++n; } }
        }
        return make_float4(e[0], e[1], e[2], e[3]);
    }
};

struct FiltersOverWindows {     // weight gradient: r = filter, k = window (n, oy, ox); dY is [N][F][OH*OW]
    const float* dy; ConvGeom g;
    __device__ __forceinline__ float at(int, int r, int k) const {
        const int per = g.OH * g.OW;
        const int n = g.by_per.div(k), j = k - n * per;
        return __ldg(dy + ((size_t)n * g.F + r) * per + j);
    }
    __device__ __forceinline__ float4 quad(int b, int r, int k, int K) const {   // contiguous within an image
        const int per = g.OH * g.OW;
        const int n = g.by_per.div(k), j = k - n * per;
        if (k + 3 >= K || j + 3 >= per) return quad_by_elements(*this, b, r, k, K);
        const float* p = dy + ((size_t)n * g.F + r) * per + j;
        return make_float4(__ldg(p), __ldg(p + 1), __ldg(p + 2), __ldg(p + 3));
    }
};

// Input gradient: the index k runs over (ky, kx, f) with the filter f fastest (any order gives the same
// exact sum as long as both operands use it), so four consecutive k are usually four filters at one tap:
// one window lookup, four loads a whole output map apart.
struct ChannelsOverTaps {       // r = input channel, k = (tap, f); weights are [F][C][KH][KW]
    const float* w; ConvGeom g;
    __device__ __forceinline__ float at(int, int r, int k) const {
        const int tap = g.by_f.div(k), f = k - tap * g.F;
        return __ldg(w + ((size_t)f * g.C + r) * (g.KH * g.KW) + tap);
    }
    RGB_QUAD_BY_ELEMENTS
};

struct PixelsOverTaps {         // b = image, r = pixel (y, x), k = (tap, f)
    const float* dy; ConvGeom g;
    // dY[b, 0, oy, ox] of the window whose tap lies on pixel r, or null when the strides and edges allow none
    __device__ __forceinline__ const float* window_at_tap(int b, int r, int tap) const {
        const int ky = g.by_kw.div(tap), kx = tap - ky * g.KW;
        const int y = g.by_w.div(r), xx = r - y * g.W;
        const int ry = y + g.PY - ky, rx = xx + g.PX - kx;
        if (ry < 0 || rx < 0) return nullptr;
        const int oy = g.by_sy.div(ry), ox = g.by_sx.div(rx);
        if (oy * g.SY != ry || ox * g.SX != rx || oy >= g.OH || ox >= g.OW) return nullptr;
        return dy + ((size_t)b * g.F * g.OH + oy) * g.OW + ox;
    }
    __device__ __forceinline__ float at(int b, int r, int k) const {
        const int tap = g.by_f.div(k), f = k - tap * g.F;
        const float* p = window_at_tap(b, r, tap);
        return p ? __ldg(p + (size_t)f * (g.OH * g.OW)) : 0.0f;
    }
    __device__ __forceinline__ float4 quad(int b, int r, int k, int K) const {
        if (g.F < 4) return quad_by_elements(*this, b, r, k, K);        // a quad could span three taps
        if (k >= K) return make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        // elements 0 .. first-1 are filters f .. of this tap, the rest filters 0 .. of the next tap (none after the last)
        const int tap = g.by_f.div(k), f = k - tap * g.F;
        const int first = min(4, g.F - f);
        const size_t per = (size_t)g.OH * g.OW;
        const float* p0 = window_at_tap(b, r, tap);
        const float* p1 = (first < 4 && tap + 1 < g.KH * g.KW) ? window_at_tap(b, r, tap + 1) : nullptr;
        if (p0) p0 += f * per;
        if (p1) p1 -= first * per;                                      // so that element i reads p1 + i * per
        float e[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float* p = i < first ? p0 : p1;
            e[i] = p ? __ldg(p + i * per) : 0.0f;
        }
        return make_float4(e[0], e[1], e[2], e[3]);
    }
};

struct AllPixelsOverTaps {      // r = pixel (n, y, x) over all images, k = (tap, f)
    const float* dy; ConvGeom g; FastDiv by_hw;
    __device__ __forceinline__ float at(int, int r, int k) const {
        const int n = by_hw.div(r);
        return PixelsOverTaps{dy, g}.at(n, r - n * (g.H * g.W), k);
    }
    __device__ __forceinline__ float4 quad(int, int r, int k, int K) const {
        const int n = by_hw.div(r);
        return PixelsOverTaps{dy, g}.quad(n, r - n * (g.H * g.W), k, K);
    }
};

struct StoredRows {             // a stored matrix [R][K]: used for the maxima of whole tensors
    const float* src; long long row_len;
    __device__ __forceinline__ float at(int, int r, int k) const { return __ldg(src + (size_t)r * row_len + k); }
    RGB_QUAD_BY_ELEMENTS
};

// ---------------------------------------------------------------------------------------------
// Pre-pass over an index map, two launches of the same shape: maxima (integer atomicMax on the bit
// patterns, exact and order-free; the slots must be zero on entry), then scale and split.
// One warp works on one row and one chunk of GATHER_CHUNK indices, so short rows (a window) and
// long rows (all windows of a position) both spread over the GPU.
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
    for (int k = k_lo + lane * 4; k < k_hi; k += 128) m = abs4max(m, src.quad(b, row, k, K));
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
    for (int k = k_lo + lane * 4; k < k_hi; k += 128) {          // a warp writes 128 contiguous bytes per plane
        store_quad<S>(src.quad(b, row, k, K), q, plain, out, plane_stride, (size_t)k);   // zeros from K up to Kp
    }
}

// Short rows (Kp <= 128 * QUADS): a group of LANES lanes keeps a whole row in registers between the maximum
// and the split, so the index map is evaluated once per element and one launch does both steps.  Rows of
// at most 32 or 64 values take 8 or 16 lanes (4 or 2 rows per warp) and fill the rest of the 128-byte
// plane row with 16-byte zero stores.  With OWN_MAX = false the scale comes from a maximum reduced
// beforehand (shared by several rows).
// grid = (ceil(R / (8 * 32 / LANES)), 1, batch), 256 threads
template <int S, class Source, int QUADS, int LANES, bool OWN_MAX>
__global__ void __launch_bounds__(PREPASS_THREADS)
gather_rows_kernel(const Source src, const uint32_t* __restrict__ maxbits, int8_t* __restrict__ planes,
                   int* __restrict__ expo, int R, int K, int Kp, int slot_batch_mul, int slot_row_mul, FastDiv slot_div) {
    static_assert(LANES == 32 || QUADS == 1, "narrow row groups hold one quad per lane");
    constexpr int ROWS_PER_WARP = 32 / LANES;
    const int lane = threadIdx.x & 31, sub = lane % LANES;
    const int row = (blockIdx.x * (PREPASS_THREADS / 32) + (threadIdx.x >> 5)) * ROWS_PER_WARP + lane / LANES;
    const int b = blockIdx.z;
    const bool live = row < R;
    const int r = live ? row : R - 1;               // idle groups of the last warp redo the last row and store nothing
    float4 v[QUADS];
    float m = 0.0f;
#pragma unroll
    for (int i = 0; i < QUADS; ++i) {
        v[i] = src.quad(b, r, (sub + LANES * i) * 4, K);
        if (OWN_MAX) m = abs4max(m, v[i]);
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
    for (int i = 0; i < QUADS; ++i) {
        const int k = (sub + LANES * i) * 4;
        if (k < Kp) store_quad<S>(v[i], q, plain, out, plane_stride, (size_t)k);
    }
    if (LANES < 32) {                                 // bytes [4 * LANES, Kp) of every plane row are padding
        for (int c = sub; c < (Kp - 4 * LANES) / 16; c += LANES)
#pragma unroll
            for (int p = 0; p < S; ++p)
                *reinterpret_cast<uint4*>(out + p * plane_stride + 4 * LANES + 16 * c) = make_uint4(0u, 0u, 0u, 0u);
    }
}

template <int S, class Source, bool OWN_MAX>
void launch_gather_rows_s(const Source& src, const uint32_t* maxbits, int8_t* planes, int* expo, int R, int K, int Kp,
                          int batch, int slot_batch_mul, int slot_row_mul, FastDiv slot_div, cudaStream_t st) {
#define RGB_ROWS(Q, LN)                                                                                          \
    gather_rows_kernel<S, Source, Q, LN, OWN_MAX><<<dim3((R + 8 * (32 / LN) - 1) / (8 * (32 / LN)), 1, batch),     \
                                                    PREPASS_THREADS, 0, st>>>(                                   \
        src, maxbits, planes, expo, R, K, Kp, slot_batch_mul, slot_row_mul, slot_div)
    if (K <= 32) RGB_ROWS(1, 8);
    else if (K <= 64) RGB_ROWS(1, 16);
    else if (Kp <= 128) RGB_ROWS(1, 32);
    else if (Kp <= 256) RGB_ROWS(2, 32);
    else if (Kp <= 512) RGB_ROWS(4, 32);
    else RGB_ROWS(8, 32);
#undef RGB_ROWS
}

constexpr int GATHER_ROWS_MAX_KP = 1024;       // longest padded row the one-launch form keeps in registers

// One operand through the gather pre-pass.  own_max: every row has its own scale (its slot is
// b * R + r); otherwise the maxima were reduced beforehand into the given slots.
template <class Source>
void launch_gather_operand(int S, const Source& src, uint32_t* maxbits, int8_t* planes, int* expo, int R, int K, int Kp,
                           int batch, bool own_max, int slot_batch_mul, int slot_row_mul, FastDiv slot_div, cudaStream_t st);

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

template <class Source>
void launch_gather_operand(int S, const Source& src, uint32_t* maxbits, int8_t* planes, int* expo, int R, int K, int Kp,
                           int batch, bool own_max, int slot_batch_mul, int slot_row_mul, FastDiv slot_div, cudaStream_t st) {
    if (Kp > GATHER_ROWS_MAX_KP) {             // long rows: maxima by atomics over chunks, then the split
        if (own_max) {
            slot_batch_mul = R; slot_row_mul = 1; slot_div = FastDiv();
            launch_gather_max(src, maxbits, R, K, batch, slot_batch_mul, slot_row_mul, st);
        }
        launch_gather_split(S, src, maxbits, planes, expo, R, K, Kp, batch, slot_batch_mul, slot_row_mul, slot_div, st);
        return;
    }
#define RGB_OPERAND(SS)                                                                                                  \
    do {                                                                                                                 \
        if (own_max) launch_gather_rows_s<SS, Source, true>(src, maxbits, planes, expo, R, K, Kp, batch, 0, 0, FastDiv(), st); \
        else launch_gather_rows_s<SS, Source, false>(src, maxbits, planes, expo, R, K, Kp, batch, slot_batch_mul, slot_row_mul, slot_div, st); \
    } while (0)
    if (S == 1) RGB_OPERAND(1); else if (S == 2) RGB_OPERAND(2); else RGB_OPERAND(3);
#undef RGB_OPERAND
}

}  // namespace rgb200
