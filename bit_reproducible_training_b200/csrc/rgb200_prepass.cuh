// Scale-and-split pre-pass: row/column maxima -> power-of-two scale exponents -> S int8 digit planes.
//
// Output layout in HBM (what the TMA descriptors of the MMA kernel read):
//   planes[batch][S][R][Kp] int8, k contiguous ("K-major") for BOTH operands: op(A) as [M][Kp] and
//   op(B) transposed as [N][Kp].  Kp = K rounded up to 128; the k padding is written as zeros, rows
//   beyond R do not exist (TMA zero-fills them).  expo[batch][R] int32 holds the scale exponents.
// Algorithmic traffic: (4 + S) bytes per input element (+ 4 per row).
//
// Reference counterparts: quantize_kmajor / quantize_kstrided (repro_gemm_cuda/repro_gemm.cu:54-121),
// which read every operand twice with scalar loads and one block per row or 32 rows.
#pragma once
#include "rgb200_math.cuh"

namespace rgb200 {

constexpr int PREPASS_THREADS = 256;
constexpr int KMAJOR_MAX_CHUNKS = 16;     // most float4 chunks a thread keeps in registers

__device__ __forceinline__ float abs4max(float m, float4 v) {
    return fmaxf(fmaxf(m, fmaxf(fabsf(v.x), fabsf(v.y))), fmaxf(fabsf(v.z), fabsf(v.w)));
}

// Fixed-point value of x plus the digit bias, Y = X + 64 * (128^(S-2) + ... + 1), by float arithmetic:
// clamp in float (RNE commutes with clamping to an integer), then add 1.5 * 2^23 so that the FP32
// adder itself performs the round-to-nearest-even to an integer (|v| < 2^22), and read the integer
// from the mantissa.  With the bias every lower digit becomes an unsigned 7-bit field of Y:
//   d[S-1] + 64 = Y & 127,  d[S-2] + 64 = (Y >> 7) & 127,  ...,  d[0] = Y >> 7(S-1)  (arithmetic shift).
// PLAIN rows (scale exponent e > -113, all but rows of denormal-range magnitude) need neither the
// second factor (2^n fits one float) nor the clamp (it can only trigger when max|x|/127 is subnormal
// and loses relative precision), so they take three instructions per element.
template <int S, bool PLAIN>
__device__ __forceinline__ int biased_fixed_point(float x, const QuantScale& q, float limf) {
    float v = __fmul_rn(x, q.f1);
    if (!PLAIN) {
        v = __fmul_rn(v, q.f2);
        v = fminf(fmaxf(v, -limf), limf);
    }
    constexpr int BIAS = S == 1 ? 0 : (S == 2 ? 64 : 64 * 129);
    return __float_as_int(__fadd_rn(v, 12582912.0f)) - (0x4B400000 - BIAS);
}

// True when the row can take the PLAIN path: the scaling is a single normal factor and the quotient
// max|x| / 127 that defined e was a normal float (e >= -126 + 7 leaves a wide margin).
__device__ __forceinline__ bool plain_row(int e) { return e > -113; }

// Bytes 0 of four words -> one word (three byte permutes).
__device__ __forceinline__ uint32_t pack_low_bytes(int a, int b, int c, int d) {
    return __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(c, d, 0x0040), 0x5410);
}
// Four packed 7-bit fields (value + 64 each) -> four packed signed bytes, without borrows between bytes.
__device__ __forceinline__ uint32_t unbias_bytes(uint32_t w) {
    return (((w & 0x7F7F7F7Fu) | 0x80808080u) - 0x40404040u) ^ 0x80808080u;
}

// Quantise four consecutive k values and store them as one 32-bit word per digit plane.
template <int S, bool PLAIN>
__device__ __forceinline__ void store_quad_impl(float4 v, const QuantScale& q, int8_t* plane0, size_t plane_stride, size_t idx) {
    const float limf = (float)q.lim;
    int y0 = biased_fixed_point<S, PLAIN>(v.x, q, limf), y1 = biased_fixed_point<S, PLAIN>(v.y, q, limf);
    int y2 = biased_fixed_point<S, PLAIN>(v.z, q, limf), y3 = biased_fixed_point<S, PLAIN>(v.w, q, limf);
#pragma unroll
    for (int p = S - 1; p >= 0; --p) {
        uint32_t w = pack_low_bytes(y0, y1, y2, y3);
        if (p > 0) { w = unbias_bytes(w); y0 >>= 7; y1 >>= 7; y2 >>= 7; y3 >>= 7; }
        *reinterpret_cast<uint32_t*>(plane0 + p * plane_stride + idx) = w;
    }
}
template <int S>
__device__ __forceinline__ void store_quad(float4 v, const QuantScale& q, bool plain, int8_t* plane0, size_t plane_stride, size_t idx) {
    if (plain) store_quad_impl<S, true>(v, q, plane0, plane_stride, idx);
    else store_quad_impl<S, false>(v, q, plane0, plane_stride, idx);
}

// Max over the TPR threads that share a row (TPR = 32, 64, 128 or 256; a CTA holds 256 / TPR rows).
// Every thread of the CTA must call it when TPR > 32 (it contains a CTA-wide barrier).
template <int TPR>
__device__ __forceinline__ float row_group_max(float m, float* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    if (TPR > 32) {
        constexpr int WPG = TPR / 32;                  // warps per row group
        const int w = threadIdx.x >> 5;
        if ((threadIdx.x & 31) == 0) red[w] = m;
        __syncthreads();
        const int g0 = (w / WPG) * WPG;
        m = red[g0];
#pragma unroll
        for (int i = 1; i < WPG; ++i) m = fmaxf(m, red[g0 + i]);
    }
    return m;
}

// ---------------------------------------------------------------------------------------------
// k-contiguous operand: element (r, k) at src[r*K + k]   (A without trans_a, B with trans_b).
// One read of the operand: a group of TPR threads keeps its row in registers (CHUNKS float4 per
// thread) between the max and the split.  VEC = false is the general path (any K, any alignment):
// scalar loads, and the row is read a second time (it is still in L2).
// grid = (ceil(R / (256 / TPR)), batch)
// ---------------------------------------------------------------------------------------------
// One k-contiguous operand of a split launch.
struct KmajorOperand {
    const float* src;
    const float* given_max;     // externally reduced row maxima, or null
    int8_t* planes;
    int* expo;
    int R;
    long long batch_stride;
};

// The kernel takes up to two operands of the same row length (op(A) and op(B)^T of one product when
// both are stored k-contiguous): blocks [0, blocks_first) work on `first`, the rest on `second`, so
// the forward GEMM of a linear layer needs one pre-pass launch.  `zero_word`, if not null, is cleared
// by one thread (the workspace's status word, when no memset precedes this launch).
template <int S, int TPR, int CHUNKS, bool VEC>
__device__ __forceinline__ void split_kmajor_body(const KmajorOperand& first, const KmajorOperand& second, int blocks_first,
                                                  int K, int Kp, int* zero_word) {
    __shared__ float red[PREPASS_THREADS / 32];
    constexpr int rows_per_cta = PREPASS_THREADS / TPR;
    if (zero_word && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) *zero_word = 0;
    const bool is_first = (int)blockIdx.x < blocks_first;
    const KmajorOperand& op = is_first ? first : second;
    const float* __restrict__ src = op.src;
    const float* __restrict__ given_max = op.given_max;
    int8_t* __restrict__ planes = op.planes;
    int* __restrict__ expo = op.expo;
    const int R = op.R;
    const long long src_batch_stride = op.batch_stride;
    const int row = ((int)blockIdx.x - (is_first ? 0 : blocks_first)) * rows_per_cta + threadIdx.x / TPR;
    const int t = threadIdx.x % TPR;
    const int b = blockIdx.y;
    const bool live = row < R;
    const size_t plane_stride = (size_t)R * Kp;
    const float* a = src + (size_t)b * src_batch_stride + (size_t)(live ? row : 0) * K;
    int8_t* out = planes + (size_t)b * S * plane_stride + (size_t)(live ? row : 0) * Kp;

    float m = 0.0f;
    if (VEC) {
        const float4* a4 = reinterpret_cast<const float4*>(a);
        const int nq = K >> 2, nqp = Kp >> 2;
        float4 v[CHUNKS];
#pragma unroll
        for (int i = 0; i < CHUNKS; ++i) {
            int c = t + i * TPR;
            v[i] = (live && c < nq) ? __ldg(a4 + c) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int i = 0; i < CHUNKS; ++i) m = abs4max(m, v[i]);
        m = row_group_max<TPR>(m, red);
        if (!live) return;
        if (given_max) m = given_max[(size_t)b * R + row];
        const int e = scale_exponent(m);
        if (t == 0) expo[(size_t)b * R + row] = e;
        const QuantScale q = quant_scale(e, S);
        if (plain_row(e)) {                      // uniform over the row group
#pragma unroll
            for (int i = 0; i < CHUNKS; ++i) {
                int c = t + i * TPR;
                if (c < nqp) store_quad_impl<S, true>(v[i], q, out, plane_stride, (size_t)c * 4);   // c >= nq: zeros (k padding)
            }
        } else {
#pragma unroll
            for (int i = 0; i < CHUNKS; ++i) {
                int c = t + i * TPR;
                if (c < nqp) store_quad_impl<S, false>(v[i], q, out, plane_stride, (size_t)c * 4);
            }
        }
    } else {
        if (live && !given_max)
            for (int k = t; k < K; k += TPR) m = fmaxf(m, fabsf(__ldg(a + k)));
        m = row_group_max<TPR>(m, red);
        if (!live) return;
        if (given_max) m = given_max[(size_t)b * R + row];
        const int e = scale_exponent(m);
        if (t == 0) expo[(size_t)b * R + row] = e;
        const QuantScale q = quant_scale(e, S);
        for (int k = t * 4; k < Kp; k += TPR * 4) {
            float4 v;
            v.x = k + 0 < K ? __ldg(a + k + 0) : 0.f;
            v.y = k + 1 < K ? __ldg(a + k + 1) : 0.f;
            v.z = k + 2 < K ? __ldg(a + k + 2) : 0.f;
            v.w = k + 3 < K ? __ldg(a + k + 3) : 0.f;
            store_quad<S>(v, q, plain_row(e), out, plane_stride, (size_t)k);
        }
    }
}

// Programmatic dependent launch: this kernel lets a kernel launched behind it with programmatic stream
// serialization start early (the other operand's split, which does not depend on it), and, when it is itself
// launched that way, does not complete before the kernel in front of it has: the ordinary launch that follows
// (the MMA kernel) then finds both operands' planes complete.  Both instructions do nothing in an ordinary launch.
template <int S, int TPR, int CHUNKS, bool VEC>
__global__ void __launch_bounds__(PREPASS_THREADS)
split_kmajor_kernel(const KmajorOperand first, const KmajorOperand second, int blocks_first,
                    int K, int Kp, int* zero_word) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    split_kmajor_body<S, TPR, CHUNKS, VEC>(first, second, blocks_first, K, Kp, zero_word);
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

// Short rows (K <= 128, one padded k block per row; 16-byte aligned rows): a warp per row - or, for K <= 64, a
// half-warp per row, so that every lane loads - and every warp walks over many rows so that the grid stays
// small: the per-row work (maximum, exponent, scale) is a large part of the cost of so short a row, and with
// one row per warp the launch of tens of thousands of tiny CTAs costs more than the rows' traffic.  Four row
// slots are in flight per warp.  Same two-operand convention as split_kmajor_kernel.
// grid = (CTAs, batch); any CTA count works.
template <int S, bool HALF>
__global__ void __launch_bounds__(PREPASS_THREADS)
split_kmajor_short_kernel(const KmajorOperand first, const KmajorOperand second, int K, int* zero_word) {
    constexpr int KP = 128;
    constexpr int LANES = HALF ? 16 : 32;                 // lanes per row
    constexpr int RPW = 32 / LANES;                       // rows per warp and slot
    if (zero_word && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) *zero_word = 0;
    const int lane = threadIdx.x & 31;
    const int c = lane % LANES, sub = lane / LANES;
    const int b = blockIdx.y;
    const int nq = K >> 2;
    const int rows_total = first.R + second.R;
    const int slots_total = gridDim.x * (PREPASS_THREADS / 32) * RPW;     // rows handled side by side
    // the operand's fields are picked one by one (a pointer to a kernel parameter would force it into local memory)
    struct RowRef { const float* src; const float* given_max; int8_t* planes; int* expo; int R; int r; };
    auto locate = [&](int row) {
        const bool f = row < first.R;
        RowRef x;
        x.R = f ? first.R : second.R;
        x.r = f ? row : row - first.R;
        x.src = (f ? first.src : second.src) + (size_t)b * (f ? first.batch_stride : second.batch_stride) + (size_t)x.r * K;
        x.given_max = f ? first.given_max : second.given_max;
        x.planes = f ? first.planes : second.planes;
        x.expo = f ? first.expo : second.expo;
        return x;
    };
    auto load = [&](const RowRef& x) {
        return c < nq ? __ldg(reinterpret_cast<const float4*>(x.src) + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    };
    auto finish = [&](const RowRef& x, float4 v, bool valid) {
        float m = abs4max(0.0f, v);
#pragma unroll
        for (int o = LANES / 2; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));     // over the row's lanes
        if (!valid) return;
        if (x.given_max) m = x.given_max[(size_t)b * x.R + x.r];
        const int e = scale_exponent(m);
        if (c == 0) x.expo[(size_t)b * x.R + x.r] = e;
        const size_t plane_stride = (size_t)x.R * KP;
        int8_t* out = x.planes + (size_t)b * S * plane_stride + (size_t)x.r * KP;
        store_quad<S>(v, quant_scale(e, S), plain_row(e), out, plane_stride, (size_t)c * 4);
        if (HALF) {                                       // k 64..127 of the padded row: zeros
#pragma unroll
            for (int p = 0; p < S; ++p) *reinterpret_cast<uint32_t*>(out + p * plane_stride + 64 + c * 4) = 0u;
        }
    };
    constexpr int INFLIGHT = 4;                           // row slots whose loads are issued before the first one is consumed
    const int first_row = (blockIdx.x * (PREPASS_THREADS / 32) + (threadIdx.x >> 5)) * RPW + sub;
    // every lane of a warp runs the same number of iterations (the shuffles need the whole warp)
    for (int base = first_row - sub; base < rows_total; base += INFLIGHT * slots_total) {
        float4 v[INFLIGHT];
#pragma unroll
        for (int i = 0; i < INFLIGHT; ++i) {
            const int ri = base + sub + i * slots_total;
            v[i] = ri < rows_total ? load(locate(ri)) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int i = 0; i < INFLIGHT; ++i) {
            const int ri = base + sub + i * slots_total;
            finish(locate(ri < rows_total ? ri : 0), v[i], ri < rows_total);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// k-strided operand: element (r, k) at src[k*R + r]   (B without trans_b, A with trans_a).
// Pass 1: column maxima over K with an integer atomicMax (|x| >= 0 orders like its bit pattern,
// so the result is exact and order-free).  maxbits[batch][R] must be zero on entry.
// grid = (ceil(R / 128), min(ceil(K / 64), 65535), batch), block = 256 threads = 32 column groups x 8 k-rows.
// ---------------------------------------------------------------------------------------------
constexpr int COLMAX_K_PER_CTA = 64;
constexpr int COLMAX_MAX_GRID_Y = 65535;       // hardware limit on gridDim.y; longer K is walked by the CTAs

__global__ void __launch_bounds__(PREPASS_THREADS)
colmax_kstrided_kernel(const float* __restrict__ src, uint32_t* __restrict__ maxbits, int R, int K,
                       long long src_batch_stride) {
    __shared__ float red[8][128 + 4];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int b = blockIdx.z;
    const float* s = src + (size_t)b * src_batch_stride;
    const int r0 = blockIdx.x * 128 + tx * 4;
    float m0 = 0.f, m1 = 0.f, m2 = 0.f, m3 = 0.f;
    const bool vec = (R & 3) == 0 && ((reinterpret_cast<uintptr_t>(s) & 15) == 0);
    // a CTA takes the k chunks blockIdx.y, blockIdx.y + gridDim.y, ... (the launch caps gridDim.y at the hardware limit)
    for (long long k_lo_ll = (long long)blockIdx.y * COLMAX_K_PER_CTA; k_lo_ll < K; k_lo_ll += (long long)gridDim.y * COLMAX_K_PER_CTA) {
    const int k_lo = (int)k_lo_ll;
    const int k_hi = (int)min((long long)K, k_lo_ll + COLMAX_K_PER_CTA);
    if (vec) {
        if (r0 < R) {
            const float4* p = reinterpret_cast<const float4*>(s + (size_t)(k_lo + ty) * R + r0);
            const size_t step = (size_t)2 * R;       // 8 k-rows ahead, in float4 units (R % 4 == 0)
            const int n = (k_hi - k_lo - ty + 7) / 8;
            int i = 0;
            for (; i + 4 <= n; i += 4) {             // four independent 16-byte loads in flight per thread
                float4 v0 = __ldg(p), v1 = __ldg(p + step), v2 = __ldg(p + 2 * step), v3 = __ldg(p + 3 * step);
                p += 4 * step;
                m0 = fmaxf(fmaxf(m0, fmaxf(fabsf(v0.x), fabsf(v1.x))), fmaxf(fabsf(v2.x), fabsf(v3.x)));
                m1 = fmaxf(fmaxf(m1, fmaxf(fabsf(v0.y), fabsf(v1.y))), fmaxf(fabsf(v2.y), fabsf(v3.y)));
                m2 = fmaxf(fmaxf(m2, fmaxf(fabsf(v0.z), fabsf(v1.z))), fmaxf(fabsf(v2.z), fabsf(v3.z)));
                m3 = fmaxf(fmaxf(m3, fmaxf(fabsf(v0.w), fabsf(v1.w))), fmaxf(fabsf(v2.w), fabsf(v3.w)));
            }
            for (; i < n; ++i, p += step) {
                float4 v = __ldg(p);
                m0 = fmaxf(m0, fabsf(v.x)); m1 = fmaxf(m1, fabsf(v.y));
                m2 = fmaxf(m2, fabsf(v.z)); m3 = fmaxf(m3, fabsf(v.w));
            }
        }
    } else {
        for (int k = k_lo + ty; k < k_hi; k += 8) {
            const float* p = s + (size_t)k * R + r0;
            if (r0 + 0 < R) m0 = fmaxf(m0, fabsf(__ldg(p + 0)));
            if (r0 + 1 < R) m1 = fmaxf(m1, fabsf(__ldg(p + 1)));
            if (r0 + 2 < R) m2 = fmaxf(m2, fabsf(__ldg(p + 2)));
            if (r0 + 3 < R) m3 = fmaxf(m3, fabsf(__ldg(p + 3)));
        }
    }
    }
    red[ty][tx * 4 + 0] = m0; red[ty][tx * 4 + 1] = m1; red[ty][tx * 4 + 2] = m2; red[ty][tx * 4 + 3] = m3;
    __syncthreads();
    if (threadIdx.x < 128) {
        float m = red[0][threadIdx.x];
#pragma unroll
        for (int i = 1; i < 8; ++i) m = fmaxf(m, red[i][threadIdx.x]);
        int r = blockIdx.x * 128 + threadIdx.x;
        if (r < R && m > 0.0f) atomicMax(maxbits + (size_t)b * R + r, f32_bits(m));
    }
}

// Row maxima of a k-contiguous operand, written as floats (the K-sharded path's first step).
// One warp per row; 16-byte loads, four in flight per lane, when the rows are 16-byte aligned.  grid = ceil(R / 8).
__global__ void __launch_bounds__(PREPASS_THREADS)
rowmax_kmajor_kernel(const float* __restrict__ src, float* __restrict__ out, int R, int K) {
    const int row = blockIdx.x * (PREPASS_THREADS / 32) + (threadIdx.x >> 5);
    if (row >= R) return;
    const int lane = threadIdx.x & 31;
    const float* a = src + (size_t)row * K;
    float m = 0.f;
    if ((K & 3) == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
        const float4* a4 = reinterpret_cast<const float4*>(a);
        const int nq = K >> 2;
        int c = lane;
        for (; c + 96 < nq; c += 128) {
            const float4 v0 = __ldg(a4 + c), v1 = __ldg(a4 + c + 32), v2 = __ldg(a4 + c + 64), v3 = __ldg(a4 + c + 96);
            m = abs4max(abs4max(abs4max(abs4max(m, v0), v1), v2), v3);
        }
        for (; c < nq; c += 32) m = abs4max(m, __ldg(a4 + c));
    } else {
        for (int k = lane; k < K; k += 32) m = fmaxf(m, fabsf(__ldg(a + k)));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    if (lane == 0) out[row] = m;
}

// Pass 2 for the k-strided operand: 32 (r) x 128 (k) tiles are read with r contiguous (16-byte loads
// where R allows), transposed through shared memory and written with k contiguous, 128 bytes per
// row and plane.  Shared layout: tile[r][k] with the 16-byte column index XOR-ed by (r / 4) % 8, which
// makes both the transposing stores and the row reads bank-conflict free.  A CTA walks over several
// k tiles of its 32 rows and loads the next tile into registers while it splits the current one.
// grid = (ceil(R / 32), k-tile walkers <= Kp / 128, batch)
template <int S>
__global__ void __launch_bounds__(PREPASS_THREADS)
split_kstrided_kernel(const float* __restrict__ src, const uint32_t* __restrict__ maxbits,
                      int8_t* __restrict__ planes, int* __restrict__ expo,
                      int R, int K, int Kp, long long src_batch_stride) {
    __shared__ __align__(16) float tile[32 * 128];
    __shared__ int e_sh[32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int b = blockIdx.z;
    const int r0 = blockIdx.x * 32;
    const int k_tiles = Kp / 128;
    const float* s = src + (size_t)b * src_batch_stride;
    const size_t plane_stride = (size_t)R * Kp;
    int8_t* out = planes + (size_t)b * S * plane_stride;
    auto slot = [](int r, int k) { return r * 128 + ((((k >> 2) ^ ((r >> 2) & 7))) << 2) + (k & 3); };

    if (threadIdx.x < 32) {
        int r = r0 + threadIdx.x;
        int e = r < R ? scale_exponent(bits_f32(maxbits[(size_t)b * R + r])) : 0;
        e_sh[threadIdx.x] = e;
        if (r < R && blockIdx.y == 0) expo[(size_t)b * R + r] = e;
    }
    const bool vec = (R & 3) == 0 && ((reinterpret_cast<uintptr_t>(s) & 15) == 0);
    // vector path: a warp covers 4 k-rows x 32 r per load, lane = (k sub-row, group of four r);
    // scalar path: a warp covers one k-row, lane = r.  Either way a thread holds 16 values of a tile.
    const int kk4 = lane >> 3, rq = lane & 7;
    float4 reg[4];
    auto load_tile = [&](int kt) {
        const int k0 = kt * 128;
        if (vec) {
            const int r = r0 + rq * 4;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int k = k0 + warp * 4 + kk4 + 32 * i;
                reg[i] = (r < R && k < K) ? __ldg(reinterpret_cast<const float4*>(s + (size_t)k * R + r))
                                          : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        } else {
            const int r = r0 + lane;
            float* f = reinterpret_cast<float*>(reg);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int k = k0 + warp + 8 * i;
                f[i] = (r < R && k < K) ? __ldg(s + (size_t)k * R + r) : 0.0f;
            }
        }
    };
    auto stage_tile = [&]() {
        if (vec) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int kk = warp * 4 + kk4 + 32 * i;
                tile[slot(rq * 4 + 0, kk)] = reg[i].x;
                tile[slot(rq * 4 + 1, kk)] = reg[i].y;
                tile[slot(rq * 4 + 2, kk)] = reg[i].z;
                tile[slot(rq * 4 + 3, kk)] = reg[i].w;
            }
        } else {
            const float* f = reinterpret_cast<const float*>(reg);
#pragma unroll
            for (int i = 0; i < 16; ++i) tile[slot(lane, warp + 8 * i)] = f[i];
        }
    };

    int kt = blockIdx.y;
    if (kt < k_tiles) load_tile(kt);
    for (; kt < k_tiles; kt += gridDim.y) {
        stage_tile();
        __syncthreads();
        const int next = kt + gridDim.y;
        if (next < k_tiles) load_tile(next);            // in flight while this tile is split
        // split: warp w takes rows w, w + 8, ...; lanes run along k in groups of four
#pragma unroll
        for (int rr = warp; rr < 32; rr += 8) {
            const int r = r0 + rr;
            if (r >= R) continue;
            const int e = e_sh[rr];
            const QuantScale q = quant_scale(e, S);
            const float4 v = *reinterpret_cast<const float4*>(&tile[slot(rr, lane * 4)]);
            store_quad<S>(v, q, plain_row(e), out, plane_stride, (size_t)r * Kp + kt * 128 + lane * 4);   // uniform over the warp
        }
        __syncthreads();                                 // the tile is rewritten by the next round
    }
}

// Turns float maxima (as exchanged between ranks) into the bit form split_kstrided_kernel reads.
__global__ void maxima_to_bits_kernel(const float* __restrict__ in, uint32_t* __restrict__ out, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = f32_bits(fmaxf(in[i], 0.0f));
}

}  // namespace rgb200
