// Scalar arithmetic that defines the output bits, written for both host and device.
//
// The definition (reference: repro_gemm_cuda/repro_gemm_math.cuh:47-119, README there lines 9-15):
//   e   = smallest integer with 2^e >= RN32(max|x| / 127)               per row of op(A), column of op(B)
//   X   = clamp(RNE(x * 2^(7(S-1) - e)), +-127 * 2^(7(S-1)))             one rounding per input
//   T   = sum_k X[i,k] * Y[j,k]                                          exact integer
//   C   = RNE_fp32(T * 2^(eA[i] + eB[j] - 14(S-1)))                      one rounding per output
// Everything below is either exact or a single IEEE operation with a fixed rounding mode, so host
// and device agree bit for bit.  Build without fast-math, FTZ or approximate division.
#pragma once
#include <cstdint>
#include <cstring>
#if defined(__CUDACC__)
#include <cuda_runtime.h>
#define RGB_HD __host__ __device__ __forceinline__
#else
#define RGB_HD inline
#endif

namespace rgb200 {

RGB_HD uint32_t f32_bits(float x) {
#ifdef __CUDA_ARCH__
    return __float_as_uint(x);
#else
    uint32_t b; std::memcpy(&b, &x, 4); return b;
#endif
}
RGB_HD float bits_f32(uint32_t b) {
#ifdef __CUDA_ARCH__
    return __uint_as_float(b);
#else
    float x; std::memcpy(&x, &b, 4); return x;
#endif
}
RGB_HD int top_bit32(uint32_t v) {   // v != 0
#ifdef __CUDA_ARCH__
    return 31 - __clz((int)v);
#else
    return 31 - __builtin_clz(v);
#endif
}
RGB_HD int top_bit64(uint64_t v) {   // v != 0
#ifdef __CUDA_ARCH__
    return 63 - __clzll((long long)v);
#else
    return 63 - __builtin_clzll(v);
#endif
}

// 2^n as a float, n in [-126, 127].
RGB_HD float pow2f(int n) { return bits_f32((uint32_t)(n + 127) << 23); }

// Smallest e with 2^e >= RN32(m / 127); 0 for m <= 0 and when the quotient underflows to zero.
RGB_HD int scale_exponent(float m) {
    if (!(m > 0.0f)) return 0;
#ifdef __CUDA_ARCH__
    float q = __fdiv_rn(m, 127.0f);
#else
    volatile float q = m / 127.0f;
#endif
    uint32_t b = f32_bits(q);
    uint32_t expo = (b >> 23) & 0xFFu, frac = b & 0x7FFFFFu;
    if (expo != 0) return (int)expo - 127 + (frac != 0 ? 1 : 0);
    if (frac == 0) return 0;
    return top_bit32(frac) - 149 + ((frac & (frac - 1)) != 0 ? 1 : 0);   // subnormal quotient
}

// The scaling x * 2^n with n = 7(S-1) - e is applied as two factors because 2^n can exceed the float
// range upwards (n <= 163).  The first product is exact whenever the final value can round to a
// non-zero integer, so the only rounding is the conversion to integer.
struct QuantScale { float f1, f2; int lim; };

RGB_HD QuantScale quant_scale(int e, int S) {
    int n = 7 * (S - 1) - e;
    int n1 = n > 127 ? 127 : n;
    QuantScale q;
    q.f1 = pow2f(n1);
    q.f2 = pow2f(n - n1);
    q.lim = 127 << (7 * (S - 1));
    return q;
}

RGB_HD int fixed_point(float x, const QuantScale& q) {
#ifdef __CUDA_ARCH__
    int X = __float2int_rn(__fmul_rn(__fmul_rn(x, q.f1), q.f2));
#else
    volatile float v = x * q.f1;
    v = v * q.f2;
    // |v| stays far below 2^31 for finite inputs within their row maximum; ties go to even
    float r = __builtin_nearbyintf(v);
    int X = (int)r;
#endif
    return X > q.lim ? q.lim : (X < -q.lim ? -q.lim : X);
}

// Digits: X is split into S balanced base-128 digits, most significant first, X = sum d[p] * 128^(S-1-p)
// with |d[0]| <= 127 and d[p>0] in [-64, 63] (the split itself lives in the pre-pass, which extracts
// biased 7-bit fields).  Any exact split gives the same T; this one keeps every slice-pair sum of a
// level within INT32 for 105517 values of k (S = 3), see max_k_per_pass().

// Largest number of k values whose level sums are guaranteed to fit INT32 in one accumulation pass.
// Level L collects the digit products d_p(x) * d_q(y) with p + q = L; per k its magnitude is at most
//   S=1: 127^2 = 16129;  S=2: max(16129, 2*127*64, 64^2) = 16256;  S=3: level 2: 2*127*64 + 64^2 = 20352.
RGB_HD int max_k_per_pass(int S) {
    return S == 1 ? 133143 : (S == 2 ? 132103 : 105516);   // floor((2^31 - 1) / bound), minus one for slack
}

RGB_HD uint64_t shr_rne(uint64_t m, int s) {   // s in [1, 63]
    uint64_t q = m >> s, rest = m & ((1ull << s) - 1), half = 1ull << (s - 1);
    return q + ((rest > half || (rest == half && (q & 1))) ? 1 : 0);
}

// Correctly rounded (nearest-even) binary32 bit pattern of the exact value m * 2^E (m > 0) by integer
// arithmetic only: subnormals, overflow to infinity, values that round to zero.
RGB_HD uint32_t round_magnitude_exact(uint64_t m, int E) {
    if (m == 0) return 0u;
    int p = top_bit64(m);
    int e = p + E;
    if (e > 127) return 0x7F800000u;
    if (e >= -126) {
        int s = p - 23;
        uint64_t q = s <= 0 ? m << (-s) : shr_rne(m, s);
        if (q == (1ull << 24)) { q >>= 1; ++e; }
        if (e > 127) return 0x7F800000u;
        return ((uint32_t)(e + 127) << 23) | ((uint32_t)q & 0x7FFFFFu);
    }
    int s = -(E + 149);
    uint64_t q = s <= 0 ? m << (-s) : (s >= 64 ? 0ull : shr_rne(m, s));
    return (uint32_t)q;     // q == 2^23 encodes the smallest normal number, as it should
}

#ifdef __CUDA_ARCH__
// Out of line on the device: it is rare (subnormal or overflowing results only) and inlining it at
// every output of the unrolled epilogue would multiply the code size.
__device__ __noinline__ uint32_t round_magnitude_rare(uint64_t m, int E) { return round_magnitude_exact(m, E); }
#endif

// Correctly rounded (nearest-even) binary32 bit pattern of the exact value T * 2^E: subnormals,
// overflow to infinity, +0 for T == 0, and -0 for a negative value that rounds to zero.
RGB_HD uint32_t round_to_f32_bits(long long T, int E) {
    if (T == 0) return 0u;
    uint32_t sign = T < 0 ? 0x80000000u : 0u;
    uint64_t m = T < 0 ? 0ull - (uint64_t)T : (uint64_t)T;
#ifdef __CUDA_ARCH__
    // Fast path: one hardware RNE conversion to 24 bits, then an exact exponent adjustment,
    // valid whenever the scaled result is a normal number.
    uint32_t fb = f32_bits(__ull2float_rn(m));
    int e = (int)(fb >> 23) - 127 + E;
    if (e >= -126 && e <= 127) return sign | (fb + ((uint32_t)E << 23));
    return sign | round_magnitude_rare(m, E);
#else
    return sign | round_magnitude_exact(m, E);
#endif
}

#ifdef __CUDA_ARCH__
// Branch-free common case of round_to_f32_bits for unrolled epilogues: returns the result that is
// valid when *ok stays true (the scaled value is a non-zero normal number); the caller redoes the
// few outputs with ok == false through round_to_f32_bits.  Keeping branches out of the per-output
// code lets the compiler interleave the independent outputs of a thread.  The signed hardware conversion
// rounds the magnitude to nearest-even and carries the sign (round-to-nearest-even is symmetric in the
// sign), so neither the absolute value nor the sign bit has to be formed separately.
__device__ __forceinline__ uint32_t round_to_f32_bits_signed(long long T, int E, bool* ok) {
    const uint32_t fb = f32_bits(__ll2float_rn(T));
    const int e = (int)((fb >> 23) & 0xFFu) + E;             // biased exponent of the scaled result
    *ok = (unsigned)(e - 1) <= 253u && (fb << 1) != 0u;      // a normal number; T == 0 converts to +0 and is redone
    return fb + ((uint32_t)E << 23);
}
#endif

}  // namespace rgb200
