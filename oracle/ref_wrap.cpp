// TEST INFRASTRUCTURE, NOT PRODUCT CODE.
//
// C entry points around the reference's own CPU implementation, compiled from the reference's
// source files where they lie (the Makefile passes their directory with -I; nothing is copied).
// The resulting library (oracle/_ref/librepro_ref.so) validates oracle.c and serves as the timed
// CPU baseline.  Wrapped: repro_gemm_cuda/repro_gemm_cpu.h:25 (cpu_gemm) and
// repro_gemm_cuda/repro_gemm_math.cuh:59,74,96 (scale_exponent, fixed_point, round_to_float).
#include "repro_gemm_cpu.h"
#include <cstdint>

extern "C" {

// Thread count follows the reference: REPRO_CPU_THREADS or every hardware thread.
void ref_cpu_gemm(const float* A, const float* B, float* C, int M, int N, int K, int ta, int tb, int S) {
    repro_gemm::cpu_gemm(A, B, C, M, N, K, ta != 0, tb != 0, S);
}
int ref_scale_exponent(float m) { return repro_gemm::scale_exponent(m); }
int ref_fixed_point(float x, int se, int S) { return repro_gemm::fixed_point(x, se, S); }
float ref_round_to_float(int64_t T, int E) { return repro_gemm::round_to_float(T, E); }

}
