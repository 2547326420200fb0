// Source-compatible replacement for the reference's repro_gemm_cuda/repro_gemm.cuh (lines 25-75):
// the same namespace, types, defaults and signatures.  librgb200.so defines these functions (thin
// C++ wrappers over its C ABI, include/rgb200.h), so a program written against the reference header
// or against this one links -lrgb200 instead of compiling the reference's repro_gemm.cu.
#pragma once
#include <cuda_runtime.h>
#include <cstddef>
#include <cstdint>
#include "rgb200.h"

namespace repro_gemm {

#ifndef REPRO_GEMM_MAX_SLICES_DEFINED
#define REPRO_GEMM_MAX_SLICES_DEFINED
// The reference defines this constant in repro_gemm_math.cuh:22; programs that also include that
// header (its test tools do) should define REPRO_GEMM_MAX_SLICES_DEFINED before this one.
constexpr int MAX_SLICES = 3;
#endif

enum class Algo {
    Auto,        // the tcgen05 tensor-core path on sm_100
    Reference,   // one-thread-per-output INT64 kernel; slow, for verification
    Tiled,       // the reference's dp4a path: not available here (cudaErrorNotSupported)
    TensorCore,  // same as Auto
};

struct Config {
    int split_k = 1;          // >= 1. May be raised automatically to keep INT32 sums exact.
    int tile_m = 16;          // ignored; kept for source compatibility
    int tile_n = 16;          // ignored
    int tile_k = 32;          // ignored
    Algo algo = Algo::Auto;
    int slices = 3;           // S, 1..MAX_SLICES
    bool trans_a = false;     // false: A is MxK row-major.  true: A is KxM row-major (use A^T)
    bool trans_b = false;     // false: B is KxN row-major.  true: B is NxK row-major (use B^T)
};

struct Plan {
    Algo algo;               // resolved (never Auto)
    int split_k;             // effective split count
    size_t workspace_bytes;  // size needed by repro_gemm_fp32_ws
};

// Defined in librgb200.so with exactly these C++ signatures, so a program compiled against the
// reference's own header links against the library as well.
cudaError_t make_plan(int M, int N, int K, Config cfg, Plan* plan);

cudaError_t repro_gemm_fp32_ws(const float* A, const float* B, float* C, int M, int N, int K, Config cfg,
                               void* workspace, size_t workspace_bytes, cudaStream_t stream = nullptr,
                               const cudaEvent_t* stage_events = nullptr);

cudaError_t repro_gemm_fp32(const float* A, const float* B, float* C, int M, int N, int K, Config cfg = Config(),
                            cudaStream_t stream = nullptr);

const char* algo_name(Algo a);

}  // namespace repro_gemm
