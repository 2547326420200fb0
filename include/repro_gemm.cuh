// Source-compatible replacement for the reference's repro_gemm_cuda/repro_gemm.cuh (lines 25-75):
// the same namespace, types, defaults and signatures, implemented as thin inline calls into the
// C ABI of librgb200.so (include/rgb200.h).  A program written against the reference header builds
// against this one unchanged; instead of compiling the reference's repro_gemm.cu it links -lrgb200.
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

namespace detail {
inline rgb200_config to_c(const Config& c) {
    rgb200_config r;
    r.split_k = c.split_k; r.tile_m = c.tile_m; r.tile_n = c.tile_n; r.tile_k = c.tile_k;
    r.algo = static_cast<int>(c.algo); r.slices = c.slices;
    r.trans_a = c.trans_a ? 1 : 0; r.trans_b = c.trans_b ? 1 : 0;
    return r;
}
}  // namespace detail

inline cudaError_t make_plan(int M, int N, int K, Config cfg, Plan* plan) {
    if (!plan) return cudaErrorInvalidValue;
    rgb200_config c = detail::to_c(cfg);
    rgb200_plan p;
    int rc = rgb200_make_plan(M, N, K, &c, &p);
    if (rc == 0) { plan->algo = static_cast<Algo>(p.algo); plan->split_k = p.split_k; plan->workspace_bytes = p.workspace_bytes; }
    return static_cast<cudaError_t>(rc);
}

inline cudaError_t repro_gemm_fp32_ws(const float* A, const float* B, float* C, int M, int N, int K, Config cfg,
                                      void* workspace, size_t workspace_bytes, cudaStream_t stream = nullptr,
                                      const cudaEvent_t* stage_events = nullptr) {
    rgb200_config c = detail::to_c(cfg);
    return static_cast<cudaError_t>(rgb200_gemm_fp32_ws(A, B, C, M, N, K, &c, workspace, workspace_bytes, stream,
                                                        reinterpret_cast<void* const*>(stage_events)));
}

inline cudaError_t repro_gemm_fp32(const float* A, const float* B, float* C, int M, int N, int K, Config cfg = Config(),
                                   cudaStream_t stream = nullptr) {
    rgb200_config c = detail::to_c(cfg);
    return static_cast<cudaError_t>(rgb200_gemm_fp32(A, B, C, M, N, K, &c, stream));
}

inline const char* algo_name(Algo a) { return rgb200_algo_name(static_cast<int>(a)); }

}  // namespace repro_gemm
