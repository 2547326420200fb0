// C++ entry points with the reference's exact signatures (repro_gemm_cuda/repro_gemm.cuh:53-75),
// forwarding to the C ABI.  They let the reference's own programs (test_repro_gemm.cu,
// hash_repro_gemm.cu, gpt2_ops_suite.cu, the torch extension) link against librgb200.so unchanged.
#include "../../include/repro_gemm.cuh"

namespace repro_gemm {

static rgb200_config to_c(const Config& c) {
    rgb200_config r;
    r.split_k = c.split_k; r.tile_m = c.tile_m; r.tile_n = c.tile_n; r.tile_k = c.tile_k;
    r.algo = static_cast<int>(c.algo); r.slices = c.slices;
    r.trans_a = c.trans_a ? 1 : 0; r.trans_b = c.trans_b ? 1 : 0;
    return r;
}

cudaError_t make_plan(int M, int N, int K, Config cfg, Plan* plan) {
    if (!plan) return cudaErrorInvalidValue;
    rgb200_config c = to_c(cfg);
    rgb200_plan p;
    int rc = rgb200_make_plan(M, N, K, &c, &p);
    if (rc == 0) { plan->algo = static_cast<Algo>(p.algo); plan->split_k = p.split_k; plan->workspace_bytes = p.workspace_bytes; }
    return static_cast<cudaError_t>(rc);
}

cudaError_t repro_gemm_fp32_ws(const float* A, const float* B, float* C, int M, int N, int K, Config cfg,
                               void* workspace, size_t workspace_bytes, cudaStream_t stream,
                               const cudaEvent_t* stage_events) {
    rgb200_config c = to_c(cfg);
    return static_cast<cudaError_t>(rgb200_gemm_fp32_ws(A, B, C, M, N, K, &c, workspace, workspace_bytes, stream,
                                                        reinterpret_cast<void* const*>(stage_events)));
}

cudaError_t repro_gemm_fp32(const float* A, const float* B, float* C, int M, int N, int K, Config cfg, cudaStream_t stream) {
    rgb200_config c = to_c(cfg);
    return static_cast<cudaError_t>(rgb200_gemm_fp32(A, B, C, M, N, K, &c, stream));
}

const char* algo_name(Algo a) { return rgb200_algo_name(static_cast<int>(a)); }

}  // namespace repro_gemm
