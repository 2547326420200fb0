// TEST INFRASTRUCTURE, NOT PRODUCT CODE.
//
// C entry points around the reference's own CUDA implementation (repro_gemm_cuda/repro_gemm.cu,
// compiled unmodified for sm_100a by oracle/Makefile; its tensor-core path is WMMA int8).  Used on the
// GPU box as a second checker ("bit-identical to the reference's existing CUDA kernel") and as the
// same-box timing comparison.  Wrapped: make_plan (repro_gemm.cuh:53) and repro_gemm_fp32_ws (:60).
#include "repro_gemm.cuh"

static repro_gemm::Config make_cfg(int split_k, int algo, int slices, int ta, int tb) {
    repro_gemm::Config c;
    c.split_k = split_k;
    c.algo = static_cast<repro_gemm::Algo>(algo);
    c.slices = slices;
    c.trans_a = ta != 0;
    c.trans_b = tb != 0;
    return c;
}

extern "C" {

int refcuda_plan(int M, int N, int K, int split_k, int algo, int slices, int ta, int tb, int* eff_split, size_t* ws_bytes) {
    repro_gemm::Plan p;
    cudaError_t e = repro_gemm::make_plan(M, N, K, make_cfg(split_k, algo, slices, ta, tb), &p);
    if (e == cudaSuccess) { *eff_split = p.split_k; *ws_bytes = p.workspace_bytes; }
    return (int)e;
}

int refcuda_gemm_ws(const float* A, const float* B, float* C, int M, int N, int K, int split_k, int algo, int slices,
                    int ta, int tb, void* ws, size_t ws_bytes, void* stream, void* const* events4) {
    return (int)repro_gemm::repro_gemm_fp32_ws(A, B, C, M, N, K, make_cfg(split_k, algo, slices, ta, tb), ws, ws_bytes,
                                               static_cast<cudaStream_t>(stream),
                                               reinterpret_cast<const cudaEvent_t*>(events4));
}

}
