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

// The convolution entry points with the reference's signatures (repro_conv_cuda/repro_conv.cuh:22-32).
#include "../../include/repro_conv.cuh"

namespace repro_conv {

static_assert(sizeof(ConvShape) == sizeof(rgb200_conv_shape), "ConvShape and rgb200_conv_shape are the same eleven ints");
static const rgb200_conv_shape* to_c(const ConvShape& g) { return reinterpret_cast<const rgb200_conv_shape*>(&g); }

cudaError_t conv2d_workspace(const ConvShape& g, int S, size_t* bytes) {
    return static_cast<cudaError_t>(rgb200_conv2d_workspace(to_c(g), S, bytes));
}
cudaError_t conv2d_grad_weight_workspace(const ConvShape& g, int S, size_t* bytes) {
    return static_cast<cudaError_t>(rgb200_conv2d_grad_weight_workspace(to_c(g), S, bytes));
}
cudaError_t conv2d_grad_input_workspace(const ConvShape& g, int S, size_t* bytes) {
    return static_cast<cudaError_t>(rgb200_conv2d_grad_input_workspace(to_c(g), S, bytes));
}
cudaError_t repro_conv2d_ws(const float* x, const float* weight, float* out, const ConvShape& g, int S,
                            void* workspace, size_t workspace_bytes, cudaStream_t stream) {
    return static_cast<cudaError_t>(rgb200_conv2d_ws(x, weight, out, to_c(g), S, workspace, workspace_bytes, stream));
}
cudaError_t repro_conv2d_grad_weight_ws(const float* dy, const float* x, float* dw, const ConvShape& g, int S,
                                        void* workspace, size_t workspace_bytes, cudaStream_t stream) {
    return static_cast<cudaError_t>(rgb200_conv2d_grad_weight_ws(dy, x, dw, to_c(g), S, workspace, workspace_bytes, stream));
}
cudaError_t repro_conv2d_grad_input_ws(const float* dy, const float* weight, float* dx, const ConvShape& g, int S,
                                       void* workspace, size_t workspace_bytes, cudaStream_t stream) {
    return static_cast<cudaError_t>(rgb200_conv2d_grad_input_ws(dy, weight, dx, to_c(g), S, workspace, workspace_bytes, stream));
}

}  // namespace repro_conv
