/*
 * rgb200 - C ABI of the B200-native integer-exact FP32 GEMM  (librgb200.so)
 *
 * C[M,N] = op(A)[M,K] * op(B)[K,N], FP32 in and out, row-major, with the output bits defined by
 * the reference project's "repro_gemm" arithmetic alone: every row of op(A) and column of op(B)
 * gets a power-of-two scale, every input is rounded once to a 7*S-bit fixed-point integer, the
 * integer dot products are formed exactly, and the exact sum is rounded once to FP32.
 *
 * Every entry point takes plain pointers and sizes.  All device work is enqueued on the stream
 * that is passed in (a cudaStream_t cast to void*; NULL = the default stream).  Return values are
 * cudaError_t codes as int (0 = success, 1 = cudaErrorInvalidValue, 801 = cudaErrorNotSupported).
 *
 * File:line citations name the interface of the reference project that each declaration stands
 * in for (paths inside that project).
 */
#ifndef RGB200_H
#define RGB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* repro_gemm_cuda/repro_gemm.cuh:25-30  enum class Algo */
enum {
    RGB200_ALGO_AUTO = 0,        /* the tcgen05 tensor-core path */
    RGB200_ALGO_REFERENCE = 1,   /* one thread per output, INT64 on CUDA cores; slow, for verification */
    RGB200_ALGO_TILED = 2,       /* the reference's dp4a fallback: not built here, always "not supported" */
    RGB200_ALGO_TENSORCORE = 3   /* same as AUTO */
};

/* repro_gemm_cuda/repro_gemm.cuh:32-41  struct Config (same fields, same order, same defaults) */
typedef struct rgb200_config {
    int split_k;   /* >= 1; a hint that never changes the output bits */
    int tile_m;    /* ignored, as in the reference */
    int tile_n;    /* ignored */
    int tile_k;    /* ignored */
    int algo;      /* RGB200_ALGO_* */
    int slices;    /* S, 1..3 */
    int trans_a;   /* 0: A is M x K row-major; 1: A is K x M row-major (use A^T) */
    int trans_b;   /* 0: B is K x N row-major; 1: B is N x K row-major (use B^T) */
} rgb200_config;

/* repro_gemm_cuda/repro_gemm.cuh:44-48  struct Plan */
typedef struct rgb200_plan {
    int algo;                /* resolved, never AUTO */
    int split_k;             /* effective number of K ranges */
    size_t workspace_bytes;  /* what the _ws entry points need */
} rgb200_plan;

/* Fills *cfg with the reference's defaults (split_k 1, tiles 16/16/32, AUTO, 3 slices, no transposes). */
void rgb200_default_config(rgb200_config* cfg);

/* repro_gemm_cuda/repro_gemm.cuh:53  make_plan
 * 1 (invalid value): null plan, M/N/K/split_k <= 0, slices outside 1..3, K too large for an exact
 * INT64 sum at this S.  801 (not supported): the algorithm cannot run on the current device. */
int rgb200_make_plan(int M, int N, int K, const rgb200_config* cfg, rgb200_plan* plan);

/* repro_gemm_cuda/repro_gemm.cuh:60-66  repro_gemm_fp32_ws
 * Asynchronous and allocation-free.  A, B, C and workspace are device pointers; workspace holds at
 * least plan.workspace_bytes (256-byte aligned).  events4, if not NULL, points to four cudaEvent_t
 * recorded before the split pre-pass, after it, after the MMA kernel and after the final step. */
int rgb200_gemm_fp32_ws(const float* A, const float* B, float* C, int M, int N, int K,
                        const rgb200_config* cfg, void* workspace, size_t workspace_bytes,
                        void* stream, void* const* events4);

/* repro_gemm_cuda/repro_gemm.cuh:69-73  repro_gemm_fp32
 * Convenience form: allocates the workspace, runs, synchronises the stream, frees.  Also reports
 * (as 702, launch timeout) a kernel that gave up on one of its bounded waits. */
int rgb200_gemm_fp32(const float* A, const float* B, float* C, int M, int N, int K,
                     const rgb200_config* cfg, void* stream);

/* repro_gemm_cuda/repro_gemm.cuh:75  algo_name  ("auto", "ref", "tiled", "tc") */
const char* rgb200_algo_name(int algo);

/* Strided-batched form: `batch` independent products, matrix b of each operand starting
 * stride_x * b elements after the first.  The reference lists batched attention GEMMs as pending
 * (gpt2_ops_suite/gpt2_ops_suite.cu:543-548); semantics are those of `batch` calls of
 * repro_gemm_fp32_ws (repro_gemm_cuda/repro_gemm.cuh:60). */
int rgb200_make_plan_batched(int M, int N, int K, int batch, const rgb200_config* cfg, rgb200_plan* plan);
int rgb200_gemm_fp32_batched_ws(const float* A, const float* B, float* C, int M, int N, int K, int batch,
                                long long stride_a, long long stride_b, long long stride_c,
                                const rgb200_config* cfg, void* workspace, size_t workspace_bytes,
                                void* stream, void* const* events4);

/* K-sharded operation (one K range per GPU).  The reference has no multi-GPU path
 * (README.md:29-30 lists it as still needed); these three calls split its single-GPU sequence
 * repro_gemm_cuda/repro_gemm.cu:451-489 at the two points where ranks must exchange data.
 *
 *  1. rgb200_absmax: out[r] = max over k of |op(X)[r,k]| for this rank's K range.  `k_strided` = 1 when
 *     k is the slow index of the stored matrix (B without trans_b, A with trans_a).  Ranks then take
 *     an element-wise max of `out` (exact, order-free) so every rank derives the same scales.
 *  2. rgb200_gemm_partial_ws: with the global maxima given, writes the exact INT64 sums T[M,N] over
 *     this rank's K range.  Ranks then add their T (integer addition: exact in any order).
 *  3. rgb200_round_partial: C = the single rounding of (sum of `parts` stacked T) * 2^(eA + eB - 14(S-1)),
 *     the job of reduce_round at repro_gemm_cuda/repro_gemm.cu:156-165.
 * K is this rank's extent; total_k (the sum over ranks) is checked against the INT64 bound. */
int rgb200_absmax(const float* X, int R, int K, int k_strided, float* out, void* stream);
int rgb200_make_plan_partial(int M, int N, int K, long long total_k, const rgb200_config* cfg, rgb200_plan* plan);
int rgb200_gemm_partial_ws(const float* A, const float* B, const float* max_a, const float* max_b,
                           long long* T, int M, int N, int K, long long total_k, const rgb200_config* cfg,
                           void* workspace, size_t workspace_bytes, void* stream);
int rgb200_round_partial(const long long* T, int parts, const float* max_a, const float* max_b, float* C,
                         int M, int N, int slices, void* stream);

/* Step 2 fused with the first half of the reduction (no counterpart in the reference): instead of
 * writing its INT64 sums locally and leaving the exchange to a collective, the MMA kernel's epilogue
 * stores each block of M / world rows straight into the memory of the rank that owns those rows
 * (ordinary peer stores over NVLink while other tiles are still being computed).  owner_buffers[o]
 * is the device address, valid on THIS device, of rank o's receive buffer of
 * rgb200_scatter_buffer_elems(M, N, world, S) INT64 elements: `world` slots, slot `rank` written by this
 * call (on every owner, its own included).  A slot keeps the owner's rows tile by tile in the order
 * the epilogue produces them, so each warp-wide store covers one contiguous kilobyte.
 * After all ranks' kernels have completed (any stream-ordered cross-rank barrier), owner o calls
 * rgb200_round_scattered(buffer_o, world, max_a + o * M / world, max_b, C_rows, M / world, N, S), which
 * adds the slots, rounds once and writes its rows of C densely.
 * world <= 8, M a multiple of 128 * world, buffers 32-byte aligned.  The buffers are peer-mapped
 * memory supplied by the caller (for example torch symmetric memory); this library maps nothing. */
size_t rgb200_scatter_buffer_elems(int M, int N, int world, int slices);
int rgb200_round_scattered(const long long* buffer, int world, const float* max_a_own, const float* max_b,
                           float* C_own, int rows_own, int N, int slices, void* stream);
int rgb200_gemm_partial_scatter_ws(const float* A, const float* B, const float* max_a, const float* max_b,
                                   long long* const* owner_buffers, int world, int rank, int M, int N, int K,
                                   long long total_k, const rgb200_config* cfg, void* workspace,
                                   size_t workspace_bytes, void* stream);

/* Host-buffer form: A, B and C live in HOST memory (pinned memory for the copies to overlap; pageable
 * memory works but serialises).  It stands in for the sequence the reference's tools run around every
 * product - cudaMemcpy of A and B, repro_gemm_fp32, cudaMemcpy of C
 * (repro_gemm_cuda/hash_repro_gemm.cu:117-118,139; test_repro_gemm.cu:35-44) - as one pipelined call:
 * B is copied first, A follows in blocks of rows, and for every block the split pre-pass, the MMA kernel
 * and the copy of the finished rows of C back to the host overlap the transfer of the next block.
 * Row blocks are independent products, so the result has the bits of a single call.
 *   rgb200_host_gemm_create   allocates the device copies of A, B, C, the workspace, three streams and the
 *                             events for one (M, N, K, cfg) on the current device; block_rows <= 0 picks 256.
 *   rgb200_gemm_fp32_host     enqueues one product; allocates nothing and does not synchronise.  Work starts
 *                             after what is already enqueued on `stream`, and `stream` continues after the
 *                             last byte of C has landed: synchronise it (or record an event on it) before
 *                             reading C_host.  One call at a time per handle.
 *   rgb200_host_gemm_info     number of row blocks, kernels launched per call, device bytes held.
 *   rgb200_host_gemm_status   after synchronising: 0, or the code of an expired bounded wait (see below).
 *   rgb200_host_gemm_destroy  synchronises the device and frees everything. */
typedef struct rgb200_host_gemm rgb200_host_gemm;
int rgb200_host_gemm_create(int M, int N, int K, const rgb200_config* cfg, int block_rows, rgb200_host_gemm** handle);
int rgb200_gemm_fp32_host(rgb200_host_gemm* handle, const float* A_host, const float* B_host, float* C_host, void* stream);
int rgb200_host_gemm_info(const rgb200_host_gemm* handle, int* blocks, int* launches, size_t* device_bytes);
int rgb200_host_gemm_status(const rgb200_host_gemm* handle, int* status);
int rgb200_host_gemm_destroy(rgb200_host_gemm* handle);

/* Call after the stream has been synchronised.  *status = 0 if the last run that used this workspace
 * completed, else the code a kernel left when one of its bounded waits expired (it then stopped
 * without hanging; the output is incomplete).  The reference reports kernel failures only through
 * cudaGetLastError (repro_gemm_cuda/repro_gemm.cu:527); this is the same channel for that one case. */
int rgb200_workspace_status(const void* workspace, int* status);

/* Self-test of the kernels' bounded waits (no counterpart in the reference, which has no waits): a probe
 * kernel waits on a barrier that nothing completes, with `limit_clocks` (at most 2e9) as its limit.
 * *status receives the code the waiting role stored when it gave up (2), *waited_clocks how long it
 * waited, *both_left = 1 if a second role waiting with the normal two-second limit also left at once
 * because it saw the first one's abort flag.  The device stays usable; nothing hangs or traps. */
int rgb200_selftest_bounded_wait(long long limit_clocks, int* status, long long* waited_clocks, int* both_left);

/* Allocation-free variant of rgb200_gemm_fp32 (it has no counterpart in the reference, whose
 * convenience call repro_gemm_fp32 allocates and frees its workspace on every call).
 *
 * Who needs it: code that is handed device pointers for A, B and C but has no way to obtain device
 * memory of its own - an operator running under a host framework whose caching allocator owns all
 * device memory (a raw cudaMalloc next to it synchronises the device and takes memory the allocator
 * believes it can still hand out), a step of a latency-critical loop that must not hit the implicit
 * device-wide synchronisation of cudaMalloc / cudaFree, or a plug-in layer that only sees tensors.
 * Such callers cannot use rgb200_gemm_fp32 (it allocates) and have nothing to pass as the workspace of
 * rgb200_gemm_fp32_ws.
 *
 * This call takes the digit planes, exponents and partial sums from a fixed array of
 * RGB200_STATIC_WORKSPACE_BYTES that is part of the library image: every GPU that loads the library
 * holds that much memory until the process exits.  It calls no cudaMalloc, cudaFree or allocating
 * library routine.  Same arithmetic, same bits as the other entry points; asynchronous on `stream`.
 *   - 2 (cudaErrorMemoryAllocation) is returned, and nothing is launched, when the problem needs more
 *     workspace than the fixed array holds (rgb200_layout reports the need; 32 MiB covers for example
 *     2048 x 2048 x 1024 or 1024 x 3072 x 768 at S = 3).  Other errors are those of rgb200_gemm_fp32_ws.
 *   - The first call on each device looks up the array's device address (and, like the first call of
 *     any entry point here, creates the library's per-device helper stream and events and sets kernel
 *     attributes); make that first call outside any stream capture.  Later calls only enqueue work.
 *   - All calls share the one array.  The library re-zeroes the part that must start at zero on every
 *     call, but two calls that overlap on the GPU (different streams, or different threads without
 *     ordering) race on it: issue them on one stream, or order them with events. */
#define RGB200_STATIC_WORKSPACE_BYTES (32u << 20)
int rgb200_gemm_fp32_static(const float* A, const float* B, float* C, int M, int N, int K,
                            const rgb200_config* cfg, void* stream);
/* The counterpart of rgb200_workspace_status for the fixed array (its callers hold no workspace pointer):
 * after synchronising the stream, *status = 0 if the last rgb200_gemm_fp32_static run on the current device
 * completed, else the code of the bounded wait that expired. */
int rgb200_static_status(int* status);

/* ------------------------------------------------------------------------------------------------
 * 2-D convolution and its two gradients in PyTorch layouts (x[N,C,H,W], weight[F,C,KH,KW], output and
 * its gradient [N,F,OH,OW]), with stride and zero padding, no groups or dilation.  They replace
 * repro_conv_cuda/repro_conv.cuh:22-32: conv2d_workspace, conv2d_grad_weight_workspace,
 * conv2d_grad_input_workspace, repro_conv2d_ws, repro_conv2d_grad_weight_ws and
 * repro_conv2d_grad_input_ws.  The shape struct has the field order of the reference's ConvShape
 * (repro_conv_cuda/repro_conv_math.cuh:29-34); stride defaults there are 1, padding 0.
 * Definition (repro_conv_math.cuh:10-17): forward and weight gradient are the GEMM definition applied
 * to the im2col matrix (scales per window and per filter; per filter of dY and per window position);
 * the input gradient uses one scale per image of dY and one for all weights.  No im2col matrix is
 * stored: the pre-pass reads the tensors through an index map and the tensor-core kernel runs on the
 * resulting digit planes.  Asynchronous on `stream`, allocation-free; the workspace size depends only
 * on (shape, slices).  cudaErrorInvalidValue for unsupported shapes (the reference's checks,
 * repro_conv.cu:157-167, except that windows may exceed 1024 values and filters 256) and for a null
 * or short workspace.  Bias is not included (add it with one IEEE addition). */
typedef struct rgb200_conv_shape {
    int N, C, H, W;      /* input  [N, C, H, W] */
    int F, KH, KW;       /* weight [F, C, KH, KW] */
    int SY, SX;          /* stride (>= 1) */
    int PY, PX;          /* zero padding (>= 0) */
} rgb200_conv_shape;

int rgb200_conv2d_workspace(const rgb200_conv_shape* shape, int slices, size_t* bytes);
int rgb200_conv2d_grad_weight_workspace(const rgb200_conv_shape* shape, int slices, size_t* bytes);
int rgb200_conv2d_grad_input_workspace(const rgb200_conv_shape* shape, int slices, size_t* bytes);
int rgb200_conv2d_ws(const float* x, const float* weight, float* out, const rgb200_conv_shape* shape, int slices,
                     void* workspace, size_t workspace_bytes, void* stream);
int rgb200_conv2d_grad_weight_ws(const float* dy, const float* x, float* dw, const rgb200_conv_shape* shape, int slices,
                                 void* workspace, size_t workspace_bytes, void* stream);
int rgb200_conv2d_grad_input_ws(const float* dy, const float* weight, float* dx, const rgb200_conv_shape* shape, int slices,
                                void* workspace, size_t workspace_bytes, void* stream);

/* Host-side helpers matching repro_gemm_cuda/repro_test_util.h:20-24 (FNV-1a-64 over raw bytes) and
 * repro_gemm_cuda/repro_gemm_math.cuh:59,74,96 (the three scalar functions, computed by this
 * library's own host code so callers can cross-check them without a GPU). */
uint64_t rgb200_fnv1a64(const void* data, size_t bytes, uint64_t h);
int rgb200_scale_exponent(float absmax);
int rgb200_fixed_point(float x, int scale_exponent, int slices);
uint32_t rgb200_round_to_float_bits(long long T, int E);
/* floor(n / divisor) for 0 <= n < 2^31 and divisor >= 1 by the multiply-high form the convolution index maps
 * use on the device (same constants, host arithmetic), so the form can be checked without a GPU. */
int rgb200_fast_div(int divisor, int n);

/* Pure host planning (no device query): padded K, number of 128-wide K blocks, the K-range count
 * the INT32 accumulators force, and the workspace size, for tests and capacity planning.
 * Mirrors the arithmetic of make_layout at repro_gemm_cuda/repro_gemm.cu:390-439. */
typedef struct rgb200_layout_info {
    int k_padded, k_blocks, min_split, split_k, tile_n;
    size_t planes_a, planes_b, partial_bytes, workspace_bytes;
} rgb200_layout_info;
int rgb200_layout(int M, int N, int K, int batch, const rgb200_config* cfg, rgb200_layout_info* info);

#ifdef __cplusplus
}
#endif
#endif /* RGB200_H */
