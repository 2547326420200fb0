// Host side of librgb200.so: planning, workspace layout, TMA descriptors, launch sequence and the
// extern "C" entry points declared in include/rgb200.h.
//
// Reference counterparts: make_layout / launch_quantize / launch_all / make_plan /
// repro_gemm_fp32_ws / repro_gemm_fp32 (repro_gemm_cuda/repro_gemm.cu:390-542).
#include <cuda.h>
#include <cuda_runtime.h>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <new>
#include <vector>

#include "../../include/rgb200.h"
#include "rgb200_math.cuh"
#include "rgb200_mma.cuh"
#include "rgb200_smallk.cuh"
#include "rgb200_rowfused.cuh"
#include "rgb200_prepass.cuh"
#include "rgb200_prepass_cluster.cuh"
#include "rgb200_conv.cuh"
#include "rgb200_conv_direct.cuh"

namespace rgb200 {
namespace {

constexpr size_t ALIGN = 256;
constexpr int MAX_DEVICES = 64;
inline size_t align_up(size_t x) { return (x + ALIGN - 1) / ALIGN * ALIGN; }
inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Columns of C per CTA tile (the MMA is S * tile wide).  TMEM holds (2S-1) * tile INT32 columns and the
// epilogue keeps tile/2 exact sums per thread in registers, which bounds the tile at 64 (S=3), 96 (S=2)
// and 256 (S=1); narrow outputs take the 64-wide tile so little of the MMA is spent on padding.
constexpr int TILE_N_BASE = 64;
inline int tile_n_for(int S, int N) {
    if (S == 1 && N >= 512) return 256;
    if (S == 2 && N >= 192) return 96;
    return TILE_N_BASE;
}

// ------------------------------------------------------------------------------------------
// Planning (pure host arithmetic)
// ------------------------------------------------------------------------------------------
struct Layout {
    int S, M, N, K, batch;
    int Kp, k_blocks, min_split, split;
    bool partial_out;          // the caller receives INT64 sums instead of C
    bool use_partial_ws;       // K ranges are reduced through the workspace
    size_t qa, qb, ea, eb, part;            // byte offsets into the workspace
    size_t max_a, max_b, status;            // inside the two zero-initialised blocks
    size_t zero_b_bytes, zero_a_bytes, total;
    int algo;
};

// Largest |X| after the split: 127*128^(S-1) + 64*(128^(S-2) + ... + 1).
double max_fixed_point(int S) {
    double top = 127.0 * std::ldexp(1.0, 7 * (S - 1)), low = 0.0;
    for (int t = 0; t + 1 < S; ++t) low += 64.0 * std::ldexp(1.0, 7 * t);
    return top + low;
}

// K-range count chosen when the caller leaves split_k at 1 and the output has too few tiles to occupy
// the GPU (for example 1024 x 768 x 50257: 96 tiles on 148 SMs, each 393 k blocks long).  Picks the
// count that minimises the number of sequential k blocks per SM; never changes the output bits.
constexpr int PLAN_SM_COUNT = 148;       // B200; the plan must not depend on a device query
int auto_split(int M, int N, int batch, int k_blocks, int tile_n) {
    const long long tiles = (long long)batch * ceil_div(M, BLOCK_M) * ceil_div(N, tile_n);
    if (tiles >= PLAN_SM_COUNT || k_blocks < 16) return 1;
    const double out_bytes = (double)M * N * batch * sizeof(long long);
    if (out_bytes > 32.0 * 1024 * 1024) return 1;   // keep the partial buffers small
    // Cost in units of one k block of MMA work on one SM (about 0.35 us, the time HBM moves 2.3 MB): sequential
    // k blocks per SM, a fixed charge for the extra reduction kernel, and per range a small tail charge plus
    // the write and read of that range's INT64 sums.  A tiny output (the weight gradient of a small
    // convolution: 6 x 25 outputs over 78 400 windows) therefore spreads its K over up to 64 SMs.
    const double per_range = 0.25 + 2.0 * out_bytes / 2.3e6;
    int best = 1;
    double best_cost = (double)ceil_div((int)tiles, PLAN_SM_COUNT) * k_blocks;
    for (int s = 2; s <= 64 && s * 8 <= k_blocks; ++s) {
        double cost = (double)((tiles * s + PLAN_SM_COUNT - 1) / PLAN_SM_COUNT) * ceil_div(k_blocks, s) + 8.0 + s * per_range;
        if (cost < best_cost * 0.9) { best_cost = cost; best = s; }
    }
    return best;
}

// sum_limit bounds total_k * max|X|^2, the largest magnitude an exact sum can reach.
cudaError_t plan_layout(int M, int N, int K, long long total_k, int batch, const rgb200_config& cfg,
                        bool partial_out, Layout& L, double sum_limit = 4611686018427387904.0 /* 2^62 */,
                        bool auto_ranges = true) {
    if (M <= 0 || N <= 0 || K <= 0 || batch <= 0 || cfg.split_k <= 0 || total_k < K) return cudaErrorInvalidValue;
    if (cfg.slices < 1 || cfg.slices > 3) return cudaErrorInvalidValue;
    if (cfg.algo < RGB200_ALGO_AUTO || cfg.algo > RGB200_ALGO_TENSORCORE) return cudaErrorInvalidValue;
    const int S = cfg.slices;
    const double d = max_fixed_point(S);
    if ((double)total_k * d * d > sum_limit) return cudaErrorInvalidValue;   // INT64 must hold any sum
    if ((long long)K + BLOCK_K > 0x7FFFFFFFll) return cudaErrorInvalidValue;
    // launch-geometry limits: the batch index is a grid y/z coordinate, row counts times batch are 32-bit
    if (batch > 65535 || (long long)batch * (M > N ? M : N) > 0x7FFFFFFFll) return cudaErrorInvalidValue;

    L.S = S; L.M = M; L.N = N; L.K = K; L.batch = batch;
    L.Kp = ceil_div(K, BLOCK_K) * BLOCK_K;
    L.k_blocks = L.Kp / BLOCK_K;
    const int blocks_per_pass = max_k_per_pass(S) / BLOCK_K;
    L.min_split = ceil_div(L.k_blocks, blocks_per_pass);
    L.algo = cfg.algo == RGB200_ALGO_AUTO ? RGB200_ALGO_TENSORCORE : cfg.algo;
    if (L.algo == RGB200_ALGO_REFERENCE) {
        L.split = 1;            // the INT64 verification kernel never needs K ranges
    } else {
        int want = cfg.split_k;
        if (want == 1 && !partial_out && auto_ranges) want = auto_split(M, N, batch, L.k_blocks, tile_n_for(S, N));
        L.split = want > L.min_split ? want : L.min_split;
        if (L.split > L.k_blocks) L.split = L.k_blocks;
    }
    L.partial_out = partial_out;
    if (partial_out && L.split != 1) {
        // INT64 output for the caller: K ranges would need a second buffer; one pass covers 105k values of k
        if (L.min_split > 1) return cudaErrorInvalidValue;
        L.split = 1;
    }
    L.use_partial_ws = !partial_out && L.split > 1;

    const size_t qa_bytes = (size_t)batch * S * M * L.Kp, qb_bytes = (size_t)batch * S * N * L.Kp;
    const size_t part_bytes = L.use_partial_ws ? (size_t)L.split * batch * M * N * sizeof(long long) : 0;
    // Everything that belongs to op(B) comes first and its offsets do not depend on M, so consecutive calls on
    // row blocks of one product can share B's digit planes (see RunArgs::reuse_b).  Two zero-initialised
    // blocks: [status word | integer column maxima of B] at the start, the maxima of A in front of A's planes.
    L.status = 0;
    L.max_b = ALIGN;
    L.zero_b_bytes = L.max_b + align_up((size_t)batch * N * sizeof(uint32_t));
    L.qb = L.zero_b_bytes;
    L.eb = L.qb + align_up(qb_bytes);
    L.max_a = L.eb + align_up((size_t)batch * N * sizeof(int));
    L.zero_a_bytes = align_up((size_t)batch * M * sizeof(uint32_t));
    L.qa = L.max_a + L.zero_a_bytes;
    L.ea = L.qa + align_up(qa_bytes);
    L.part = L.ea + align_up((size_t)batch * M * sizeof(int));
    L.total = L.part + align_up(part_bytes);
    return cudaSuccess;
}

// ------------------------------------------------------------------------------------------
// Per-device facts, looked up once (immutable afterwards)
// ------------------------------------------------------------------------------------------
struct DeviceInfo {
    int sm_count = 0; int cc = 0; bool attrs_set = false; cudaError_t err = cudaSuccess;
};
DeviceInfo g_dev[MAX_DEVICES];
std::once_flag g_dev_once[MAX_DEVICES];

template <int S, int NT, bool IMAGE_MAJOR_C = false>
cudaError_t set_kernel_attrs() {
    return cudaFuncSetAttribute(gemm_i8_tcgen05_kernel<S, NT, IMAGE_MAJOR_C>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                GemmTraits<S, NT>::SMEM_BYTES);
}

template <int S>
cudaError_t set_cluster_split_attrs() {
    const int bytes = KSC_MAX_SLAB_BYTES + 128;
    cudaError_t e = cudaFuncSetAttribute(split_kstrided_cluster_kernel<S, 32>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(split_kstrided_cluster_kernel<S, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(split_kstrided_cluster_kernel<S, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    return e;
}

cudaError_t device_info(const DeviceInfo** out) {
    int dev;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= MAX_DEVICES) return cudaErrorInvalidDevice;
    std::call_once(g_dev_once[dev], [dev] {
        DeviceInfo& d = g_dev[dev];
        int major = 0, minor = 0;
        cudaError_t e2;
        if ((e2 = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev)) != cudaSuccess ||
            (e2 = cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev)) != cudaSuccess ||
            (e2 = cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) {
            d.err = e2;
            return;
        }
        d.cc = major * 10 + minor;
        if (d.cc == 100) {   // the only architecture this library carries code for
            if ((e2 = set_kernel_attrs<1, 64>()) != cudaSuccess || (e2 = set_kernel_attrs<2, 64>()) != cudaSuccess ||
                (e2 = set_kernel_attrs<3, 64>()) != cudaSuccess || (e2 = set_kernel_attrs<1, 256>()) != cudaSuccess ||
                (e2 = set_kernel_attrs<2, 96>()) != cudaSuccess || (e2 = set_kernel_attrs<1, 64, true>()) != cudaSuccess ||
                (e2 = set_kernel_attrs<2, 64, true>()) != cudaSuccess || (e2 = set_kernel_attrs<3, 64, true>()) != cudaSuccess) {
                d.err = e2;
                return;
            }
            if ((e2 = cudaFuncSetAttribute(gemm_i8_smallk_kernel<1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SmallKTraits<1>::SMEM_BYTES)) != cudaSuccess ||
                (e2 = cudaFuncSetAttribute(gemm_i8_smallk_kernel<2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SmallKTraits<2>::SMEM_BYTES)) != cudaSuccess ||
                (e2 = cudaFuncSetAttribute(gemm_i8_smallk_kernel<3, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SmallKTraits<3>::SMEM_BYTES)) != cudaSuccess ||
                (e2 = cudaFuncSetAttribute(gemm_i8_smallk_kernel<1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SmallKTraits<1>::SMEM_BYTES)) != cudaSuccess ||
                (e2 = cudaFuncSetAttribute(gemm_i8_smallk_kernel<2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SmallKTraits<2>::SMEM_BYTES)) != cudaSuccess ||
                (e2 = cudaFuncSetAttribute(gemm_i8_smallk_kernel<3, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SmallKTraits<3>::SMEM_BYTES)) != cudaSuccess) {
                d.err = e2;
                return;
            }
            if ((e2 = cudaFuncSetAttribute(gemm_i8_rowfused_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, RowFusedTraits<1>::SMEM_BYTES)) != cudaSuccess ||
                (e2 = cudaFuncSetAttribute(gemm_i8_rowfused_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, RowFusedTraits<2>::SMEM_BYTES)) != cudaSuccess ||
                (e2 = cudaFuncSetAttribute(gemm_i8_rowfused_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, RowFusedTraits<3>::SMEM_BYTES)) != cudaSuccess) {
                d.err = e2;
                return;
            }
            if ((e2 = set_cluster_split_attrs<1>()) != cudaSuccess || (e2 = set_cluster_split_attrs<2>()) != cudaSuccess ||
                (e2 = set_cluster_split_attrs<3>()) != cudaSuccess) {
                d.err = e2;
                return;
            }
            d.attrs_set = true;
        }
    });
    if (g_dev[dev].err != cudaSuccess) return g_dev[dev].err;
    *out = &g_dev[dev];
    return cudaSuccess;
}

// Resolves the algorithm against the current device, as make_layout does in the reference
// (repro_gemm_cuda/repro_gemm.cu:398-409): "not supported" when the device cannot run it.
cudaError_t check_device(int algo, const DeviceInfo** dev) {
    if (algo == RGB200_ALGO_TILED) return cudaErrorNotSupported;   // dp4a fallback is not part of this library
    cudaError_t e = device_info(dev);
    if (e != cudaSuccess) return e;
    if ((*dev)->cc != 100) return cudaErrorNotSupported;
    return cudaSuccess;
}

// ------------------------------------------------------------------------------------------
// TMA descriptors.  The driver entry point is fetched at run time so that the library loads on
// machines without a driver (planning and the host helpers still work there).
// ------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
std::once_flag g_encode_once;

bool ensure_encode() {
    std::call_once(g_encode_once, [] {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qr) == cudaSuccess &&
            qr == cudaDriverEntryPointSuccess)
            g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    });
    return g_encode != nullptr;
}

cudaError_t encode_planes_map(CUtensorMap* map, const void* planes, int rows, int Kp, int S, int batch, int box_rows) {
    if (!ensure_encode()) return cudaErrorNotSupported;
    // dims (fastest first): k, row, digit plane, batch.  Rows beyond `rows` read as zero.
    cuuint64_t dims[4] = {(cuuint64_t)Kp, (cuuint64_t)rows, (cuuint64_t)S, (cuuint64_t)batch};
    cuuint64_t strides[3] = {(cuuint64_t)Kp, (cuuint64_t)rows * Kp, (cuuint64_t)rows * Kp * S};
    cuuint32_t box[4] = {(cuuint32_t)BLOCK_K, (cuuint32_t)box_rows, (cuuint32_t)S, 1u};
    cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(planes), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

// FP32 operand stored [batch][K][R] (r contiguous), as the cluster split reads it: dims (r, k, batch), box (W, 64, 1).
cudaError_t encode_kstrided_map(CUtensorMap* map, const float* src, int R, int K, int batch, long long batch_stride, int W) {
    if (!ensure_encode()) return cudaErrorNotSupported;
    cuuint64_t dims[3] = {(cuuint64_t)R, (cuuint64_t)K, (cuuint64_t)batch};
    cuuint64_t strides[2] = {(cuuint64_t)R * 4, (cuuint64_t)(batch > 1 ? batch_stride : (long long)R * K) * 4};
    cuuint32_t box[3] = {(cuuint32_t)W, (cuuint32_t)KSC_BOX_K, 1u};
    cuuint32_t estr[3] = {1u, 1u, 1u};
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(src), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

// FP32 operand stored [batch][M][K] (k contiguous), as the fused-split kernel streams it: dims (k, row, batch),
// box (64 k, 128 rows, 1), zero fill beyond K and M.
cudaError_t encode_kmajor_f32_map(CUtensorMap* map, const float* src, int M, int K, int batch, long long batch_stride) {
    if (!ensure_encode()) return cudaErrorNotSupported;
    cuuint64_t dims[3] = {(cuuint64_t)K, (cuuint64_t)M, (cuuint64_t)batch};
    cuuint64_t strides[2] = {(cuuint64_t)K * 4, (cuuint64_t)(batch > 1 ? batch_stride : (long long)M * K) * 4};
    cuuint32_t box[3] = {(cuuint32_t)RF_CHUNK_K, (cuuint32_t)BLOCK_M, 1u};
    cuuint32_t estr[3] = {1u, 1u, 1u};
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(src), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

// FP32 view of C as [batch][M][N] for the tensor stores of the short-K kernel: boxes of `cols` columns x 128 rows,
// written from a shared-memory image with the swizzle that matches the box's row length (128 or 64 bytes).
cudaError_t encode_c_store_map(CUtensorMap* map, float* C, int M, int N, int batch, long long batch_stride, int cols) {
    if (!ensure_encode()) return cudaErrorNotSupported;
    cuuint64_t dims[3] = {(cuuint64_t)N, (cuuint64_t)M, (cuuint64_t)batch};
    cuuint64_t strides[2] = {(cuuint64_t)N * 4, (cuuint64_t)(batch > 1 ? batch_stride : (long long)M * N) * 4};
    cuuint32_t box[3] = {(cuuint32_t)cols, (cuuint32_t)BLOCK_M, 1u};
    cuuint32_t estr[3] = {1u, 1u, 1u};
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, C, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          cols * 4 == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                          CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

// The cluster form of the k-strided split (one read of the operand, rgb200_prepass_cluster.cuh).  Returns false when
// the operand cannot take it (rows not a multiple of four floats, unaligned base or batch stride, K too long for a
// slab), and the caller then runs the two-kernel form.  `overlap`: launch with programmatic stream serialization,
// so that the kernel may start while the previous kernel of the stream - the other operand's split, which it does
// not depend on - is still draining; the next ordinary launch of the stream waits for both, as stream order demands.
template <int S, int W>
cudaError_t launch_cluster_split(const CUtensorMap& map, const float* given_max, int8_t* planes, int* expo, int R, int K, int Kp,
                                 int KC, int batch, int* status, bool overlap, cudaStream_t st) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(KSC_CLUSTER * ceil_div(R, W), batch);
    cfg.blockDim = dim3(PREPASS_THREADS);
    cfg.dynamicSmemBytes = (size_t)KC * W * 4 + 128;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, split_kstrided_cluster_kernel<S, W>, map, given_max, planes, expo, R, K, Kp, KC, status);
}

// Whether a k-strided operand of R rows (16-byte aligned base and batch stride taken for granted) takes the cluster form.
bool cluster_split_fits(int R, int Kp) {
    const int KC = ceil_div(ceil_div(Kp, KSC_CLUSTER), KSC_BOX_K) * KSC_BOX_K;
    return R % 4 == 0 && (size_t)KC * 8 * 4 <= (size_t)KSC_MAX_SLAB_BYTES;
}

template <int S>
bool try_cluster_split(const float* src, const float* given_max, int8_t* planes, int* expo, int R, int K, int Kp, int batch,
                       long long batch_stride, int* status, bool overlap, cudaStream_t st) {
    if (R % 4 != 0 || (reinterpret_cast<uintptr_t>(src) & 15) != 0 || (batch > 1 && batch_stride % 4 != 0)) return false;
    if (!ensure_encode()) return false;
    const int KC = ceil_div(ceil_div(Kp, KSC_CLUSTER), KSC_BOX_K) * KSC_BOX_K;
    int W = 32;
    while (W > 8 && (size_t)KC * W * 4 > (size_t)KSC_MAX_SLAB_BYTES) W >>= 1;
    if ((size_t)KC * W * 4 > (size_t)KSC_MAX_SLAB_BYTES) return false;
    while (W > 8 && (long long)ceil_div(R, W) * KSC_CLUSTER * batch < PLAN_SM_COUNT) W >>= 1;   // few columns: narrower panels, more CTAs
    CUtensorMap map;
    if (encode_kstrided_map(&map, src, R, K, batch, batch_stride, W) != cudaSuccess) return false;
    cudaError_t e;
    if (W == 32) e = launch_cluster_split<S, 32>(map, given_max, planes, expo, R, K, Kp, KC, batch, status, overlap, st);
    else if (W == 16) e = launch_cluster_split<S, 16>(map, given_max, planes, expo, R, K, Kp, KC, batch, status, overlap, st);
    else e = launch_cluster_split<S, 8>(map, given_max, planes, expo, R, K, Kp, KC, batch, status, overlap, st);
    if (e != cudaSuccess) (void)cudaGetLastError();      // not launched: the caller falls back to the two-kernel form
    return e == cudaSuccess;
}

// ------------------------------------------------------------------------------------------
// Launch sequence
// ------------------------------------------------------------------------------------------
// Launches the k-contiguous split for one operand (second.src == nullptr) or for two operands of the same
// row length in one grid.
template <int S>
void launch_kmajor(const KmajorOperand& first, const KmajorOperand& second, int K, int Kp, int batch, int* zero_word,
                   cudaStream_t st) {
    const bool two = second.src != nullptr;
    auto aligned_op = [&](const KmajorOperand& o) {
        return (K % 4 == 0) && ((reinterpret_cast<uintptr_t>(o.src) & 15) == 0) && (o.batch_stride % 4 == 0);
    };
    const bool aligned = aligned_op(first) && (!two || aligned_op(second));
    const int nq = Kp / 4;     // float4 chunks per padded row
#define RGB_KMAJOR(TPR, CH, VEC)                                                                              \
    do {                                                                                                      \
        const int rpc = PREPASS_THREADS / TPR;                                                                \
        const int b1 = ceil_div(first.R, rpc), b2 = two ? ceil_div(second.R, rpc) : 0;                        \
        split_kmajor_kernel<S, TPR, CH, VEC><<<dim3(b1 + b2, batch), PREPASS_THREADS, 0, st>>>(               \
            first, second, b1, K, Kp, zero_word);                                                             \
    } while (0)
    if (aligned && Kp == 128) {                          // short rows: a small grid of warps, each walking over many rows
        const long long rows = (long long)first.R + (two ? second.R : 0);
        const long long want = (rows + 63) / 64;         // eight rows per warp at least
        const int ctas = (int)(want < 1 ? 1 : (want > PLAN_SM_COUNT * 8 ? PLAN_SM_COUNT * 8 : want));
        if (K <= 64) split_kmajor_short_kernel<S, true><<<dim3(ctas, batch), PREPASS_THREADS, 0, st>>>(first, second, K, zero_word);
        else split_kmajor_short_kernel<S, false><<<dim3(ctas, batch), PREPASS_THREADS, 0, st>>>(first, second, K, zero_word);
        return;
    }
    if (!aligned || nq > 256 * KMAJOR_MAX_CHUNKS) {      // general path: any K, any alignment; row group sized to the row
        if (nq <= 64) RGB_KMAJOR(32, 1, false);
        else if (nq <= 256) RGB_KMAJOR(64, 1, false);
        else if (nq <= 1024) RGB_KMAJOR(128, 1, false);
        else RGB_KMAJOR(256, 1, false);
    }
    else if (nq <= 32 * 2) RGB_KMAJOR(32, 2, true);
    else if (nq <= 32 * 4) RGB_KMAJOR(32, 4, true);
    else if (nq <= 64 * 4) RGB_KMAJOR(64, 4, true);
    else if (nq <= 128 * 4) RGB_KMAJOR(128, 4, true);
    else if (nq <= 256 * 4) RGB_KMAJOR(256, 4, true);
    else if (nq <= 256 * 8) RGB_KMAJOR(256, 8, true);
    else RGB_KMAJOR(256, 16, true);
#undef RGB_KMAJOR
}

// One operand through the pre-pass.  k_major: element (r, k) at src[r*K + k].
template <int S>
void launch_split(const float* src, bool k_major, const float* given_max, uint32_t* maxbits, int8_t* planes, int* expo,
                  int R, int K, int Kp, int batch, long long batch_stride, int* status, cudaStream_t st, bool overlap = false) {
    if (k_major) {
        const KmajorOperand op{src, given_max, planes, expo, R, batch_stride};
        const KmajorOperand none{nullptr, nullptr, nullptr, nullptr, 0, 0};
        launch_kmajor<S>(op, none, K, Kp, batch, nullptr, st);
    } else if (try_cluster_split<S>(src, given_max, planes, expo, R, K, Kp, batch, batch_stride, status, overlap, st)) {
        // one read of the operand; the zeroed maxima words stay unused
    } else {
        if (given_max)
            maxima_to_bits_kernel<<<ceil_div(batch * R, 256), 256, 0, st>>>(given_max, maxbits, batch * R);
        else
            colmax_kstrided_kernel<<<dim3(ceil_div(R, 128), (ceil_div(K, COLMAX_K_PER_CTA) < COLMAX_MAX_GRID_Y ? ceil_div(K, COLMAX_K_PER_CTA) : COLMAX_MAX_GRID_Y), batch), PREPASS_THREADS, 0, st>>>(
                src, maxbits, R, K, batch_stride);
        // about eight CTAs per SM in total; each walks over the k tiles of its 32 rows
        const int r_blocks = ceil_div(R, 32), k_tiles = Kp / BLOCK_K;
        int walkers = ceil_div(PLAN_SM_COUNT * 8, r_blocks * batch);
        walkers = walkers < 1 ? 1 : (walkers > k_tiles ? k_tiles : walkers);
        split_kstrided_kernel<S><<<dim3(r_blocks, walkers, batch), PREPASS_THREADS, 0, st>>>(
            src, maxbits, planes, expo, R, K, Kp, batch_stride);
    }
}

// Picks the four-wide form of the rounding kernel when rows, strides and base addresses allow it.
void launch_round(const long long* partial, int parts, size_t part_stride, const int* ea, const int* eb,
                  const float* max_a, const float* max_b, float* C, int M, int N, int batch, long long stride_c, int e0,
                  int sm_count, cudaStream_t st) {
    const size_t total = (size_t)batch * M * N;
    const bool vec = N % 4 == 0 && part_stride % 4 == 0 && stride_c % 4 == 0 &&
                     (reinterpret_cast<uintptr_t>(partial) & 31) == 0 && (reinterpret_cast<uintptr_t>(C) & 15) == 0;
    const size_t items = vec ? total / 4 : total;
    const size_t want = (items + 255) / 256, cap = (size_t)sm_count * 32;
    const int blocks = (int)(want < cap ? want : cap);
    if (vec) round_partial_kernel<true><<<blocks, 256, 0, st>>>(partial, parts, part_stride, ea, eb, max_a, max_b, C, M, N, batch, stride_c, e0);
    else round_partial_kernel<false><<<blocks, 256, 0, st>>>(partial, parts, part_stride, ea, eb, max_a, max_b, C, M, N, batch, stride_c, e0);
}

// A pre-pass supplied by the caller of run(): fills both operands' digit planes and exponents
// (the convolutions read their operands through index maps instead of stored matrices).
// max_a / max_b are zeroed scratch words, batch * M and batch * N of them.
struct PrepassHook {
    cudaError_t (*launch)(const void* ctx, const Layout& L, uint32_t* max_a, uint32_t* max_b, int8_t* qa, int8_t* qb,
                          int* ea, int* eb, cudaStream_t st);
    const void* ctx;
};

struct RunArgs {
    const float *A, *B;
    float* C;
    long long* T_out;                 // INT64 output for the caller (partial mode), else null
    const float *max_a, *max_b;       // externally reduced maxima (partial mode), else null
    long long stride_a, stride_b, stride_c;
    bool trans_a, trans_b;
    char* ws;
    cudaStream_t st;
    const cudaEvent_t* ev;
    long long* const* scatter = nullptr;   // per-owner destination buffers of the INT64 sums (K-sharded), or null
    int scatter_world = 0, scatter_rank = 0;
    const PrepassHook* hook = nullptr;
    int c_image_rows = 0;                  // > 0: image-major C (see GemmParams::c_image_rows); needs split == 1
    // B's digit planes and exponents already sit in the workspace from the previous call on it with the same
    // N, K, S and transposition (row blocks of one product): skip B's pre-pass.
    bool reuse_b = false;
};

template <int S>
cudaError_t run(const Layout& L, const RunArgs& a, const DeviceInfo& dev) {
    auto record = [&](int i) { if (a.ev) cudaEventRecord(a.ev[i], a.st); };
    int8_t* qa = reinterpret_cast<int8_t*>(a.ws + L.qa);
    int8_t* qb = reinterpret_cast<int8_t*>(a.ws + L.qb);
    int* ea = reinterpret_cast<int*>(a.ws + L.ea);
    int* eb = reinterpret_cast<int*>(a.ws + L.eb);
    uint32_t* max_a = reinterpret_cast<uint32_t*>(a.ws + L.max_a);
    uint32_t* max_b = reinterpret_cast<uint32_t*>(a.ws + L.max_b);
    int* status = reinterpret_cast<int*>(a.ws + L.status);
    long long* part = L.use_partial_ws ? reinterpret_cast<long long*>(a.ws + L.part) : a.T_out;
    const int e0 = -14 * (S - 1);

    cudaError_t e = cudaSuccess;
    // Skinny output (N <= 64) with a k-contiguous A: A's split is fused into the MMA kernel's producer and its
    // digit planes never reach HBM (rgb200_rowfused.cuh); only B goes through the pre-pass.
    const bool fused_a = !a.hook && !a.trans_a && !a.max_a && !part && !a.scatter && !a.c_image_rows &&
                         L.algo == RGB200_ALGO_TENSORCORE && L.N <= RF_NT && L.split == 1 && L.k_blocks > 1 &&
                         L.K % 4 == 0 && (reinterpret_cast<uintptr_t>(a.A) & 15) == 0 && (L.batch == 1 || a.stride_a % 4 == 0);
    // Both operands k-contiguous (the forward product of a linear layer, C = A B^T): one launch splits both
    // and clears the status word; no column maxima are needed, hence no memset either.
    const bool both_kmajor = !a.trans_a && a.trans_b;
    if (fused_a) {
        if (!a.reuse_b) {
            if ((e = cudaMemsetAsync(a.ws, 0, L.zero_b_bytes, a.st)) != cudaSuccess) return e;   // status word + column maxima of B
            record(0);
            launch_split<S>(a.B, a.trans_b, a.max_b, max_b, qb, eb, L.N, L.K, L.Kp, L.batch, a.stride_b, status, a.st);
        } else {
            record(0);
        }
        record(1);
        CUtensorMap map_a, map_b;
        if ((e = encode_kmajor_f32_map(&map_a, a.A, L.M, L.K, L.batch, a.stride_a)) != cudaSuccess) return e;
        if ((e = encode_planes_map(&map_b, qb, L.N, L.Kp, S, L.batch, RF_NT)) != cudaSuccess) return e;
        RowFusedParams Q;
        Q.expo_b = eb; Q.C = a.C; Q.status = status;
        Q.M = L.M; Q.N = L.N; Q.K = L.K; Q.batch = L.batch; Q.stride_c = a.stride_c;
        Q.m_tiles = ceil_div(L.M, BLOCK_M); Q.k_blocks = L.k_blocks; Q.e0 = e0;
        const long long rf_tiles = (long long)L.batch * Q.m_tiles;
        const int rf_grid = (int)(rf_tiles < dev.sm_count ? rf_tiles : dev.sm_count);
        gemm_i8_rowfused_kernel<S><<<rf_grid, RF_THREADS, RowFusedTraits<S>::SMEM_BYTES, a.st>>>(map_a, map_b, Q);
        record(2);
        record(3);
        return cudaGetLastError();
    }
    if (a.hook) {
        if ((e = cudaMemsetAsync(a.ws, 0, L.zero_b_bytes, a.st)) != cudaSuccess) return e;
        if ((e = cudaMemsetAsync(a.ws + L.max_a, 0, L.zero_a_bytes, a.st)) != cudaSuccess) return e;
        record(0);
        if ((e = a.hook->launch(a.hook->ctx, L, max_a, max_b, qa, qb, ea, eb, a.st)) != cudaSuccess) return e;
        record(1);
    } else if (a.reuse_b) {
        // B's planes and exponents are those of the previous call on this workspace (same N, K, S): only A is split
        if (a.trans_a && (e = cudaMemsetAsync(a.ws + L.max_a, 0, L.zero_a_bytes, a.st)) != cudaSuccess) return e;
        record(0);
        launch_split<S>(a.A, !a.trans_a, a.max_a, max_a, qa, ea, L.M, L.K, L.Kp, L.batch, a.stride_a, status, a.st);
        record(1);
    } else if (both_kmajor) {
        record(0);
        const KmajorOperand opa{a.A, a.max_a, qa, ea, L.M, a.stride_a};
        const KmajorOperand opb{a.B, a.max_b, qb, eb, L.N, a.stride_b};
        launch_kmajor<S>(opa, opb, L.K, L.Kp, L.batch, status, a.st);
        record(1);
    } else {
        if ((e = cudaMemsetAsync(a.ws, 0, L.zero_b_bytes, a.st)) != cudaSuccess) return e;   // status word + column maxima of B
        if (a.trans_a && (e = cudaMemsetAsync(a.ws + L.max_a, 0, L.zero_a_bytes, a.st)) != cudaSuccess) return e;
        record(0);
        // both splits on the caller's stream, one after the other: each saturates the memory system by itself, and
        // the library keeps no stream or event of its own
        launch_split<S>(a.A, !a.trans_a, a.max_a, max_a, qa, ea, L.M, L.K, L.Kp, L.batch, a.stride_a, status, a.st);
        launch_split<S>(a.B, a.trans_b, a.max_b, max_b, qb, eb, L.N, L.K, L.Kp, L.batch, a.stride_b, status, a.st, true);
        record(1);
    }

    if (L.algo == RGB200_ALGO_REFERENCE) {
        gemm_int64_check_kernel<S><<<dim3(ceil_div(L.N, 16), ceil_div(L.M, 16), L.batch), dim3(16, 16), 0, a.st>>>(
            qa, qb, ea, eb, a.C, L.M, L.N, L.Kp, a.stride_c, e0);
        record(2);
        record(3);
        return cudaGetLastError();
    }

    if (a.c_image_rows && (L.split != 1 || L.batch != 1 || part)) return cudaErrorInvalidValue;
    CUtensorMap map_a, map_b;
    if (L.k_blocks == 1 && !part && !a.c_image_rows && !a.scatter) {
        // the whole K fits one k block (attention scores and the like): the epilogue-centred kernel
        if ((e = encode_planes_map(&map_a, qa, L.M, L.Kp, S, L.batch, BLOCK_M)) != cudaSuccess) return e;
        if ((e = encode_planes_map(&map_b, qb, L.N, L.Kp, S, L.batch, SK_NT)) != cudaSuccess) return e;
        SmallKParams Q;
        Q.expo_a = ea; Q.expo_b = eb; Q.C = a.C; Q.status = status;
        Q.M = L.M; Q.N = L.N; Q.batch = L.batch; Q.stride_c = a.stride_c;
        Q.m_tiles = ceil_div(L.M, BLOCK_M); Q.n_tiles = ceil_div(L.N, SK_NT);
        Q.k_steps = ceil_div(L.K, UMMA_K);
        Q.e0 = e0;
        // full-line output through shared memory and TMA stores where C's layout allows a tensor map
        CUtensorMap map_cx = map_a, map_cy = map_a;
        bool staged = (reinterpret_cast<uintptr_t>(a.C) & 15) == 0 && L.N % 4 == 0 && (L.batch == 1 || a.stride_c % 4 == 0) &&
                   getenv("RGB200_SMALLK_DIRECT_STORES") == nullptr;
        if (staged &&
            (encode_c_store_map(&map_cx, a.C, L.M, L.N, L.batch, a.stride_c, SK_STAGE_X_COLS) != cudaSuccess ||
             encode_c_store_map(&map_cy, a.C, L.M, L.N, L.batch, a.stride_c, SK_NT - SK_STAGE_X_COLS) != cudaSuccess)) {
            staged = false;                     // a layout the encoder refuses: the threads store their rows themselves
            map_cx = map_cy = map_a;
        }
        const long long sk_tiles = (long long)L.batch * Q.m_tiles * Q.n_tiles;
        const int sk_grid = (int)(sk_tiles < dev.sm_count ? sk_tiles : dev.sm_count);
        if (staged) gemm_i8_smallk_kernel<S, true><<<sk_grid, SK_THREADS, SmallKTraits<S>::SMEM_BYTES, a.st>>>(map_a, map_b, map_cx, map_cy, Q);
        else gemm_i8_smallk_kernel<S, false><<<sk_grid, SK_THREADS, SmallKTraits<S>::SMEM_BYTES, a.st>>>(map_a, map_b, map_cx, map_cy, Q);
        record(2);
        record(3);
        return cudaGetLastError();
    }
    const int tile_n = a.c_image_rows ? TILE_N_BASE : tile_n_for(S, L.N);
    if ((e = encode_planes_map(&map_a, qa, L.M, L.Kp, S, L.batch, BLOCK_M)) != cudaSuccess) return e;
    if ((e = encode_planes_map(&map_b, qb, L.N, L.Kp, S, L.batch, tile_n)) != cudaSuccess) return e;
    GemmParams P;
    P.expo_a = ea; P.expo_b = eb;
    P.C = part ? nullptr : a.C;
    P.partial = part;
    P.status = status;
    P.M = L.M; P.N = L.N; P.batch = L.batch;
    P.stride_c = a.stride_c;
    P.k_blocks = L.k_blocks;
    P.split = L.split;
    P.m_tiles = ceil_div(L.M, BLOCK_M);
    P.n_tiles = ceil_div(L.N, tile_n);
    P.e0 = e0;
    P.scatter_rows = 0; P.scatter_slot = 0; P.scatter_rot = 0;
    P.c_image_rows = a.c_image_rows;
    for (int i = 0; i < 8; ++i) P.scatter[i] = nullptr;
    if (a.scatter) {
        P.scatter_rows = L.M / a.scatter_world;
        P.scatter_slot = a.scatter_rank;
        // start with the rows of the next rank, end with this rank's own (see GemmParams::scatter_rot)
        P.scatter_rot = ((a.scatter_rank + 1) % a.scatter_world) * (P.scatter_rows / BLOCK_M);
        for (int i = 0; i < a.scatter_world; ++i) P.scatter[i] = a.scatter[i];
        P.partial = a.scatter[a.scatter_rank];      // non-null marks the INT64 path; every row is redirected
        P.C = nullptr;
    }
    const long long tiles = (long long)L.batch * L.split * P.m_tiles * P.n_tiles;
    const int grid = (int)(tiles < dev.sm_count ? tiles : dev.sm_count);
    if (a.c_image_rows)
        gemm_i8_tcgen05_kernel<S, TILE_N_BASE, true><<<grid, GEMM_THREADS, GemmTraits<S, TILE_N_BASE>::SMEM_BYTES, a.st>>>(map_a, map_b, P);
    else if (S == 1 && tile_n == 256)
        gemm_i8_tcgen05_kernel<1, 256><<<grid, GEMM_THREADS, GemmTraits<1, 256>::SMEM_BYTES, a.st>>>(map_a, map_b, P);
    else if (S == 2 && tile_n == 96)
        gemm_i8_tcgen05_kernel<2, 96><<<grid, GEMM_THREADS, GemmTraits<2, 96>::SMEM_BYTES, a.st>>>(map_a, map_b, P);
    else
        gemm_i8_tcgen05_kernel<S, TILE_N_BASE><<<grid, GEMM_THREADS, GemmTraits<S, TILE_N_BASE>::SMEM_BYTES, a.st>>>(map_a, map_b, P);
    record(2);
    if (L.use_partial_ws) {
        const size_t total = (size_t)L.batch * L.M * L.N;
        launch_round(part, L.split, total, ea, eb, nullptr, nullptr, a.C, L.M, L.N, L.batch, a.stride_c, e0, dev.sm_count, a.st);
    }
    record(3);
    return cudaGetLastError();
}

cudaError_t dispatch(const Layout& L, const RunArgs& a, const DeviceInfo& dev) {
    switch (L.S) {
        case 1: return run<1>(L, a, dev);
        case 2: return run<2>(L, a, dev);
        case 3: return run<3>(L, a, dev);
    }
    return cudaErrorInvalidValue;
}

cudaError_t gemm_ws(const float* A, const float* B, float* C, int M, int N, int K, int batch, long long sa, long long sb,
                    long long sc, const rgb200_config* cfg, void* ws, size_t ws_bytes, void* stream, void* const* events4) {
    if (!A || !B || !C || !cfg) return cudaErrorInvalidValue;
    Layout L;
    cudaError_t e = plan_layout(M, N, K, K, batch, *cfg, false, L);
    if (e != cudaSuccess) return e;
    const DeviceInfo* dev = nullptr;
    if ((e = check_device(L.algo, &dev)) != cudaSuccess) return e;
    if (!ws || ws_bytes < L.total) return cudaErrorInvalidValue;
    if (batch > 1 && (sa < (long long)M * K || sb < (long long)K * N || sc < (long long)M * N)) return cudaErrorInvalidValue;
    RunArgs a{A, B, C, nullptr, nullptr, nullptr, sa, sb, sc, cfg->trans_a != 0, cfg->trans_b != 0,
              static_cast<char*>(ws), static_cast<cudaStream_t>(stream), reinterpret_cast<const cudaEvent_t*>(events4)};
    return dispatch(L, a, *dev);
}


// ------------------------------------------------------------------------------------------
// Host-buffer pipeline.  The reference's tools surround every product with whole-matrix copies
// (repro_gemm_cuda/hash_repro_gemm.cu:117-118,139); here B travels first, A follows in row blocks, and
// for each block the split, the MMA kernel and the copy of the finished rows of C back to the host run
// while the next block of A is still on the link (three streams: copy-in, compute, copy-out).  Row
// blocks are independent products (scales and sums never cross rows), so the bits equal one call's.
// B is split once, by the first block's call; later blocks reuse its planes (RunArgs::reuse_b).
// ------------------------------------------------------------------------------------------
struct HostBlock { int lo, rows; };
}  // namespace
}  // namespace rgb200

struct rgb200_host_gemm {
    int M, N, K, device;
    rgb200_config cfg;
    std::vector<rgb200::HostBlock> blocks;
    std::vector<rgb200::Layout> layouts;      // one per block
    float *dA = nullptr, *dB = nullptr, *dC = nullptr;
    char* ws = nullptr;
    size_t ws_bytes = 0;
    cudaStream_t s_in = nullptr, s_run = nullptr, s_out = nullptr;
    cudaEvent_t ev_fork = nullptr, ev_b = nullptr, ev_in_done = nullptr, ev_run_done = nullptr, ev_out_done = nullptr;
    std::vector<cudaEvent_t> ev_a, ev_c;
    int launches = 0;
};

namespace rgb200 {
namespace {

void host_gemm_free(rgb200_host_gemm* h) {
    if (!h) return;
    cudaFree(h->dA); cudaFree(h->dB); cudaFree(h->dC); cudaFree(h->ws);
    for (cudaStream_t st : {h->s_in, h->s_run, h->s_out}) if (st) cudaStreamDestroy(st);
    for (cudaEvent_t ev : {h->ev_fork, h->ev_b, h->ev_in_done, h->ev_run_done, h->ev_out_done}) if (ev) cudaEventDestroy(ev);
    for (cudaEvent_t ev : h->ev_a) if (ev) cudaEventDestroy(ev);
    for (cudaEvent_t ev : h->ev_c) if (ev) cudaEventDestroy(ev);
    (void)cudaGetLastError();
    delete h;
}

// ------------------------------------------------------------------------------------------
// Convolutions (reference: repro_conv_cuda/repro_conv.cu:157-238).  Each call is one (batched)
// product on digit planes that a gather pre-pass writes; see rgb200_conv.cuh for the mapping.
// ------------------------------------------------------------------------------------------
enum ConvKind { CONV_FORWARD, CONV_GRAD_WEIGHT, CONV_GRAD_INPUT };

// The reference's shape check (repro_conv.cu:157-167) without its kernel-specific limits on the
// window size (1024) and the filter count (256), which this implementation does not have.
bool conv_geometry(const rgb200_conv_shape* s, int S, ConvGeom& g) {
    if (!s || S < 1 || S > 3) return false;
    if (s->N <= 0 || s->C <= 0 || s->H <= 0 || s->W <= 0 || s->F <= 0 || s->KH <= 0 || s->KW <= 0) return false;
    if (s->SY <= 0 || s->SX <= 0 || s->PY < 0 || s->PX < 0) return false;
    if ((long long)s->H + 2ll * s->PY < s->KH || (long long)s->W + 2ll * s->PX < s->KW) return false;
    if (s->N > 65535) return false;
    const long long OH = ((long long)s->H + 2ll * s->PY - s->KH) / s->SY + 1, OW = ((long long)s->W + 2ll * s->PX - s->KW) / s->SX + 1;
    const double K = (double)s->C * s->KH * s->KW, windows = (double)s->N * OH * OW;
    const double out_size = windows * s->F, in_size = (double)s->N * s->C * s->H * s->W;
    if (out_size >= 2147483648.0 || in_size >= 2147483648.0 || K * s->F >= 2147483648.0) return false;
    const double lim = 127.0 * (double)(1 << (7 * (S - 1))), max_terms = 9.0e18 / (lim * lim);   // keeps |sum| < 2^63
    if (windows > max_terms || (double)s->KH * s->KW * s->F > max_terms || K > max_terms) return false;
    g.N = s->N; g.C = s->C; g.H = s->H; g.W = s->W; g.F = s->F; g.KH = s->KH; g.KW = s->KW;
    g.SY = s->SY; g.SX = s->SX; g.PY = s->PY; g.PX = s->PX;
    g.OH = (int)OH; g.OW = (int)OW; g.K = s->C * s->KH * s->KW;
    g.prepare();
    return true;
}

// Orientation of forward and input gradient: the many-row operand (windows, pixels) on the row side with
// the image-major store, unless K needs several INT32 accumulation passes (then one product per image).
bool conv_rows_are_places(ConvKind kind, const ConvGeom& g, int S) {
    if (kind == CONV_GRAD_WEIGHT) return false;
    const long long k = kind == CONV_FORWARD ? (long long)g.K : (long long)g.F * g.KH * g.KW;
    const long long rows = kind == CONV_FORWARD ? (long long)g.N * g.OH * g.OW : (long long)g.N * g.H * g.W;
    return k <= max_k_per_pass(S) / BLOCK_K * BLOCK_K && rows <= 0x7FFFFFFFll;
}

cudaError_t conv_layout(ConvKind kind, const ConvGeom& g, int S, Layout& L) {
    rgb200_config cfg;
    rgb200_default_config(&cfg);
    cfg.slices = S;
    cfg.algo = RGB200_ALGO_TENSORCORE;
    const double no_limit = 1.0e300;             // conv_geometry has bounded the sums already
    const bool places = conv_rows_are_places(kind, g, S);
    switch (kind) {
        case CONV_FORWARD:
            if (places) return plan_layout(g.N * g.OH * g.OW, g.F, g.K, g.K, 1, cfg, false, L, no_limit, false);
            return plan_layout(g.F, g.OH * g.OW, g.K, g.K, g.N, cfg, false, L, no_limit);
        case CONV_GRAD_WEIGHT: { const int w = g.N * g.OH * g.OW; return plan_layout(g.F, g.K, w, w, 1, cfg, false, L, no_limit); }
        case CONV_GRAD_INPUT: {
            const int t = g.F * g.KH * g.KW;
            if (places) return plan_layout(g.N * g.H * g.W, g.C, t, t, 1, cfg, false, L, no_limit, false);
            return plan_layout(g.C, g.H * g.W, t, t, g.N, cfg, false, L, no_limit);
        }
    }
    return cudaErrorInvalidValue;
}

// (p, q) = (x, weight), (dy, x) or (dy, weight); pixmax: C*H*W words behind the product's workspace (weight gradient)
struct ConvCall { ConvKind kind; ConvGeom g; const float* p; const float* q; bool places; uint32_t* pixmax; };

size_t conv_extra_bytes(ConvKind kind, const ConvGeom& g) {
    return kind == CONV_GRAD_WEIGHT ? align_up((size_t)g.C * g.H * g.W * sizeof(uint32_t)) : 0;
}

cudaError_t conv_prepass(const void* ctx, const Layout& L, uint32_t* max_a, uint32_t* max_b, int8_t* qa, int8_t* qb,
                         int* ea, int* eb, cudaStream_t st) {
    const ConvCall& c = *static_cast<const ConvCall*>(ctx);
    const ConvGeom& g = c.g;
    const int S = L.S;
    const FastDiv one;
    switch (c.kind) {
        case CONV_FORWARD: {
            // k runs (tap, channel) when there are at least four channels, else (c, ky, kx) as the weights are stored
            const bool tap_major = g.C >= 4;
            const size_t khw = (size_t)g.KH * g.KW;
            const TapMajorWeights wt{c.q, g, g.C, g.by_c, (size_t)g.C * khw, khw};
            const StoredRows ws{c.q, g.K};
            if (c.places) {           // A: every window of every image; B: the weights
                if (tap_major) {
                    launch_gather_operand<true>(S, AllWindowTaps{c.p, g}, max_a, qa, ea, L.M, L.K, L.Kp, 1, 0, 0, one, st);
                    launch_gather_operand<true>(S, wt, max_b, qb, eb, L.N, L.K, L.Kp, 1, 0, 0, one, st);
                } else {
                    launch_gather_operand<true>(S, AllWindows{c.p, g}, max_a, qa, ea, L.M, L.K, L.Kp, 1, 0, 0, one, st);
                    launch_gather_operand<true>(S, ws, max_b, qb, eb, L.N, L.K, L.Kp, 1, 0, 0, one, st);
                }
            } else {                  // per image: A the weights (one copy of the planes per image), B the windows of image b
                if (tap_major) {
                    launch_gather_operand<true>(S, wt, max_a, qa, ea, L.M, L.K, L.Kp, L.batch, 0, 0, one, st);
                    launch_gather_operand<true>(S, WindowTapsOfImage{c.p, g}, max_b, qb, eb, L.N, L.K, L.Kp, L.batch, 0, 0, one, st);
                } else {
                    launch_gather_operand<true>(S, ws, max_a, qa, ea, L.M, L.K, L.Kp, L.batch, 0, 0, one, st);
                    launch_gather_operand<true>(S, WindowsOfImage{c.p, g}, max_b, qb, eb, L.N, L.K, L.Kp, L.batch, 0, 0, one, st);
                }
            }
            break;
        }
        case CONV_GRAD_WEIGHT:        // A: dY by filter over all windows; B: window values by position over all windows
            launch_gather_operand<true>(S, FiltersOverWindows{c.p, g}, max_a, qa, ea, L.M, L.K, L.Kp, 1, 0, 0, one, st);
            // the position maxima come from a per-pixel maximum over the images instead of a second gather
            pixel_max_over_images_kernel<<<dim3(ceil_div(g.H * g.W, PREPASS_THREADS), g.C < 65535 ? g.C : 65535), PREPASS_THREADS, 0, st>>>(
                c.q, c.pixmax, g.N, g.C, g.H * g.W);
            position_max_kernel<<<g.K, PREPASS_THREADS, 0, st>>>(c.pixmax, max_b, g);
            launch_gather_operand<false>(S, PositionsOverWindows{c.q, g}, max_b, qb, eb, L.N, L.K, L.Kp, 1, 0, 1, one, st);
            break;
        case CONV_GRAD_INPUT: {       // k runs (tap, filter); dY taps per pixel with one scale per image, weights by channel with one scale
            uint32_t* max_w = c.places ? max_b : max_a;
            uint32_t* max_img = c.places ? max_a : max_b;     // N words: both regions hold at least N (rows >= N, batch >= N)
            const size_t khw = (size_t)g.KH * g.KW;
            const TapMajorWeights wt{c.q, g, g.F, g.by_f, khw, (size_t)g.C * khw};
            launch_gather_max(StoredRows{c.q, (long long)g.F * g.K}, max_w, 1, g.F * g.K, 1, 0, 0, st);
            launch_gather_max(StoredRows{c.p, (long long)g.F * g.OH * g.OW}, max_img, g.N, g.F * g.OH * g.OW, 1, 0, 1, st);
            if (c.places) {
                launch_gather_operand<false>(S, AllPixelTaps{c.p, g}, max_img, qa, ea, L.M, L.K, L.Kp, 1, 0, 1, g.by_hw, st);
                launch_gather_operand<false>(S, wt, max_w, qb, eb, L.N, L.K, L.Kp, 1, 0, 0, one, st);
            } else {
                launch_gather_operand<false>(S, wt, max_w, qa, ea, L.M, L.K, L.Kp, L.batch, 0, 0, one, st);
                launch_gather_operand<false>(S, PixelTapsOfImage{c.p, g}, max_img, qb, eb, L.N, L.K, L.Kp, L.batch, 1, 0, one, st);
            }
            break;
        }
    }
    return cudaGetLastError();
}

cudaError_t conv_workspace(ConvKind kind, const rgb200_conv_shape* shape, int S, size_t* bytes) {
    ConvGeom g;
    if (!bytes || !conv_geometry(shape, S, g)) return cudaErrorInvalidValue;
    Layout L;
    cudaError_t e = conv_layout(kind, g, S, L);
    if (e == cudaSuccess) *bytes = L.total + conv_extra_bytes(kind, g);
    return e;
}

cudaError_t conv_run(ConvKind kind, const float* p, const float* q, float* out, const rgb200_conv_shape* shape, int S,
                     void* ws, size_t ws_bytes, void* stream) {
    ConvGeom g;
    if (!conv_geometry(shape, S, g)) return cudaErrorInvalidValue;
    Layout L;
    cudaError_t e = conv_layout(kind, g, S, L);
    if (e != cudaSuccess) return e;
    if (!p || !q || !out || !ws || ws_bytes < L.total + conv_extra_bytes(kind, g)) return cudaErrorInvalidValue;
    const DeviceInfo* dev = nullptr;
    if ((e = check_device(L.algo, &dev)) != cudaSuccess) return e;
    // The smallest layers (a LeNet-style first convolution) skip the tensor cores: one thread per output
    // evaluates the definition directly (rgb200_conv_direct.cuh); one launch, no workspace traffic.
    {
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        const long long weights = (long long)g.F * g.K;
        if (kind == CONV_FORWARD && g.K <= CONV_DIRECT_MAX_K && g.F <= CONV_DIRECT_MAX_F) {
            const long long windows = (long long)g.N * g.OH * g.OW;
            const unsigned grid = (unsigned)((windows + CONV_DIRECT_THREADS - 1) / CONV_DIRECT_THREADS);
            if (S == 1) conv_direct_forward_kernel<1><<<grid, CONV_DIRECT_THREADS, 0, st>>>(p, q, out, g);
            else if (S == 2) conv_direct_forward_kernel<2><<<grid, CONV_DIRECT_THREADS, 0, st>>>(p, q, out, g);
            else conv_direct_forward_kernel<3><<<grid, CONV_DIRECT_THREADS, 0, st>>>(p, q, out, g);
            return cudaGetLastError();
        }
        // the per-image maximum of dY is recomputed by every CTA of the image: worth it only for small images
        if (kind == CONV_GRAD_INPUT && weights <= CONV_DIRECT_MAX_WEIGHTS && (long long)g.F * g.KH * g.KW <= 256 &&
            (long long)g.F * g.OH * g.OW <= 16384) {
            const dim3 grid((unsigned)((g.C * g.H * g.W + CONV_DIRECT_THREADS - 1) / CONV_DIRECT_THREADS), (unsigned)g.N);
            if (S == 1) conv_direct_grad_input_kernel<1><<<grid, CONV_DIRECT_THREADS, 0, st>>>(p, q, out, g);
            else if (S == 2) conv_direct_grad_input_kernel<2><<<grid, CONV_DIRECT_THREADS, 0, st>>>(p, q, out, g);
            else conv_direct_grad_input_kernel<3><<<grid, CONV_DIRECT_THREADS, 0, st>>>(p, q, out, g);
            return cudaGetLastError();
        }
    }
    const ConvCall call{kind, g, p, q, conv_rows_are_places(kind, g, S),
                        reinterpret_cast<uint32_t*>(static_cast<char*>(ws) + L.total)};
    const PrepassHook hook{conv_prepass, &call};
    RunArgs a{nullptr, nullptr, out, nullptr, nullptr, nullptr, 0, 0, (long long)L.M * L.N, false, true,
              static_cast<char*>(ws), static_cast<cudaStream_t>(stream), nullptr};
    a.hook = &hook;
    if (call.places) a.c_image_rows = kind == CONV_FORWARD ? g.OH * g.OW : g.H * g.W;
    return dispatch(L, a, *dev);
}

}  // namespace
}  // namespace rgb200

using namespace rgb200;

// Fixed workspace of rgb200_gemm_fp32_static.  In host code this name is only a stand-in for the
// device object: the address a kernel can use comes from cudaGetSymbolAddress, looked up once per
// device with that device current (static_workspace_address below).
static __device__ __align__(256) unsigned char rgb200_static_scratch[RGB200_STATIC_WORKSPACE_BYTES];
// Scratch of the bounded-wait self-test (status word and three result words); separate from the array above so
// that the self-test never touches a rgb200_gemm_fp32_static call in flight.
static __device__ __align__(256) unsigned char rgb200_probe_scratch[256];

namespace {
void* g_static_ptr[MAX_DEVICES];
cudaError_t g_static_err[MAX_DEVICES];
std::once_flag g_static_once[MAX_DEVICES];

cudaError_t static_workspace_address(void** out) {
    int dev;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= MAX_DEVICES) return cudaErrorInvalidDevice;
    std::call_once(g_static_once[dev], [dev] {
        void* p = nullptr;
        g_static_err[dev] = cudaGetSymbolAddress(&p, rgb200_static_scratch);   // the current device's copy
        g_static_ptr[dev] = p;
    });
    if (g_static_err[dev] != cudaSuccess) return g_static_err[dev];
    if (!g_static_ptr[dev]) return cudaErrorInvalidSymbol;
    *out = g_static_ptr[dev];
    return cudaSuccess;
}
}  // namespace

extern "C" {

int rgb200_gemm_fp32_static(const float* A, const float* B, float* C, int M, int N, int K, const rgb200_config* cfg,
                            void* stream) {
    rgb200_config def;
    if (!cfg) { rgb200_default_config(&def); cfg = &def; }
    if (!A || !B || !C) return cudaErrorInvalidValue;
    Layout L;
    cudaError_t e = plan_layout(M, N, K, K, 1, *cfg, false, L);
    if (e != cudaSuccess) return e;
    if (L.total > (size_t)RGB200_STATIC_WORKSPACE_BYTES) return cudaErrorMemoryAllocation;   // does not fit the fixed array
    const DeviceInfo* dev = nullptr;
    if ((e = check_device(L.algo, &dev)) != cudaSuccess) return e;       // "not supported" before any symbol lookup
    void* ws = nullptr;
    if ((e = static_workspace_address(&ws)) != cudaSuccess) return e;
    return gemm_ws(A, B, C, M, N, K, 1, 0, 0, 0, cfg, ws, RGB200_STATIC_WORKSPACE_BYTES, stream, nullptr);
}

int rgb200_static_status(int* status) {
    if (!status) return cudaErrorInvalidValue;
    void* ws = nullptr;
    cudaError_t e = static_workspace_address(&ws);
    if (e != cudaSuccess) return e;
    return cudaMemcpy(status, ws, sizeof(int), cudaMemcpyDeviceToHost);    // the status word leads the array
}

void rgb200_default_config(rgb200_config* cfg) {
    if (!cfg) return;
    cfg->split_k = 1; cfg->tile_m = 16; cfg->tile_n = 16; cfg->tile_k = 32;
    cfg->algo = RGB200_ALGO_AUTO; cfg->slices = 3; cfg->trans_a = 0; cfg->trans_b = 0;
}

const char* rgb200_algo_name(int algo) {
    switch (algo) {
        case RGB200_ALGO_AUTO: return "auto";
        case RGB200_ALGO_REFERENCE: return "ref";
        case RGB200_ALGO_TILED: return "tiled";
        case RGB200_ALGO_TENSORCORE: return "tc";
    }
    return "?";
}

int rgb200_fast_div(int divisor, int n) {
    if (divisor < 1 || n < 0) return -1;
    return FastDiv(divisor).div(n);
}

int rgb200_layout(int M, int N, int K, int batch, const rgb200_config* cfg, rgb200_layout_info* info) {
    if (!cfg || !info) return cudaErrorInvalidValue;
    Layout L;
    cudaError_t e = plan_layout(M, N, K, K, batch, *cfg, false, L);
    if (e != cudaSuccess) return e;
    info->k_padded = L.Kp; info->k_blocks = L.k_blocks; info->min_split = L.min_split; info->split_k = L.split;
    info->tile_n = tile_n_for(L.S, N);
    info->planes_a = (size_t)batch * L.S * M * L.Kp; info->planes_b = (size_t)batch * L.S * N * L.Kp;
    info->partial_bytes = L.total - L.part;
    info->workspace_bytes = L.total;
    return cudaSuccess;
}

static int make_plan_common(int M, int N, int K, long long total_k, int batch, const rgb200_config* cfg, bool partial,
                            rgb200_plan* plan) {
    if (!plan || !cfg) return cudaErrorInvalidValue;
    Layout L;
    cudaError_t e = plan_layout(M, N, K, total_k, batch, *cfg, partial, L);
    if (e != cudaSuccess) return e;
    const DeviceInfo* dev = nullptr;
    if ((e = check_device(L.algo, &dev)) != cudaSuccess) return e;
    plan->algo = L.algo;
    plan->split_k = L.split;
    plan->workspace_bytes = L.total;
    return cudaSuccess;
}

int rgb200_make_plan(int M, int N, int K, const rgb200_config* cfg, rgb200_plan* plan) {
    return make_plan_common(M, N, K, K, 1, cfg, false, plan);
}
int rgb200_make_plan_batched(int M, int N, int K, int batch, const rgb200_config* cfg, rgb200_plan* plan) {
    return make_plan_common(M, N, K, K, batch, cfg, false, plan);
}
int rgb200_make_plan_partial(int M, int N, int K, long long total_k, const rgb200_config* cfg, rgb200_plan* plan) {
    return make_plan_common(M, N, K, total_k, 1, cfg, true, plan);
}

int rgb200_gemm_fp32_ws(const float* A, const float* B, float* C, int M, int N, int K, const rgb200_config* cfg,
                        void* workspace, size_t workspace_bytes, void* stream, void* const* events4) {
    return gemm_ws(A, B, C, M, N, K, 1, 0, 0, 0, cfg, workspace, workspace_bytes, stream, events4);
}

int rgb200_conv2d_workspace(const rgb200_conv_shape* shape, int slices, size_t* bytes) {
    return conv_workspace(CONV_FORWARD, shape, slices, bytes);
}
int rgb200_conv2d_grad_weight_workspace(const rgb200_conv_shape* shape, int slices, size_t* bytes) {
    return conv_workspace(CONV_GRAD_WEIGHT, shape, slices, bytes);
}
int rgb200_conv2d_grad_input_workspace(const rgb200_conv_shape* shape, int slices, size_t* bytes) {
    return conv_workspace(CONV_GRAD_INPUT, shape, slices, bytes);
}
int rgb200_conv2d_ws(const float* x, const float* weight, float* out, const rgb200_conv_shape* shape, int slices,
                     void* workspace, size_t workspace_bytes, void* stream) {
    return conv_run(CONV_FORWARD, x, weight, out, shape, slices, workspace, workspace_bytes, stream);
}
int rgb200_conv2d_grad_weight_ws(const float* dy, const float* x, float* dw, const rgb200_conv_shape* shape, int slices,
                                 void* workspace, size_t workspace_bytes, void* stream) {
    return conv_run(CONV_GRAD_WEIGHT, dy, x, dw, shape, slices, workspace, workspace_bytes, stream);
}
int rgb200_conv2d_grad_input_ws(const float* dy, const float* weight, float* dx, const rgb200_conv_shape* shape, int slices,
                                void* workspace, size_t workspace_bytes, void* stream) {
    return conv_run(CONV_GRAD_INPUT, dy, weight, dx, shape, slices, workspace, workspace_bytes, stream);
}

int rgb200_gemm_fp32_batched_ws(const float* A, const float* B, float* C, int M, int N, int K, int batch,
                                long long stride_a, long long stride_b, long long stride_c, const rgb200_config* cfg,
                                void* workspace, size_t workspace_bytes, void* stream, void* const* events4) {
    return gemm_ws(A, B, C, M, N, K, batch, stride_a, stride_b, stride_c, cfg, workspace, workspace_bytes, stream, events4);
}

int rgb200_host_gemm_create(int M, int N, int K, const rgb200_config* cfg, int block_rows, rgb200_host_gemm** handle) {
    if (!handle || !cfg) return cudaErrorInvalidValue;
    *handle = nullptr;
    if (block_rows <= 0) block_rows = 256;
    rgb200_host_gemm* h = new (std::nothrow) rgb200_host_gemm();
    if (!h) return cudaErrorMemoryAllocation;
    h->M = M; h->N = N; h->K = K; h->cfg = *cfg;
    cudaError_t e = cudaGetDevice(&h->device);
    // Row blocks: block_rows each; the last full block is halved repeatedly (down to 128 rows) so that little
    // compute and little of C remain after the last byte of A has arrived.
    if (e == cudaSuccess) {
        Layout probe;
        e = plan_layout(M, N, K, K, 1, *cfg, false, probe);
    }
    const DeviceInfo* dev = nullptr;
    if (e == cudaSuccess) e = check_device(cfg->algo == RGB200_ALGO_AUTO ? RGB200_ALGO_TENSORCORE : cfg->algo, &dev);
    if (e != cudaSuccess) { host_gemm_free(h); return e; }
    int lo = 0;
    while (lo < M) {
        int rows = M - lo < block_rows ? M - lo : block_rows;
        if (M - lo <= block_rows) {                       // the tail: 1/2, 1/4, ... of what is left
            while (rows > 128 && rows > (M - lo + 1) / 2) rows = (rows + 1) / 2;
            if (M - lo - rows < 64) rows = M - lo;
        }
        h->blocks.push_back({lo, rows});
        lo += rows;
    }
    for (const HostBlock& b : h->blocks) {
        Layout L;
        if ((e = plan_layout(b.rows, N, K, K, 1, *cfg, false, L)) != cudaSuccess) { host_gemm_free(h); return e; }
        h->layouts.push_back(L);
        h->ws_bytes = L.total > h->ws_bytes ? L.total : h->ws_bytes;
        // launches per block: A's split (a k-strided operand that cannot take the cluster form needs two kernels),
        // the MMA kernel, the K-range reduction
        h->launches += (cfg->trans_a && !cluster_split_fits(b.rows, L.Kp) ? 2 : 1) + 1 + (L.use_partial_ws ? 1 : 0);
    }
    // B's split, once per product: one kernel, two when B is stored k-strided and cannot take the cluster form, and none
    // extra when both operands are k-contiguous (the first block's launch then splits both)
    h->launches += cfg->trans_b ? (cfg->trans_a ? 1 : 0) : (cluster_split_fits(N, h->layouts[0].Kp) ? 1 : 2);
    const size_t na = (size_t)M * K, nb = (size_t)K * N, nc = (size_t)M * N;
    if ((e = cudaMalloc(&h->dA, na * sizeof(float))) != cudaSuccess || (e = cudaMalloc(&h->dB, nb * sizeof(float))) != cudaSuccess ||
        (e = cudaMalloc(&h->dC, nc * sizeof(float))) != cudaSuccess || (e = cudaMalloc(&h->ws, h->ws_bytes)) != cudaSuccess ||
        (e = cudaStreamCreateWithFlags(&h->s_in, cudaStreamNonBlocking)) != cudaSuccess ||
        (e = cudaStreamCreateWithFlags(&h->s_run, cudaStreamNonBlocking)) != cudaSuccess ||
        (e = cudaStreamCreateWithFlags(&h->s_out, cudaStreamNonBlocking)) != cudaSuccess) { host_gemm_free(h); return e; }
    for (cudaEvent_t* ev : {&h->ev_fork, &h->ev_b, &h->ev_in_done, &h->ev_run_done, &h->ev_out_done})
        if ((e = cudaEventCreateWithFlags(ev, cudaEventDisableTiming)) != cudaSuccess) { host_gemm_free(h); return e; }
    h->ev_a.assign(h->blocks.size(), nullptr);
    h->ev_c.assign(h->blocks.size(), nullptr);
    for (size_t i = 0; i < h->blocks.size(); ++i)
        if ((e = cudaEventCreateWithFlags(&h->ev_a[i], cudaEventDisableTiming)) != cudaSuccess ||
            (e = cudaEventCreateWithFlags(&h->ev_c[i], cudaEventDisableTiming)) != cudaSuccess) { host_gemm_free(h); return e; }
    *handle = h;
    return cudaSuccess;
}

int rgb200_host_gemm_destroy(rgb200_host_gemm* handle) {
    if (!handle) return cudaErrorInvalidValue;
    cudaError_t e = cudaSetDevice(handle->device);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    host_gemm_free(handle);
    return e;
}

int rgb200_host_gemm_info(const rgb200_host_gemm* handle, int* blocks, int* launches, size_t* device_bytes) {
    if (!handle) return cudaErrorInvalidValue;
    if (blocks) *blocks = (int)handle->blocks.size();
    if (launches) *launches = handle->launches;
    if (device_bytes)
        *device_bytes = ((size_t)handle->M * handle->K + (size_t)handle->K * handle->N + (size_t)handle->M * handle->N) * sizeof(float) +
                        handle->ws_bytes;
    return cudaSuccess;
}

int rgb200_gemm_fp32_host(rgb200_host_gemm* h, const float* A_host, const float* B_host, float* C_host, void* stream) {
    if (!h || !A_host || !B_host || !C_host) return cudaErrorInvalidValue;
    int cur = -1;
    cudaError_t e = cudaGetDevice(&cur);
    if (e != cudaSuccess) return e;
    if (cur != h->device) return cudaErrorInvalidDevice;
    const DeviceInfo* dev = nullptr;
    if ((e = check_device(h->cfg.algo == RGB200_ALGO_AUTO ? RGB200_ALGO_TENSORCORE : h->cfg.algo, &dev)) != cudaSuccess) return e;
    cudaStream_t user = static_cast<cudaStream_t>(stream);
    const int M = h->M, N = h->N, K = h->K;
    const bool ta = h->cfg.trans_a != 0;
#define RGB_CK(call) do { if ((e = (call)) != cudaSuccess) return e; } while (0)
    // fork: the three pipeline streams start after whatever the caller has enqueued on `stream`
    RGB_CK(cudaEventRecord(h->ev_fork, user));
    RGB_CK(cudaStreamWaitEvent(h->s_in, h->ev_fork, 0));
    RGB_CK(cudaStreamWaitEvent(h->s_run, h->ev_fork, 0));
    RGB_CK(cudaStreamWaitEvent(h->s_out, h->ev_fork, 0));
    // copy-in: B, then A block by block.  With trans_a the stored matrix is K x M and a row block of op(A) is a
    // band of columns: a pitched copy packs it into a dense K x rows block at element offset lo * K.
    RGB_CK(cudaMemcpyAsync(h->dB, B_host, (size_t)K * N * sizeof(float), cudaMemcpyHostToDevice, h->s_in));
    RGB_CK(cudaEventRecord(h->ev_b, h->s_in));
    for (size_t i = 0; i < h->blocks.size(); ++i) {
        const HostBlock& b = h->blocks[i];
        float* dst = h->dA + (size_t)b.lo * K;
        if (!ta) RGB_CK(cudaMemcpyAsync(dst, A_host + (size_t)b.lo * K, (size_t)b.rows * K * sizeof(float), cudaMemcpyHostToDevice, h->s_in));
        else RGB_CK(cudaMemcpy2DAsync(dst, (size_t)b.rows * sizeof(float), A_host + b.lo, (size_t)M * sizeof(float),
                                      (size_t)b.rows * sizeof(float), (size_t)K, cudaMemcpyHostToDevice, h->s_in));
        RGB_CK(cudaEventRecord(h->ev_a[i], h->s_in));
    }
    RGB_CK(cudaEventRecord(h->ev_in_done, h->s_in));
    // compute
    RGB_CK(cudaStreamWaitEvent(h->s_run, h->ev_b, 0));
    for (size_t i = 0; i < h->blocks.size(); ++i) {
        const HostBlock& b = h->blocks[i];
        RGB_CK(cudaStreamWaitEvent(h->s_run, h->ev_a[i], 0));
        RunArgs a{h->dA + (size_t)b.lo * K, h->dB, h->dC + (size_t)b.lo * N, nullptr, nullptr, nullptr, 0, 0, 0, ta,
                  h->cfg.trans_b != 0, h->ws, h->s_run, nullptr};
        a.reuse_b = i > 0;
        RGB_CK(dispatch(h->layouts[i], a, *dev));
        RGB_CK(cudaEventRecord(h->ev_c[i], h->s_run));
    }
    RGB_CK(cudaEventRecord(h->ev_run_done, h->s_run));
    // copy-out
    for (size_t i = 0; i < h->blocks.size(); ++i) {
        const HostBlock& b = h->blocks[i];
        RGB_CK(cudaStreamWaitEvent(h->s_out, h->ev_c[i], 0));
        RGB_CK(cudaMemcpyAsync(C_host + (size_t)b.lo * N, h->dC + (size_t)b.lo * N, (size_t)b.rows * N * sizeof(float),
                               cudaMemcpyDeviceToHost, h->s_out));
    }
    RGB_CK(cudaEventRecord(h->ev_out_done, h->s_out));
    // join: the caller's stream continues after the last copy into C_host
    RGB_CK(cudaStreamWaitEvent(user, h->ev_in_done, 0));
    RGB_CK(cudaStreamWaitEvent(user, h->ev_run_done, 0));
    RGB_CK(cudaStreamWaitEvent(user, h->ev_out_done, 0));
#undef RGB_CK
    return cudaSuccess;
}

int rgb200_host_gemm_status(const rgb200_host_gemm* handle, int* status) {
    if (!handle || !status) return cudaErrorInvalidValue;
    return cudaMemcpy(status, handle->ws, sizeof(int), cudaMemcpyDeviceToHost);
}

int rgb200_workspace_status(const void* workspace, int* status) {
    if (!workspace || !status) return cudaErrorInvalidValue;
    return cudaMemcpy(status, workspace, sizeof(int), cudaMemcpyDeviceToHost);   // the status word leads the workspace
}

int rgb200_gemm_fp32(const float* A, const float* B, float* C, int M, int N, int K, const rgb200_config* cfg, void* stream) {
    rgb200_config def;
    if (!cfg) { rgb200_default_config(&def); cfg = &def; }
    rgb200_plan plan;
    int rc = rgb200_make_plan(M, N, K, cfg, &plan);
    if (rc != cudaSuccess) return rc;
    void* ws = nullptr;
    cudaError_t e = cudaMalloc(&ws, plan.workspace_bytes);
    if (e != cudaSuccess) return e;
    rc = rgb200_gemm_fp32_ws(A, B, C, M, N, K, cfg, ws, plan.workspace_bytes, stream, nullptr);
    if (rc == cudaSuccess) rc = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
    if (rc == cudaSuccess) {
        int st = 0;
        rc = rgb200_workspace_status(ws, &st);
        if (rc == cudaSuccess && st != 0) rc = cudaErrorLaunchTimeout;
    }
    cudaFree(ws);
    return rc;
}

int rgb200_absmax(const float* X, int R, int K, int k_strided, float* out, void* stream) {
    if (!X || !out || R <= 0 || K <= 0) return cudaErrorInvalidValue;
    const DeviceInfo* dev = nullptr;
    cudaError_t e = check_device(RGB200_ALGO_TENSORCORE, &dev);
    if (e != cudaSuccess) return e;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (!k_strided) {
        rowmax_kmajor_kernel<<<ceil_div(R, PREPASS_THREADS / 32), PREPASS_THREADS, 0, st>>>(X, out, R, K);
    } else {
        // non-negative floats order like their bit patterns: accumulate the maxima in place as integers
        if ((e = cudaMemsetAsync(out, 0, (size_t)R * sizeof(float), st)) != cudaSuccess) return e;
        colmax_kstrided_kernel<<<dim3(ceil_div(R, 128), (ceil_div(K, COLMAX_K_PER_CTA) < COLMAX_MAX_GRID_Y ? ceil_div(K, COLMAX_K_PER_CTA) : COLMAX_MAX_GRID_Y), 1), PREPASS_THREADS, 0, st>>>(
            X, reinterpret_cast<uint32_t*>(out), R, K, 0);
    }
    return cudaGetLastError();
}

int rgb200_gemm_partial_ws(const float* A, const float* B, const float* max_a, const float* max_b, long long* T,
                           int M, int N, int K, long long total_k, const rgb200_config* cfg, void* workspace,
                           size_t workspace_bytes, void* stream) {
    if (!A || !B || !max_a || !max_b || !T || !cfg) return cudaErrorInvalidValue;
    Layout L;
    cudaError_t e = plan_layout(M, N, K, total_k, 1, *cfg, true, L);
    if (e != cudaSuccess) return e;
    if (L.algo == RGB200_ALGO_REFERENCE) return cudaErrorNotSupported;
    const DeviceInfo* dev = nullptr;
    if ((e = check_device(L.algo, &dev)) != cudaSuccess) return e;
    if (!workspace || workspace_bytes < L.total) return cudaErrorInvalidValue;
    RunArgs a{A, B, nullptr, T, max_a, max_b, 0, 0, 0, cfg->trans_a != 0, cfg->trans_b != 0,
              static_cast<char*>(workspace), static_cast<cudaStream_t>(stream), nullptr};
    return dispatch(L, a, *dev);
}

int rgb200_gemm_partial_scatter_ws(const float* A, const float* B, const float* max_a, const float* max_b,
                                   long long* const* owner_buffers, int world, int rank, int M, int N, int K,
                                   long long total_k, const rgb200_config* cfg, void* workspace, size_t workspace_bytes,
                                   void* stream) {
    if (!A || !B || !max_a || !max_b || !owner_buffers || !cfg) return cudaErrorInvalidValue;
    if (world < 1 || world > 8 || rank < 0 || rank >= world || M % (world * BLOCK_M) != 0) return cudaErrorInvalidValue;
    for (int i = 0; i < world; ++i)
        if (!owner_buffers[i] || (reinterpret_cast<uintptr_t>(owner_buffers[i]) & 31)) return cudaErrorInvalidValue;
    Layout L;
    cudaError_t e = plan_layout(M, N, K, total_k, 1, *cfg, true, L);
    if (e != cudaSuccess) return e;
    if (L.algo == RGB200_ALGO_REFERENCE) return cudaErrorNotSupported;
    const DeviceInfo* dev = nullptr;
    if ((e = check_device(L.algo, &dev)) != cudaSuccess) return e;
    if (!workspace || workspace_bytes < L.total) return cudaErrorInvalidValue;
    RunArgs a{A, B, nullptr, owner_buffers[rank], max_a, max_b, 0, 0, 0, cfg->trans_a != 0, cfg->trans_b != 0,
              static_cast<char*>(workspace), static_cast<cudaStream_t>(stream), nullptr};
    a.scatter = owner_buffers;
    a.scatter_world = world;
    a.scatter_rank = rank;
    return dispatch(L, a, *dev);
}

size_t rgb200_scatter_buffer_elems(int M, int N, int world, int slices) {
    if (M <= 0 || N <= 0 || world < 1 || world > 8 || slices < 1 || slices > 3 || M % (world * BLOCK_M) != 0) return 0;
    const int nt = tile_n_for(slices, N);
    return (size_t)world * (M / world) * ceil_div(N, nt) * nt;
}

int rgb200_round_scattered(const long long* buffer, int world, const float* max_a_own, const float* max_b, float* C_own,
                           int rows_own, int N, int slices, void* stream) {
    if (!buffer || !max_a_own || !max_b || !C_own || world < 1 || world > 8 || rows_own <= 0 || rows_own % BLOCK_M != 0 ||
        N <= 0 || slices < 1 || slices > 3 || (reinterpret_cast<uintptr_t>(buffer) & 31))
        return cudaErrorInvalidValue;
    const DeviceInfo* dev = nullptr;
    cudaError_t e = check_device(RGB200_ALGO_TENSORCORE, &dev);
    if (e != cudaSuccess) return e;
    const int nt = tile_n_for(slices, N), n_tiles = ceil_div(N, nt);
    const size_t chunks = (size_t)rows_own * n_tiles * nt / 4;
    const size_t want = (chunks + 255) / 256, cap = (size_t)dev->sm_count * 32;
    const int blocks = (int)(want < cap ? want : cap);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int e0 = -14 * (slices - 1);
    if (nt == 256) round_scattered_kernel<256><<<blocks, 256, 0, st>>>(buffer, world, max_a_own, max_b, C_own, rows_own, N, n_tiles, e0);
    else if (nt == 96) round_scattered_kernel<96><<<blocks, 256, 0, st>>>(buffer, world, max_a_own, max_b, C_own, rows_own, N, n_tiles, e0);
    else round_scattered_kernel<64><<<blocks, 256, 0, st>>>(buffer, world, max_a_own, max_b, C_own, rows_own, N, n_tiles, e0);
    return cudaGetLastError();
}

int rgb200_round_partial(const long long* T, int parts, const float* max_a, const float* max_b, float* C, int M, int N,
                         int slices, void* stream) {
    if (!T || !max_a || !max_b || !C || parts <= 0 || M <= 0 || N <= 0 || slices < 1 || slices > 3)
        return cudaErrorInvalidValue;
    const DeviceInfo* dev = nullptr;
    cudaError_t e = check_device(RGB200_ALGO_TENSORCORE, &dev);
    if (e != cudaSuccess) return e;
    const size_t total = (size_t)M * N;
    launch_round(T, parts, total, nullptr, nullptr, max_a, max_b, C, M, N, 1, (long long)total, -14 * (slices - 1),
                 dev->sm_count, static_cast<cudaStream_t>(stream));
    return cudaGetLastError();
}

int rgb200_selftest_bounded_wait(long long limit_clocks, int* status, long long* waited_clocks, int* both_left) {
    if (!status || !waited_clocks || !both_left || limit_clocks <= 0 || limit_clocks > 2000000000ll) return cudaErrorInvalidValue;
    const DeviceInfo* dev = nullptr;
    cudaError_t e = check_device(RGB200_ALGO_TENSORCORE, &dev);
    if (e != cudaSuccess) return e;
    void* base = nullptr;
    if ((e = cudaGetSymbolAddress(&base, rgb200_probe_scratch)) != cudaSuccess) return e;   // no allocation
    int* d_status = static_cast<int*>(base);
    long long* d_out = reinterpret_cast<long long*>(static_cast<char*>(base) + 64);
    if ((e = cudaMemset(base, 0, 256)) != cudaSuccess) return e;
    bounded_wait_probe_kernel<<<1, 64>>>(d_status, limit_clocks, d_out);
    if ((e = cudaDeviceSynchronize()) != cudaSuccess) return e;
    long long out[3];
    if ((e = cudaMemcpy(status, d_status, sizeof(int), cudaMemcpyDeviceToHost)) != cudaSuccess) return e;
    if ((e = cudaMemcpy(out, d_out, sizeof out, cudaMemcpyDeviceToHost)) != cudaSuccess) return e;
    *both_left = (out[0] == 1 && out[1] == 1) ? 1 : 0;
    *waited_clocks = out[2];
    return cudaSuccess;
}

uint64_t rgb200_fnv1a64(const void* data, size_t bytes, uint64_t h) {
    const unsigned char* p = static_cast<const unsigned char*>(data);
    for (size_t i = 0; i < bytes; ++i) { h ^= p[i]; h *= 0x100000001b3ull; }
    return h;
}
int rgb200_scale_exponent(float absmax) { return scale_exponent(absmax); }
int rgb200_fixed_point(float x, int se, int slices) { return fixed_point(x, quant_scale(se, slices)); }
uint32_t rgb200_round_to_float_bits(long long T, int E) { return round_to_f32_bits(T, E); }

}  // extern "C"
