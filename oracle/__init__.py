"""TEST INFRASTRUCTURE, NOT PRODUCT CODE: ctypes access to the CPU checkers.

``liboracle.so`` is the plain-C restatement of the reference's integer-exact GEMM definition
(``oracle/oracle.c``); ``_ref/librepro_ref.so`` is the reference's own ``cpu_gemm``
(repro_gemm_cuda/repro_gemm_cpu.h:25) compiled from its sources.  Only the tests, the smoke check
and the CPU-baseline legs of the benchmark may import this module; the shipped package never does.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, "liboracle.so")
_REF = os.path.join(_HERE, "_ref", "librepro_ref.so")
_REF_CUDA = os.path.join(_HERE, "_ref", "librepro_ref_cuda.so")
_REF_CONV = os.path.join(_HERE, "_ref", "librepro_ref_conv.so")
REF_CONV_TEST_TOOL = os.path.join(_HERE, "_ref", "test_repro_conv_rgb200")
REF_CONV_BENCH_TOOL = os.path.join(_HERE, "_ref", "bench_repro_conv_rgb200")
REF_CONV_BENCH_REF = os.path.join(_HERE, "_ref", "bench_repro_conv_ref")
REF_TEST_TOOL = os.path.join(_HERE, "_ref", "test_repro_gemm_rgb200")
REF_HASH_TOOL = os.path.join(_HERE, "_ref", "hash_repro_gemm_rgb200")

FNV_OFFSET = 0xCBF29CE484222325


def reference_root():
    """Where a checkout of the reference project lives: $REPRO_REFERENCE_ROOT, else a directory named
    ``reference`` beside this repository; None when neither holds the GEMM sources."""
    for cand in (os.environ.get("REPRO_REFERENCE_ROOT"), os.path.join(_HERE, "..", "..", "reference")):
        if cand and os.path.isfile(os.path.join(cand, "repro_gemm_cuda", "repro_gemm_cpu.h")):
            return os.path.abspath(cand)
    return None


def build(force=False):
    """Compile the checkers with oracle/Makefile (the reference build only where its sources exist)."""
    if force or not os.path.exists(_LIB) or os.path.getmtime(_LIB) < os.path.getmtime(os.path.join(_HERE, "oracle.c")):
        subprocess.run(["make", "-C", _HERE, "-B", "liboracle.so"], check=True, capture_output=True)
    root = reference_root()
    if root is None:
        return                      # keep whatever was built where the sources were present
    ref_arg = "REF_ROOT=" + root
    if force or not os.path.exists(_REF) or not os.path.exists(_REF_CONV):
        subprocess.run(["make", "-C", _HERE, "ref", ref_arg], check=True, capture_output=True)
    if force or not os.path.exists(_REF_CUDA) or not os.path.exists(REF_CONV_TEST_TOOL):
        subprocess.run(["make", "-C", _HERE, "ref_gpu", ref_arg], check=True, capture_output=True)
    # the reference's torch extension with its GEMM and convolution kernels replaced by librgb200.so
    from . import build_ref_torch
    if force or build_ref_torch.built_module() is None:
        build_ref_torch.build(root)


def _f32(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(C.POINTER(C.c_float))


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB)
        fp, ip, i64p = C.POINTER(C.c_float), C.c_int, C.POINTER(C.c_int64)
        L.orc_scale_exponent.argtypes = [C.c_float]
        L.orc_scale_exponent.restype = C.c_int
        L.orc_fixed_point.argtypes = [C.c_float, C.c_int, C.c_int]
        L.orc_fixed_point.restype = C.c_int
        L.orc_round_to_float_bits.argtypes = [C.c_int64, C.c_int]
        L.orc_round_to_float_bits.restype = C.c_uint32
        L.orc_digits.argtypes = [C.c_int, C.c_int, C.POINTER(C.c_int8)]
        L.orc_gemm.argtypes = [fp, fp, fp] + [ip] * 7
        L.orc_gemm.restype = C.c_int
        L.orc_gemm_partial.argtypes = [fp, fp, i64p, fp, fp] + [ip] * 9
        L.orc_gemm_partial.restype = C.c_int
        L.orc_absmax.argtypes = [fp, fp, ip, ip, ip]
        L.orc_round_partials.argtypes = [i64p, ip, fp, fp, fp, ip, ip, ip]
        ip11 = C.POINTER(C.c_int)
        for name in ("orc_conv2d", "orc_conv2d_grad_weight", "orc_conv2d_grad_input"):
            getattr(L, name).argtypes = [fp, fp, fp, ip11, ip, ip]
            getattr(L, name).restype = C.c_int
        L.orc_fnv1a64.argtypes = [C.c_void_p, C.c_size_t, C.c_uint64]
        L.orc_fnv1a64.restype = C.c_uint64
        st = C.POINTER(C.c_uint64)
        L.orc_fill_uniform_pm1.argtypes = [fp, C.c_size_t, st]
        L.orc_fill_normal.argtypes = [fp, C.c_size_t, C.c_double, st]
        L.orc_fill_u01.argtypes = [fp, C.c_size_t, C.c_double, st]
        L.orc_fill_wide.argtypes = [fp, C.c_size_t, C.c_int, C.c_int, st]
        L.orc_fill_wide_mixed.argtypes = [fp, C.c_size_t, C.c_int, C.c_int, st]
        L.orc_fill_prob_rows.argtypes = [fp, C.c_size_t, C.c_size_t, st]
        _lib = L
    return _lib


_ref = None


def ref():
    """The reference's own CPU implementation, or None where it has not been built."""
    global _ref
    if _ref is None and os.path.exists(_REF):
        R = C.CDLL(_REF)
        fp = C.POINTER(C.c_float)
        R.ref_cpu_gemm.argtypes = [fp, fp, fp] + [C.c_int] * 6
        R.ref_scale_exponent.argtypes = [C.c_float]
        R.ref_scale_exponent.restype = C.c_int
        R.ref_fixed_point.argtypes = [C.c_float, C.c_int, C.c_int]
        R.ref_fixed_point.restype = C.c_int
        R.ref_round_to_float.argtypes = [C.c_int64, C.c_int]
        R.ref_round_to_float.restype = C.c_float
        _ref = R
    return _ref


_ref_cuda = None


def ref_cuda():
    """The reference's own CUDA kernels recompiled for sm_100a, or None where not built."""
    global _ref_cuda
    if _ref_cuda is None and os.path.exists(_REF_CUDA):
        R = C.CDLL(_REF_CUDA)
        vp, i = C.c_void_p, C.c_int
        R.refcuda_plan.argtypes = [i] * 8 + [C.POINTER(C.c_int), C.POINTER(C.c_size_t)]
        R.refcuda_gemm_ws.argtypes = [vp, vp, vp] + [i] * 8 + [vp, C.c_size_t, vp, C.POINTER(vp)]
        _ref_cuda = R
    return _ref_cuda


def ref_cuda_gemm(A, B, M, N, K, ta=False, tb=False, S=3, split_k=1, algo=0, events=None):
    """Runs the reference's repro_gemm_fp32_ws on CUDA tensors A, B (torch); returns C [M, N]."""
    import torch
    R = ref_cuda()
    eff, nbytes = C.c_int(0), C.c_size_t(0)
    rc = R.refcuda_plan(M, N, K, split_k, algo, S, int(ta), int(tb), C.byref(eff), C.byref(nbytes))
    if rc != 0:
        raise RuntimeError("reference make_plan: cudaError %d" % rc)
    ws = torch.empty(nbytes.value, dtype=torch.uint8, device=A.device)
    out = torch.empty((M, N), dtype=torch.float32, device=A.device)
    ev = None
    if events is not None:
        ev = (C.c_void_p * 4)(*[C.c_void_p(e.cuda_event) for e in events])
    rc = R.refcuda_gemm_ws(A.data_ptr(), B.data_ptr(), out.data_ptr(), M, N, K, split_k, algo, S, int(ta), int(tb),
                           ws.data_ptr(), nbytes.value, torch.cuda.current_stream().cuda_stream, ev)
    if rc != 0:
        raise RuntimeError("reference repro_gemm_fp32_ws: cudaError %d" % rc)
    return out


def default_threads():
    env = os.environ.get("REPRO_CPU_THREADS")
    return int(env) if env else (os.cpu_count() or 1)


def gemm(A, B, M, N, K, ta=False, tb=False, S=3, threads=None):
    """C[M,N] = op(A) op(B) by the restated definition (float32 numpy in, float32 [M,N] out)."""
    A, pa = _f32(A)
    B, pb = _f32(B)
    assert A.size == M * K and B.size == K * N
    out = np.empty((M, N), dtype=np.float32)
    rc = lib().orc_gemm(pa, pb, out.ctypes.data_as(C.POINTER(C.c_float)), M, N, K, int(ta), int(tb), S,
                        threads or default_threads())
    if rc != 0:
        raise MemoryError("oracle gemm: allocation failed")
    return out


def ref_gemm(A, B, M, N, K, ta=False, tb=False, S=3):
    """The same product by the reference's own cpu_gemm (needs oracle/_ref)."""
    R = ref()
    if R is None:
        raise RuntimeError("oracle/_ref/librepro_ref.so has not been built")
    A, pa = _f32(A)
    B, pb = _f32(B)
    assert A.size == M * K and B.size == K * N
    out = np.empty((M, N), dtype=np.float32)
    R.ref_cpu_gemm(pa, pb, out.ctypes.data_as(C.POINTER(C.c_float)), M, N, K, int(ta), int(tb), S)
    return out


# --- convolution: shape = (N, C, H, W, F, KH, KW, SY, SX, PY, PX) -----------------------------------
def conv_dims(shape):
    N, Cc, H, W, F, KH, KW, SY, SX, PY, PX = shape
    return (H + 2 * PY - KH) // SY + 1, (W + 2 * PX - KW) // SX + 1


def _conv_call(fn, a, b, out_shape, shape, S, threads=None):
    a, pa = _f32(a)
    b, pb = _f32(b)
    out = np.empty(out_shape, dtype=np.float32)
    arr = (C.c_int * 11)(*shape)
    args = [pa, pb, out.ctypes.data_as(C.POINTER(C.c_float)), arr, S]
    if threads is not False:
        args.append(threads or default_threads())
    rc = fn(*args)
    if rc not in (0, None):
        raise MemoryError("oracle convolution: allocation failed")
    return out


def conv2d(x, w, shape, S=3):
    """out[N, F, OH, OW] by the restated definition."""
    oh, ow = conv_dims(shape)
    return _conv_call(lib().orc_conv2d, x, w, (shape[0], shape[4], oh, ow), shape, S)


def conv2d_grad_weight(dy, x, shape, S=3):
    return _conv_call(lib().orc_conv2d_grad_weight, dy, x, (shape[4], shape[1], shape[5], shape[6]), shape, S)


def conv2d_grad_input(dy, w, shape, S=3):
    return _conv_call(lib().orc_conv2d_grad_input, dy, w, shape[:4], shape, S)


_ref_conv = None


def ref_conv():
    """The reference's own CPU convolutions, or None where they have not been built."""
    global _ref_conv
    if _ref_conv is None and os.path.exists(_REF_CONV):
        R = C.CDLL(_REF_CONV)
        fp = C.POINTER(C.c_float)
        for name in ("ref_cpu_conv2d", "ref_cpu_conv2d_grad_weight", "ref_cpu_conv2d_grad_input"):
            getattr(R, name).argtypes = [fp, fp, fp, C.POINTER(C.c_int), C.c_int]
            getattr(R, name).restype = None
        _ref_conv = R
    return _ref_conv


def ref_conv2d(x, w, shape, S=3):
    oh, ow = conv_dims(shape)
    return _conv_call(ref_conv().ref_cpu_conv2d, x, w, (shape[0], shape[4], oh, ow), shape, S, threads=False)


def ref_conv2d_grad_weight(dy, x, shape, S=3):
    return _conv_call(ref_conv().ref_cpu_conv2d_grad_weight, dy, x, (shape[4], shape[1], shape[5], shape[6]), shape, S, threads=False)


def ref_conv2d_grad_input(dy, w, shape, S=3):
    return _conv_call(ref_conv().ref_cpu_conv2d_grad_input, dy, w, shape[:4], shape, S, threads=False)


def absmax(src, R, K, k_strided):
    src, ps = _f32(src)
    out = np.empty(R, dtype=np.float32)
    lib().orc_absmax(ps, out.ctypes.data_as(C.POINTER(C.c_float)), R, K, int(k_strided))
    return out


def gemm_partial(A, B, maxA, maxB, M, N, K, ta, tb, S, k0, k1, threads=None):
    """Exact int64 sums over k in [k0, k1) with scales fixed by the given whole-K maxima."""
    A, pa = _f32(A)
    B, pb = _f32(B)
    maxA, pma = _f32(maxA)
    maxB, pmb = _f32(maxB)
    T = np.empty((M, N), dtype=np.int64)
    rc = lib().orc_gemm_partial(pa, pb, T.ctypes.data_as(C.POINTER(C.c_int64)), pma, pmb, M, N, K, int(ta), int(tb), S,
                                k0, k1, threads or default_threads())
    if rc != 0:
        raise MemoryError("oracle gemm_partial: allocation failed")
    return T


def round_partials(T, maxA, maxB, M, N, S):
    T = np.ascontiguousarray(T, dtype=np.int64).reshape(-1, M, N)
    maxA, pma = _f32(maxA)
    maxB, pmb = _f32(maxB)
    out = np.empty((M, N), dtype=np.float32)
    lib().orc_round_partials(T.ctypes.data_as(C.POINTER(C.c_int64)), T.shape[0], pma, pmb,
                             out.ctypes.data_as(C.POINTER(C.c_float)), M, N, S)
    return out


def fnv1a64(arr, h=FNV_OFFSET):
    """FNV-1a-64 of the raw bytes of a numpy array, chained from ``h``."""
    arr = np.ascontiguousarray(arr)
    return int(lib().orc_fnv1a64(arr.ctypes.data, arr.nbytes, h))


def hexhash(arr, h=FNV_OFFSET):
    return "%016x" % fnv1a64(arr, h)


class Rng:
    """SplitMix64 stream with the reference's derived draws; fills are sequential like its tools."""

    def __init__(self, seed):
        self.state = C.c_uint64(seed)

    def _fill(self, fn, n, *args):
        out = np.empty(n, dtype=np.float32)
        fn(out.ctypes.data_as(C.POINTER(C.c_float)), n, *args, C.byref(self.state))
        return out

    def uniform_pm1(self, n):
        return self._fill(lib().orc_fill_uniform_pm1, n)

    def normal(self, n, scale=1.0):
        return self._fill(lib().orc_fill_normal, n, scale)

    def u01(self, n, scale=1.0):
        return self._fill(lib().orc_fill_u01, n, scale)

    def wide(self, n, elo, ehi):
        return self._fill(lib().orc_fill_wide, n, elo, ehi)

    def wide_mixed(self, n, elo=-20, ehi=20):
        return self._fill(lib().orc_fill_wide_mixed, n, elo, ehi)

    def prob_rows(self, rows, cols):
        out = np.empty(rows * cols, dtype=np.float32)
        lib().orc_fill_prob_rows(out.ctypes.data_as(C.POINTER(C.c_float)), rows, cols, C.byref(self.state))
        return out
