"""ctypes binding of librgb200.so (the C ABI declared in include/rgb200.h)."""
import ctypes as C
import os

from . import build as _build


class Config(C.Structure):
    _fields_ = [("split_k", C.c_int), ("tile_m", C.c_int), ("tile_n", C.c_int), ("tile_k", C.c_int),
                ("algo", C.c_int), ("slices", C.c_int), ("trans_a", C.c_int), ("trans_b", C.c_int)]


class Plan(C.Structure):
    _fields_ = [("algo", C.c_int), ("split_k", C.c_int), ("workspace_bytes", C.c_size_t)]


class LayoutInfo(C.Structure):
    _fields_ = [("k_padded", C.c_int), ("k_blocks", C.c_int), ("min_split", C.c_int), ("split_k", C.c_int),
                ("tile_n", C.c_int), ("planes_a", C.c_size_t), ("planes_b", C.c_size_t),
                ("partial_bytes", C.c_size_t), ("workspace_bytes", C.c_size_t)]


class ConvShape(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("N", "C", "H", "W", "F", "KH", "KW", "SY", "SX", "PY", "PX")]


_lib = None


def lib():
    """The loaded library.  There is no fallback: a missing library is an error."""
    global _lib
    if _lib is not None:
        return _lib
    path = os.environ.get("RGB200_LIBRARY") or _build.LIB      # explicit path override, e.g. for a tuned build
    if not os.path.exists(path):
        raise RuntimeError("%s is missing: run `python -m bit_reproducible_training_b200.build` "
                           "(or __graft_entry__.build()) first; there is no CPU fallback" % path)
    L = C.CDLL(path)
    vp, i, ll, fp = C.c_void_p, C.c_int, C.c_longlong, C.c_void_p
    cfgp, planp = C.POINTER(Config), C.POINTER(Plan)
    L.rgb200_default_config.argtypes = [cfgp]
    L.rgb200_default_config.restype = None
    L.rgb200_make_plan.argtypes = [i, i, i, cfgp, planp]
    L.rgb200_make_plan_batched.argtypes = [i, i, i, i, cfgp, planp]
    L.rgb200_make_plan_partial.argtypes = [i, i, i, ll, cfgp, planp]
    L.rgb200_gemm_fp32_ws.argtypes = [fp, fp, fp, i, i, i, cfgp, vp, C.c_size_t, vp, C.POINTER(vp)]
    L.rgb200_gemm_fp32.argtypes = [fp, fp, fp, i, i, i, cfgp, vp]
    L.rgb200_gemm_fp32_batched_ws.argtypes = [fp, fp, fp, i, i, i, i, ll, ll, ll, cfgp, vp, C.c_size_t, vp,
                                              C.POINTER(vp)]
    L.rgb200_gemm_fp32_static.argtypes = [fp, fp, fp, i, i, i, cfgp, vp]
    L.rgb200_static_status.argtypes = [C.POINTER(C.c_int)]
    L.rgb200_host_gemm_create.argtypes = [i, i, i, cfgp, i, C.POINTER(vp)]
    L.rgb200_gemm_fp32_host.argtypes = [vp, fp, fp, fp, vp]
    L.rgb200_host_gemm_info.argtypes = [vp, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_size_t)]
    L.rgb200_host_gemm_status.argtypes = [vp, C.POINTER(C.c_int)]
    L.rgb200_host_gemm_destroy.argtypes = [vp]
    L.rgb200_selftest_bounded_wait.argtypes = [ll, C.POINTER(C.c_int), C.POINTER(ll), C.POINTER(C.c_int)]
    L.rgb200_absmax.argtypes = [fp, i, i, i, fp, vp]
    L.rgb200_gemm_partial_ws.argtypes = [fp, fp, fp, fp, vp, i, i, i, ll, cfgp, vp, C.c_size_t, vp]
    L.rgb200_gemm_partial_scatter_ws.argtypes = [fp, fp, fp, fp, C.POINTER(vp), i, i, i, i, i, ll, cfgp, vp, C.c_size_t, vp]
    L.rgb200_scatter_buffer_elems.argtypes = [i, i, i, i]
    L.rgb200_scatter_buffer_elems.restype = C.c_size_t
    L.rgb200_round_scattered.argtypes = [vp, i, fp, fp, fp, i, i, i, vp]
    L.rgb200_round_partial.argtypes = [vp, i, fp, fp, fp, i, i, i, vp]
    L.rgb200_workspace_status.argtypes = [vp, C.POINTER(C.c_int)]
    L.rgb200_algo_name.argtypes = [i]
    L.rgb200_algo_name.restype = C.c_char_p
    L.rgb200_fnv1a64.argtypes = [vp, C.c_size_t, C.c_uint64]
    L.rgb200_fnv1a64.restype = C.c_uint64
    L.rgb200_scale_exponent.argtypes = [C.c_float]
    L.rgb200_fixed_point.argtypes = [C.c_float, i, i]
    L.rgb200_round_to_float_bits.argtypes = [ll, i]
    L.rgb200_round_to_float_bits.restype = C.c_uint32
    L.rgb200_fast_div.argtypes = [i, i]
    L.rgb200_layout.argtypes = [i, i, i, i, cfgp, C.POINTER(LayoutInfo)]
    shp = C.POINTER(ConvShape)
    for name in ("rgb200_conv2d", "rgb200_conv2d_grad_weight", "rgb200_conv2d_grad_input"):
        getattr(L, name + "_workspace").argtypes = [shp, i, C.POINTER(C.c_size_t)]
        getattr(L, name + "_ws").argtypes = [fp, fp, fp, shp, i, vp, C.c_size_t, vp]
    _lib = L
    return L
