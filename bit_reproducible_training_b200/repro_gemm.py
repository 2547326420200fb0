"""Host-side mirror of the reference's repro_gemm interface, on top of the C ABI.

Names, argument meaning and error behaviour follow repro_gemm_cuda/repro_gemm.cuh:25-75
(``Algo``, ``Config``, ``Plan``, ``make_plan``, ``repro_gemm_fp32_ws``, ``repro_gemm_fp32``,
``algo_name``) and the torch binding repro_torch/src/bindings.cpp:43-66 (``gemm``).  PyTorch is used
only for device memory and streams; all arithmetic happens in librgb200.so.  There is no CPU path:
the reference's binding sends CPU tensors to its CPU implementation, this one refuses them.
"""
import ctypes as C
import os
import enum
from dataclasses import dataclass

import torch

from . import _lib

cudaSuccess = 0
cudaErrorInvalidValue = 1
cudaErrorLaunchTimeout = 702
cudaErrorNotSupported = 801
MAX_SLICES = 3


class Algo(enum.IntEnum):
    Auto = 0
    Reference = 1
    Tiled = 2
    TensorCore = 3


@dataclass
class Config:
    split_k: int = 1
    tile_m: int = 16      # ignored, kept for source compatibility like the reference's field
    tile_n: int = 16      # ignored
    tile_k: int = 32      # ignored
    algo: Algo = Algo.Auto
    slices: int = 3
    trans_a: bool = False
    trans_b: bool = False

    def c(self):
        return _lib.Config(self.split_k, self.tile_m, self.tile_n, self.tile_k, int(self.algo), self.slices,
                           int(self.trans_a), int(self.trans_b))


@dataclass
class Plan:
    algo: Algo
    split_k: int
    workspace_bytes: int


class ReproGemmError(RuntimeError):
    """A non-zero cudaError_t from the library; ``code`` holds the number."""

    def __init__(self, code, where):
        super().__init__("%s: cudaError %d" % (where, code))
        self.code = code


def algo_name(a):
    return _lib.lib().rgb200_algo_name(int(a)).decode()


def make_plan(M, N, K, cfg=None, batch=1):
    """Returns (code, Plan or None); code is a cudaError_t number as in the reference."""
    cfg = cfg or Config()
    p = _lib.Plan()
    c = cfg.c()
    if batch == 1:
        rc = _lib.lib().rgb200_make_plan(M, N, K, C.byref(c), C.byref(p))
    else:
        rc = _lib.lib().rgb200_make_plan_batched(M, N, K, batch, C.byref(c), C.byref(p))
    return rc, (Plan(Algo(p.algo), p.split_k, p.workspace_bytes) if rc == cudaSuccess else None)


def _ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def _stream(stream):
    s = stream if stream is not None else torch.cuda.current_stream()
    return C.c_void_p(s.cuda_stream)


def _events(events):
    if events is None:
        return None
    arr = (C.c_void_p * 4)(*[C.c_void_p(e.cuda_event) for e in events])
    return arr


def repro_gemm_fp32_ws(A, B, Cout, M, N, K, cfg, workspace, stream=None, stage_events=None):
    """Asynchronous, allocation-free run on `stream` (default: torch's current stream).

    A, B, Cout, workspace are CUDA tensors (workspace: uint8).  stage_events: four recorded-capable
    ``torch.cuda.Event(enable_timing=True)`` objects that have been created on the device
    (record each once beforehand so their handles exist).  Returns the cudaError_t number.
    """
    c = cfg.c()
    return _lib.lib().rgb200_gemm_fp32_ws(_ptr(A), _ptr(B), _ptr(Cout), M, N, K, C.byref(c), _ptr(workspace),
                                         workspace.numel() if workspace is not None else 0, _stream(stream),
                                         _events(stage_events))


def repro_gemm_fp32(A, B, Cout, M, N, K, cfg=None, stream=None):
    """Convenience form: the library allocates the workspace, runs, synchronises and frees."""
    c = (cfg or Config()).c()
    return _lib.lib().rgb200_gemm_fp32(_ptr(A), _ptr(B), _ptr(Cout), M, N, K, C.byref(c), _stream(stream))


STATIC_WORKSPACE_BYTES = 32 << 20
cudaErrorMemoryAllocation = 2


def repro_gemm_fp32_static(A, B, Cout, M, N, K, cfg=None, stream=None):
    """Allocation-free run for callers that own no device memory besides A, B and C (for example
    an operator living under a framework whose caching allocator must not be bypassed): the
    workspace is a fixed STATIC_WORKSPACE_BYTES array inside the library.  Asynchronous on `stream`.
    Returns the cudaError_t number; 2 means the problem needs more workspace than the array holds.
    Calls share the array, so calls that overlap on the GPU race; keep them on one stream."""
    c = (cfg or Config()).c()
    return _lib.lib().rgb200_gemm_fp32_static(_ptr(A), _ptr(B), _ptr(Cout), M, N, K, C.byref(c), _stream(stream))


def repro_gemm_fp32_batched_ws(A, B, Cout, M, N, K, batch, stride_a, stride_b, stride_c, cfg, workspace, stream=None,
                               stage_events=None):
    c = cfg.c()
    return _lib.lib().rgb200_gemm_fp32_batched_ws(_ptr(A), _ptr(B), _ptr(Cout), M, N, K, batch, stride_a, stride_b,
                                                 stride_c, C.byref(c), _ptr(workspace), workspace.numel(),
                                                 _stream(stream), _events(stage_events))


def static_status():
    """Status word of the fixed array behind repro_gemm_fp32_static (0, or the code of an expired wait)."""
    st = C.c_int(0)
    rc = _lib.lib().rgb200_static_status(C.byref(st))
    if rc != cudaSuccess:
        raise ReproGemmError(rc, "static_status")
    return st.value


def workspace_status(workspace):
    st = C.c_int(0)
    rc = _lib.lib().rgb200_workspace_status(_ptr(workspace), C.byref(st))
    if rc != cudaSuccess:
        raise ReproGemmError(rc, "workspace_status")
    return st.value


_ws_cache = {}


def _workspace(nbytes, device):
    """One growing scratch tensor per device and stream, the role torch.empty plays in bindings.cpp:57."""
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    ws = _ws_cache.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _ws_cache[key] = ws
    return ws


class ReproGemmIncomplete(RuntimeError):
    """A kernel gave up a bounded wait and left its output incomplete; ``status`` holds the code of the wait."""

    def __init__(self, status, where):
        super().__init__("%s: a bounded wait inside the kernel expired (status %d); the result is incomplete" % (where, status))
        self.status = status


def check_status_enabled():
    """Opt-in check of the workspace's status word after the allocating wrappers (gemm, gemm_batched): set
    RGB200_CHECK_STATUS=1.  It synchronises the stream, so it is off by default."""
    return os.environ.get("RGB200_CHECK_STATUS", "0") not in ("", "0")


def _raise_if_incomplete(ws, where):
    if check_status_enabled():
        torch.cuda.current_stream(ws.device).synchronize()
        st = workspace_status(ws)
        if st != 0:
            raise ReproGemmIncomplete(st, where)


def _check(t, n, name):
    if t.dtype != torch.float32:
        raise TypeError("%s must be float32" % name)
    if not t.is_cuda:
        raise RuntimeError("%s is not a CUDA tensor: this library has no CPU path" % name)
    if t.numel() != n:
        raise ValueError("%s has %d elements, expected %d" % (name, t.numel(), n))
    return t.contiguous()


def gemm(A, B, M, N, K, trans_a=False, trans_b=False, slices=3, split_k=1, algo=Algo.Auto):
    """C[M,N] = op(A) op(B) on the current stream; the counterpart of ``_backend.gemm``
    (repro_torch/src/bindings.cpp:43-66).  Returns a new [M, N] float32 CUDA tensor."""
    A = _check(A, M * K, "A")
    B = _check(B, K * N, "B")
    cfg = Config(split_k=split_k, algo=algo, slices=slices, trans_a=trans_a, trans_b=trans_b)
    rc, plan = make_plan(M, N, K, cfg)
    if rc != cudaSuccess:
        raise ReproGemmError(rc, "make_plan")
    with torch.cuda.device(A.device):
        ws = _workspace(plan.workspace_bytes, A.device)
        out = torch.empty((M, N), dtype=torch.float32, device=A.device)
        rc = repro_gemm_fp32_ws(A, B, out, M, N, K, cfg, ws)
    if rc != cudaSuccess:
        raise ReproGemmError(rc, "repro_gemm_fp32_ws")
    _raise_if_incomplete(ws, "gemm")
    return out


def gemm_batched(A, B, batch, M, N, K, trans_a=False, trans_b=False, slices=3):
    """`batch` independent products of densely stacked matrices: A [batch, M*K], B [batch, K*N]."""
    A = _check(A, batch * M * K, "A")
    B = _check(B, batch * K * N, "B")
    cfg = Config(slices=slices, trans_a=trans_a, trans_b=trans_b)
    rc, plan = make_plan(M, N, K, cfg, batch=batch)
    if rc != cudaSuccess:
        raise ReproGemmError(rc, "make_plan_batched")
    with torch.cuda.device(A.device):
        ws = _workspace(plan.workspace_bytes, A.device)
        out = torch.empty((batch, M, N), dtype=torch.float32, device=A.device)
        rc = repro_gemm_fp32_batched_ws(A, B, out, M, N, K, batch, M * K, K * N, M * N, cfg, ws)
    if rc != cudaSuccess:
        raise ReproGemmError(rc, "repro_gemm_fp32_batched_ws")
    _raise_if_incomplete(ws, "gemm_batched")
    return out


class HostGemm:
    """C = op(A) op(B) for operands and result in pinned HOST memory, with the PCIe copies overlapped:
    the Python face of rgb200_host_gemm_create / rgb200_gemm_fp32_host / rgb200_host_gemm_destroy.

    The library copies B first; A then travels in blocks of rows, and for each block the split pre-pass,
    the MMA kernel and the copy of the finished rows of C back to the host run while the next block of A
    is still on its way.  Row blocks are independent products, so the bits equal those of one call.
    Device buffers, workspace, streams and events are created once; a call allocates nothing."""

    def __init__(self, M, N, K, cfg=None, block_rows=0, device=None):
        self.M, self.N, self.K, self.cfg = M, N, K, cfg or Config()
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        self._h = C.c_void_p()
        c = self.cfg.c()
        with torch.cuda.device(self.device):
            rc = _lib.lib().rgb200_host_gemm_create(M, N, K, C.byref(c), block_rows, C.byref(self._h))
        if rc != cudaSuccess:
            raise ReproGemmError(rc, "host_gemm_create")
        nb, nl, nbytes = C.c_int(0), C.c_int(0), C.c_size_t(0)
        _lib.lib().rgb200_host_gemm_info(self._h, C.byref(nb), C.byref(nl), C.byref(nbytes))
        self.blocks, self.launches, self.device_bytes = nb.value, nl.value, nbytes.value

    def __call__(self, hA, hB, hC, stream=None):
        """Enqueues the whole product; on return the stream (default: torch's current one) is ordered after
        the last copy into hC: synchronise it, or record an event on it, to know when hC is ready."""
        for t, n, name in ((hA, self.M * self.K, "A"), (hB, self.K * self.N, "B"), (hC, self.M * self.N, "C")):
            if t.is_cuda or t.dtype != torch.float32 or t.numel() != n or not t.is_contiguous():
                raise ValueError("%s must be a contiguous float32 host tensor of %d elements" % (name, n))
        with torch.cuda.device(self.device):
            rc = _lib.lib().rgb200_gemm_fp32_host(self._h, _ptr(hA), _ptr(hB), _ptr(hC), _stream(stream))
        if rc != cudaSuccess:
            raise ReproGemmError(rc, "gemm_fp32_host")

    def status(self):
        st = C.c_int(0)
        rc = _lib.lib().rgb200_host_gemm_status(self._h, C.byref(st))
        if rc != cudaSuccess:
            raise ReproGemmError(rc, "host_gemm_status")
        return st.value

    def close(self):
        if self._h:
            with torch.cuda.device(self.device):
                _lib.lib().rgb200_host_gemm_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


# ------------------------------------------------------------------------------------------------
# K-sharded building blocks (one K range per rank); see bit_reproducible_training_b200/sharded.py
# ------------------------------------------------------------------------------------------------
def absmax(X, R, K, k_strided, out=None):
    """max over k of |op(X)[r, k]| as a float32 [R] tensor (written into `out` when given)."""
    if out is None:
        out = torch.empty(R, dtype=torch.float32, device=X.device)
    rc = _lib.lib().rgb200_absmax(_ptr(X), R, K, int(k_strided), _ptr(out), _stream(None))
    if rc != cudaSuccess:
        raise ReproGemmError(rc, "absmax")
    return out


def gemm_partial(A, B, max_a, max_b, M, N, K, total_k, cfg):
    """Exact INT64 sums over this rank's K range, scales fixed by the global maxima."""
    c = cfg.c()
    p = _lib.Plan()
    rc = _lib.lib().rgb200_make_plan_partial(M, N, K, total_k, C.byref(c), C.byref(p))
    if rc != cudaSuccess:
        raise ReproGemmError(rc, "make_plan_partial")
    ws = _workspace(p.workspace_bytes, A.device)
    T = torch.empty((M, N), dtype=torch.int64, device=A.device)
    rc = _lib.lib().rgb200_gemm_partial_ws(_ptr(A), _ptr(B), _ptr(max_a), _ptr(max_b), _ptr(T), M, N, K, total_k,
                                          C.byref(c), _ptr(ws), ws.numel(), _stream(None))
    if rc != cudaSuccess:
        raise ReproGemmError(rc, "gemm_partial_ws")
    return T


def gemm_partial_scatter(A, B, max_a, max_b, owner_ptrs, world, rank, M, N, K, total_k, cfg):
    """Exact INT64 sums over this rank's K range, stored by row block into the owners' receive buffers
    (owner_ptrs: device addresses valid on this device; slot `rank` of each buffer of scatter_buffer_elems)."""
    c = cfg.c()
    p = _lib.Plan()
    rc = _lib.lib().rgb200_make_plan_partial(M, N, K, total_k, C.byref(c), C.byref(p))
    if rc != cudaSuccess:
        raise ReproGemmError(rc, "make_plan_partial")
    ws = _workspace(p.workspace_bytes, A.device)
    ptrs = (C.c_void_p * world)(*[C.c_void_p(int(x)) for x in owner_ptrs])
    rc = _lib.lib().rgb200_gemm_partial_scatter_ws(_ptr(A), _ptr(B), _ptr(max_a), _ptr(max_b), ptrs, world, rank, M, N, K,
                                                  total_k, C.byref(c), _ptr(ws), ws.numel(), _stream(None))
    if rc != cudaSuccess:
        raise ReproGemmError(rc, "gemm_partial_scatter_ws")


def scatter_buffer_elems(M, N, world, slices):
    """INT64 elements of one rank's receive buffer for gemm_partial_scatter (0: shape not supported)."""
    return int(_lib.lib().rgb200_scatter_buffer_elems(M, N, world, slices))


def round_scattered(buffer, world, max_a_own, max_b, rows_own, N, slices, out=None):
    """Owner-side finish of the scattered reduction: sum of the `world` slots, one rounding, dense rows of C."""
    if out is None:
        out = torch.empty((rows_own, N), dtype=torch.float32, device=buffer.device)
    rc = _lib.lib().rgb200_round_scattered(_ptr(buffer), world, _ptr(max_a_own), _ptr(max_b), _ptr(out), rows_own, N,
                                          slices, _stream(None))
    if rc != cudaSuccess:
        raise ReproGemmError(rc, "round_scattered")
    return out


def round_partial(T, max_a, max_b, M, N, slices):
    """C = single rounding of (sum over the leading axis of T) * 2^(eA + eB - 14 (S - 1))."""
    T = T.contiguous()
    parts = T.numel() // (M * N)
    out = torch.empty((M, N), dtype=torch.float32, device=T.device)
    rc = _lib.lib().rgb200_round_partial(_ptr(T), parts, _ptr(max_a), _ptr(max_b), _ptr(out), M, N, slices,
                                        _stream(None))
    if rc != cudaSuccess:
        raise ReproGemmError(rc, "round_partial")
    return out


def fnv1a64(t, h=0xCBF29CE484222325):
    """FNV-1a-64 of a CPU tensor's / numpy array's raw bytes (repro_test_util.h:20-24)."""
    import numpy as np
    a = t.detach().cpu().contiguous().numpy() if isinstance(t, torch.Tensor) else np.ascontiguousarray(t)
    return int(_lib.lib().rgb200_fnv1a64(C.c_void_p(a.ctypes.data), a.nbytes, h))
