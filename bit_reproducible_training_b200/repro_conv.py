"""Host-side mirror of the reference's convolution interface (repro_conv_cuda/repro_conv.cuh:22-32)
over librgb200.so: the shape type, the three workspace queries, the three allocation-free calls,
and tensor-level conveniences.  CUDA tensors only; there is no CPU path.

Layouts are PyTorch's: x[N, C, H, W], weight[F, C, KH, KW], output and its gradient [N, F, OH, OW].
Bias is not part of these calls (the reference adds it with one IEEE addition)."""
import ctypes as C
from dataclasses import dataclass

import torch

from . import _lib
from .repro_gemm import ReproGemmError, _ptr, _stream, _workspace, cudaSuccess


@dataclass
class ConvShape:
    """Field for field the reference's ConvShape (repro_conv_cuda/repro_conv_math.cuh:29-45)."""
    N: int
    C: int
    H: int
    W: int
    F: int
    KH: int
    KW: int
    SY: int = 1
    SX: int = 1
    PY: int = 0
    PX: int = 0

    def K(self):
        return self.C * self.KH * self.KW

    def OH(self):
        return (self.H + 2 * self.PY - self.KH) // self.SY + 1

    def OW(self):
        return (self.W + 2 * self.PX - self.KW) // self.SX + 1

    def windows(self):
        return self.N * self.OH() * self.OW()

    def input_size(self):
        return self.N * self.C * self.H * self.W

    def weight_size(self):
        return self.F * self.K()

    def output_size(self):
        return self.N * self.F * self.OH() * self.OW()

    def c(self):
        return _lib.ConvShape(self.N, self.C, self.H, self.W, self.F, self.KH, self.KW, self.SY, self.SX, self.PY, self.PX)


def _workspace_query(name, g, S):
    n = C.c_size_t(0)
    s = g.c()
    rc = getattr(_lib.lib(), name)(C.byref(s), S, C.byref(n))
    return rc, n.value


def conv2d_workspace(g, S=3):
    """(cudaError code, bytes) for repro_conv2d_ws."""
    return _workspace_query("rgb200_conv2d_workspace", g, S)


def conv2d_grad_weight_workspace(g, S=3):
    return _workspace_query("rgb200_conv2d_grad_weight_workspace", g, S)


def conv2d_grad_input_workspace(g, S=3):
    return _workspace_query("rgb200_conv2d_grad_input_workspace", g, S)


def _call(name, a, b, out, g, S, ws, stream):
    s = g.c()
    return getattr(_lib.lib(), name)(_ptr(a), _ptr(b), _ptr(out), C.byref(s), S, _ptr(ws),
                                     0 if ws is None else ws.numel(), _stream(stream))


def repro_conv2d_ws(x, weight, out, g, S, ws, stream=None):
    """out[N,F,OH,OW] from x and weight; asynchronous, allocation-free; returns the cudaError code."""
    return _call("rgb200_conv2d_ws", x, weight, out, g, S, ws, stream)


def repro_conv2d_grad_weight_ws(dy, x, dw, g, S, ws, stream=None):
    """dw[F,C,KH,KW] from dy[N,F,OH,OW] and x."""
    return _call("rgb200_conv2d_grad_weight_ws", dy, x, dw, g, S, ws, stream)


def repro_conv2d_grad_input_ws(dy, weight, dx, g, S, ws, stream=None):
    """dx[N,C,H,W] from dy[N,F,OH,OW] and weight."""
    return _call("rgb200_conv2d_grad_input_ws", dy, weight, dx, g, S, ws, stream)


def _run(query, call, a, b, out_shape, g, S):
    if not (a.is_cuda and b.is_cuda):
        raise RuntimeError("repro_conv runs on CUDA tensors only; there is no CPU path")
    if a.dtype != torch.float32 or b.dtype != torch.float32:
        raise TypeError("repro_conv takes float32 tensors")
    rc, nbytes = query(g, S)
    if rc != cudaSuccess:
        raise ReproGemmError(rc, query.__name__)
    ws = _workspace(nbytes, a.device)
    out = torch.empty(out_shape, dtype=torch.float32, device=a.device)
    rc = call(a.contiguous(), b.contiguous(), out, g, S, ws)
    if rc != cudaSuccess:
        raise ReproGemmError(rc, call.__name__)
    return out


def conv2d(x, weight, g, S=3):
    """Tensor-level forward: allocates the workspace and the result through torch's allocator."""
    return _run(conv2d_workspace, repro_conv2d_ws, x, weight, (g.N, g.F, g.OH(), g.OW()), g, S)


def conv2d_grad_weight(dy, x, g, S=3):
    return _run(conv2d_grad_weight_workspace, repro_conv2d_grad_weight_ws, dy, x, (g.F, g.C, g.KH, g.KW), g, S)


def conv2d_grad_input(dy, weight, g, S=3):
    return _run(conv2d_grad_input_workspace, repro_conv2d_grad_input_ws, dy, weight, (g.N, g.C, g.H, g.W), g, S)
