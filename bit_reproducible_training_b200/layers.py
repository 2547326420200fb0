"""Linear and Conv2d layers on the reproducible GEMM and convolutions: the counterparts of ``_LinearFn`` /
``Linear`` and ``_ConvFn`` / ``Conv2d`` in the reference's repro_torch/repro_torch/layers.py:70-135.

Forward  Y  = X W^T     gemm(x,  W, m, n, k, trans_a=False, trans_b=True)     (layers.py:85)
Backward dX = dY W      gemm(dy, W, m, k, n, False, False)                    (layers.py:89)
         dW = dY^T X    gemm(dy, x, n, k, m, True,  False)                    (layers.py:90)

The bias gradient of the reference is an exact superaccumulator sum from another component
(repro_sum, layers.py:92), which is not part of this library.  A layer with a bias therefore needs
the caller's column-sum function (``set_bias_grad``); without one, asking for the bias gradient
raises instead of silently falling back to a sum whose bits depend on the reduction order.
"""
import torch

from . import repro_conv as rc
from . import repro_gemm as rg

_slices = 3
_bias_grad = None


def set_slices(s):
    """Number of int8 slices for all layers (1..3), like the reference's set_slices (layers.py:10-13)."""
    global _slices
    if s not in (1, 2, 3):
        raise ValueError("slices must be 1, 2 or 3")
    _slices = s


def set_bias_grad(fn):
    """fn(dy[m, n]) -> db[n]: the reproducible column sum to use for bias gradients (Conv2d passes dY as
    [N * OH * OW, F] rows)."""
    global _bias_grad
    _bias_grad = fn


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias):
        ctx.save_for_backward(x, weight)
        m, k, n = x.shape[0], weight.shape[1], weight.shape[0]
        y = rg.gemm(x, weight, m, n, k, False, True, _slices)
        return y + bias if bias is not None else y      # one IEEE addition per element

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        dy = dy.contiguous()
        m, k, n = x.shape[0], weight.shape[1], weight.shape[0]
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = rg.gemm(dy, weight, m, k, n, False, False, _slices)
        if ctx.needs_input_grad[1]:
            dw = rg.gemm(dy, x, n, k, m, True, False, _slices)
        if ctx.needs_input_grad[2]:
            if _bias_grad is None:
                raise NotImplementedError("bias gradient needs a reproducible column sum: call set_bias_grad(fn)")
            db = _bias_grad(dy)
        return dx, dw, db


class Linear(torch.nn.Linear):
    """torch.nn.Linear whose three matrix products are bit-reproducible (2-D input [tokens, features])."""

    def forward(self, x):
        return _LinearFn.apply(x.contiguous(), self.weight, self.bias)


class _ConvFn(torch.autograd.Function):
    """Y = conv(x, W), dX and dW through the three reproducible calls (layers.py:103-126 in the reference)."""

    @staticmethod
    def forward(ctx, x, weight, bias, stride, padding):
        ctx.save_for_backward(x, weight)
        n, c, h, w = x.shape
        f, _, kh, kw = weight.shape
        ctx.shape = rc.ConvShape(n, c, h, w, f, kh, kw, stride[0], stride[1], padding[0], padding[1])
        y = rc.conv2d(x, weight, ctx.shape, _slices)
        return y + bias[None, :, None, None] if bias is not None else y      # one IEEE addition per element

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        dy = dy.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = rc.conv2d_grad_input(dy, weight, ctx.shape, _slices)
        if ctx.needs_input_grad[1]:
            dw = rc.conv2d_grad_weight(dy, x, ctx.shape, _slices)
        if ctx.needs_input_grad[2]:
            if _bias_grad is None:
                raise NotImplementedError("bias gradient needs a reproducible column sum: call set_bias_grad(fn)")
            db = _bias_grad(dy.permute(0, 2, 3, 1).reshape(-1, dy.shape[1]))
        return dx, dw, db, None, None


class Conv2d(torch.nn.Conv2d):
    """torch.nn.Conv2d whose forward and both gradients are bit-reproducible: stride and zero padding only,
    like the reference's layer (layers.py:129-135)."""

    def forward(self, x):
        if self.groups != 1 or self.dilation != (1, 1) or isinstance(self.padding, str) or self.padding_mode != "zeros":
            raise NotImplementedError("Conv2d supports stride and zero padding only")
        return _ConvFn.apply(x.contiguous(), self.weight, self.bias, self.stride, self.padding)
