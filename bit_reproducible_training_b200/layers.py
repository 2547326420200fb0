"""Linear layer on the reproducible GEMM: the counterpart of ``_LinearFn`` / ``Linear`` in the
reference's repro_torch/repro_torch/layers.py:70-99.

Forward  Y  = X W^T     gemm(x,  W, m, n, k, trans_a=False, trans_b=True)     (layers.py:85)
Backward dX = dY W      gemm(dy, W, m, k, n, False, False)                    (layers.py:89)
         dW = dY^T X    gemm(dy, x, n, k, m, True,  False)                    (layers.py:90)

The bias gradient of the reference is an exact superaccumulator sum from another component
(repro_sum, layers.py:92), which is not part of this library.  A layer with a bias therefore needs
the caller's column-sum function (``set_bias_grad``); without one, asking for the bias gradient
raises instead of silently falling back to a sum whose bits depend on the reduction order.
"""
import torch

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
    """fn(dy[m, n]) -> db[n]: the reproducible column sum to use for bias gradients."""
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
