"""The reference project's own PyTorch extension, built against librgb200.so, on a GPU.

oracle/build_ref_torch.py compiles the reference's repro_torch/_backend with the two textual includes of its
GEMM and convolution kernels (repro_torch/src/kernels.cu:2,5) dropped and -lrgb200 in their place; everything
else (bindings.cpp, layers.py, the exact-sum / softmax / pooling / Adam kernels) is the reference's, unchanged.
These tests run its Linear and Conv2d layers (repro_torch/repro_torch/layers.py:70-135) forward and backward on
CUDA tensors, so every GEMM and convolution goes bindings.cpp -> repro_gemm.cuh / repro_conv.cuh -> this library,
and compare the results bit for bit with the CPU oracle.
"""
import os
import sys

import numpy as np
import pytest
import torch

import oracle
from bit_reproducible_training_b200 import fixtures as fx

pytestmark = pytest.mark.gpu
BUILD = os.path.join(os.path.dirname(os.path.abspath(oracle.__file__)), "_ref", "repro_torch_rgb200")


@pytest.fixture(scope="module")
def rt():
    if not os.path.isdir(os.path.join(BUILD, "repro_torch")):
        pytest.skip("the reference's torch extension has not been built against librgb200.so (oracle/build_ref_torch.py)")
    sys.path.insert(0, BUILD)
    try:
        import repro_torch
    finally:
        sys.path.remove(BUILD)
    assert repro_torch.has_cuda
    return repro_torch


def bits(t):
    return t.detach().cpu().contiguous().numpy().view(np.uint32).reshape(-1)


@pytest.mark.parametrize("S", [1, 2, 3])
def test_reference_linear_layer_runs_on_this_library(rt, S):
    rt.set_slices(S)
    try:
        m, k, n = 200, 96, 144
        g = fx.Rng(50 + S)
        x, w, dy = g.normal(m * k), g.normal(n * k, 0.05), g.normal(m * n, 1e-3)
        layer = rt.Linear(k, n, bias=False).cuda()
        with torch.no_grad():
            layer.weight.copy_(torch.from_numpy(w).view(n, k))
        xt = torch.from_numpy(x).view(m, k).cuda().requires_grad_(True)
        y = layer(xt)
        y.backward(torch.from_numpy(dy).view(m, n).cuda())
        assert np.array_equal(bits(y), oracle.gemm(x, w, m, n, k, False, True, S).view(np.uint32).reshape(-1))
        assert np.array_equal(bits(xt.grad), oracle.gemm(dy, w, m, k, n, False, False, S).view(np.uint32).reshape(-1))
        assert np.array_equal(bits(layer.weight.grad), oracle.gemm(dy, x, n, k, m, True, False, S).view(np.uint32).reshape(-1))
        rt.layers.guard().check()
    finally:
        rt.set_slices(3)


@pytest.mark.parametrize("shape", [(10, 1, 28, 28, 6, 5, 5, 1, 1, 2, 2), (4, 3, 17, 23, 8, 3, 5, 2, 2, 1, 1),
                                   (2, 16, 12, 12, 24, 3, 3, 1, 1, 1, 1)])
def test_reference_conv_layer_runs_on_this_library(rt, shape):
    N, C, H, W, F, KH, KW, SY, SX, PY, PX = shape
    x, w, dy = fx.conv_inputs(shape)
    layer = rt.Conv2d(C, F, (KH, KW), stride=(SY, SX), padding=(PY, PX), bias=False).cuda()
    with torch.no_grad():
        layer.weight.copy_(torch.from_numpy(w).view(F, C, KH, KW))
    xt = torch.from_numpy(x).view(N, C, H, W).cuda().requires_grad_(True)
    y = layer(xt)
    y.backward(torch.from_numpy(dy).view(y.shape).cuda())
    assert np.array_equal(bits(y), oracle.conv2d(x, w, shape).view(np.uint32).reshape(-1))
    assert np.array_equal(bits(layer.weight.grad), oracle.conv2d_grad_weight(dy, x, shape).view(np.uint32).reshape(-1))
    assert np.array_equal(bits(xt.grad), oracle.conv2d_grad_input(dy, w, shape).view(np.uint32).reshape(-1))


def test_reference_binding_refuses_what_the_reference_refuses(rt):
    a = torch.zeros(4, 4, device="cuda", dtype=torch.float64)
    with pytest.raises(Exception):
        rt._backend.gemm(a, a, 4, 4, 4, False, False, 3)          # float32 only (bindings.cpp:36-38)
    b = torch.zeros(4, 4, device="cuda")
    with pytest.raises(Exception):
        rt._backend.gemm(b, b, 4, 5, 4, False, False, 3)          # shape mismatch (bindings.cpp:48)
