"""Convolution forward and both gradients on the GPU, through the C ABI, against the CPU oracle, the
committed hashes of the reference's CPU code, the reference's own test program, and the GEMM entry
point applied to an explicit im2col matrix."""
import os
import subprocess

import numpy as np
import pytest
import torch

import oracle
from bit_reproducible_training_b200 import fixtures as fx
from bit_reproducible_training_b200 import repro_conv as rc
from bit_reproducible_training_b200 import repro_gemm as rg

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def bits(t):
    return t.detach().cpu().numpy().reshape(-1).view(np.uint32)


@pytest.mark.parametrize("name,shape,dist", fx.CONV_CASES, ids=[c[0] for c in fx.CONV_CASES])
def test_convolutions_match_oracle_and_reference_hashes(name, shape, dist, conv_golden):
    x, w, dy = fx.conv_inputs(shape, dist)
    g = rc.ConvShape(*shape)
    dx_, dw_, ddy = dev(x), dev(w), dev(dy)
    for S in (1, 2, 3):
        rec = conv_golden[(name, S)]
        y = rc.conv2d(dx_, dw_, g, S)
        gw = rc.conv2d_grad_weight(ddy, dx_, g, S)
        gi = rc.conv2d_grad_input(ddy, dw_, g, S)
        assert np.array_equal(bits(y), oracle.conv2d(x, w, shape, S).reshape(-1).view(np.uint32)), (name, S, "forward")
        assert np.array_equal(bits(gw), oracle.conv2d_grad_weight(dy, x, shape, S).reshape(-1).view(np.uint32)), (name, S, "dW")
        assert np.array_equal(bits(gi), oracle.conv2d_grad_input(dy, w, shape, S).reshape(-1).view(np.uint32)), (name, S, "dX")
        assert "%016x" % rg.fnv1a64(y.cpu().numpy()) == rec["forward"]
        assert "%016x" % rg.fnv1a64(gw.cpu().numpy()) == rec["grad_weight"]
        assert "%016x" % rg.fnv1a64(gi.cpu().numpy()) == rec["grad_input"]


def test_forward_and_weight_gradient_equal_gemm_on_im2col():
    """The identities the reference tests (repro_conv_cuda/test_repro_conv.cu:84-112), with this
    library's own GEMM entry point on a stored im2col matrix."""
    shape = (4, 3, 17, 23, 8, 3, 5, 2, 2, 1, 1)
    N, C, H, W, F, KH, KW, SY, SX, PY, PX = shape
    x, w, dy = fx.conv_inputs(shape)
    g = rc.ConvShape(*shape)
    oh, ow, K, windows = g.OH(), g.OW(), g.K(), g.windows()
    cols = torch.nn.functional.unfold(torch.from_numpy(x).reshape(N, C, H, W), (KH, KW), padding=(PY, PX), stride=(SY, SX))
    X = cols.permute(0, 2, 1).reshape(windows, K).contiguous().cuda()          # [window][position]
    DY = torch.from_numpy(dy).reshape(N, F, oh * ow).permute(0, 2, 1).reshape(windows, F).contiguous().cuda()
    for S in (1, 3):
        y = rc.conv2d(dev(x), dev(w), g, S)
        y_rows = y.reshape(N, F, oh * ow).permute(0, 2, 1).reshape(windows, F)
        via_gemm = rg.gemm(X, dev(w), windows, F, K, trans_b=True, slices=S)
        assert torch.equal(via_gemm.view(torch.int32), y_rows.contiguous().view(torch.int32))
        gw = rc.conv2d_grad_weight(dev(dy), dev(x), g, S)
        via_gemm = rg.gemm(DY, X, F, K, windows, trans_a=True, slices=S)
        assert torch.equal(via_gemm.view(torch.int32).reshape(-1), gw.view(torch.int32).reshape(-1))


def test_allocation_free_calls_errors_and_repeatability():
    shape = (2, 4, 12, 12, 100, 3, 3, 1, 1, 1, 1)
    x, w, dy = fx.conv_inputs(shape)
    g = rc.ConvShape(*shape)
    dx_, dw_, ddy = dev(x), dev(w), dev(dy)
    code, nbytes = rc.conv2d_workspace(g, 3)
    assert code == 0
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    out = torch.full((g.output_size(),), float("nan"), device="cuda")
    assert rc.repro_conv2d_ws(dx_, dw_, out, g, 3, ws[:nbytes - 1]) == rg.cudaErrorInvalidValue
    assert rc.repro_conv2d_ws(dx_, dw_, out, g, 3, None) == rg.cudaErrorInvalidValue
    assert rc.repro_conv2d_ws(dx_, dw_, out, g, 4, ws) == rg.cudaErrorInvalidValue
    assert rc.repro_conv2d_ws(dx_, dw_, out, rc.ConvShape(2, 4, 2, 2, 100, 3, 3), 3, ws) == rg.cudaErrorInvalidValue
    assert torch.isnan(out).all()                          # nothing ran
    s = torch.cuda.Stream()
    torch.cuda.synchronize()
    assert rc.repro_conv2d_ws(dx_, dw_, out, g, 3, ws, stream=s) == 0
    s.synchronize()
    first = out.clone()
    assert np.array_equal(bits(first), oracle.conv2d(x, w, shape, 3).reshape(-1).view(np.uint32))
    ws.fill_(0xFF)                                         # leftovers in the workspace must not matter
    assert rc.repro_conv2d_ws(dx_, dw_, out, g, 3, ws) == 0
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.int32), first.view(torch.int32))
    assert rg.workspace_status(ws) == 0
    with pytest.raises(RuntimeError):
        rc.conv2d(torch.from_numpy(x), torch.from_numpy(w), g)      # CPU tensors: there is no CPU path


def test_reference_conv_test_program_passes_against_this_library():
    """repro_conv_cuda/test_repro_conv.cu, unmodified, linked against librgb200.so: GPU == the reference's
    CPU code for all three functions on its six shapes, repeat runs identical, forward and weight
    gradient == repro_gemm on im2col."""
    if not os.path.exists(oracle.REF_CONV_TEST_TOOL):
        pytest.skip("oracle/_ref/test_repro_conv_rgb200 has not been built (reference sources absent)")
    res = subprocess.run([oracle.REF_CONV_TEST_TOOL], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert "OVERALL: PASS" in res.stdout and "FAIL " not in res.stdout
    assert res.stdout.count("  ok ") == 36


def test_conv2d_layer_autograd_matches_oracle():
    """The torch layer: forward, input gradient and weight gradient through autograd equal the oracle's three
    results; a bias adds one IEEE addition per output."""
    from bit_reproducible_training_b200 import layers
    shape = (3, 5, 11, 9, 12, 3, 3, 1, 2, 1, 0)
    N, C, H, W, F, KH, KW, SY, SX, PY, PX = shape
    x, w, dy = fx.conv_inputs(shape)
    layer = layers.Conv2d(C, F, (KH, KW), stride=(SY, SX), padding=(PY, PX), bias=True).cuda()
    bias = torch.linspace(-1.0, 1.0, F)
    with torch.no_grad():
        layer.weight.copy_(torch.from_numpy(w).reshape(F, C, KH, KW))
        layer.bias.copy_(bias)
    layer.bias.requires_grad_(False)
    xin = torch.from_numpy(x).reshape(N, C, H, W).cuda().requires_grad_(True)
    y = layer(xin)
    want = torch.from_numpy(oracle.conv2d(x, w, shape, 3)) + bias[None, :, None, None]
    assert np.array_equal(bits(y), want.numpy().reshape(-1).view(np.uint32))
    y.backward(torch.from_numpy(dy).reshape(y.shape).cuda())
    assert np.array_equal(bits(xin.grad), oracle.conv2d_grad_input(dy, w, shape, 3).reshape(-1).view(np.uint32))
    assert np.array_equal(bits(layer.weight.grad), oracle.conv2d_grad_weight(dy, x, shape, 3).reshape(-1).view(np.uint32))
    with pytest.raises(NotImplementedError):
        layers.Conv2d(C, F, 3, dilation=2).cuda()(xin)


def test_random_geometries_match_the_oracle():
    """Forty seeded random layers: kernels up to 5 x 4, strides up to 3 (different per axis), padding up to
    kernel size, 1 to 40 channels and filters, both input distributions, every S."""
    rng = np.random.default_rng(20241125)
    for case in range(40):
        KH, KW = int(rng.integers(1, 6)), int(rng.integers(1, 5))
        SY, SX = int(rng.integers(1, 4)), int(rng.integers(1, 4))
        PY, PX = int(rng.integers(0, KH + 1)), int(rng.integers(0, KW + 1))
        H, W = max(1, KH - 2 * PY) + int(rng.integers(0, 12)), max(1, KW - 2 * PX) + int(rng.integers(0, 12))
        N, C, F = int(rng.integers(1, 5)), int(rng.choice([1, 2, 3, 4, 5, 8, 16, 17, 40])), int(rng.choice([1, 3, 4, 7, 16, 20, 33]))
        shape = (N, C, H, W, F, KH, KW, SY, SX, PY, PX)
        S = int(rng.integers(1, 4))
        x, w, dy = fx.conv_inputs(shape, "wide" if case % 3 == 0 else "normal", seed=1000 + case)
        g = rc.ConvShape(*shape)
        assert g.OH() >= 1 and g.OW() >= 1
        dx_, dw_, ddy = dev(x), dev(w), dev(dy)
        assert np.array_equal(bits(rc.conv2d(dx_, dw_, g, S)), oracle.conv2d(x, w, shape, S).reshape(-1).view(np.uint32)), (shape, S, "forward")
        assert np.array_equal(bits(rc.conv2d_grad_weight(ddy, dx_, g, S)),
                              oracle.conv2d_grad_weight(dy, x, shape, S).reshape(-1).view(np.uint32)), (shape, S, "dW")
        assert np.array_equal(bits(rc.conv2d_grad_input(ddy, dw_, g, S)),
                              oracle.conv2d_grad_input(dy, w, shape, S).reshape(-1).view(np.uint32)), (shape, S, "dX")
