"""Pins the CPU restatement of the convolutions (oracle/oracle.c: orc_conv2d*) before the CUDA path
is checked against it.

Sources of truth, produced by the reference's own code:
  * tests/golden/conv_hashes.json - output hashes of cpu_conv2d, cpu_conv2d_grad_weight and
    cpu_conv2d_grad_input (repro_conv_cuda/repro_conv_cpu.h:25,45,72) for seeded inputs
  * oracle/_ref/librepro_ref_conv.so (those functions compiled from their sources), where present
"""
import numpy as np
import pytest

import oracle
from bit_reproducible_training_b200 import fixtures as fx


@pytest.mark.parametrize("name,shape,dist", fx.CONV_CASES, ids=[c[0] for c in fx.CONV_CASES])
def test_oracle_convolutions_match_golden_hashes(name, shape, dist, conv_golden):
    x, w, dy = fx.conv_inputs(shape, dist)
    for S in (1, 2, 3):
        rec = conv_golden[(name, S)]
        assert tuple(rec["shape"]) == shape
        assert "%016x" % oracle.fnv1a64(dy, oracle.fnv1a64(w, oracle.fnv1a64(x))) == rec["in_hash"]
        assert oracle.hexhash(oracle.conv2d(x, w, shape, S)) == rec["forward"]
        assert oracle.hexhash(oracle.conv2d_grad_weight(dy, x, shape, S)) == rec["grad_weight"]
        assert oracle.hexhash(oracle.conv2d_grad_input(dy, w, shape, S)) == rec["grad_input"]


def test_oracle_convolutions_against_reference_library():
    if oracle.ref_conv() is None:
        pytest.skip("oracle/_ref/librepro_ref_conv.so not built (reference sources absent)")
    rng = np.random.default_rng(5)
    for _ in range(12):
        N, C, F = (int(v) for v in rng.integers(1, 5, size=3))
        KH, KW, SY, SX = (int(v) for v in rng.integers(1, 4, size=4))
        PY, PX = (int(v) for v in rng.integers(0, 3, size=2))
        H, W = KH + int(rng.integers(0, 9)), KW + int(rng.integers(0, 9))
        shape = (N, C, H, W, F, KH, KW, SY, SX, PY, PX)
        x, w, dy = fx.conv_inputs(shape, "wide" if rng.random() < 0.5 else "normal", seed=int(rng.integers(1, 1 << 30)))
        for S in (1, 2, 3):
            assert np.array_equal(oracle.conv2d(x, w, shape, S).view(np.uint32), oracle.ref_conv2d(x, w, shape, S).view(np.uint32)), shape
            assert np.array_equal(oracle.conv2d_grad_weight(dy, x, shape, S).view(np.uint32),
                                  oracle.ref_conv2d_grad_weight(dy, x, shape, S).view(np.uint32)), shape
            assert np.array_equal(oracle.conv2d_grad_input(dy, w, shape, S).view(np.uint32),
                                  oracle.ref_conv2d_grad_input(dy, w, shape, S).view(np.uint32)), shape


def test_adjoint_identities_hold_to_rounding():
    """<dY, Y> = <dX, x> = <dW, W> up to the quantisation of the operands (the reference's own check
    of its gradients, repro_conv_cuda/README.md:19); the tolerance is relative to |dY| |Y|, since the
    inner product itself nearly cancels."""
    name, shape, dist = fx.CONV_CASES[3]
    x, w, dy = fx.conv_inputs(shape, dist)
    y = oracle.conv2d(x, w, shape, 3).astype(np.float64).reshape(-1)
    dw = oracle.conv2d_grad_weight(dy, x, shape, 3).astype(np.float64).reshape(-1)
    dx = oracle.conv2d_grad_input(dy, w, shape, 3).astype(np.float64).reshape(-1)
    a, b, c = float(dy.astype(np.float64) @ y), float(dx @ x.astype(np.float64)), float(dw @ w.astype(np.float64))
    scale = float(np.linalg.norm(dy.astype(np.float64)) * np.linalg.norm(y))
    assert abs(a - b) <= 1e-6 * scale and abs(a - c) <= 1e-6 * scale
