"""Bit-exact parity of the CUDA path (through the C ABI) with the CPU oracle and the golden hashes.

Mirrors the reference's own correctness tools: test_repro_gemm.cu (ragged shape, every S, split_k
values, all transpositions, poisoned output), hash_repro_gemm.cu / run_repro.sh (shapes and input
distributions, hash stability over split_k) and bench_repro_gemm.cu (every algorithm must equal the
verification kernel).
"""
import numpy as np
import pytest
import torch

import oracle
from bit_reproducible_training_b200 import fixtures as fx
from bit_reproducible_training_b200 import repro_gemm as rg

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def run(A, B, M, N, K, ta=False, tb=False, S=3, split_k=1, algo=rg.Algo.Auto):
    """One GEMM through repro_gemm_fp32_ws with a poisoned output and a poisoned workspace."""
    cfg = rg.Config(split_k=split_k, algo=algo, slices=S, trans_a=ta, trans_b=tb)
    rc, plan = rg.make_plan(M, N, K, cfg)
    assert rc == 0, rc
    ws = torch.full((plan.workspace_bytes,), 0xA5, dtype=torch.uint8, device="cuda")
    out = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
    rc = rg.repro_gemm_fp32_ws(dev(A), dev(B), out, M, N, K, cfg, ws)
    assert rc == 0, rc
    torch.cuda.synchronize()
    assert rg.workspace_status(ws) == 0
    return out.cpu().numpy()


def same_bits(x, y):
    return np.array_equal(np.asarray(x).view(np.uint32).reshape(-1), np.asarray(y).view(np.uint32).reshape(-1))


def first_diff(x, y):
    x = np.asarray(x).view(np.uint32).reshape(-1)
    y = np.asarray(y).view(np.uint32).reshape(-1)
    bad = np.nonzero(x != y)[0]
    return "%d differing of %d; first at %d: %08x vs %08x" % (len(bad), x.size, bad[0], x[bad[0]], y[bad[0]]) if len(bad) else "equal"


def transposed(A, rows, cols):
    return np.ascontiguousarray(A.reshape(rows, cols).T).reshape(-1)


@pytest.mark.parametrize("S", [1, 2, 3])
def test_config1_matches_oracle_and_golden(S, golden):
    c = fx.config1()[0]
    got = run(c["A"], c["B"], 512, 512, 512, S=S)
    want = oracle.gemm(c["A"], c["B"], 512, 512, 512, S=S)
    assert same_bits(got, want), first_diff(got, want)
    assert oracle.hexhash(got) == golden[("c1.512", S)]["out_hash"]


@pytest.mark.parametrize("S", [1, 2, 3])
@pytest.mark.parametrize("algo", [rg.Algo.TensorCore, rg.Algo.Reference])
def test_ragged_shape_splits_and_transposes(S, algo, golden):
    """The reference's test_repro_gemm.cu: 133 x 77 x 301, N(0,1) with a 1e6 outlier."""
    M, N, K = 133, 77, 301
    A, B = fx.ragged_test_inputs(M, N, K)
    At, Bt = transposed(A, M, K), transposed(B, K, N)
    want = oracle.gemm(A, B, M, N, K, S=S)
    assert oracle.hexhash(want) == golden[("ragged.133x77x301", S)]["out_hash"]
    for split in (1, 2, 3, 7, 64):
        for (a, b, ta, tb) in ((A, B, False, False), (A, B, False, False), (At, B, True, False),
                               (At, Bt, True, True), (A, Bt, False, True)):
            got = run(a, b, M, N, K, ta, tb, S, split, algo)
            assert same_bits(got, want), "S=%d split=%d ta=%d tb=%d: %s" % (S, split, ta, tb, first_diff(got, want))


def test_tiled_algo_is_reported_unsupported():
    rc, _ = rg.make_plan(64, 64, 64, rg.Config(algo=rg.Algo.Tiled))
    assert rc == rg.cudaErrorNotSupported


@pytest.mark.parametrize("shape,splits", [((256, 256, 1024), (1, 2, 3, 4, 7, 8, 16, 64)),
                                          ((129, 77, 1000), (1, 2, 3, 5, 7, 13, 64)),
                                          ((64, 64, 7), (1, 2, 3, 7, 16))])
@pytest.mark.parametrize("dist", ["uniform", "normal", "weights", "wide", "stress"])
@pytest.mark.parametrize("S", [1, 3])
def test_hash_tool_shapes(shape, splits, dist, S, golden):
    """run_repro.sh's shapes x distributions: identical bits for every split_k, equal to the oracle."""
    M, N, K = shape
    A, B = fx.hash_tool_inputs(dist, M, N, K)
    want = oracle.gemm(A, B, M, N, K, S=S)
    assert oracle.hexhash(want) == golden[("hash.%s.%dx%dx%d" % (dist, M, N, K), S)]["out_hash"]
    for split in splits:
        got = run(A, B, M, N, K, S=S, split_k=split)
        assert same_bits(got, want), "%s split=%d: %s" % (dist, split, first_diff(got, want))
