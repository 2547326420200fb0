"""Edge cases of the GPU path: degenerate and ragged sizes, misaligned pointers, zeros, extreme
magnitudes, results that underflow or overflow.  Everything is compared bit for bit with the oracle."""
import numpy as np
import pytest
import torch

import oracle
from bit_reproducible_training_b200 import fixtures as fx
from bit_reproducible_training_b200 import repro_gemm as rg

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def check(A, B, M, N, K, ta=False, tb=False, S=3, split_k=1):
    got = rg.gemm(dev(A), dev(B), M, N, K, ta, tb, S, split_k).cpu().numpy()
    want = oracle.gemm(A, B, M, N, K, ta, tb, S)
    bad = np.nonzero(got.view(np.uint32).reshape(-1) != want.view(np.uint32).reshape(-1))[0]
    assert len(bad) == 0, "M=%d N=%d K=%d ta=%d tb=%d S=%d: %d differ, first at %d (%r vs %r)" % (
        M, N, K, ta, tb, S, len(bad), bad[0], got.reshape(-1)[bad[0]], want.reshape(-1)[bad[0]])
    return got


@pytest.mark.parametrize("shape", [(1, 1, 1), (1, 1, 129), (1, 300, 5), (300, 1, 5), (2, 3, 4), (127, 63, 127),
                                   (128, 64, 128), (129, 65, 129), (257, 130, 1), (5, 4099, 33), (4099, 5, 33),
                                   (64, 64, 4097), (100, 100, 515)])
def test_degenerate_and_ragged_shapes(shape):
    M, N, K = shape
    g = fx.Rng(M * 1000003 + N * 1009 + K)
    A, B = g.normal(M * K), g.wide(K * N, -8, 8)
    for S in (1, 2, 3):
        for ta, tb in ((False, False), (True, True)):
            a = np.ascontiguousarray(A.reshape(M, K).T).reshape(-1) if ta else A
            b = np.ascontiguousarray(B.reshape(K, N).T).reshape(-1) if tb else B
            check(a, b, M, N, K, ta, tb, S)


def test_misaligned_pointers_and_output():
    """A, B and C start 4, 8 or 12 bytes past a 16-byte boundary: the vector paths must step aside."""
    M, N, K = 200, 136, 264            # all multiples of 4, so only the base pointers are misaligned
    g = fx.Rng(808)
    A, B = g.normal(M * K), g.normal(K * N)
    want = oracle.gemm(A, B, M, N, K)
    for off in (1, 2, 3):
        bufA = torch.zeros(M * K + 8, device="cuda")
        bufB = torch.zeros(K * N + 8, device="cuda")
        bufC = torch.full((M * N + 8,), float("nan"), device="cuda")
        bufA[off:off + M * K] = dev(A)
        bufB[off:off + K * N] = dev(B)
        for ta, tb, a, b in ((False, False, A, B),
                             (True, True, np.ascontiguousarray(A.reshape(M, K).T).reshape(-1),
                              np.ascontiguousarray(B.reshape(K, N).T).reshape(-1))):
            bufA[off:off + M * K] = dev(a)
            bufB[off:off + K * N] = dev(b)
            cfg = rg.Config(trans_a=ta, trans_b=tb)
            rc, plan = rg.make_plan(M, N, K, cfg)
            ws = torch.empty(plan.workspace_bytes, dtype=torch.uint8, device="cuda")
            bufC.fill_(float("nan"))
            assert rg.repro_gemm_fp32_ws(bufA[off:], bufB[off:], bufC[off:], M, N, K, cfg, ws) == 0
            torch.cuda.synchronize()
            out = bufC.cpu().numpy()
            assert np.array_equal(out[off:off + M * N].view(np.uint32), want.view(np.uint32).reshape(-1)), (off, ta, tb)
            assert np.isnan(out[:off]).all() and np.isnan(out[off + M * N:]).all()       # nothing written outside C


def test_zeros_signed_zeros_and_zero_rows():
    M, N, K = 70, 90, 300
    A = np.zeros(M * K, dtype=np.float32)
    B = fx.Rng(3).normal(K * N)
    got = check(A, B, M, N, K)
    assert (got.view(np.uint32) == 0).all()                 # exact zero sums give +0, never -0
    A = np.where(np.arange(M * K) % 2 == 0, np.float32(-0.0), np.float32(0.0)).astype(np.float32)
    got = check(A, B, M, N, K)
    assert (got.view(np.uint32) == 0).all()
    A = fx.Rng(4).normal(M * K)
    A.reshape(M, K)[::3] = 0.0                                # zero rows next to ordinary rows
    Bz = B.copy()
    Bz.reshape(K, N)[:, ::4] = 0.0                            # zero columns
    check(A, Bz, M, N, K)


def test_extreme_magnitudes_overflow_and_underflow():
    M, N, K = 96, 80, 260
    g = fx.Rng(99)
    # rows of A near FLT_MAX against columns of B of ordinary size: finite inputs, results overflow to +-inf
    A = g.normal(M * K)
    A.reshape(M, K)[::2] *= np.float32(3e37)
    B = g.normal(K * N)
    B.reshape(K, N)[:, ::2] *= np.float32(10.0)
    got = check(A, B, M, N, K)
    assert np.isinf(got).any() and np.isfinite(got).any()
    # subnormal inputs and subnormal / underflowing results
    A = np.ldexp(g.normal64(M * K), -140).astype(np.float32)
    B = np.ldexp(g.normal64(K * N), -5).astype(np.float32)
    got = check(A, B, M, N, K)
    assert ((np.abs(got) < 1.2e-38) & (got != 0)).any()       # some outputs are subnormal
    A = np.ldexp(g.normal64(M * K), -120).astype(np.float32)
    B = np.ldexp(g.normal64(K * N), -60).astype(np.float32)
    got = check(A, B, M, N, K)
    assert (got == 0).all() and (got.view(np.uint32) == 0x80000000).any()    # negative underflow keeps its sign
    # largest finite inputs everywhere
    A = np.full(M * K, np.finfo(np.float32).max, dtype=np.float32)
    B = np.full(K * N, -np.finfo(np.float32).max, dtype=np.float32)
    got = check(A, B, M, N, K)
    assert np.isneginf(got).all()


def test_one_outlier_per_row_and_column():
    """A single huge element fixes the scale of its row: every other element rounds to a few bits or to zero."""
    M, N, K = 133, 77, 301
    A, B = fx.ragged_test_inputs(M, N, K)
    A = A.copy()
    B = B.copy()
    A.reshape(M, K)[np.arange(M), np.arange(M) % K] = np.float32(1e20)
    B.reshape(K, N)[np.arange(N) % K, np.arange(N)] = np.float32(-1e-20)
    for S in (1, 2, 3):
        check(A, B, M, N, K, S=S)


def test_batched_ragged_shapes():
    batch, M, N, K = 5, 131, 67, 200
    g = fx.Rng(606)
    A, B = g.normal(batch * M * K), g.normal(batch * K * N)
    for ta, tb in ((False, False), (True, False), (False, True)):
        out = rg.gemm_batched(dev(A), dev(B), batch, M, N, K, ta, tb, 3).cpu().numpy()
        for b in range(batch):
            want = oracle.gemm(A[b * M * K:(b + 1) * M * K], B[b * K * N:(b + 1) * K * N], M, N, K, ta, tb, 3)
            assert np.array_equal(out[b].view(np.uint32), want.view(np.uint32)), (b, ta, tb)


def test_batched_with_k_ranges_and_every_slice_count():
    """Batches, explicit K ranges (INT64 partials per batch and range) and padded strides together."""
    batch, M, N, K = 4, 140, 200, 700
    g = fx.Rng(707)
    sa, sb, sc = M * K + 8, K * N + 4, M * N + 12
    A, B = g.normal(batch * sa), g.wide(batch * sb, -6, 6)
    dA, dB = dev(A), dev(B)
    for S in (1, 2, 3):
        for split in (1, 3):
            cfg = rg.Config(slices=S, split_k=split)
            rc, plan = rg.make_plan(M, N, K, cfg, batch=batch)
            assert rc == 0 and plan.split_k == split
            ws = torch.empty(plan.workspace_bytes, dtype=torch.uint8, device="cuda")
            out = torch.full((batch * sc,), float("nan"), device="cuda")
            assert rg.repro_gemm_fp32_batched_ws(dA, dB, out, M, N, K, batch, sa, sb, sc, cfg, ws) == 0
            torch.cuda.synchronize()
            o = out.cpu().numpy()
            for b in range(batch):
                want = oracle.gemm(A[b * sa:b * sa + M * K], B[b * sb:b * sb + K * N], M, N, K, S=S)
                assert np.array_equal(o[b * sc:b * sc + M * N].view(np.uint32), want.view(np.uint32).reshape(-1)), (S, split, b)
                assert np.isnan(o[b * sc + M * N:(b + 1) * sc]).all()


def test_k_strided_operands_longer_than_the_grid_limit():
    """K above 65535 x 64: the column-maximum pass of a k-strided operand cannot give every 64-k chunk a CTA of
    its own along grid.y and has to walk them; both operands are k-strided here (A transposed, B not)."""
    M, N, K = 16, 16, 65535 * 64 + 777
    g = fx.Rng(4242)
    A, B = g.normal(M * K), g.normal(K * N)
    At = np.ascontiguousarray(A.reshape(M, K).T).reshape(-1)
    check(At, B, M, N, K, True, False, 1)
