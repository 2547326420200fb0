"""Bit-exact parity of the two kernels for skinny products with the CPU oracle.

* short K (K <= 128, one k block): the epilogue-centred kernel with two accumulator sets (attention scores);
* narrow output (N <= 64) with a k-contiguous A: A's split fused into the MMA kernel's producer (attention P V).
Both are chosen by the library from the shape alone; the cases below sit on and around the conditions that
select them (ragged edges, every slice count, transposed storage, batches with padded strides, rows of
zeros and of subnormal magnitude, unaligned operands that must fall back to the general path).
The reference lists these batched attention products as pending (gpt2_ops_suite/gpt2_ops_suite.cu:543-548);
its per-matrix definition (repro_gemm_cuda/repro_gemm_cpu.h:25) is what the oracle restates.
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


def transposed(A, rows, cols):
    return np.ascontiguousarray(A.reshape(rows, cols).T).reshape(-1)


def run(A, B, M, N, K, ta=False, tb=False, S=3):
    cfg = rg.Config(slices=S, trans_a=ta, trans_b=tb)
    rc, plan = rg.make_plan(M, N, K, cfg)
    assert rc == 0, rc
    ws = torch.full((plan.workspace_bytes,), 0xA5, dtype=torch.uint8, device="cuda")
    out = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
    assert rg.repro_gemm_fp32_ws(dev(A), dev(B), out, M, N, K, cfg, ws) == 0
    torch.cuda.synchronize()
    assert rg.workspace_status(ws) == 0
    return out.cpu().numpy()


def check(got, want, what):
    g, w = got.view(np.uint32).reshape(-1), want.view(np.uint32).reshape(-1)
    bad = np.nonzero(g != w)[0]
    assert len(bad) == 0, "%s: %d of %d differ, first at %d: %08x vs %08x" % (what, len(bad), g.size, bad[0], g[bad[0]], w[bad[0]])


@pytest.mark.parametrize("S", [1, 2, 3])
@pytest.mark.parametrize("shape", [(133, 77, 64), (300, 200, 100), (129, 1000, 128), (64, 64, 7), (1, 1, 1),
                                   (513, 33, 31), (128, 32, 32), (1024, 1024, 64), (257, 4100, 96),
                                   (40, 8, 64), (200, 20, 100), (130, 44, 64)])   # N below one store box, and a clipped second box
def test_short_k_every_transposition(shape, S):
    M, N, K = shape
    g = fx.Rng(1000 + M + N + K)
    A, B = g.wide(M * K, -8, 8), g.normal(K * N)
    want = oracle.gemm(A, B, M, N, K, S=S)
    At, Bt = transposed(A, M, K), transposed(B, K, N)
    for a, b, ta, tb in ((A, B, False, False), (A, Bt, False, True), (At, B, True, False), (At, Bt, True, True)):
        check(run(a, b, M, N, K, ta, tb, S), want, "%s S=%d ta=%d tb=%d" % (shape, S, ta, tb))


@pytest.mark.parametrize("S", [1, 2, 3])
@pytest.mark.parametrize("shape", [(300, 64, 1000), (200, 17, 260), (1024, 64, 1024), (129, 1, 132), (128, 33, 4096),
                                   (1000, 48, 256), (77, 64, 10240)])
def test_narrow_output_with_fused_split_of_a(shape, S):
    M, N, K = shape
    g = fx.Rng(2000 + M + N + K)
    A, B = g.wide(M * K, -8, 8), g.normal(K * N)
    want = oracle.gemm(A, B, M, N, K, S=S)
    Bt = transposed(B, K, N)
    check(run(A, B, M, N, K, False, False, S), want, "%s S=%d" % (shape, S))
    check(run(A, Bt, M, N, K, False, True, S), want, "%s S=%d tb" % (shape, S))


def test_narrow_output_special_rows():
    """Rows of zeros, of subnormal magnitude (the two-factor scaling path), of huge magnitude, signed zeros and a
    single outlier, in a product that takes the fused split; plus exact zeros and subnormals sprinkled everywhere."""
    M, N, K = 256, 64, 512
    A, B = fx.hash_tool_inputs("stress", M, N, K)
    for S in (1, 2, 3):
        check(run(A, B, M, N, K, S=S), oracle.gemm(A, B, M, N, K, S=S), "stress S=%d" % S)
    g = fx.Rng(31)
    A, B = g.wide_mixed(M * K), g.wide_mixed(K * N)
    check(run(A, B, M, N, K), oracle.gemm(A, B, M, N, K), "wide_mixed")


def test_short_k_special_rows():
    M, N, K = 200, 150, 64
    A, B = fx.hash_tool_inputs("stress", M, N, K)
    for S in (1, 2, 3):
        check(run(A, B, M, N, K, S=S), oracle.gemm(A, B, M, N, K, S=S), "stress S=%d" % S)


def test_operands_the_fused_split_cannot_take_fall_back():
    """K not a multiple of four, or A not 16-byte aligned: the general path must give the same bits."""
    M, N = 260, 40
    g = fx.Rng(77)
    for K in (301, 514):
        A, B = g.normal(M * K), g.normal(K * N)
        check(run(A, B, M, N, K), oracle.gemm(A, B, M, N, K), "K=%d" % K)
    K = 512
    A, B = g.normal(M * K), g.normal(K * N)
    buf = torch.zeros(M * K + 1, dtype=torch.float32, device="cuda")
    buf[1:].copy_(torch.from_numpy(A))
    cfg = rg.Config()
    rc, plan = rg.make_plan(M, N, K, cfg)
    ws = torch.empty(plan.workspace_bytes, dtype=torch.uint8, device="cuda")
    out = torch.full((M, N), float("nan"), device="cuda")
    assert rg.repro_gemm_fp32_ws(buf[1:], dev(B), out, M, N, K, cfg, ws) == 0
    torch.cuda.synchronize()
    check(out.cpu().numpy(), oracle.gemm(A, B, M, N, K), "unaligned A")


@pytest.mark.parametrize("case", [(5, 131, 67, 64, False, True), (3, 300, 64, 520, False, False),
                                  (4, 129, 40, 260, False, True), (6, 64, 200, 17, True, False)])
def test_batched_with_padded_strides(case):
    batch, M, N, K, ta, tb = case
    g = fx.Rng(909 + M)
    sa, sb, sc = M * K + 8, K * N + 4, M * N + 12
    A, B = g.normal(batch * sa), g.wide(batch * sb, -6, 6)
    for S in (1, 3):
        cfg = rg.Config(slices=S, trans_a=ta, trans_b=tb)
        rc, plan = rg.make_plan(M, N, K, cfg, batch=batch)
        assert rc == 0
        ws = torch.full((plan.workspace_bytes,), 0x5A, dtype=torch.uint8, device="cuda")
        out = torch.full((batch * sc,), float("nan"), device="cuda")
        assert rg.repro_gemm_fp32_batched_ws(dev(A), dev(B), out, M, N, K, batch, sa, sb, sc, cfg, ws) == 0
        torch.cuda.synchronize()
        assert rg.workspace_status(ws) == 0
        o = out.cpu().numpy()
        for b in range(batch):
            want = oracle.gemm(A[b * sa:b * sa + M * K], B[b * sb:b * sb + K * N], M, N, K, ta, tb, S)
            check(o[b * sc:b * sc + M * N], want, "batch %d S=%d" % (b, S))
            assert np.isnan(o[b * sc + M * N:(b + 1) * sc]).all()


def test_attention_shapes_full_batch_by_golden_hash(golden):
    """Configuration 5 at its full size through the batched entry: 96 x (1024 x 1024 x 64) and 96 x (1024 x 64 x 1024)."""
    Q, Km, V, P = fx.config5_device("cuda")
    for name, A, B, M, N, K, tb in (("c5.QKt.b96", Q, Km, 1024, 1024, 64, True), ("c5.PV.b96", P, V, 1024, 64, 1024, False)):
        out = rg.gemm_batched(A, B, 96, M, N, K, False, tb, 3)
        assert "%016x" % rg.fnv1a64(out) == golden[(name, 3)]["out_hash"], name


@pytest.mark.parametrize("shape", [(64, 64, 30000), (256, 320, 20000), (512, 512, 12000), (300, 1000, 50000), (128, 36, 200),
                                   (72, 4100, 640)])
def test_single_read_split_of_k_strided_operands(shape):
    """The cluster form of the k-strided split at every panel width (32, 16 and 8 columns), at the longest K a slab
    holds and just beyond it (two-kernel form), for B and for a transposed A, with ragged last panels."""
    M, N, K = shape
    g = fx.Rng(4000 + M + N + K)
    A, B = g.wide(M * K, -6, 6), g.wide_mixed(K * N)
    for S in (1, 3):
        want = oracle.gemm(A, B, M, N, K, S=S)
        check(run(A, B, M, N, K, False, False, S), want, "%s S=%d" % (shape, S))
        check(run(transposed(A, M, K), B, M, N, K, True, False, S), want, "%s S=%d ta" % (shape, S))
