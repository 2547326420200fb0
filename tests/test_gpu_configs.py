"""The five benchmark configurations and the conformance-suite operations on the GPU, bit for bit.

Small cases are compared element-wise with the CPU oracle; full-size cases with the golden hashes
that the reference's cpu_gemm produced (tests/golden/gemm_hashes.json) and with the hashes the
reference itself commits (gpt2_ops_suite/results/*/cpu.txt), plus size-independent properties.
"""
import numpy as np
import pytest
import torch

import oracle
from bit_reproducible_training_b200 import fixtures as fx
from bit_reproducible_training_b200 import repro_gemm as rg
from test_oracle import SUITE_HASHES

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def bits(t):
    return t.detach().cpu().numpy().view(np.uint32).reshape(-1)


def gpu_gemm(c, S=3, split_k=1):
    return rg.gemm(dev(c["A"]), dev(c["B"]), c["M"], c["N"], c["K"], c["trans_a"], c["trans_b"], S, split_k)


@pytest.mark.parametrize("S", [1, 2, 3])
def test_config3_small_matches_oracle(S, golden):
    c = fx.config3(1024)[0]
    got = gpu_gemm(c, S).cpu().numpy()
    want = oracle.gemm(c["A"], c["B"], 1024, 1024, 1024, S=S)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    assert oracle.hexhash(got) == golden[("c3.1024", S)]["out_hash"]


@pytest.mark.parametrize("S", [1, 2, 3])
def test_config3_full_size_matches_golden(S, golden):
    c = fx.config3(4096)[0]
    rec = golden[("c3.4096", S)]
    assert "%016x" % oracle.fnv1a64(c["B"], oracle.fnv1a64(c["A"])) == rec["in_hash"]
    for split in (1, 4):
        assert oracle.hexhash(gpu_gemm(c, S, split).cpu().numpy()) == rec["out_hash"], "split_k=%d" % split


def test_config2_linear_layer_triple_matches_golden(golden):
    for c in fx.config2():
        rec = golden[(c["name"], 3)]
        assert "%016x" % oracle.fnv1a64(c["B"], oracle.fnv1a64(c["A"])) == rec["in_hash"]
        assert oracle.hexhash(gpu_gemm(c).cpu().numpy()) == rec["out_hash"], c["name"]


def test_config2_one_op_elementwise_against_oracle():
    c = fx.config2(1024)[1]          # dX at 1024 tokens: 1024 x 768 x 3072
    got = gpu_gemm(c).cpu().numpy()
    want = oracle.gemm(c["A"], c["B"], c["M"], c["N"], c["K"], c["trans_a"], c["trans_b"], 3)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("batch", [4, 96])
def test_config5_strided_batched(batch, golden):
    for c in fx.config5(batch):
        rec = golden[("%s.b%d" % (c["name"], batch), 3)]
        assert "%016x" % oracle.fnv1a64(c["B"], oracle.fnv1a64(c["A"])) == rec["in_hash"]
        out = rg.gemm_batched(dev(c["A"]), dev(c["B"]), batch, c["M"], c["N"], c["K"], c["trans_a"], c["trans_b"], 3)
        assert oracle.hexhash(out.cpu().numpy()) == rec["out_hash"], c["name"]
        if batch == 4:
            M, N, K = c["M"], c["N"], c["K"]
            for b in range(batch):       # each batch equals a plain call and the oracle
                a, bb = c["A"][b * M * K:(b + 1) * M * K], c["B"][b * K * N:(b + 1) * K * N]
                want = oracle.gemm(a, bb, M, N, K, c["trans_a"], c["trans_b"], 3)
                assert np.array_equal(bits(out[b]), want.view(np.uint32).reshape(-1))
                single = rg.gemm(dev(a), dev(bb), M, N, K, c["trans_a"], c["trans_b"], 3)
                assert np.array_equal(bits(single), bits(out[b]))


def test_batched_with_padded_strides():
    batch, M, N, K = 3, 70, 50, 200
    g = fx.Rng(77)
    sa, sb, sc = M * K + 64, K * N + 32, M * N + 16
    A, B = g.normal(batch * sa), g.normal(batch * sb)
    dA, dB = dev(A), dev(B)
    out = torch.full((batch * sc,), float("nan"), device="cuda")
    cfg = rg.Config()
    rc, plan = rg.make_plan(M, N, K, cfg, batch=batch)
    assert rc == 0
    ws = torch.empty(plan.workspace_bytes, dtype=torch.uint8, device="cuda")
    assert rg.repro_gemm_fp32_batched_ws(dA, dB, out, M, N, K, batch, sa, sb, sc, cfg, ws) == 0
    torch.cuda.synchronize()
    o = out.cpu().numpy()
    for b in range(batch):
        want = oracle.gemm(A[b * sa:b * sa + M * K], B[b * sb:b * sb + K * N], M, N, K)
        assert np.array_equal(o[b * sc:b * sc + M * N].view(np.uint32), want.view(np.uint32).reshape(-1))
        assert np.isnan(o[b * sc + M * N:(b + 1) * sc]).all()      # the gaps between matrices stay untouched


def test_config4_scaled_down_matches_golden(golden):
    c = fx.config4(2048)[0]
    rec = golden[("c4.2048", 3)]
    assert oracle.hexhash(gpu_gemm(c).cpu().numpy()) == rec["out_hash"]


def test_config4_full_size_hash_and_row_blocks(golden):
    """16384^3: the whole matrix against the golden hash; row blocks computed separately (the row
    sharding of the multi-GPU mode) give the same bits block by block."""
    rec = golden.get(("c4.16384", 3))
    if rec is None:
        pytest.skip("golden for 16384^3 not generated")
    n = 16384
    c = fx.config4(n)[0]
    dA, dB = dev(c["A"]), dev(c["B"])
    full = rg.gemm(dA, dB, n, n, n).cpu().numpy()
    assert oracle.hexhash(full) == rec["out_hash"]
    rows = rec["row_block_hashes"]["rows"]
    for i, want in enumerate(rec["row_block_hashes"]["hashes"]):
        assert oracle.hexhash(full[i * rows:(i + 1) * rows]) == want
    for i in (0, 5):
        block = rg.gemm(dA[i * rows * n:(i + 1) * rows * n], dB, rows, n, n).cpu().numpy()
        assert oracle.hexhash(block) == rec["row_block_hashes"]["hashes"][i]


@pytest.mark.parametrize("name", list(SUITE_HASHES))
def test_conformance_suite_hashes(name):
    """All 21 GEMM operations of the reference's GPT-2 conformance suite (tokens = 1024, S = 3),
    including the ragged vocabulary shapes (N, M or K = 50257)."""
    op = [o for o in fx.suite_gemm_ops(1024) if o[0] == name][0]
    A, B = fx.suite_inputs(op)
    assert "%016x" % rg.fnv1a64(B, rg.fnv1a64(A)) == SUITE_HASHES[name][0]
    out = rg.gemm(dev(A), dev(B), op[1], op[2], op[3], op[4], op[5], 3)
    assert "%016x" % rg.fnv1a64(out) == SUITE_HASHES[name][1]


def test_properties_at_full_size():
    """Size-independent properties on 4096^3 wide-range data: exact scaling by powers of two,
    invariance under a permutation of k, and row permutation equivariance."""
    n = 4096
    c = fx.config3(n)[0]
    A, B = dev(c["A"]).reshape(n, n), dev(c["B"]).reshape(n, n)
    base = rg.gemm(A, B, n, n, n)
    scaled = rg.gemm(A * 8.0, B * 0.25, n, n, n)             # |values| stay far from overflow and underflow ...
    finite = torch.isfinite(base) & (base.abs() > 1e-30) & (base.abs() < 1e30)
    assert torch.equal((base * 2.0)[finite], scaled[finite])   # ... so C scales exactly by 8 * 0.25
    perm = torch.randperm(n, device="cuda", generator=torch.Generator(device="cuda").manual_seed(1))
    assert torch.equal(rg.gemm(A[:, perm].contiguous(), B[perm].contiguous(), n, n, n).view(torch.int32),
                       base.view(torch.int32))
    assert torch.equal(rg.gemm(A[perm].contiguous(), B, n, n, n).view(torch.int32), base[perm].view(torch.int32))
    # transposed storage of either operand does not change a bit
    assert torch.equal(rg.gemm(A.t().contiguous(), B.t().contiguous(), n, n, n, True, True).view(torch.int32),
                       base.view(torch.int32))


def test_device_generated_operands_have_the_golden_input_hashes(golden):
    """The operands bench.py generates on the GPU carry the bits the golden outputs were computed from."""
    A, B = fx.config3_device("cuda", 4096)
    assert "%016x" % rg.fnv1a64(B, rg.fnv1a64(A)) == golden[("c3.4096", 3)]["in_hash"]
    A, B = fx.config4_device("cuda", 2048)
    assert "%016x" % rg.fnv1a64(B, rg.fnv1a64(A)) == golden[("c4.2048", 3)]["in_hash"]
    Q, Km, V, P = fx.config5_device("cuda", 4)
    assert "%016x" % rg.fnv1a64(Km, rg.fnv1a64(Q)) == golden[("c5.QKt.b4", 3)]["in_hash"]
    assert "%016x" % rg.fnv1a64(V, rg.fnv1a64(P)) == golden[("c5.PV.b4", 3)]["in_hash"]
