"""Pins the CPU oracle (oracle/oracle.c) before anything is checked against it.

Sources of truth, all produced by the reference's own code:
  * tests/golden/scalar_vectors.json  - repro_gemm_math.cuh's scale_exponent / fixed_point / round_to_float
  * tests/golden/gemm_hashes.json     - cpu_gemm (repro_gemm_cpu.h:25) output hashes for seeded inputs
  * the FNV-1a-64 hashes the reference commits for its conformance suite
    (gpt2_ops_suite/results/mac/cpu.txt:2-22, identical in all its result files), restated below
  * oracle/_ref (the reference's cpu_gemm compiled from its sources), where present
"""
import numpy as np
import pytest

import oracle
from bit_reproducible_training_b200 import fixtures as fx

# name -> (input hash, output hash) at tokens = 1024, S = 3, as committed by the reference
SUITE_HASHES = {
    "attn_qkv.fwd": ("f717589d12c07658", "0694c9bba1a03388"),
    "attn_qkv.dX": ("1def0bbe8aa4626e", "4403cea1ec942a80"),
    "attn_qkv.dW": ("4cf53ab57e3ce5ab", "014bb47372fe46df"),
    "attn_proj.fwd": ("46dd3a91b61dc793", "2ad24a70eb9b78a4"),
    "attn_proj.dX": ("a47a950cdbdbad69", "7965e353dbd38c2b"),
    "attn_proj.dW": ("8875bcd8658fbce5", "41796587ec48e228"),
    "mlp_fc.fwd": ("fdae6f3970f3fe8b", "4078a224b3834789"),
    "mlp_fc.dX": ("d057b521131a9f2c", "a69e67f97ebfb1cd"),
    "mlp_fc.dW": ("d7077130e5007894", "0f81482aaee505a0"),
    "mlp_proj.fwd": ("4852be59efa2ee0a", "5f3e342869c293a3"),
    "mlp_proj.dX": ("71dc25c7240fbde6", "48d8a391ce9d2bb3"),
    "mlp_proj.dW": ("e741de491c78c56a", "e0147ab9ccbd914a"),
    "lm_head.fwd": ("b265644b15ea5c6e", "f8779013fd9bc98e"),
    "lm_head.dX": ("91d5f60ef9811d69", "df619a9df0ddc2ae"),
    "lm_head.dW": ("d47d89b75a0d5d91", "041cc60891e7c1ef"),
    "attn_head.scores QK^T": ("5583f430f0a27d10", "ea40462e9fd9a0ee"),
    "attn_head.PV": ("a51050319f40a2a8", "e4930c3f6bba0f08"),
    "attn_head.dP = dO V^T": ("cba8e43dcd4f8afa", "dfc5ed268bb253b7"),
    "attn_head.dV = P^T dO": ("1a057d6d2ce2411d", "915aa015fe5cbe02"),
    "attn_head.dQ = dS K": ("fda2db40fb04de38", "5154b62e4776d7d7"),
    "attn_head.dK = dS^T Q": ("4060ea8764645983", "6a48b39e45a17b10"),
}


def f32(bits):
    return float(np.uint32(bits).view(np.float32))


def test_scale_exponent_vectors(scalar_vectors):
    L = oracle.lib()
    for bits, want in scalar_vectors["scale_exponent"]:
        assert L.orc_scale_exponent(f32(bits)) == want, hex(bits)


def test_fixed_point_vectors(scalar_vectors):
    L = oracle.lib()
    for bits, se, x1, x2, x3 in scalar_vectors["fixed_point"]:
        got = [L.orc_fixed_point(f32(bits), se, S) for S in (1, 2, 3)]
        assert got == [x1, x2, x3], (hex(bits), se)


def test_round_to_float_vectors(scalar_vectors):
    L = oracle.lib()
    for T, E, want in scalar_vectors["round_to_float"]:
        assert L.orc_round_to_float_bits(T, E) == want, (T, E)


def test_digits_are_an_exact_balanced_split():
    L = oracle.lib()
    import ctypes as C
    rng = np.random.default_rng(5)
    for S in (1, 2, 3):
        lim = 127 << (7 * (S - 1))
        xs = list(rng.integers(-lim, lim + 1, size=4000)) + [lim, -lim, lim - 1, -lim + 1, 0, 63, 64, -64, -65]
        for X in xs:
            d = (C.c_int8 * 3)()
            L.orc_digits(int(X), S, d)
            assert sum(int(d[p]) * 128 ** (S - 1 - p) for p in range(S)) == X
            assert abs(d[0]) <= 127 and all(-64 <= d[p] <= 63 for p in range(1, S))


def test_scalar_functions_against_reference_library():
    R = oracle.ref()
    if R is None:
        pytest.skip("oracle/_ref not built on this machine")
    L = oracle.lib()
    rng = np.random.default_rng(99)
    for bits in rng.integers(0, 0x7F800000, size=20000):
        m = f32(int(bits))
        assert L.orc_scale_exponent(m) == R.ref_scale_exponent(m)
    for _ in range(20000):
        T = int(rng.integers(-(1 << 62), 1 << 62)) >> int(rng.integers(0, 62))
        E = int(rng.integers(-326, 245))
        want = int(np.float32(R.ref_round_to_float(T, E)).view(np.uint32))
        assert L.orc_round_to_float_bits(T, E) == want, (T, E)


@pytest.mark.parametrize("name", [n for n in SUITE_HASHES if not n.startswith("lm_head")])
def test_committed_suite_hashes(name):
    """Inputs from the numpy SplitMix64 fixture and outputs from the oracle reproduce the hashes the
    reference commits for its GPT-2-shaped GEMM operations."""
    op = [o for o in fx.suite_gemm_ops(1024) if o[0] == name][0]
    A, B = fx.suite_inputs(op)
    assert "%016x" % oracle.fnv1a64(B, oracle.fnv1a64(A)) == SUITE_HASHES[name][0]
    C = oracle.gemm(A, B, op[1], op[2], op[3], op[4], op[5], 3)
    assert oracle.hexhash(C) == SUITE_HASHES[name][1]


def test_committed_suite_hash_ragged_vocab():
    """lm_head.dW: M = 50257 (ragged), A^T; the largest-M case of the suite."""
    op = [o for o in fx.suite_gemm_ops(1024) if o[0] == "lm_head.dW"][0]
    A, B = fx.suite_inputs(op)
    assert "%016x" % oracle.fnv1a64(B, oracle.fnv1a64(A)) == SUITE_HASHES["lm_head.dW"][0]
    C = oracle.gemm(A, B, op[1], op[2], op[3], op[4], op[5], 3)
    assert oracle.hexhash(C) == SUITE_HASHES["lm_head.dW"][1]


SMALL_GOLDEN = [("c1.512", 1), ("c1.512", 2), ("c1.512", 3), ("ragged.133x77x301", 1), ("ragged.133x77x301", 2),
                ("ragged.133x77x301", 3), ("c3.1024", 1), ("c3.1024", 2), ("c3.1024", 3)]


@pytest.mark.parametrize("name,S", SMALL_GOLDEN)
def test_oracle_matches_golden_hashes(name, S, golden):
    rec = golden[(name, S)]
    if name.startswith("c1"):
        c = fx.config1()[0]
        A, B = c["A"], c["B"]
    elif name.startswith("ragged"):
        A, B = fx.ragged_test_inputs()
    else:
        c = fx.config3(1024)[0]
        A, B = c["A"], c["B"]
    assert "%016x" % oracle.fnv1a64(B, oracle.fnv1a64(A)) == rec["in_hash"]
    C = oracle.gemm(A, B, rec["M"], rec["N"], rec["K"], rec["trans_a"], rec["trans_b"], S)
    assert oracle.hexhash(C) == rec["out_hash"]


@pytest.mark.parametrize("dist", ["uniform", "normal", "weights", "wide", "stress"])
def test_oracle_matches_golden_on_hash_tool_distributions(dist, golden):
    for (M, N, K) in ((129, 77, 1000), (64, 64, 7)):
        A, B = fx.hash_tool_inputs(dist, M, N, K)
        for S in (1, 3):
            rec = golden[("hash.%s.%dx%dx%d" % (dist, M, N, K), S)]
            assert "%016x" % oracle.fnv1a64(B, oracle.fnv1a64(A)) == rec["in_hash"]
            assert oracle.hexhash(oracle.gemm(A, B, M, N, K, S=S)) == rec["out_hash"]


def test_batched_golden_is_per_batch_gemm(golden):
    for c in fx.config5(4):
        rec = golden[("%s.b4" % c["name"], 3)]
        M, N, K = c["M"], c["N"], c["K"]
        outs = [oracle.gemm(c["A"][b * M * K:(b + 1) * M * K], c["B"][b * K * N:(b + 1) * K * N], M, N, K,
                            c["trans_a"], c["trans_b"], 3) for b in range(4)]
        assert oracle.hexhash(np.concatenate([o.reshape(-1) for o in outs])) == rec["out_hash"]


def test_transposed_storage_gives_the_same_bits():
    M, N, K = 45, 37, 130
    A, B = fx.ragged_test_inputs(M, N, K)
    At = np.ascontiguousarray(A.reshape(M, K).T).reshape(-1)
    Bt = np.ascontiguousarray(B.reshape(K, N).T).reshape(-1)
    base = oracle.gemm(A, B, M, N, K, S=3)
    for a, b, ta, tb in ((At, B, True, False), (A, Bt, False, True), (At, Bt, True, True)):
        assert np.array_equal(oracle.gemm(a, b, M, N, K, ta, tb, 3).view(np.uint32), base.view(np.uint32))


def test_k_ranges_sum_to_the_whole():
    """Partial sums over K ranges with shared scales, added and rounded once, equal the one-pass result."""
    M, N, K = 33, 29, 700
    A, B = fx.hash_tool_inputs("stress", M, N, K)
    maxA = oracle.absmax(A, M, K, False)
    maxB = oracle.absmax(B, N, K, True)
    for S in (1, 2, 3):
        parts = [oracle.gemm_partial(A, B, maxA, maxB, M, N, K, False, False, S, lo, hi)
                 for lo, hi in ((0, 100), (100, 101), (101, 700))]
        got = oracle.round_partials(np.stack(parts), maxA, maxB, M, N, S)
        want = oracle.gemm(A, B, M, N, K, S=S)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
