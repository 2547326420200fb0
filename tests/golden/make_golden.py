"""Generates the committed golden fixtures from the reference's own CPU code.

Run where the reference sources are mounted (they are compiled, in place, into oracle/_ref by
oracle/Makefile):

    python tests/golden/make_golden.py scalar        # tests/golden/scalar_vectors.json
    python tests/golden/make_golden.py gemm          # tests/golden/gemm_hashes.json (seconds to minutes)
    python tests/golden/make_golden.py c4            # adds the 16384^3 case (about ten minutes, 6 GiB)
    python tests/golden/make_golden.py conv          # tests/golden/conv_hashes.json

Every GEMM entry records the FNV-1a-64 of the inputs (A then B, chained) and of the output that
repro_gemm_cuda/repro_gemm_cpu.h:25 (cpu_gemm) produced for them, so a test can regenerate the
inputs from their seed, check that it has the same bits, and compare its result by hash.
"""
import json
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
import oracle  # noqa: E402
from bit_reproducible_training_b200 import fixtures as fx  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def f32_bits(x):
    return int(np.float32(x).view(np.uint32))


def scalar_vectors():
    R = oracle.ref()
    rng = np.random.default_rng(20240607)
    out = {"scale_exponent": [], "fixed_point": [], "round_to_float": []}

    m_bits = [0x00000000, 0x00000001, 0x0000007F, 0x00000080, 0x00800000, 0x3C23D70A, 0x3F800000, 0x42FE0000,
              0x42FE0001, 0x42FF0000, 0x437E0000, 0x437E0001, 0x49742400, 0x7F7FFFFF, 0x3B810204, 0x3B810205,
              0x007FFFFF, 0x00000100, 0x000000FE, 0x000000FF, 0x3F7FFFFF, 0x40000000]
    m_bits += [int(b) for b in rng.integers(0, 0x7F800000, size=2000)]
    m_bits += [int(b) for b in rng.integers(0, 0x00010000, size=500)]          # deep subnormals
    m_bits += [f32_bits(127.0 * 2.0 ** e) for e in range(-140, 100, 7)]           # exact powers of two after /127
    for b in m_bits:
        m = np.uint32(b).view(np.float32)
        out["scale_exponent"].append([b, int(R.ref_scale_exponent(float(m)))])

    fp_cases = [(0x3F800000, -6), (0xBF800000, -6), (0x3EAAAAAB, -6), (0x3DCCCCCD, -6), (0x3C23D70A, -12),
                (0x42FE0000, 0), (0xC2FE0000, 0), (0x3F7FFFFF, -6), (0x33800000, -6), (0x00000001, -149),
                (0x80000040, -149), (0x7F7FFFFF, 122), (0x3F000000, 0), (0x3FC00000, 0), (0x40200000, 0),
                (0xBF000000, 0), (0x00000000, 0), (0x80000000, 5)]
    for _ in range(3000):
        se = int(rng.integers(-149, 123))
        # a value whose magnitude is at most about 127 * 2^se, as the row maximum guarantees
        mag = rng.random() * 127.0 * 2.0 ** se * (2.0 ** -int(rng.integers(0, 30)))
        x = np.float32(mag if rng.random() < 0.5 else -mag)
        if np.isfinite(x):
            fp_cases.append((f32_bits(x), se))
    for b, se in fp_cases:
        x = float(np.uint32(b).view(np.float32))
        out["fixed_point"].append([b, se] + [int(R.ref_fixed_point(x, se, S)) for S in (1, 2, 3)])

    rt_cases = [(0, 0), (1, 0), (-1, 0), (16777216, 0), (16777217, 0), (16777218, 0), (16777219, 0), (-16777219, 0),
                (33554434, 0), (33554438, 0), (1 << 62, -62), ((1 << 62) + (1 << 38), -62),
                ((1 << 62) + (1 << 38) + 1, -62), (-(1 << 62), -28), (1, -149), (1, -150), (3, -151), (2, -151),
                (6, -152), (5, -152), (-5, -152), (-1, -151), (16777215, -173), (16777215, 104), (16777216, 104),
                (4294967167, 96), (4294967168, 96), (-4294967168, 96), (1, 127), (1, 128), (-1, 244),
                (123456789012345678, -80), (-987654321098765, -326), (4611686018427387903, -326)]
    for _ in range(6000):
        bits = int(rng.integers(1, 63))
        T = int(rng.integers(0, 1 << bits))
        if rng.random() < 0.3:      # force ties and near-ties at the 24-bit boundary
            T = (T | 1) << int(rng.integers(0, 38))
            T = min(T, (1 << 62))
        if rng.random() < 0.5:
            T = -T
        E = int(rng.integers(-326, 245))
        if rng.random() < 0.4:      # concentrate on the subnormal and overflow edges
            p = max(abs(T), 1).bit_length() - 1
            E = int(rng.choice([-126, -149, -150, -127, 127, 128, 104])) - p + int(rng.integers(-3, 4))
            E = max(-326, min(244, E))
        rt_cases.append((T, E))
    for T, E in rt_cases:
        out["round_to_float"].append([T, E, f32_bits(R.ref_round_to_float(T, E))])

    with open(os.path.join(HERE, "scalar_vectors.json"), "w") as f:
        json.dump(out, f, separators=(",", ":"))
    print("scalar vectors:", {k: len(v) for k, v in out.items()})


def entry(name, A, B, M, N, K, ta, tb, S, recipe, batch=1):
    """One GEMM (or `batch` back-to-back GEMMs) through the reference; returns the JSON record."""
    outs = []
    for b in range(batch):
        a = A[b * M * K:(b + 1) * M * K]
        bb = B[b * K * N:(b + 1) * K * N]
        outs.append(oracle.ref_gemm(a, bb, M, N, K, ta, tb, S))
    Cm = np.concatenate([o.reshape(-1) for o in outs])
    rec = dict(name=name, M=M, N=N, K=K, trans_a=bool(ta), trans_b=bool(tb), S=S, batch=batch, recipe=recipe,
               in_hash="%016x" % oracle.fnv1a64(B, oracle.fnv1a64(A)), out_hash=oracle.hexhash(Cm))
    print(rec, flush=True)
    return rec, Cm


def transposed(A, rows, cols):
    return np.ascontiguousarray(A.reshape(rows, cols).T).reshape(-1)


def gemm_hashes(path):
    recs = []
    # configuration 1
    c = fx.config1()[0]
    for S in (1, 2, 3):
        recs.append(entry("c1.512", c["A"], c["B"], 512, 512, 512, False, False, S, "config1()")[0])
    # the reference's ragged correctness shape, every transposition (all must equal the plain result)
    A, B = fx.ragged_test_inputs()
    M, N, K = 133, 77, 301
    for S in (1, 2, 3):
        base, _ = entry("ragged.133x77x301", A, B, M, N, K, False, False, S, "ragged_test_inputs()")
        recs.append(base)
    # the hash tool's shapes and distributions
    for (M, N, K) in ((256, 256, 1024), (129, 77, 1000), (64, 64, 7)):
        for dist in ("uniform", "normal", "weights", "wide", "stress"):
            A, B = fx.hash_tool_inputs(dist, M, N, K)
            for S in (1, 3):
                recs.append(entry("hash.%s.%dx%dx%d" % (dist, M, N, K), A, B, M, N, K, False, False, S,
                                  "hash_tool_inputs(%r,%d,%d,%d)" % (dist, M, N, K))[0])
    # configuration 2: the linear-layer triple at 8192 tokens
    for c in fx.config2():
        recs.append(entry(c["name"], c["A"], c["B"], c["M"], c["N"], c["K"], c["trans_a"], c["trans_b"], 3,
                          "config2()")[0])
    # configuration 3: wide dynamic range, S = 1, 2, 3 (also at 1024 for quick checks)
    for n in (1024, 4096):
        c = fx.config3(n)[0]
        for S in (1, 2, 3):
            recs.append(entry(c["name"], c["A"], c["B"], n, n, n, False, False, S, "config3(%d)" % n)[0])
    # configuration 5: strided-batched attention shapes (also a 4-batch cut for quick checks)
    for batch in (4, 96):
        for c in fx.config5(batch):
            recs.append(entry("%s.b%d" % (c["name"], batch), c["A"], c["B"], c["M"], c["N"], c["K"], c["trans_a"],
                              c["trans_b"], 3, "config5(%d)" % batch, batch=batch)[0])
    # uniform squares used by the scaling tests
    for n in (2048,):
        c = fx.config4(n)[0]
        recs.append(entry(c["name"], c["A"], c["B"], n, n, n, False, False, 3, "config4(%d)" % n)[0])
    with open(path, "w") as f:
        json.dump(recs, f, indent=0)


def c4(path):
    recs = json.load(open(path))
    recs = [r for r in recs if r["name"] != "c4.16384"]
    c = fx.config4()[0]
    n = 16384
    rec, Cm = entry("c4.16384", c["A"], c["B"], n, n, n, False, False, 3, "config4()")
    # per-row-block hashes let a row-sharded run check its own slice without the whole matrix
    Cm = Cm.reshape(n, n)
    rec["row_block_hashes"] = {"rows": 2048, "hashes": [oracle.hexhash(Cm[i:i + 2048]) for i in range(0, n, 2048)]}
    recs.append(rec)
    with open(path, "w") as f:
        json.dump(recs, f, indent=0)


def kcat(path):
    """Configuration 3's operands repeated w times along K (A = [A0 A0 ...], B = [B0; B0; ...]): the product a
    K-sharded run forms when each of w ranks holds one K range.  Appends records c3.4096.kcat<w>."""
    recs = [r for r in json.load(open(path)) if ".kcat" not in r["name"]]
    n = 4096
    c = fx.config3(n)[0]
    A0, B0 = c["A"].reshape(n, n), c["B"].reshape(n, n)
    for w in (2, 4, 8):
        A = np.ascontiguousarray(np.tile(A0, (1, w))).reshape(-1)
        B = np.ascontiguousarray(np.tile(B0, (w, 1))).reshape(-1)
        recs.append(entry("c3.4096.kcat%d" % w, A, B, n, n, n * w, False, False, 3, "config3(4096) tiled %d times along K" % w)[0])
    with open(path, "w") as f:
        json.dump(recs, f, indent=0)


def conv_hashes():
    """Forward, weight-gradient and input-gradient hashes from repro_conv_cuda/repro_conv_cpu.h:25,45,72."""
    recs = []
    for name, shape, dist in fx.CONV_CASES:
        x, w, dy = fx.conv_inputs(shape, dist)
        for S in (1, 2, 3):
            rec = dict(name=name, shape=list(shape), dist=dist, S=S,
                       in_hash="%016x" % oracle.fnv1a64(dy, oracle.fnv1a64(w, oracle.fnv1a64(x))),
                       forward=oracle.hexhash(oracle.ref_conv2d(x, w, shape, S)),
                       grad_weight=oracle.hexhash(oracle.ref_conv2d_grad_weight(dy, x, shape, S)),
                       grad_input=oracle.hexhash(oracle.ref_conv2d_grad_input(dy, w, shape, S)))
            print(rec, flush=True)
            recs.append(rec)
    with open(os.path.join(HERE, "conv_hashes.json"), "w") as f:
        json.dump(recs, f, indent=0)


if __name__ == "__main__":
    what = sys.argv[1] if len(sys.argv) > 1 else "all"
    oracle.build()
    if oracle.ref() is None:
        sys.exit("the reference library oracle/_ref/librepro_ref.so could not be built here")
    path = os.path.join(HERE, "gemm_hashes.json")
    if what in ("scalar", "all"):
        scalar_vectors()
    if what in ("gemm", "all"):
        gemm_hashes(path)
    if what == "c4":
        c4(path)
    if what == "kcat":
        kcat(path)
    if what in ("conv", "all"):
        if oracle.ref_conv() is None:
            sys.exit("the reference library oracle/_ref/librepro_ref_conv.so could not be built here")
        conv_hashes()
