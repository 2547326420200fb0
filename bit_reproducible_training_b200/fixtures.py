"""Portable seeded inputs and the five benchmark configurations.

The reference generates every test input from a SplitMix64 stream using only exact integer-to-float
conversions, additions and ldexp, so the same seed gives the same input bits on every machine
(repro_gemm_cuda/repro_test_util.h:30-48; gpt2_ops_suite/gpt2_ops_suite.cu:59-76).  SplitMix64 is a
counter generator (state_i = seed + i * gamma), which lets numpy produce the identical stream in
vectorised chunks.  The distributions here reproduce the reference's draws one for one:

  u01          (next() >> 40) * 2^-24                       exact, in [0, 1)
  uniform_pm1  float32(2 * u01 - 1)
  normal       sum of 12 u01 minus 6 (exact in float64), times a scale, then float32
  wide         +-(1 + u01) * 2^e, e = lo + next() % (hi - lo + 1); draws: mantissa, exponent, sign
"""
import numpy as np

_GAMMA = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)
_CHUNK = 1 << 22


class Rng:
    """SplitMix64 stream; every method consumes draws in the reference's order."""

    def __init__(self, seed):
        self.state = int(seed) & 0xFFFFFFFFFFFFFFFF

    def next(self, n):
        """The next n raw 64-bit outputs."""
        idx = np.arange(1, n + 1, dtype=np.uint64)
        with np.errstate(over="ignore"):
            z = np.uint64(self.state) + idx * _GAMMA
            self.state = (self.state + n * int(_GAMMA)) & 0xFFFFFFFFFFFFFFFF
            z = (z ^ (z >> np.uint64(30))) * _M1
            z = (z ^ (z >> np.uint64(27))) * _M2
            return z ^ (z >> np.uint64(31))

    def _u01(self, n):
        return (self.next(n) >> np.uint64(40)).astype(np.float64) * (1.0 / 16777216.0)

    def _chunks(self, n, per_chunk):
        out = np.empty(n, dtype=np.float32)
        for lo in range(0, n, _CHUNK):
            hi = min(n, lo + _CHUNK)
            out[lo:hi] = per_chunk(hi - lo)
        return out

    def u01(self, n, scale=1.0):
        return self._chunks(n, lambda m: (scale * self._u01(m)).astype(np.float32))

    def uniform_pm1(self, n):
        return self._chunks(n, lambda m: (2.0 * self._u01(m) - 1.0).astype(np.float32))

    def normal(self, n, scale=1.0):
        def one(m):
            u = self._u01(12 * m).reshape(m, 12)
            t = np.zeros(m, dtype=np.float64)
            for i in range(12):          # same left-to-right order as the reference's loop
                t = t + u[:, i]
            return (scale * (t - 6.0)).astype(np.float32)
        return self._chunks(n, one)

    def normal64(self, n):
        """n standard-normal draws left in float64 (callers scale and round themselves)."""
        u = self._u01(12 * n).reshape(n, 12)
        t = np.zeros(n, dtype=np.float64)
        for i in range(12):
            t = t + u[:, i]
        return t - 6.0

    def range(self, lo, hi):
        """One integer in [lo, hi] from one draw."""
        return lo + int(self.next(1)[0] % np.uint64(hi - lo + 1))

    def weights(self, n):
        """N(0, 0.02) with 0.1 % outliers x100; per element 12 draws for the normal, then one for the
        outlier decision (repro_gemm_cuda/hash_repro_gemm.cu:30)."""
        def one(m):
            z = self.next(13 * m).reshape(m, 13)
            u = (z[:, :12] >> np.uint64(40)).astype(np.float64) * (1.0 / 16777216.0)
            t = np.zeros(m, dtype=np.float64)
            for i in range(12):
                t = t + u[:, i]
            v = 0.02 * (t - 6.0)
            return np.where(z[:, 12] % np.uint64(1000) == 0, v * 100.0, v).astype(np.float32)
        return self._chunks(n, one)

    def wide(self, n, elo, ehi):
        def one(m):
            z = self.next(3 * m).reshape(m, 3)
            mant = 1.0 + (z[:, 0] >> np.uint64(40)).astype(np.float64) * (1.0 / 16777216.0)
            e = elo + (z[:, 1] % np.uint64(ehi - elo + 1)).astype(np.int64)
            v = np.ldexp(mant, e.astype(np.int32))
            return np.where((z[:, 2] & np.uint64(1)) != 0, -v, v).astype(np.float32)
        return self._chunks(n, one)

    def wide_mixed(self, n, elo=-20, ehi=20):
        """Wide dynamic range with 1 % exact zeros and 0.1 % subnormals; four draws per element:
        r = next() % 1000, mantissa, exponent word w, sign.  r < 10 -> +0; r == 10 -> subnormal
        +-m * 2^(-149 + w % 23); otherwise +-m * 2^(elo + w % (ehi - elo + 1))."""
        def one(m):
            z = self.next(4 * m).reshape(m, 4)
            r = z[:, 0] % np.uint64(1000)
            mant = 1.0 + (z[:, 1] >> np.uint64(40)).astype(np.float64) * (1.0 / 16777216.0)
            e_norm = elo + (z[:, 2] % np.uint64(ehi - elo + 1)).astype(np.int64)
            e_sub = -149 + (z[:, 2] % np.uint64(23)).astype(np.int64)
            e = np.where(r == 10, e_sub, e_norm).astype(np.int32)
            v = np.ldexp(mant, e)
            v = np.where((z[:, 3] & np.uint64(1)) != 0, -v, v)
            return np.where(r < 10, 0.0, v).astype(np.float32)
        return self._chunks(n, one)

    def prob_rows(self, rows, cols):
        """Row-softmax-like matrix: u = u01 + 2^-25, row sum in float64 in index order, p = u / sum."""
        out = np.empty((rows, cols), dtype=np.float32)
        step = max(1, _CHUNK // cols)
        for lo in range(0, rows, step):
            hi = min(rows, lo + step)
            u = self._u01((hi - lo) * cols).reshape(hi - lo, cols) + 1.0 / 33554432.0
            s = np.zeros(hi - lo, dtype=np.float64)
            for c in range(cols):        # sequential sum, the order is part of the recipe
                s = s + u[:, c]
            out[lo:hi] = (u / s[:, None]).astype(np.float32)
        return out.reshape(-1)


def gen_normal(n, scale, seed):
    """A fresh generator per tensor, as the conformance suite does (gpt2_ops_suite.cu:71-76)."""
    return Rng(seed).normal(n, scale)


def hash_tool_inputs(dist, M, N, K, seed=12345):
    """A[M,K] and B[K,N] as the reference's hash tool fills them for one of its five named
    distributions (repro_gemm_cuda/hash_repro_gemm.cu:20-56): one generator, A first, then B, then
    (for "stress") the special rows of A and columns of B in index order."""
    g = Rng(seed)
    if dist == "uniform":
        return g.uniform_pm1(M * K), g.uniform_pm1(K * N)
    if dist == "normal":
        return g.normal(M * K), g.normal(K * N)
    if dist == "weights":
        return g.weights(M * K), g.weights(K * N)
    if dist == "wide":
        return g.wide(M * K, -40, 40), g.wide(K * N, -40, 40)
    if dist != "stress":
        raise ValueError("unknown distribution %r" % dist)
    A = g.normal(M * K).reshape(M, K)
    B = g.normal(K * N).reshape(K, N)
    for r in range(M):
        case = r % 8
        if case == 1:
            A[r] = 0.0
        elif case == 2:
            A[r] = np.ldexp(g.normal64(K), -140).astype(np.float32)
        elif case == 3:
            A[r] = (1e30 * g.normal64(K)).astype(np.float32)
        elif case == 4:
            A[r, g.range(0, K - 1)] = np.float32(1e6)
        elif case == 5:
            A[r] = np.where(np.arange(K) & 1, np.float32(-0.0), np.float32(0.0))
    for c in range(N):
        case = c % 6
        if case == 1:
            B[:, c] = 0.0
        elif case == 2:
            B[:, c] = g.wide(K, -60, 60)
        elif case == 3:
            B[:, c] = np.ldexp(g.normal64(K), -120).astype(np.float32)
    return A.reshape(-1), B.reshape(-1)


def ragged_test_inputs(M=133, N=77, K=301):
    """Inputs of the reference's correctness test: Rng{2024}, N(0,1), and one 1e6 outlier in A
    (repro_gemm_cuda/test_repro_gemm.cu:18-27)."""
    g = Rng(2024)
    A = g.normal(M * K)
    B = g.normal(K * N)
    A[5] = np.float32(1e6)
    return A, B


# GPT-2-small operations of the conformance suite: name -> (M, N, K, trans_a, trans_b, scale_a, scale_b)
# in the order gpt2_ops_suite.cu:463-483 creates them; seeds start at 1010 and advance by 10.
def suite_gemm_ops(tokens=1024):
    D, FF, V, HD, T = 768, 3072, 50257, 64, 1024
    ops, seed = [], 1000
    for name, fin, fout in (("attn_qkv", D, 3 * D), ("attn_proj", D, D), ("mlp_fc", D, FF), ("mlp_proj", FF, D),
                            ("lm_head", D, V)):
        seed += 10
        ops.append((name + ".fwd", tokens, fout, fin, False, True, 1.0, 0.02, seed))
        seed += 10
        ops.append((name + ".dX", tokens, fin, fout, False, False, 1e-3, 0.02, seed))
        seed += 10
        ops.append((name + ".dW", fout, fin, tokens, True, False, 1e-3, 1.0, seed))
    for name, M, N, K, ta, tb, sa, sb in (
            ("attn_head.scores QK^T", T, T, HD, False, True, 1.0, 1.0),
            ("attn_head.PV", T, HD, T, False, False, 2.0 / T, 1.0),
            ("attn_head.dP = dO V^T", T, T, HD, False, True, 1e-3, 1.0),
            ("attn_head.dV = P^T dO", T, HD, T, True, False, 2.0 / T, 1e-3),
            ("attn_head.dQ = dS K", T, HD, T, False, False, 1e-4, 1.0),
            ("attn_head.dK = dS^T Q", T, HD, T, True, False, 1e-4, 1.0)):
        seed += 10
        ops.append((name, M, N, K, ta, tb, sa, sb, seed))
    return ops


def suite_inputs(op):
    """The two input tensors of one suite operation (flat float32 arrays)."""
    _, M, N, K, _, _, sa, sb, seed = op
    return gen_normal(M * K, sa, seed), gen_normal(K * N, sb, seed + 1)


# ---------------------------------------------------------------------------------------------
# The five benchmark configurations.  Each returns a list of cases
#   dict(name, M, N, K, trans_a, trans_b, A, B [, batch])
# A and B are flat float32 arrays; batched cases hold `batch` matrices back to back.
# ---------------------------------------------------------------------------------------------
def config1(n=512):
    g = Rng(0)
    A = g.uniform_pm1(n * n)
    B = g.uniform_pm1(n * n)
    return [dict(name="c1.%d" % n, M=n, N=n, K=n, trans_a=False, trans_b=False, A=A, B=B)]


def config2(tokens=8192):
    cases = []
    for op in suite_gemm_ops(tokens)[6:9]:
        A, B = suite_inputs(op)
        cases.append(dict(name="c2." + op[0], M=op[1], N=op[2], K=op[3], trans_a=op[4], trans_b=op[5], A=A, B=B))
    return cases


def config3(n=4096):
    g = Rng(3)
    A = g.wide_mixed(n * n)
    B = g.wide_mixed(n * n)
    return [dict(name="c3.%d" % n, M=n, N=n, K=n, trans_a=False, trans_b=False, A=A, B=B)]


def config4(n=16384):
    g = Rng(4)
    A = g.uniform_pm1(n * n)
    B = g.uniform_pm1(n * n)
    return [dict(name="c4.%d" % n, M=n, N=n, K=n, trans_a=False, trans_b=False, A=A, B=B)]


def config5(batch=96, T=1024, HD=64):
    g = Rng(5)
    Q = g.normal(batch * T * HD)
    Km = g.normal(batch * T * HD)
    V = g.normal(batch * T * HD)
    P = g.prob_rows(batch * T, T)
    return [dict(name="c5.QKt", batch=batch, M=T, N=T, K=HD, trans_a=False, trans_b=True, A=Q, B=Km),
            dict(name="c5.PV", batch=batch, M=T, N=HD, K=T, trans_a=False, trans_b=False, A=P, B=V)]


# ------------------------------------------------------------------------------------------------
# Convolution cases: shape = (N, C, H, W, F, KH, KW, SY, SX, PY, PX)
# ------------------------------------------------------------------------------------------------
CONV_CASES = [
    # the six shapes of the reference's own GPU test (repro_conv_cuda/test_repro_conv.cu:126-131)
    ("lenet1", (100, 1, 28, 28, 6, 5, 5, 1, 1, 2, 2), "normal"),
    ("lenet2", (100, 6, 14, 14, 16, 5, 5, 1, 1, 0, 0), "normal"),
    ("lenet1.small", (10, 1, 28, 28, 6, 5, 5, 1, 1, 2, 2), "normal"),
    ("stride2.pad1", (4, 3, 17, 23, 8, 3, 5, 2, 2, 1, 1), "normal"),
    ("stride3x1", (2, 2, 19, 11, 5, 4, 3, 3, 1, 0, 2), "normal"),
    ("filters100", (2, 4, 12, 12, 100, 3, 3, 1, 1, 1, 1), "normal"),
    # beyond the reference kernels' limits (more than 1024 values per window, more than 256 filters)
    ("big.window", (2, 160, 9, 9, 40, 3, 3, 1, 1, 1, 1), "normal"),
    ("many.filters", (1, 8, 10, 10, 300, 3, 3, 1, 1, 0, 0), "normal"),
    # stride larger than the kernel (pixels no window touches), 1x1 kernel, one window, padding wider than the kernel
    ("skipping", (3, 2, 13, 14, 7, 2, 2, 3, 4, 0, 0), "normal"),
    ("pointwise", (2, 64, 7, 7, 96, 1, 1, 1, 1, 0, 0), "normal"),
    ("one.window", (5, 3, 4, 6, 9, 4, 6, 1, 1, 0, 0), "normal"),
    ("wide.padding", (2, 2, 5, 5, 4, 3, 3, 1, 1, 4, 5), "normal"),
    # wide dynamic range with exact zeros and subnormals in every tensor
    ("wide.range", (3, 5, 11, 9, 12, 3, 3, 1, 2, 1, 0), "wide"),
    # enough windows that the weight gradient is cut into several accumulation ranges
    ("many.windows", (64, 3, 48, 48, 8, 3, 3, 1, 1, 1, 1), "normal"),
    # row lengths that take the remaining lane layouts of the one-launch pre-pass (padded K of 512, 640 and 768)
    ("k432", (1, 48, 6, 6, 8, 3, 3, 1, 1, 1, 1), "normal"),
    ("k576.window", (2, 64, 8, 8, 24, 3, 3, 1, 1, 1, 1), "normal"),
    ("k576.taps", (2, 8, 8, 8, 64, 3, 3, 1, 1, 1, 1), "wide"),
    ("k700", (1, 28, 7, 9, 76, 5, 5, 2, 1, 2, 2), "normal"),
    # more than 105 472 values per window / taps per pixel: the forward (first) and the input gradient
    # (second) need several INT32 accumulation passes at S = 3 and take the one-product-per-image form
    ("long.window", (2, 300, 19, 19, 2, 19, 19, 1, 1, 9, 9), "normal"),
    ("long.taps", (2, 2, 19, 19, 300, 19, 19, 1, 1, 9, 9), "normal"),
]


def conv_output_dims(shape):
    N, C, H, W, F, KH, KW, SY, SX, PY, PX = shape
    return (H + 2 * PY - KH) // SY + 1, (W + 2 * PX - KW) // SX + 1


def conv_inputs(shape, dist="normal", seed=2024):
    """x, weight and dY for a convolution case, drawn in that order from one stream; magnitudes follow the
    reference's test (repro_conv_cuda/test_repro_conv.cu:63-65): x ~ 1, weights ~ 0.1, dY ~ 1e-3."""
    N, C, H, W, F, KH, KW, SY, SX, PY, PX = shape
    oh, ow = conv_output_dims(shape)
    g = Rng(seed)
    sizes = (N * C * H * W, F * C * KH * KW, N * F * oh * ow)
    if dist == "wide":
        return tuple(g.wide_mixed(n) for n in sizes)
    return g.normal(sizes[0]), g.normal(sizes[1], 0.1), g.normal(sizes[2], 1e-3)


# ------------------------------------------------------------------------------------------------
# The same streams produced with torch tensor arithmetic on any device (the 16384^2 operands of
# configuration 4 take minutes with the numpy generator and milliseconds on a GPU).  Every step is an
# exact integer or float64 operation followed by one IEEE rounding to float32, so the bits equal the
# numpy generator's; tests compare the two element for element and against the committed input hashes.
# ------------------------------------------------------------------------------------------------
class DeviceRng:
    """SplitMix64 stream on a torch device; methods consume draws in the same order as ``Rng``."""

    _CHUNK = 1 << 24

    def __init__(self, seed, device):
        import torch
        self.t = torch
        self.state = int(seed) & 0xFFFFFFFFFFFFFFFF
        self.device = torch.device(device)

    @staticmethod
    def _i64(x):
        x &= 0xFFFFFFFFFFFFFFFF
        return x - (1 << 64) if x >= (1 << 63) else x

    def skip(self, n):
        """Advances the stream by n draws without producing them (the generator is a counter)."""
        self.state = (self.state + n * int(_GAMMA)) & 0xFFFFFFFFFFFFFFFF

    def _lsr(self, z, k):
        return (z >> k) & ((1 << (64 - k)) - 1)          # logical shift of a 64-bit pattern held as int64

    def next(self, n):
        """The next n raw outputs as int64 bit patterns (two's-complement wrap = arithmetic mod 2^64)."""
        t = self.t
        idx = t.arange(1, n + 1, dtype=t.int64, device=self.device)
        z = idx * self._i64(int(_GAMMA)) + self._i64(self.state)
        self.skip(n)
        z = (z ^ self._lsr(z, 30)) * self._i64(int(_M1))
        z = (z ^ self._lsr(z, 27)) * self._i64(int(_M2))
        return z ^ self._lsr(z, 31)

    def _umod(self, z, m):
        """z mod m for the unsigned 64-bit value behind an int64 pattern (m < 2^31)."""
        hi, lo = self._lsr(z, 32), z & 0xFFFFFFFF
        return ((hi % m) * ((1 << 32) % m) + lo % m) % m

    def _u01_of(self, z):
        return self._lsr(z, 40).to(self.t.float64) * (1.0 / 16777216.0)

    def _pow2(self, e):
        """2^e as float64 for an int64 tensor of exponents in the normal range, built from its bit pattern."""
        return ((e + 1023) << 52).view(self.t.float64)

    def _chunks(self, n, per_elem, one):
        out = self.t.empty(n, dtype=self.t.float32, device=self.device)
        step = max(1, self._CHUNK // per_elem)
        for lo in range(0, n, step):
            hi = min(n, lo + step)
            out[lo:hi] = one(hi - lo)
        return out

    def uniform_pm1(self, n):
        return self._chunks(n, 1, lambda m: (2.0 * self._u01_of(self.next(m)) - 1.0).to(self.t.float32))

    def normal(self, n, scale=1.0):
        def one(m):
            u = self._u01_of(self.next(12 * m)).view(m, 12)
            acc = self.t.zeros(m, dtype=self.t.float64, device=self.device)
            for i in range(12):
                acc = acc + u[:, i]
            return (scale * (acc - 6.0)).to(self.t.float32)
        return self._chunks(n, 12, one)

    def wide_mixed(self, n, elo=-20, ehi=20):
        t = self.t

        def one(m):
            z = self.next(4 * m).view(m, 4)
            r = self._umod(z[:, 0], 1000)
            mant = 1.0 + self._u01_of(z[:, 1])
            e = t.where(r == 10, -149 + self._umod(z[:, 2], 23), elo + self._umod(z[:, 2], ehi - elo + 1))
            v = mant * self._pow2(e)
            v = t.where((z[:, 3] & 1) != 0, -v, v)
            return t.where(r < 10, t.zeros_like(v), v).to(t.float32)
        return self._chunks(n, 4, one)

    def prob_rows(self, rows, cols):
        t = self.t
        out = t.empty((rows, cols), dtype=t.float32, device=self.device)
        step = max(1, self._CHUNK // cols)
        for lo in range(0, rows, step):
            hi = min(rows, lo + step)
            u = self._u01_of(self.next((hi - lo) * cols)).view(hi - lo, cols) + 1.0 / 33554432.0
            s = t.zeros(hi - lo, dtype=t.float64, device=self.device)
            for c in range(cols):        # sequential sum, the order is part of the recipe
                s = s + u[:, c]
            out[lo:hi] = (u / s[:, None]).to(t.float32)
        return out.view(-1)


def config3_device(device, n=4096):
    """Configuration 3's operands generated on `device` (same bits as config3())."""
    g = DeviceRng(3, device)
    return g.wide_mixed(n * n), g.wide_mixed(n * n)


def config4_device(device, n=16384, a_rows=None, b_rows=None):
    """Configuration 4's operands generated on `device`.  a_rows / b_rows = (lo, hi) restrict the result
    to that block of rows of A / B (the stream is advanced past the rest), otherwise the whole matrix."""
    g = DeviceRng(4, device)

    def rows(block):
        lo, hi = block if block is not None else (0, n)
        g.skip(lo * n)
        x = g.uniform_pm1((hi - lo) * n)
        g.skip((n - hi) * n)
        return x
    return rows(a_rows), rows(b_rows)


def config4_device_k_range(device, n, klo, khi):
    """A[:, klo:khi] (as a dense n x (khi-klo) matrix) and B[klo:khi, :] of configuration 4 on `device`."""
    t_ = DeviceRng(4, device)
    torch = t_.t
    A = torch.empty((n, khi - klo), dtype=torch.float32, device=t_.device)
    step = max(1, DeviceRng._CHUNK // n)
    for lo in range(0, n, step):                     # whole rows are drawn, the K range is kept
        hi = min(n, lo + step)
        A[lo:hi] = t_.uniform_pm1((hi - lo) * n).view(hi - lo, n)[:, klo:khi]
    t_.skip(klo * n)
    B = t_.uniform_pm1((khi - klo) * n)
    return A.reshape(-1), B


def config5_device(device, batch=96, T=1024, HD=64):
    g = DeviceRng(5, device)
    Q = g.normal(batch * T * HD)
    Km = g.normal(batch * T * HD)
    V = g.normal(batch * T * HD)
    P = g.prob_rows(batch * T, T)
    return Q, Km, V, P
