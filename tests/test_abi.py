"""The C-ABI library: loads without a GPU, exports everything include/rgb200.h declares, and its
host-side planning and scalar helpers behave like the reference's (no kernels are launched here)."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from bit_reproducible_training_b200 import _lib, build
from bit_reproducible_training_b200 import fixtures as fx
from bit_reproducible_training_b200 import repro_gemm as rg

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def L():
    build.build()
    return _lib.lib()


def test_library_exports_every_declared_symbol(L):
    header = open(os.path.join(ROOT, "include", "rgb200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    names = set(re.findall(r"\b(rgb200_[a-z0-9_]+)\s*\(", header))
    assert len(names) >= 24
    for n in sorted(names):
        assert hasattr(L, n), "librgb200.so does not export %s" % n


def test_cxx_shim_declares_the_reference_surface():
    shim = open(os.path.join(ROOT, "include", "repro_gemm.cuh")).read()
    for needle in ("namespace repro_gemm", "enum class Algo", "struct Config", "struct Plan", "make_plan",
                   "repro_gemm_fp32_ws", "repro_gemm_fp32", "algo_name", "MAX_SLICES"):
        assert needle in shim, needle


def test_conv_shim_declares_the_reference_surface():
    shim = open(os.path.join(ROOT, "include", "repro_conv.cuh")).read()
    for needle in ("namespace repro_conv", "struct ConvShape", "conv2d_workspace", "conv2d_grad_weight_workspace",
                   "conv2d_grad_input_workspace", "repro_conv2d_ws", "repro_conv2d_grad_weight_ws",
                   "repro_conv2d_grad_input_ws", "int SY = 1, SX = 1", "int PY = 0, PX = 0"):
        assert needle in shim, needle


def test_conv_workspace_planning_and_shape_checks(L):
    """Host-only: sizes depend on (shape, slices) alone; unsupported shapes give cudaErrorInvalidValue
    (the reference's checks, repro_conv_cuda/repro_conv.cu:157-167)."""
    from bit_reproducible_training_b200 import repro_conv as rc
    g = rc.ConvShape(100, 1, 28, 28, 6, 5, 5, PY=2, PX=2)
    assert (g.K(), g.OH(), g.OW(), g.windows(), g.output_size()) == (25, 28, 28, 78400, 100 * 6 * 784)
    for query in (rc.conv2d_workspace, rc.conv2d_grad_weight_workspace, rc.conv2d_grad_input_workspace):
        code, n3 = query(g, 3)
        assert code == 0 and n3 > 0 and query(g, 3) == (0, n3)
        assert query(g, 1)[1] < n3                      # fewer digit planes
        assert query(g, 0)[0] == rg.cudaErrorInvalidValue and query(g, 4)[0] == rg.cudaErrorInvalidValue
        for bad in (dict(N=0), dict(C=0), dict(F=0), dict(KH=0), dict(SY=0), dict(PX=-1), dict(KH=40), dict(N=70000),
                    dict(N=60000, H=200, W=200)):     # the last: 2^31 or more input values
            fields = dict(N=100, C=1, H=28, W=28, F=6, KH=5, KW=5, SY=1, SX=1, PY=2, PX=2)
            fields.update(bad)
            assert query(rc.ConvShape(**fields), 3)[0] == rg.cudaErrorInvalidValue, bad
    # larger windows and filter counts than the reference's kernels take are planned here
    assert rc.conv2d_workspace(rc.ConvShape(2, 160, 9, 9, 300, 3, 3, PY=1, PX=1), 3)[0] == 0
    # more windows than an exact INT64 sum allows at S = 3 (9e18 / (127 * 128^2)^2 = 2 078 698)
    assert rc.conv2d_grad_weight_workspace(rc.ConvShape(600, 1, 60, 60, 4, 1, 1), 3)[0] == rg.cudaErrorInvalidValue
    assert rc.conv2d_grad_weight_workspace(rc.ConvShape(600, 1, 60, 60, 4, 1, 1), 2)[0] == 0


def test_index_division_by_multiply_high_is_exact(L):
    """The convolutions' index maps divide by kernel and image extents with one multiply-high and a shift;
    the library's host copy of that arithmetic must equal floor division for every n below 2^31."""
    rng = np.random.default_rng(11)
    divisors = list(range(1, 300)) + [int(v) for v in rng.integers(1, 1 << 31, size=300)] + \
        [(1 << k) + j for k in range(1, 31) for j in (-1, 0, 1)] + [(1 << 31) - 1]
    for d in divisors:
        if d < 1:
            continue
        top = (1 << 31) - 1
        ns = [0, 1, d - 1, d, d + 1, 2 * d - 1, 2 * d, top, top - 1, (top // d) * d, (top // d) * d - 1]
        ns += [int(v) for v in rng.integers(0, 1 << 31, size=40)]
        for n in ns:
            if 0 <= n <= top:
                assert L.rgb200_fast_div(d, n) == n // d, (d, n)
    assert L.rgb200_fast_div(0, 5) == -1 and L.rgb200_fast_div(3, -1) == -1


def test_default_config_matches_reference_defaults(L):
    c = _lib.Config()
    L.rgb200_default_config(C.byref(c))
    assert (c.split_k, c.tile_m, c.tile_n, c.tile_k, c.algo, c.slices, c.trans_a, c.trans_b) == (1, 16, 16, 32, 0, 3, 0, 0)
    d = rg.Config().c()
    assert bytes(c) == bytes(d)


def test_algo_names(L):
    assert [rg.algo_name(a) for a in (rg.Algo.Auto, rg.Algo.Reference, rg.Algo.Tiled, rg.Algo.TensorCore)] == \
        ["auto", "ref", "tiled", "tc"]


def layout(L, M, N, K, batch=1, **kw):
    info = _lib.LayoutInfo()
    c = rg.Config(**kw).c()
    rc = L.rgb200_layout(M, N, K, batch, C.byref(c), C.byref(info))
    return rc, info


def test_layout_rejects_bad_arguments(L):
    assert layout(L, 0, 4, 4)[0] == rg.cudaErrorInvalidValue
    assert layout(L, 4, -1, 4)[0] == rg.cudaErrorInvalidValue
    assert layout(L, 4, 4, 0)[0] == rg.cudaErrorInvalidValue
    assert layout(L, 4, 4, 4, split_k=0)[0] == rg.cudaErrorInvalidValue
    assert layout(L, 4, 4, 4, slices=0)[0] == rg.cudaErrorInvalidValue
    assert layout(L, 4, 4, 4, slices=4)[0] == rg.cudaErrorInvalidValue
    assert layout(L, 4, 4, 4, batch=0)[0] == rg.cudaErrorInvalidValue
    assert layout(L, 4, 4, 4, batch=70000)[0] == rg.cudaErrorInvalidValue
    assert layout(L, 4, 4, 4, batch=65535)[0] == 0


def test_k_bound_for_exact_int64(L):
    """K * max|X|^2 <= 2^62: S = 3 allows K up to about a million (reference: repro_gemm.cu:394-396)."""
    assert layout(L, 8, 8, 1056000, slices=3)[0] == 0
    assert layout(L, 8, 8, 1057000, slices=3)[0] == rg.cudaErrorInvalidValue
    assert layout(L, 8, 8, 50_000_000, slices=2)[0] == 0


def test_split_is_clamped_and_raised(L):
    rc, info = layout(L, 64, 64, 7, split_k=16)
    assert rc == 0 and (info.k_padded, info.k_blocks, info.split_k) == (128, 1, 1)
    rc, info = layout(L, 133, 77, 301, split_k=64)
    assert rc == 0 and (info.k_blocks, info.split_k) == (3, 3)
    rc, info = layout(L, 128, 128, 4096, split_k=7)
    assert rc == 0 and info.split_k == 7 and info.partial_bytes >= 7 * 128 * 128 * 8
    # one INT32 pass holds 105516 values of k at S = 3 (824 blocks of 128): longer K is cut automatically
    rc, info = layout(L, 128, 128, 824 * 128, slices=3)
    assert rc == 0 and info.min_split == 1
    rc, info = layout(L, 128, 128, 824 * 128 + 1, slices=3)
    assert rc == 0 and info.min_split == 2 and info.split_k >= 2
    # enough tiles to fill the GPU: no K ranges unless asked for or forced
    rc, info = layout(L, 4096, 4096, 4096)
    assert rc == 0 and info.split_k == 1 and info.partial_bytes == 0
    # few tiles and a long K: the planner cuts K by itself
    rc, info = layout(L, 1024, 768, 50257)
    assert rc == 0 and info.split_k == 3 and info.partial_bytes >= 3 * 1024 * 768 * 8
    rc, info = layout(L, 128, 128, 1032 * 128 + 1, slices=2)
    assert rc == 0 and info.min_split == 2
    rc, info = layout(L, 128, 128, 1040 * 128 + 1, slices=1)
    assert rc == 0 and info.min_split == 2


def test_level_sums_fit_int32_for_one_pass():
    # worst-case per-k magnitude of one level, from the digit ranges |d0| <= 127, |d_{p>0}| <= 64
    worst = {1: 127 * 127, 2: max(127 * 127, 2 * 127 * 64, 64 * 64), 3: 2 * 127 * 64 + 64 * 64}
    blocks = {1: 1040, 2: 1032, 3: 824}
    for S in (1, 2, 3):
        assert blocks[S] * 128 * worst[S] <= 2 ** 31 - 1
        assert (blocks[S] + 1) * 128 * worst[S] > 2 ** 31 - 1


def test_workspace_size_covers_planes(L):
    rc, info = layout(L, 4096, 4096, 4096)
    assert rc == 0
    assert info.planes_a == 3 * 4096 * 4096 and info.planes_b == 3 * 4096 * 4096
    assert info.workspace_bytes >= info.planes_a + info.planes_b + 2 * 4096 * 4
    assert info.workspace_bytes < info.planes_a + info.planes_b + (1 << 20)
    rc, b = layout(L, 1024, 1024, 64, batch=96)
    assert rc == 0 and b.planes_a == 96 * 3 * 1024 * 128


def test_host_scalar_helpers_match_reference_vectors(L, scalar_vectors):
    for bits, want in scalar_vectors["scale_exponent"]:
        assert L.rgb200_scale_exponent(float(np.uint32(bits).view(np.float32))) == want
    for bits, se, x1, x2, x3 in scalar_vectors["fixed_point"]:
        x = float(np.uint32(bits).view(np.float32))
        assert [L.rgb200_fixed_point(x, se, S) for S in (1, 2, 3)] == [x1, x2, x3]
    for T, E, want in scalar_vectors["round_to_float"]:
        assert L.rgb200_round_to_float_bits(T, E) == want, (T, E)


def test_fnv_matches_reference_input_hashes(L):
    op = [o for o in fx.suite_gemm_ops(1024) if o[0] == "attn_proj.fwd"][0]
    A, B = fx.suite_inputs(op)
    assert "%016x" % rg.fnv1a64(B, rg.fnv1a64(A)) == "46dd3a91b61dc793"


def test_plan_without_a_device_fails_cleanly(L):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    rc, plan = rg.make_plan(64, 64, 64)
    assert rc != 0 and plan is None
    rc, _ = rg.make_plan(64, 64, 64, rg.Config(algo=rg.Algo.Tiled))
    assert rc == rg.cudaErrorNotSupported


def test_host_pipeline_without_a_device_fails_cleanly(L):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    h = C.c_void_p()
    c = rg.Config().c()
    assert L.rgb200_host_gemm_create(256, 256, 256, C.byref(c), 0, C.byref(h)) != 0 and not h.value
    assert L.rgb200_host_gemm_create(256, 256, 256, C.byref(c), 0, None) == rg.cudaErrorInvalidValue
    assert L.rgb200_gemm_fp32_host(None, None, None, None, None) == rg.cudaErrorInvalidValue
    assert L.rgb200_host_gemm_destroy(None) == rg.cudaErrorInvalidValue
    assert L.rgb200_static_status(None) == rg.cudaErrorInvalidValue


def test_device_generator_reproduces_the_numpy_streams():
    """The torch generator (used to create large operands on a GPU) gives the numpy generator's bits."""
    import torch

    def same(a, b):
        return np.array_equal(np.asarray(a).view(np.uint32), b.cpu().numpy().view(np.uint32))
    n = 70001
    g, d = fx.Rng(4), fx.DeviceRng(4, "cpu")
    assert same(g.uniform_pm1(n), d.uniform_pm1(n)) and same(g.uniform_pm1(33), d.uniform_pm1(33))
    g, d = fx.Rng(3), fx.DeviceRng(3, "cpu")
    assert same(g.wide_mixed(n), d.wide_mixed(n)) and same(g.wide_mixed(n), d.wide_mixed(n))
    g, d = fx.Rng(5), fx.DeviceRng(5, "cpu")
    assert same(g.normal(n), d.normal(n)) and same(g.normal(n, 0.02), d.normal(n, 0.02))
    assert same(g.prob_rows(37, 1024), d.prob_rows(37, 1024))
    c = fx.config4(192)[0]
    A, B = fx.config4_device("cpu", 192, a_rows=(64, 128))
    assert same(c["A"].reshape(192, 192)[64:128].reshape(-1), A) and same(c["B"], B)
    A, B = fx.config4_device_k_range("cpu", 192, 32, 96)
    assert same(np.ascontiguousarray(c["A"].reshape(192, 192)[:, 32:96]).reshape(-1), A)
    assert same(c["B"].reshape(192, 192)[32:96].reshape(-1), B)
    c3 = fx.config3(64)[0]
    A, B = fx.config3_device("cpu", 64)
    assert same(c3["A"], A) and same(c3["B"], B)
    c5 = fx.config5(2, 16, 64)
    Q, Km, V, P = fx.config5_device("cpu", 2, 16, 64)
    assert same(c5[0]["A"], Q) and same(c5[0]["B"], Km) and same(c5[1]["B"], V) and same(c5[1]["A"], P)


CXX_CALLER = r"""
// A caller written against the reference's C++ surface (repro_gemm_cuda/repro_gemm.cuh:25-75).
#include "repro_gemm.cuh"
#include <cstdio>
int main() {
    repro_gemm::Config cfg;                       // the reference's defaults
    cfg.slices = 2;
    cfg.trans_b = true;
    repro_gemm::Plan plan{};
    cudaError_t e = repro_gemm::make_plan(128, 64, 256, cfg, &plan);
    cudaError_t bad = repro_gemm::make_plan(128, 64, 256, cfg, nullptr);
    cfg.algo = repro_gemm::Algo::Tiled;
    cudaError_t tiled = repro_gemm::make_plan(128, 64, 256, cfg, &plan);
    std::printf("%d %d %d %s %s %d\n", (int)e, (int)bad, (int)tiled, repro_gemm::algo_name(repro_gemm::Algo::TensorCore),
                repro_gemm::algo_name(repro_gemm::Algo::Reference), repro_gemm::MAX_SLICES);
    return 0;
}
"""


def test_cxx_caller_builds_against_the_shim_and_links_the_library(L, tmp_path):
    """A C++ program using the reference's namespace, types and defaults compiles against
    include/repro_gemm.cuh and links librgb200.so; without a GPU the calls fail cleanly."""
    import shutil
    import subprocess
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc not available")
    src = tmp_path / "caller.cu"
    src.write_text(CXX_CALLER)
    exe = tmp_path / "caller"
    libdir = os.path.dirname(build.LIB)
    subprocess.run([nvcc, "-std=c++17", "-I", os.path.join(ROOT, "include"), "-o", str(exe), str(src),
                    "-L", libdir, "-lrgb200", "-Xlinker", "-rpath", "-Xlinker", libdir], check=True, capture_output=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()
    import torch
    if not torch.cuda.is_available():
        assert int(out[0]) != 0                    # no device: an error code, not a crash
    assert int(out[1]) == rg.cudaErrorInvalidValue and int(out[2]) == rg.cudaErrorNotSupported
    assert out[3:] == ["tc", "ref", "3"]


CXX_CONV_CALLER = r"""
// A caller written against the reference's convolution surface (repro_conv_cuda/repro_conv.cuh:22-32).
#include "repro_conv.cuh"
#include <cstdio>
int main() {
    repro_conv::ConvShape g;                      // stride 1 and no padding by default, as in the reference
    g.N = 100; g.C = 1; g.H = 28; g.W = 28; g.F = 6; g.KH = 5; g.KW = 5; g.PY = 2; g.PX = 2;
    size_t b0 = 0, b1 = 0, b2 = 0;
    cudaError_t e0 = repro_conv::conv2d_workspace(g, 3, &b0);
    cudaError_t e1 = repro_conv::conv2d_grad_weight_workspace(g, 3, &b1);
    cudaError_t e2 = repro_conv::conv2d_grad_input_workspace(g, 3, &b2);
    cudaError_t bad = repro_conv::conv2d_workspace(g, 4, &b0);
    cudaError_t run = repro_conv::repro_conv2d_ws(nullptr, nullptr, nullptr, g, 3, nullptr, 0);
    std::printf("%d %d %d %d %d %d %d %d %d %zu\n", (int)e0, (int)e1, (int)e2, (int)bad, (int)run, g.K(), g.OH(), g.OW(), g.windows(),
                g.output_size());
    return (b0 && b1 && b2) ? 0 : 1;
}
"""


def test_cxx_conv_caller_builds_against_the_shim_and_links_the_library(L, tmp_path):
    """A C++ program using the reference's ConvShape and workspace queries compiles against
    include/repro_conv.cuh and links librgb200.so; planning needs no GPU."""
    import shutil
    import subprocess
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc not available")
    src = tmp_path / "conv_caller.cu"
    src.write_text(CXX_CONV_CALLER)
    exe = tmp_path / "conv_caller"
    libdir = os.path.dirname(build.LIB)
    subprocess.run([nvcc, "-std=c++17", "-I", os.path.join(ROOT, "include"), "-o", str(exe), str(src),
                    "-L", libdir, "-lrgb200", "-Xlinker", "-rpath", "-Xlinker", libdir], check=True, capture_output=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()
    assert [int(v) for v in out[:5]] == [0, 0, 0, rg.cudaErrorInvalidValue, rg.cudaErrorInvalidValue]
    assert [int(v) for v in out[5:]] == [25, 28, 28, 78400, 100 * 6 * 28 * 28]


def test_status_check_of_the_python_wrappers_is_opt_in(monkeypatch):
    from bit_reproducible_training_b200 import repro_gemm as rg
    monkeypatch.delenv("RGB200_CHECK_STATUS", raising=False)
    assert not rg.check_status_enabled()
    monkeypatch.setenv("RGB200_CHECK_STATUS", "0")
    assert not rg.check_status_enabled()
    monkeypatch.setenv("RGB200_CHECK_STATUS", "1")
    assert rg.check_status_enabled()
    err = rg.ReproGemmIncomplete(4, "gemm")
    assert err.status == 4 and "incomplete" in str(err)
