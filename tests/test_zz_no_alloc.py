"""The allocation-free entry point (rgb200_gemm_fp32_static).

It serves callers that are given device pointers but cannot allocate device memory themselves (an
operator under a framework's caching allocator, a latency-critical step that must avoid the
device-wide synchronisation of cudaMalloc / cudaFree).  Its scratch is a fixed array inside the
library that every call shares and that keeps the previous call's contents, so the checks below run
two calls in a row, of different shapes, and compare each with the ordinary workspace entry point
and with the CPU oracle bit for bit.  This file is collected last on purpose: a run that stops at the first failure has
then already exercised everything else.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle

from bit_reproducible_training_b200 import _lib
from bit_reproducible_training_b200 import fixtures as fx
from bit_reproducible_training_b200 import repro_gemm as rg

pytestmark = pytest.mark.gpu


def with_workspace(dA, dB, M, N, K, cfg):
    """The existing entry point (rgb200_gemm_fp32_ws) with a caller-allocated workspace."""
    rc, plan = rg.make_plan(M, N, K, cfg)
    assert rc == 0
    ws = torch.empty(plan.workspace_bytes, dtype=torch.uint8, device="cuda")
    out = torch.full((M, N), float("nan"), device="cuda")
    assert rg.repro_gemm_fp32_ws(dA, dB, out, M, N, K, cfg, ws) == 0
    torch.cuda.synchronize()
    return out


def through_static(dA, dB, M, N, K, cfg):
    out = torch.full((M, N), float("nan"), device="cuda")
    c = cfg.c()
    rc = _lib.lib().rgb200_gemm_fp32_static(C.c_void_p(dA.data_ptr()), C.c_void_p(dB.data_ptr()),
                                           C.c_void_p(out.data_ptr()), M, N, K, C.byref(c),
                                           C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, rc
    torch.cuda.synchronize()
    return out


def test_two_calls_in_a_row_match_the_workspace_entry_point():
    # second shape smaller and with other transpositions: stale planes of the first call lie beside and
    # beyond its workspace image; a K-range run follows to use the partial-sum area as well
    cases = [(700, 520, 1300, rg.Config(slices=3)),
             (133, 77, 301, rg.Config(slices=2, trans_a=True, trans_b=True)),
             (256, 192, 2048, rg.Config(slices=3, split_k=4)),
             (700, 520, 1300, rg.Config(slices=3))]
    g = fx.Rng(2718)
    for M, N, K, cfg in cases:
        hA, hB = g.wide(M * K, -12, 12), g.normal(K * N)
        A, B = torch.from_numpy(hA).cuda(), torch.from_numpy(hB).cuda()
        want = with_workspace(A, B, M, N, K, cfg)
        cpu = oracle.gemm(hA, hB, M, N, K, cfg.trans_a, cfg.trans_b, cfg.slices)
        assert np.array_equal(want.cpu().numpy().view(np.uint32), cpu.view(np.uint32)), (M, N, K)
        for _ in range(2):
            got = through_static(A, B, M, N, K, cfg)
            assert torch.equal(got.view(torch.int32), want.view(torch.int32)), (M, N, K)
            assert np.array_equal(got.cpu().numpy().view(np.uint32), cpu.view(np.uint32)), (M, N, K)
            assert rg.static_status() == 0


def test_problems_beyond_the_fixed_array_are_refused_cleanly():
    M = N = K = 4096                          # needs about 96 MiB of workspace
    A = torch.zeros(1, device="cuda")
    out = torch.full((4,), 7.0, device="cuda")
    c = rg.Config().c()
    rc = _lib.lib().rgb200_gemm_fp32_static(C.c_void_p(A.data_ptr()), C.c_void_p(A.data_ptr()),
                                           C.c_void_p(out.data_ptr()), M, N, K, C.byref(c), None)
    assert rc == rg.cudaErrorMemoryAllocation
    torch.cuda.synchronize()
    assert torch.all(out == 7.0)              # nothing was launched
    info = _lib.LayoutInfo()
    assert _lib.lib().rgb200_layout(M, N, K, 1, C.byref(c), C.byref(info)) == 0
    assert info.workspace_bytes > rg.STATIC_WORKSPACE_BYTES
    assert rg.repro_gemm_fp32_static(None, A, out, 8, 8, 8) == rg.cudaErrorInvalidValue
