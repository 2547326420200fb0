"""The reference's own GPU code as a checker.

* Its correctness test and hash tool (test_repro_gemm.cu, hash_repro_gemm.cu), compiled unmodified
  from its sources against the reference header and linked with librgb200.so instead of
  repro_gemm.cu, must pass: that is the drop-in claim executed end to end.
* Its CUDA kernels, recompiled for sm_100a, must produce the same bits as this library.
Both come prebuilt in oracle/_ref (oracle/Makefile, target ref_gpu); absent files skip the test.
"""
import os
import subprocess

import numpy as np
import pytest
import torch

import oracle
from bit_reproducible_training_b200 import fixtures as fx
from bit_reproducible_training_b200 import repro_gemm as rg

pytestmark = pytest.mark.gpu


def run_tool(path, *args):
    if not os.path.exists(path):
        pytest.skip("%s not built" % os.path.basename(path))
    return subprocess.run([path] + [str(a) for a in args], capture_output=True, text=True, timeout=900)


def test_reference_correctness_program_passes_on_this_library():
    """S = 1..3 x {ref, tiled (skipped as unsupported), tc} x split_k {1,2,3,7,64} x five transposition
    cases on 133 x 77 x 301, each compared bit for bit with the reference's cpu_reference."""
    res = run_tool(oracle.REF_TEST_TOOL)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert "PASS: all S, algorithms, split_k values, and transposes match the CPU definition" in res.stdout
    assert res.stdout.count("skipped (not supported") == 3          # only the dp4a algorithm, once per S


@pytest.mark.parametrize("shape,splits", [("256 256 1024", "1,2,3,4,7,8,16,64"), ("129 77 1000", "1,2,3,5,7,13,64"),
                                          ("64 64 7", "1,2,3,7,16")])
@pytest.mark.parametrize("dist", ["uniform", "weights", "wide", "stress"])
def test_reference_hash_program_passes_on_this_library(shape, splits, dist, golden):
    M, N, K = (int(x) for x in shape.split())
    for S in (1, 3):
        res = run_tool(oracle.REF_HASH_TOOL, M, N, K, 2, splits, 12345, dist, "ref,tc", S)
        assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
        assert "status=PASS" in res.stdout and "exact vs CPU definition: MATCH" in res.stdout
        want = golden[("hash.%s.%dx%dx%d" % (dist, M, N, K), S)]["out_hash"]
        assert "hash=%s" % want in res.stdout      # the tool's own input generator and our fixture agree too


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_same_bits_as_the_reference_cuda_kernels():
    if oracle.ref_cuda() is None:
        pytest.skip("oracle/_ref/librepro_ref_cuda.so not built")
    cases = [fx.config1()[0], fx.config3(1024)[0]] + fx.config2(1024) + fx.config5(2)
    for c in cases:
        M, N, K, ta, tb = c["M"], c["N"], c["K"], c["trans_a"], c["trans_b"]
        A, B = c["A"][:M * K], c["B"][:K * N]          # batched cases: the first matrix
        dA, dB = dev(A), dev(B)
        for S in (1, 2, 3):
            mine = rg.gemm(dA, dB, M, N, K, ta, tb, S)
            for algo in (3, 2):                         # the reference's WMMA and dp4a kernels
                theirs = oracle.ref_cuda_gemm(dA, dB, M, N, K, ta, tb, S, algo=algo)
                assert torch.equal(mine.view(torch.int32), theirs.view(torch.int32)), (c["name"], S, algo)


def test_same_bits_as_the_reference_cuda_kernel_at_full_size():
    if oracle.ref_cuda() is None:
        pytest.skip("oracle/_ref/librepro_ref_cuda.so not built")
    c = fx.config3(4096)[0]
    dA, dB = dev(c["A"]), dev(c["B"])
    for S in (1, 2, 3):
        mine = rg.gemm(dA, dB, 4096, 4096, 4096, slices=S)
        theirs = oracle.ref_cuda_gemm(dA, dB, 4096, 4096, 4096, S=S)
        assert torch.equal(mine.view(torch.int32), theirs.view(torch.int32)), S


def test_per_gpu_hash_files_from_separate_processes(tmp_path, golden):
    """run_repro.sh's outer loop (repro_gemm_cuda/run_repro.sh:77-115) on this library: the reference's hash tool in
    three separate processes per case on every visible GPU; one hash file per GPU; all processes and all GPUs agree,
    and the hashes are the reference CPU implementation's."""
    from oracle import run_repro_hashes as rr
    if not os.path.exists(rr.TOOL):
        pytest.skip("oracle/_ref/hash_repro_gemm_rgb200 not built")
    gpus = [str(i) for i in range(torch.cuda.device_count())]
    files, failures = rr.run(str(tmp_path), procs=3, gpus=gpus, slices=("1", "3"), shapes=rr.SHAPES[1:3],
                             dists=("normal", "stress"))
    assert not failures, failures
    assert len(files) == len(gpus)
    lines = open(files[0]).read().splitlines()
    assert len(lines) == 2 * 2 * 2 and all("status=PASS" in l for l in lines)
    for l in lines:
        f = dict(kv.split("=") for kv in l.split()[1:])
        want = golden[("hash.%s.%sx%sx%s" % (f["dist"], f["M"], f["N"], f["K"]), int(f["S"]))]["out_hash"]
        assert f["hash"] == want
