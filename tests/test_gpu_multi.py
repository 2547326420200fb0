"""Multi-GPU modes over NCCL, one process per GPU (skipped with fewer than two devices).

Rows of A: no collective on the data path.  K ranges: max all-reduce of the row/column maxima and
an INT64 sum all-reduce of the exact partials, then one rounding.  Every layout must reproduce the
bits of the single-GPU product (checked against the golden hash of the reference's cpu_gemm)."""
import json
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from bit_reproducible_training_b200 import fixtures as fx
from bit_reproducible_training_b200 import repro_gemm as rg
from bit_reproducible_training_b200 import sharded

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def worker(rank, world, port, n, want_hash, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        c = fx.config4(n)[0]
        A, B = c["A"].reshape(n, n), c["B"].reshape(n, n)
        cfg = rg.Config()
        # rows of A
        lo, hi = sharded.shard_range(n, world, rank)
        C_all = sharded.gemm_row_sharded(torch.from_numpy(np.ascontiguousarray(A[lo:hi])).cuda(),
                                         torch.from_numpy(B).cuda(), hi - lo, n, n, cfg,
                                         gather_group=dist.group.WORLD)
        assert "%016x" % rg.fnv1a64(C_all) == want_hash, "row-sharded result differs"
        # K ranges
        klo, khi = sharded.shard_range(n, world, rank)
        C_k = sharded.gemm_k_sharded(torch.from_numpy(np.ascontiguousarray(A[:, klo:khi])).cuda(),
                                     torch.from_numpy(np.ascontiguousarray(B[klo:khi])).cuda(),
                                     n, n, khi - klo, n, cfg)
        assert "%016x" % rg.fnv1a64(C_k) == want_hash, "K-sharded result differs"
        # K ranges with transposed storage on both sides
        cfg_t = rg.Config(trans_a=True, trans_b=True)
        C_t = sharded.gemm_k_sharded(torch.from_numpy(np.ascontiguousarray(A[:, klo:khi].T)).cuda(),
                                     torch.from_numpy(np.ascontiguousarray(B[klo:khi].T)).cuda(),
                                     n, n, khi - klo, n, cfg_t)
        assert "%016x" % rg.fnv1a64(C_t) == want_hash, "K-sharded (transposed storage) result differs"
        # K ranges with the reduction started inside the MMA epilogue (peer stores into the row owners)
        fused = sharded.FusedKShard(n, n, cfg)
        A_k = torch.from_numpy(np.ascontiguousarray(A[:, klo:khi])).cuda()
        B_k = torch.from_numpy(np.ascontiguousarray(B[klo:khi])).cuda()
        for _ in range(3):              # the two receive buffers alternate
            C_f = fused(A_k, B_k, khi - klo, n)
            assert "%016x" % rg.fnv1a64(C_f) == want_hash, "fused K-shard result differs"
        # row-sharded output: every rank keeps its own rows only, back to back without a gather in between
        rows = n // world
        for _ in range(3):
            C_own = fused(A_k, B_k, khi - klo, n, gather=False)
            assert torch.equal(C_own.view(torch.int32), C_f.view(n, n)[rank * rows:(rank + 1) * rows].view(torch.int32))
        torch.cuda.synchronize()
        open(os.path.join(out_dir, "ok.%d" % rank), "w").close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_row_and_k_sharding_over_nccl(world, tmp_path):
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    with open(os.path.join(ROOT, "tests", "golden", "gemm_hashes.json")) as f:
        want = [r for r in json.load(f) if r["name"] == "c4.2048"][0]["out_hash"]
    mp.spawn(worker, args=(world, free_port(), 2048, want, str(tmp_path)), nprocs=world, join=True)
    assert sorted(os.listdir(tmp_path)) == ["ok.%d" % r for r in range(world)]
