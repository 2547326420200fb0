"""The sharding logic of the multi-GPU modes on CPU ranks (gloo, world size 2 and 3).

The collectives and the partitioning are the shipped code (bit_reproducible_training_b200/sharded.py);
the arithmetic backend is replaced by the CPU oracle, which only this test may do."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from bit_reproducible_training_b200 import fixtures as fx
from bit_reproducible_training_b200 import repro_gemm as rg
from bit_reproducible_training_b200 import sharded


class OracleBackend:
    """Same four operations as sharded.CudaBackend, computed by the CPU oracle on CPU tensors."""

    def gemm(self, A, B, M, N, K, cfg):
        return torch.from_numpy(oracle.gemm(A.numpy(), B.numpy(), M, N, K, cfg.trans_a, cfg.trans_b, cfg.slices))

    def absmax(self, X, R, K, k_strided):
        return torch.from_numpy(oracle.absmax(X.numpy(), R, K, k_strided))

    def gemm_partial(self, A, B, max_a, max_b, M, N, K, total_k, cfg):
        return torch.from_numpy(oracle.gemm_partial(A.numpy(), B.numpy(), max_a.numpy(), max_b.numpy(), M, N, K,
                                                    cfg.trans_a, cfg.trans_b, cfg.slices, 0, K))

    def round_partial(self, T, max_a, max_b, M, N, slices):
        return torch.from_numpy(oracle.round_partials(T.numpy(), max_a.numpy(), max_b.numpy(), M, N, slices))


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        M, N, K = 61, 45, 333
        A, B = fx.hash_tool_inputs("stress", M, N, K)
        want = oracle.gemm(A, B, M, N, K)
        be = OracleBackend()
        for ta, tb in ((False, False), (True, True)):
            cfg = rg.Config(trans_a=ta, trans_b=tb)
            Am, Bm = A.reshape(M, K), B.reshape(K, N)
            # rows of A: no collective on the data path, then an optional gather of the row blocks
            lo, hi = sharded.shard_range(M, world, rank)
            a_rows = Am[lo:hi]
            a_rows = np.ascontiguousarray(a_rows.T if ta else a_rows)
            b_full = np.ascontiguousarray(Bm.T if tb else Bm)
            C_rows = sharded.gemm_row_sharded(torch.from_numpy(a_rows), torch.from_numpy(b_full), hi - lo, N, K, cfg, be)
            assert np.array_equal(C_rows.numpy().view(np.uint32), want[lo:hi].view(np.uint32))
            C_all = sharded.gemm_row_sharded(torch.from_numpy(a_rows), torch.from_numpy(b_full), hi - lo, N, K, cfg, be,
                                             gather_group=dist.group.WORLD)
            assert np.array_equal(C_all.numpy().view(np.uint32), want.view(np.uint32))
            # K ranges: max of maxima, INT64 sum of partials, one rounding
            klo, khi = sharded.shard_range(K, world, rank)
            a_k = Am[:, klo:khi]
            b_k = Bm[klo:khi]
            a_k = np.ascontiguousarray(a_k.T if ta else a_k)
            b_k = np.ascontiguousarray(b_k.T if tb else b_k)
            C_k = sharded.gemm_k_sharded(torch.from_numpy(a_k), torch.from_numpy(b_k), M, N, khi - klo, K, cfg,
                                         backend=be)
            assert np.array_equal(C_k.numpy().view(np.uint32), want.view(np.uint32))
        open(os.path.join(out_dir, "ok.%d" % rank), "w").close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_row_and_k_sharding_over_gloo(world, tmp_path):
    mp.spawn(worker, args=(world, free_port(), str(tmp_path)), nprocs=world, join=True)
    assert sorted(os.listdir(tmp_path)) == ["ok.%d" % r for r in range(world)]


def test_shard_range_partitions_exactly():
    for n in (1, 7, 64, 16384, 50257):
        for world in (1, 2, 3, 4, 8):
            cuts = [sharded.shard_range(n, world, r) for r in range(world)]
            assert cuts[0][0] == 0 and cuts[-1][1] == n
            assert all(cuts[i][1] == cuts[i + 1][0] for i in range(world - 1))
            sizes = [hi - lo for lo, hi in cuts]
            assert max(sizes) - min(sizes) <= 1
