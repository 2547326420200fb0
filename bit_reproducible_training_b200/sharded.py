"""Multi-GPU forms of the GEMM, one process per GPU over torch.distributed.

The reference is single-GPU (its README lists a deterministic multi-GPU reduction as still needed,
README.md:29-30).  Because the products are exact integers until the single final rounding, the
work can be cut in two ways without changing one output bit:

* rows of A: every rank owns a block of rows of op(A) and the whole of B.  Row scales and every
  T[i, j] are formed entirely on one rank, so there is no collective on the data path.
* K ranges: every rank owns a K range of both operands.  Ranks first agree on the row and column
  maxima (an element-wise max, exact and order-free), then form exact INT64 partial sums with the
  shared scales, add them with an integer reduction (associative, cannot overflow: |T| <= 2^62 is
  enforced for the whole K) and round once.  Over NCCL the reduction is a reduce-scatter by row
  blocks, each rank rounds its block, and an FP32 all-gather distributes C.

The arithmetic backend is a parameter so the sharding logic can be exercised on CPU ranks (gloo)
by the tests; the default backend is the CUDA library.
"""
import torch
import torch.distributed as dist

from . import repro_gemm as rg


def shard_range(n, world, rank):
    """Contiguous, balanced range of `n` items owned by `rank` out of `world`."""
    base, extra = divmod(n, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


class CudaBackend:
    """The shipped arithmetic: librgb200.so on the current CUDA device."""

    def gemm(self, A, B, M, N, K, cfg):
        return rg.gemm(A, B, M, N, K, cfg.trans_a, cfg.trans_b, cfg.slices, cfg.split_k, cfg.algo)

    def absmax(self, X, R, K, k_strided):
        return rg.absmax(X, R, K, k_strided)

    def gemm_partial(self, A, B, max_a, max_b, M, N, K, total_k, cfg):
        return rg.gemm_partial(A, B, max_a, max_b, M, N, K, total_k, cfg)

    def round_partial(self, T, max_a, max_b, M, N, slices):
        return rg.round_partial(T, max_a, max_b, M, N, slices)


def gemm_row_sharded(A_rows, B, m_local, N, K, cfg, backend=None, gather_group=None):
    """This rank's rows of C = op(A) op(B).  A_rows holds rows [lo, hi) of op(A) (for trans_a the
    stored matrix is K x m_local).  With `gather_group` the row blocks are all-gathered into the
    full C (plain FP32 copy; sizes may differ per rank)."""
    backend = backend or CudaBackend()
    C_rows = backend.gemm(A_rows, B, m_local, N, K, cfg)
    if gather_group is None:
        return C_rows
    world = dist.get_world_size(gather_group)
    sizes = [torch.zeros(1, dtype=torch.int64, device=C_rows.device) for _ in range(world)]
    dist.all_gather(sizes, torch.tensor([m_local], dtype=torch.int64, device=C_rows.device), group=gather_group)
    parts = [torch.empty((int(s.item()), N), dtype=torch.float32, device=C_rows.device) for s in sizes]
    if len({p.shape[0] for p in parts}) == 1:
        dist.all_gather(parts, C_rows.contiguous(), group=gather_group)
    else:
        for src, p in enumerate(parts):           # ragged row blocks: one broadcast per owner
            if src == dist.get_rank(gather_group):
                p.copy_(C_rows)
            dist.broadcast(p, src=dist.get_global_rank(gather_group, src), group=gather_group)
    return torch.cat(parts, dim=0)


def gemm_k_sharded(A_k, B_k, M, N, k_local, total_k, cfg, group=None, backend=None):
    """Full C on every rank from per-rank K ranges.  A_k is this rank's [M, k_local] block of op(A)
    (stored k_local x M when trans_a), B_k its [k_local, N] block of op(B) (N x k_local when trans_b)."""
    backend = backend or CudaBackend()
    max_a = backend.absmax(A_k, M, k_local, cfg.trans_a)          # k is the slow index iff trans_a
    max_b = backend.absmax(B_k, N, k_local, not cfg.trans_b)      # ... iff B is stored K x N
    dist.all_reduce(max_a, op=dist.ReduceOp.MAX, group=group)
    dist.all_reduce(max_b, op=dist.ReduceOp.MAX, group=group)
    T = backend.gemm_partial(A_k, B_k, max_a, max_b, M, N, k_local, total_k, cfg)
    world = dist.get_world_size(group)
    if world > 1 and M % world == 0 and dist.get_backend(group) == "nccl":
        # reduce-scatter the INT64 sums by row blocks, round only the own block, all-gather FP32:
        # 12 instead of 16 bytes per output cross the links and the rounding is shared between ranks
        rank = dist.get_rank(group)
        rows = M // world
        T_own = torch.empty((rows, N), dtype=torch.int64, device=T.device)
        dist.reduce_scatter_tensor(T_own, T, op=dist.ReduceOp.SUM, group=group)
        C_own = backend.round_partial(T_own, max_a[rank * rows:(rank + 1) * rows].contiguous(), max_b, rows, N, cfg.slices)
        C = torch.empty((M, N), dtype=torch.float32, device=T.device)
        dist.all_gather_into_tensor(C, C_own, group=group)
        return C
    dist.all_reduce(T, op=dist.ReduceOp.SUM, group=group)
    return backend.round_partial(T, max_a, max_b, M, N, cfg.slices)


class FusedKShard:
    """K-sharded product whose reduction starts inside the MMA kernel.

    Every rank owns M / world rows of the result.  The MMA kernel's epilogue stores the exact INT64
    sums of each row block directly into the owner's receive buffer (ordinary peer stores over NVLink,
    one contiguous kilobyte per warp-wide store thanks to a tile-native buffer layout, issued tile by
    tile while the rest of the product is still being computed), so the reduce-scatter
    of the collective form needs no separate pass over the data: after a stream-ordered barrier each
    owner adds its `world` slots, rounds once, and an FP32 all-gather distributes C.  Integer addition
    is exact in any order, so the bits equal the single-GPU product.

    The receive buffers live in torch symmetric memory (peer-mapped at rendezvous); the object is
    created once per shape and reused, nothing is mapped per call.  NCCL only.
    """

    def __init__(self, M, N, cfg, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        elems = rg.scatter_buffer_elems(M, N, self.world, cfg.slices)
        if elems == 0:
            raise ValueError("the fused K-shard needs M to be a multiple of 128 * world and at most 8 ranks")
        self.M, self.N, self.cfg, self.rows, self.elems = M, N, cfg, M // self.world, elems
        dev = torch.device("cuda", torch.cuda.current_device())
        # two receive buffers used in turn: a rank that is one product ahead stores into the other buffer, so a
        # slow owner can still be reading the previous product's slots (a rank cannot get two products ahead,
        # because each product ends with a collective every rank takes part in)
        self.slots = symm_mem.empty((2 * elems,), dtype=torch.int64, device=dev)
        self.handle = symm_mem.rendezvous(self.slots, self.group)
        self.owner_ptrs = [[int(p) + half * elems * 8 for p in self.handle.buffer_ptrs] for half in (0, 1)]
        self.phase = 0
        self.token = torch.zeros(1, dtype=torch.int32, device=dev)
        self.maxima = torch.empty(M + N, dtype=torch.float32, device=dev)
        self.launches_per_step = 7     # row max, column max, split A, split B, MMA, rounding (+ one more when B's split takes two kernels)

    def __call__(self, A_k, B_k, k_local, total_k, out=None, gather=True):
        """gather=True: the full C on every rank (FP32 all-gather of the owners' rows).  gather=False: only this rank's
        rows [rank * M / world, (rank + 1) * M / world) are returned, for callers that go on row-sharded."""
        cfg, M, N = self.cfg, self.M, self.N
        half = self.phase
        self.phase ^= 1
        # one buffer for both sets of maxima: a single max all-reduce instead of two
        maxima = self.maxima
        rg.absmax(A_k, M, k_local, cfg.trans_a, out=maxima[:M])
        rg.absmax(B_k, N, k_local, not cfg.trans_b, out=maxima[M:])
        dist.all_reduce(maxima, op=dist.ReduceOp.MAX, group=self.group)
        max_a, max_b = maxima[:M], maxima[M:]
        rg.gemm_partial_scatter(A_k, B_k, max_a, max_b, self.owner_ptrs[half], self.world, self.rank, M, N, k_local, total_k, cfg)
        # stream-ordered barrier: no rank reads its slots before every rank's kernel has finished writing them
        dist.all_reduce(self.token, group=self.group)
        lo = self.rank * self.rows
        own = self.slots[half * self.elems:(half + 1) * self.elems]
        if not gather:
            return rg.round_scattered(own, self.world, max_a[lo:lo + self.rows], max_b, self.rows, N, cfg.slices,
                                      out=out)
        C_own = rg.round_scattered(own, self.world, max_a[lo:lo + self.rows], max_b, self.rows, N, cfg.slices)
        C = out if out is not None else torch.empty((M, N), dtype=torch.float32, device=C_own.device)
        dist.all_gather_into_tensor(C.view(M, N), C_own, group=self.group)
        return C


class KSplitState:
    """Benchmark helper: this rank's operands are one K range of an M x N x (K * world) product."""
    launches_per_step = 7   # row max, column max, split A, split B, MMA, rounding (+ one more when B's split takes two kernels)

    def __init__(self, M, N, K, world, cfg, dA, dB, fused=False, gather=True):
        self.M, self.N, self.K, self.world, self.cfg, self.dA, self.dB = M, N, K, world, cfg, dA, dB
        self.fused = FusedKShard(M, N, cfg) if fused else None
        self.gather = gather
        if self.fused is not None:
            self.launches_per_step = self.fused.launches_per_step

    def step(self, dC):
        """dC: the full C (gather=True) or this rank's rows of it (fused form with gather=False)."""
        if self.fused is not None:
            self.fused(self.dA, self.dB, self.K, self.K * self.world, out=dC, gather=self.gather)
            return
        out = gemm_k_sharded(self.dA, self.dB, self.M, self.N, self.K, self.K * self.world, self.cfg)
        dC.copy_(out.reshape(-1))
