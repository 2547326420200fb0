"""Behaviour of the entry points themselves: error codes, stage events, the convenience call,
the verification algorithm, and the K-range / row-block building blocks of the multi-GPU modes
(emulated on one GPU by running the shards one after another)."""
import numpy as np
import pytest
import torch

import oracle
from bit_reproducible_training_b200 import fixtures as fx
from bit_reproducible_training_b200 import repro_gemm as rg
from bit_reproducible_training_b200 import sharded

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_error_codes():
    M, N, K = 64, 48, 200
    A, B = dev(fx.Rng(1).normal(M * K)), dev(fx.Rng(2).normal(K * N))
    out = torch.empty(M * N, device="cuda")
    cfg = rg.Config()
    rc, plan = rg.make_plan(M, N, K, cfg)
    assert rc == 0 and plan.algo == rg.Algo.TensorCore and plan.split_k == 1
    ws = torch.empty(plan.workspace_bytes, dtype=torch.uint8, device="cuda")
    assert rg.repro_gemm_fp32_ws(None, B, out, M, N, K, cfg, ws) == rg.cudaErrorInvalidValue
    assert rg.repro_gemm_fp32_ws(A, None, out, M, N, K, cfg, ws) == rg.cudaErrorInvalidValue
    assert rg.repro_gemm_fp32_ws(A, B, None, M, N, K, cfg, ws) == rg.cudaErrorInvalidValue
    assert rg.repro_gemm_fp32_ws(A, B, out, M, N, K, cfg, ws[:plan.workspace_bytes - 1]) == rg.cudaErrorInvalidValue
    assert rg.repro_gemm_fp32_ws(A, B, out, M, N, K, cfg, None) == rg.cudaErrorInvalidValue
    assert rg.repro_gemm_fp32_ws(A, B, out, M, N, K, rg.Config(slices=4), ws) == rg.cudaErrorInvalidValue
    assert rg.repro_gemm_fp32_ws(A, B, out, M, N, K, rg.Config(split_k=0), ws) == rg.cudaErrorInvalidValue
    assert rg.repro_gemm_fp32_ws(A, B, out, 0, N, K, cfg, ws) == rg.cudaErrorInvalidValue
    assert rg.repro_gemm_fp32_ws(A, B, out, M, N, K, rg.Config(algo=rg.Algo.Tiled), ws) == rg.cudaErrorNotSupported
    assert rg.make_plan(M, N, 2_000_000, rg.Config(slices=3))[0] == rg.cudaErrorInvalidValue
    # a good call still works afterwards (no sticky error state)
    assert rg.repro_gemm_fp32_ws(A, B, out, M, N, K, cfg, ws) == 0
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError):
        rg.gemm(torch.zeros(M * K), torch.zeros(K * N), M, N, K)       # CPU tensors: there is no CPU path


def test_stage_events_are_recorded_in_order():
    n = 1024
    c = fx.config3(n)[0]
    A, B = dev(c["A"]), dev(c["B"])
    out = torch.empty(n * n, device="cuda")
    for split in (1, 4):
        cfg = rg.Config(split_k=split)
        rc, plan = rg.make_plan(n, n, n, cfg)
        ws = torch.empty(plan.workspace_bytes, dtype=torch.uint8, device="cuda")
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        for e in ev:
            e.record()
        assert rg.repro_gemm_fp32_ws(A, B, out, n, n, n, cfg, ws, stage_events=ev) == 0
        torch.cuda.synchronize()
        t = [ev[i].elapsed_time(ev[i + 1]) for i in range(3)]
        assert t[0] > 0 and t[1] > 0 and t[2] >= 0
        if split > 1:
            assert t[2] > 0          # the integer reduction + rounding kernel ran as the final step


def test_convenience_call_and_custom_stream():
    M, N, K = 200, 120, 900
    A, B = fx.hash_tool_inputs("weights", M, N, K)
    want = oracle.gemm(A, B, M, N, K)
    out = torch.full((M, N), float("nan"), device="cuda")
    assert rg.repro_gemm_fp32(dev(A), dev(B), out, M, N, K) == 0
    assert np.array_equal(out.cpu().numpy().view(np.uint32), want.view(np.uint32))
    s = torch.cuda.Stream()
    dA, dB = dev(A), dev(B)
    torch.cuda.synchronize()
    with torch.cuda.stream(s):
        got = rg.gemm(dA, dB, M, N, K)
    s.synchronize()
    assert np.array_equal(got.cpu().numpy().view(np.uint32), want.view(np.uint32))


def test_verification_algorithm_equals_tensor_core_path():
    M, N, K = 333, 257, 1500
    A, B = fx.hash_tool_inputs("stress", M, N, K)
    for S in (1, 2, 3):
        ref = rg.gemm(dev(A), dev(B), M, N, K, slices=S, algo=rg.Algo.Reference)
        tc = rg.gemm(dev(A), dev(B), M, N, K, slices=S, algo=rg.Algo.TensorCore)
        assert torch.equal(ref.view(torch.int32), tc.view(torch.int32))


def test_long_k_is_cut_into_int32_safe_ranges():
    """K beyond one INT32 pass (105516 at S = 3): the planner raises the K-range count by itself
    and the result still equals the oracle.  Inputs of maximal magnitude make the level sums as
    large as they can get."""
    M, N, K = 130, 70, 824 * 128 + 300
    A = np.ones(M * K, dtype=np.float32)
    B = np.ones(K * N, dtype=np.float32)
    A[::7] = -1.0
    rc, plan = rg.make_plan(M, N, K, rg.Config())
    assert rc == 0 and plan.split_k >= 2
    got = rg.gemm(dev(A), dev(B), M, N, K).cpu().numpy()
    want = oracle.gemm(A, B, M, N, K)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # one full pass at the bound, worst-case digits (all +-127 * 128^2 ... ) stays exact too
    K1 = 824 * 128
    A1 = np.full(8 * K1, 127.0, dtype=np.float32)
    B1 = np.full(K1 * 8, -127.0, dtype=np.float32)
    got = rg.gemm(dev(A1), dev(B1), 8, 8, K1).cpu().numpy()
    assert np.array_equal(got.view(np.uint32), oracle.gemm(A1, B1, 8, 8, K1).view(np.uint32))
    # every element with digits (-126, -64, -64): the middle level gains 2*126*64 + 64*64 = 20224 per k,
    # 2 133 066 368 over the whole pass, within 0.7 % of the INT32 limit.  156 output tiles keep the
    # planner from cutting K by itself, so this really is one accumulation pass.
    M2, N2 = 1536, 832
    rc, plan = rg.make_plan(M2, N2, K1, rg.Config())
    assert rc == 0 and plan.split_k == 1
    A2 = np.full(M2 * K1, -2072640.0, dtype=np.float32)
    B2 = np.full(K1 * N2, -2072640.0, dtype=np.float32)
    got = rg.gemm(dev(A2), dev(B2), M2, N2, K1).cpu().numpy()
    want = oracle.round_partials(np.full((1, 1, 1), 2072640 * 2072640 * K1, dtype=np.int64),
                                 np.float32([2072640.0]), np.float32([2072640.0]), 1, 1, 3)
    assert (got.view(np.uint32) == want.view(np.uint32)[0, 0]).all()      # every output is the same exact sum


@pytest.mark.parametrize("ta,tb", [(False, False), (True, False), (False, True), (True, True)])
def test_k_ranges_emulated_on_one_gpu(ta, tb):
    """The three K-shard calls, run for 3 uneven ranges one after another: maxima are combined with
    an element-wise max, the INT64 partials with an integer sum, and one rounding gives the bits of
    the unsharded product."""
    M, N, K = 150, 90, 1000
    A, B = fx.hash_tool_inputs("stress", M, N, K)
    want = oracle.gemm(A, B, M, N, K)
    Am, Bm = A.reshape(M, K), B.reshape(K, N)
    cuts = [(0, 130), (130, 131), (131, 1000)]
    shards = []
    for lo, hi in cuts:
        a = Am[:, lo:hi]
        b = Bm[lo:hi]
        shards.append((dev(a.T if ta else a), dev(b.T if tb else b), hi - lo))
    cfg = rg.Config(trans_a=ta, trans_b=tb)
    max_a = torch.stack([rg.absmax(a, M, k, ta) for a, _, k in shards]).amax(0)
    max_b = torch.stack([rg.absmax(b, N, k, not tb) for _, b, k in shards]).amax(0)
    assert np.array_equal(max_a.cpu().numpy(), oracle.absmax(A, M, K, False))
    assert np.array_equal(max_b.cpu().numpy(), oracle.absmax(B, N, K, True))
    parts = [rg.gemm_partial(a, b, max_a, max_b, M, N, k, K, cfg) for a, b, k in shards]
    for (lo, hi), T in zip(cuts, parts):
        wantT = oracle.gemm_partial(A, B, max_a.cpu().numpy(), max_b.cpu().numpy(), M, N, K, False, False, 3, lo, hi)
        assert np.array_equal(T.cpu().numpy(), wantT)
    got = rg.round_partial(torch.stack(parts).sum(0), max_a, max_b, M, N, 3)
    assert np.array_equal(got.cpu().numpy().view(np.uint32), want.view(np.uint32))
    stacked = rg.round_partial(torch.stack(parts), max_a, max_b, M, N, 3)        # the library sums the stack itself
    assert torch.equal(stacked.view(torch.int32), got.view(torch.int32))


def test_row_blocks_emulated_on_one_gpu():
    M, N, K = 500, 130, 640
    A, B = fx.hash_tool_inputs("wide", M, N, K)
    want = oracle.gemm(A, B, M, N, K)
    dB = dev(B)
    blocks = []
    for r in range(3):
        lo, hi = sharded.shard_range(M, 3, r)
        blocks.append(sharded.gemm_row_sharded(dev(A[lo * K:hi * K]), dB, hi - lo, N, K, rg.Config()))
    got = torch.cat(blocks).cpu().numpy()
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_repeated_runs_and_workspace_reuse_are_bit_stable():
    n = 768
    g = fx.Rng(9)
    A, B = dev(g.wide(n * n, -30, 30)), dev(g.normal(n * n))
    first = rg.gemm(A, B, n, n, n)
    other = rg.gemm(B, A, n, n, n)      # a different problem through the same cached workspace
    for _ in range(5):
        assert torch.equal(rg.gemm(A, B, n, n, n).view(torch.int32), first.view(torch.int32))
    assert not torch.equal(other, first)


def test_auto_k_ranges_for_few_tiles():
    """Few output tiles and a long K: the planner cuts K by itself (split_k left at 1) and the bits stay."""
    M, N, K = 256, 192, 8192
    rc, plan = rg.make_plan(M, N, K, rg.Config())
    assert rc == 0 and plan.split_k > 1
    A, B = fx.hash_tool_inputs("weights", M, N, K)
    got = rg.gemm(dev(A), dev(B), M, N, K).cpu().numpy()
    assert np.array_equal(got.view(np.uint32), oracle.gemm(A, B, M, N, K).view(np.uint32))


def test_workspace_call_inside_a_cuda_graph():
    """The allocation-free call is stream-ordered work only, so it can be captured once and replayed."""
    n = 512
    g = fx.Rng(5)
    A, B = dev(g.normal(n * n)), dev(g.normal(n * n))
    cfg = rg.Config()
    rc, plan = rg.make_plan(n, n, n, cfg)
    ws = torch.empty(plan.workspace_bytes, dtype=torch.uint8, device="cuda")
    out = torch.zeros(n * n, device="cuda")
    assert rg.repro_gemm_fp32_ws(A, B, out, n, n, n, cfg, ws) == 0          # first call: one-time set-up
    torch.cuda.synchronize()
    want = out.clone()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        assert rg.repro_gemm_fp32_ws(A, B, out, n, n, n, cfg, ws) == 0
    for _ in range(3):
        out.fill_(float("nan"))
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out.view(torch.int32), want.view(torch.int32))


def test_linear_layer_forward_and_backward():
    """Y = X W^T, dX = dY W, dW = dY^T X through autograd equal the oracle's three products."""
    from bit_reproducible_training_b200 import layers
    m, k, n = 96, 200, 72
    g = fx.Rng(31)
    X, W, dY = g.normal(m * k), g.normal(n * k, 0.02), g.normal(m * n, 1e-3)
    lin = layers.Linear(k, n, bias=False).cuda()
    with torch.no_grad():
        lin.weight.copy_(dev(W).view(n, k))
    x = dev(X).view(m, k).requires_grad_(True)
    y = lin(x)
    y.backward(dev(dY).view(m, n))
    assert np.array_equal(y.detach().cpu().numpy().view(np.uint32), oracle.gemm(X, W, m, n, k, False, True).view(np.uint32))
    assert np.array_equal(x.grad.cpu().numpy().view(np.uint32), oracle.gemm(dY, W, m, k, n).view(np.uint32))
    assert np.array_equal(lin.weight.grad.cpu().numpy().view(np.uint32),
                          oracle.gemm(dY, X, n, k, m, True, False).view(np.uint32))


def test_suite_tool_writes_reference_format(tmp_path):
    from bit_reproducible_training_b200 import suite
    from test_oracle import SUITE_HASHES
    path = tmp_path / "gpu.txt"
    lines = suite.run(tokens=1024, reps=1, out=str(path))
    assert lines[0].startswith("# GPU")
    ops = [l.split("\t") for l in lines[1:]]
    assert len(ops) == 21
    for f in ops:
        assert f[0] == "OP" and (f[3][3:], f[4][4:]) == SUITE_HASHES[f[1]]


def test_host_buffer_pipeline_matches_single_call():
    """Pinned host operands in, pinned host result out, row blocks overlapped with the copies: same bits
    as one call, for plain and transposed storage (a row block of a transposed A is a band of columns of the
    stored matrix and travels as a pitched copy)."""
    M, N, K = 1100, 260, 520
    A, B = fx.hash_tool_inputs("wide", M, N, K)
    want = oracle.gemm(A, B, M, N, K)
    hA, hB = torch.from_numpy(A).pin_memory(), torch.from_numpy(B).pin_memory()
    hC = torch.empty(M * N).pin_memory()
    for block_rows in (128, 300, 4096):
        pipe = rg.HostGemm(M, N, K, rg.Config(), block_rows=block_rows)
        for _ in range(2):
            hC.fill_(float("nan"))
            pipe(hA, hB, hC)
            torch.cuda.synchronize()
            assert np.array_equal(hC.numpy().view(np.uint32), want.view(np.uint32).reshape(-1)), block_rows
    hAt = torch.from_numpy(np.ascontiguousarray(A.reshape(M, K).T).reshape(-1)).pin_memory()
    hBt = torch.from_numpy(np.ascontiguousarray(B.reshape(K, N).T).reshape(-1)).pin_memory()
    for cfg, a, b in ((rg.Config(trans_a=True), hAt, hB), (rg.Config(trans_a=True, trans_b=True), hAt, hBt),
                      (rg.Config(trans_b=True), hA, hBt)):
        pipe = rg.HostGemm(M, N, K, cfg, block_rows=512)
        hC.fill_(float("nan"))
        pipe(a, b, hC)
        torch.cuda.synchronize()
        assert pipe.blocks == 3 and pipe.status() == 0
        assert np.array_equal(hC.numpy().view(np.uint32), want.view(np.uint32).reshape(-1)), cfg
        pipe.close()


def test_host_buffer_pipeline_short_last_block_with_own_k_ranges():
    """A short last block can plan K ranges (few tiles) and then needs more workspace than the full
    blocks do: the pipeline sizes its workspace for every block height."""
    M, N, K = 512 + 128, 2432, 4096
    assert rg.make_plan(512, N, K, rg.Config())[1].split_k == 1 and rg.make_plan(128, N, K, rg.Config())[1].split_k > 1
    g = fx.Rng(77)
    A, B = g.normal(M * K), g.normal(K * N)
    want = rg.gemm(dev(A), dev(B), M, N, K).cpu().numpy()
    hA, hB, hC = torch.from_numpy(A).pin_memory(), torch.from_numpy(B).pin_memory(), torch.empty(M * N).pin_memory()
    pipe = rg.HostGemm(M, N, K, rg.Config(), block_rows=512)
    pipe(hA, hB, hC)
    torch.cuda.synchronize()
    # kernels per call: B's split once (one kernel: the cluster form), A's split + MMA per block, one K-range reduction
    # for the short block
    assert pipe.blocks == 2 and pipe.launches == 1 + 2 + 3
    assert np.array_equal(hC.numpy().view(np.uint32), want.view(np.uint32).reshape(-1))


def test_bounded_wait_expires_and_reports():
    """Failure detection without a fault: a wait that nothing will satisfy runs into its (short) limit,
    leaves a status code, makes the other waiting role leave too, and the device keeps working."""
    import ctypes as C
    from bit_reproducible_training_b200 import _lib
    status, waited, both = C.c_int(-1), C.c_longlong(0), C.c_int(0)
    limit = 2_000_000                                   # about a millisecond
    rc = _lib.lib().rgb200_selftest_bounded_wait(limit, C.byref(status), C.byref(waited), C.byref(both))
    assert rc == 0
    assert status.value == 2                            # the code of the role that gave up
    assert both.value == 1                              # the second role saw the abort flag and left
    assert limit < waited.value < 200 * limit           # it did wait for the limit, and not much longer
    n = 256                                             # the context is intact: a GEMM still runs and is exact
    g = fx.Rng(12)
    A, B = g.normal(n * n), g.normal(n * n)
    got = rg.gemm(dev(A), dev(B), n, n, n).cpu().numpy()
    assert np.array_equal(got.view(np.uint32), oracle.gemm(A, B, n, n, n).view(np.uint32))


def test_scatter_epilogue_emulated_on_one_gpu():
    """The row-block scatter of the INT64 sums, with three "ranks" run one after another on one GPU
    and all receive buffers local: each owner's slots, added and rounded once, give its rows of C."""
    for world, M, N, K, S in ((3, 384, 200, 900, 3), (2, 512, 1000, 300, 1), (2, 256, 330, 260, 2)):
        A, B = fx.hash_tool_inputs("stress", M, N, K)
        want = oracle.gemm(A, B, M, N, K, S=S)
        Am, Bm = A.reshape(M, K), B.reshape(K, N)
        rows = M // world
        elems = rg.scatter_buffer_elems(M, N, world, S)
        assert elems >= world * rows * N
        bufs = [torch.full((elems,), -7, dtype=torch.int64, device="cuda") for _ in range(world)]
        ptrs = [b.data_ptr() for b in bufs]
        cuts = [sharded.shard_range(K, world, r) for r in range(world)]
        shards = [(dev(Am[:, lo:hi]), dev(Bm[lo:hi]), hi - lo) for lo, hi in cuts]
        cfg = rg.Config(slices=S)
        max_a = torch.stack([rg.absmax(a, M, k, False) for a, _, k in shards]).amax(0)
        max_b = torch.stack([rg.absmax(b, N, k, True) for _, b, k in shards]).amax(0)
        for r, (a, b, k) in enumerate(shards):
            rg.gemm_partial_scatter(a, b, max_a, max_b, ptrs, world, r, M, N, k, K, cfg)
        torch.cuda.synchronize()
        for o in range(world):
            got = rg.round_scattered(bufs[o], world, max_a[o * rows:(o + 1) * rows], max_b, rows, N, S).cpu().numpy()
            assert np.array_equal(got.view(np.uint32), want[o * rows:(o + 1) * rows].view(np.uint32)), (world, S, o)
    assert rg.scatter_buffer_elems(300, 64, 2, 3) == 0          # rows per owner must be whole 128-row tiles


def test_wrappers_check_the_status_word_when_asked(monkeypatch):
    """RGB200_CHECK_STATUS=1: gemm and gemm_batched synchronise and read the workspace's status word; a run whose
    waits all completed passes the check and returns the same bits."""
    import numpy as np
    g = fx.Rng(77)
    M, N, K = 130, 70, 200
    A, B = g.normal(M * K), g.normal(K * N)
    monkeypatch.delenv("RGB200_CHECK_STATUS", raising=False)
    plain = rg.gemm(torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda(), M, N, K).cpu().numpy()
    monkeypatch.setenv("RGB200_CHECK_STATUS", "1")
    checked = rg.gemm(torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda(), M, N, K).cpu().numpy()
    assert np.array_equal(plain.view(np.uint32), checked.view(np.uint32))
    out = rg.gemm_batched(torch.from_numpy(np.concatenate([A, A])).cuda(), torch.from_numpy(np.concatenate([B, B])).cuda(), 2, M, N, K)
    assert np.array_equal(out[1].cpu().numpy().view(np.uint32), plain.view(np.uint32))
