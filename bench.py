"""Benchmark of the integer-exact FP32 GEMM path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--no-ksplit] [--no-c4] [--no-cpu-baseline] [--int8-library-yardstick]
    python bench.py --workload c1|c2|c4|c5                            (the other GEMM configurations, one GPU)
    python bench.py --workload conv-lenet1|conv-lenet2|conv-mid|conv-small|conv-5x5   (one convolution layer, one GPU)

One step = one full pass of the hot path (split pre-pass, int8 MMA mainloop, fused rounding
epilogue) over one 4096 x 4096 x 4096, S = 3 GEMM with the wide-dynamic-range synthetic inputs.
With N > 1 GPUs (torchrun, one rank per GPU) the headline line shards rows of A: every rank owns a
4096-row block of a (4096 N) x 4096 x 4096 product and the whole B; no collective is on the data
path (weak scaling).  The same run then times, as sub-records of the line,
  * "ksplit" / "ksplit_fused": every rank holds a 4096-wide K range of a 4096 x 4096 x (4096 N) product;
    the exact INT64 partial sums are reduced with NCCL, or stored by the MMA epilogue straight into the
    owning rank's memory;
  * "c4": the 16384^3 product of configuration 4 sharded over the N ranks by rows of A and by K ranges
    (strong scaling: the total work is fixed).
Every timed variant's output is hashed (FNV-1a-64) and compared with the value the reference's CPU
implementation produced for the same seeded inputs; a mismatch makes the run exit with status 3, as
the reference's own benchmark refuses a timing whose hash is wrong
(repro_gemm_cuda/bench_repro_gemm.cu:62-68,116,149).

Prints one JSON line (rank 0).  `value` is 2 M N K / time summed over ranks with the inputs
resident in HBM; `e2e` repeats the measurement through the host-buffer entry point of the C ABI
(rgb200_gemm_fp32_host: pinned host memory, copies inside the timed region, overlapped with compute
block by block) and reports beside it what plain copies of the same bytes take (`e2e.pcie`).
--impl reference times the reference's CPU implementation (oracle/_ref, built from the reference's
sources) on a bounded sample of the same workload.
"""
import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SIZE = 4096
SLICES = 3
METRIC = "bit-exact FP32 GEMM TFLOP/s (2MNK/t), S=3, 4096^3"
WORKLOAD = ("C=A.B fp32, M=N=K=4096 per GPU, S=3 int8 slices, wide-dynamic-range inputs "
            "(1% zeros, 0.1% subnormals), seed 3")
NOMINAL_INT8_TOPS = 4500.0
# dram__bytes_read.sum + dram__bytes_write.sum of one MMA-kernel launch at this workload, from one ncu
# capture of that launch (193.0 MB read + 53.3 MB written); a constant, not re-measured by a bench run
MMA_DRAM_TRAFFIC_BYTES = 246.3e6
GOLDEN = os.path.join(ROOT, "tests", "golden", "gemm_hashes.json")


def golden_record(name, slices=SLICES):
    with open(GOLDEN) as f:
        return [r for r in json.load(f) if r["name"] == name and r["S"] == slices][0]


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "source": "measured"}
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """Polls SM clock and clock-event (throttle) reasons through NVML from a thread while the timed
    region runs.  Read-only: nothing about the GPU is changed."""
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, torch_index):
        self.samples, self.reasons, self.max_mhz, self.stop_flag, self.thread, self.err = [], set(), None, False, None, None
        try:
            import pynvml
            import torch
            pynvml.nvmlInit()
            self.nv = pynvml
            try:
                uuid = "GPU-" + str(torch.cuda.get_device_properties(torch_index).uuid)
                self.h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(torch_index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception as e:      # NVML missing: report that instead of clocks
            self.nv, self.err = None, repr(e)

    def _poll(self):
        nv = self.nv
        while not self.stop_flag:
            try:
                self.samples.append(float(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception as e:
                self.err = repr(e)
                return
            time.sleep(0.002)

    def start(self):
        if self.nv is not None:
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()

    def stop(self):
        self.stop_flag = True
        if self.thread is not None:
            self.thread.join(timeout=5)
        out = {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
               "reasons": sorted(self.reasons), "samples": len(self.samples)}
        if self.err:
            out["error"] = self.err
        return out


def cpu_reference_run(steps, warmup, sample_rows):
    """Times the reference's cpu_gemm (or the restated oracle if that library is absent) on the first
    `sample_rows` rows of A against the whole B.  Returns (TFLOP/s, seconds per step, info)."""
    import oracle
    g = oracle.Rng(3)                          # configuration 3's stream: A first, then B
    A = g.wide_mixed(SIZE * SIZE)[:sample_rows * SIZE]
    B = g.wide_mixed(SIZE * SIZE)
    use_ref = oracle.ref() is not None
    fn = (lambda: oracle.ref_gemm(A, B, sample_rows, SIZE, SIZE, False, False, SLICES)) if use_ref else \
         (lambda: oracle.gemm(A, B, sample_rows, SIZE, SIZE, False, False, SLICES))
    for _ in range(warmup):
        fn()
    t0 = time.perf_counter()
    for _ in range(steps):
        fn()
    dt = (time.perf_counter() - t0) / max(steps, 1)
    tflops = 2.0 * sample_rows * SIZE * SIZE / dt / 1e12
    info = {"value": tflops, "unit": "TFLOP/s", "cores": oracle.default_threads(),
            "kind": "reference" if use_ref else "port",
            "sample": "rows 0..%d of A times all of B (%dx%dx%d of the %d^3 workload), %d step(s)" %
                      (sample_rows - 1, sample_rows, SIZE, SIZE, SIZE, steps)}
    return tflops, dt, info


def reference_arm(args, rank):
    if rank != 0:
        return
    tflops, dt, info = cpu_reference_run(args.steps, min(args.warmup, 1), 512)
    line = {"impl": "reference", "metric": METRIC, "value": tflops, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": min(args.warmup, 1), "ms_per_step": dt * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "int64", "data": "synthetic",
            "config": {"workload": WORKLOAD, "sharding": "none (rank 0 only, host cores)", "cpu_sample": info["sample"]},
            "cpu_baseline": info,
            "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def auxiliary_workload(args):
    """Times one of the other four configurations on one GPU (device-resident inputs, CUDA events,
    L2 flushed between steps) and checks its output hash against the golden file."""
    import torch
    from bit_reproducible_training_b200 import fixtures as fx
    from bit_reproducible_training_b200 import repro_gemm as rg
    torch.cuda.set_device(0)
    if args.workload == "c4":       # the large operands are generated on the device (same bits, far quicker)
        A, B = fx.config4_device("cuda")
        cases = [dict(name="c4.16384", M=16384, N=16384, K=16384, trans_a=False, trans_b=False, A=A, B=B)]
    elif args.workload == "c5":
        Q, Km, V, P = fx.config5_device("cuda")
        cases = [dict(name="c5.QKt", batch=96, M=1024, N=1024, K=64, trans_a=False, trans_b=True, A=Q, B=Km),
                 dict(name="c5.PV", batch=96, M=1024, N=64, K=1024, trans_a=False, trans_b=False, A=P, B=V)]
    else:
        cases = {"c1": fx.config1, "c2": fx.config2}[args.workload]()
    with open(GOLDEN) as f:
        golden = {(r["name"], r["S"]): r["out_hash"] for r in json.load(f)}
    flush = torch.empty(512 << 20, dtype=torch.uint8, device="cuda")
    prepared, flops = [], 0.0
    for c in cases:
        batch = c.get("batch", 1)
        M, N, K = c["M"], c["N"], c["K"]
        cfg = rg.Config(slices=SLICES, trans_a=c["trans_a"], trans_b=c["trans_b"])
        rc, plan = rg.make_plan(M, N, K, cfg, batch=batch)
        if rc != 0:
            raise rg.ReproGemmError(rc, "make_plan")
        on_dev = lambda x: x if isinstance(x, torch.Tensor) else torch.from_numpy(x).cuda()
        prepared.append((c, cfg, batch, on_dev(c["A"]), on_dev(c["B"]),
                         torch.empty(batch * M * N, dtype=torch.float32, device="cuda"),
                         torch.empty(plan.workspace_bytes, dtype=torch.uint8, device="cuda")))
        flops += 2.0 * batch * M * N * K

    def run(item):
        c, cfg, batch, dA, dB, dC, ws = item
        M, N, K = c["M"], c["N"], c["K"]
        if batch == 1:
            rc = rg.repro_gemm_fp32_ws(dA, dB, dC, M, N, K, cfg, ws)
        else:
            rc = rg.repro_gemm_fp32_batched_ws(dA, dB, dC, M, N, K, batch, M * K, K * N, M * N, cfg, ws)
        if rc != 0:
            raise rg.ReproGemmError(rc, c["name"])

    warmup = max(args.warmup, 3)
    peaks = measured_peaks()
    per_case, total_ms, ok = [], 0.0, True
    for item in prepared:                      # every case is timed by itself, L2 flushed before each run
        c, cfg, batch, dA, dB, dC, ws = item
        for _ in range(warmup):
            flush.zero_()
            run(item)
        torch.cuda.synchronize()
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
        for a, b in ev:
            flush.zero_()
            a.record()
            run(item)
            b.record()
        torch.cuda.synchronize()
        ms = statistics.mean(a.elapsed_time(b) for a, b in ev)
        total_ms += ms
        name = c["name"] + (".b%d" % batch if "batch" in c else "")
        want = golden.get((name, SLICES))
        match = want is not None and ("%016x" % rg.fnv1a64(dC)) == want
        ok = ok and match
        M, N, K = c["M"], c["N"], c["K"]
        # algorithmic bytes of a whole call: (4 + S) per operand element (one FP32 read, S digit bytes) + 4 per output
        nbytes = batch * ((4.0 + SLICES) * (M * K + N * K) + 4.0 * M * N)
        gbs = nbytes / (ms * 1e-3) / 1e9
        per_case.append({"name": name, "ms": ms, "tflops": 2.0 * batch * M * N * K / (ms * 1e-3) / 1e12,
                         "output_matches_golden": match,
                         "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                      "frac": gbs / peaks["hbm_gbs"], "algorithmic_bytes": nbytes},
                         "int8_frac_of_nominal_4500": 2.0 * SLICES * SLICES * batch * M * N * K / (ms * 1e-3) / 1e12 / NOMINAL_INT8_TOPS})
    line = {"metric": "bit-exact FP32 GEMM TFLOP/s (2MNK/t), S=3", "value": flops / (total_ms * 1e-3) / 1e12,
            "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
            "ms_per_step": total_ms, "higher_is_better": True, "dtype": "int8", "data": "synthetic",
            "auxiliary": True, "output_matches_golden": ok, "cases": per_case,
            "config": {"workload": args.workload + ": " + ", ".join(
                "%s %s%dx%dx%d" % (c["name"], ("%d x " % c["batch"]) if "batch" in c else "", c["M"], c["N"], c["K"])
                for c in cases), "l2": "512 MiB buffer written between timed iterations (L2 flush)",
                "peaks": peaks["source"]}}
    worst = min(per_case, key=lambda r: r["roofline"]["frac"])
    line["roofline"] = dict(worst["roofline"], kernel="whole call of " + worst["name"] + " (pre-pass + MMA + epilogue)")
    print(json.dumps(line), flush=True)
    if not ok:
        sys.exit(3)


CONV_BENCH_SHAPES = {
    # the two layers the reference's own convolution benchmark times (repro_conv_cuda/bench_repro_conv.cu:64-66)
    "conv-lenet1": (100, 1, 28, 28, 6, 5, 5, 1, 1, 2, 2),
    "conv-lenet2": (100, 6, 14, 14, 16, 5, 5, 1, 1, 0, 0),
    # a mid-size layer (64 -> 64 channels, 3 x 3, 56 x 56 images, batch 32) where the products are large enough for tensor cores
    "conv-mid": (32, 64, 56, 56, 64, 3, 3, 1, 1, 1, 1),
    # two more layers with enough channels for tensor cores: 16 -> 32 channels 3 x 3 on 32 x 32, 32 -> 64 channels 5 x 5 on 28 x 28
    "conv-small": (32, 16, 32, 32, 32, 3, 3, 1, 1, 1, 1),
    "conv-5x5": (64, 32, 28, 28, 64, 5, 5, 1, 1, 2, 2),
}


def conv_workload(args):
    """Times the convolution forward, weight gradient and input gradient of one layer on one GPU (device-resident
    tensors, CUDA events, L2 flushed between steps), checks the three results against the reference's CPU code
    (or the restated oracle where that library is absent) and times that CPU code beside it."""
    import torch
    import oracle
    from bit_reproducible_training_b200 import fixtures as fx
    from bit_reproducible_training_b200 import repro_conv as rc
    from bit_reproducible_training_b200 import repro_gemm as rg
    torch.cuda.set_device(0)
    shape = CONV_BENCH_SHAPES[args.workload]
    g = rc.ConvShape(*shape)
    x, w, dy = fx.conv_inputs(shape)
    dx_, dw_, ddy = (torch.from_numpy(t).cuda() for t in (x, w, dy))
    calls = []
    for name, query, fn, a, b, n_out in (
            ("forward", rc.conv2d_workspace, rc.repro_conv2d_ws, dx_, dw_, g.output_size()),
            ("grad_weight", rc.conv2d_grad_weight_workspace, rc.repro_conv2d_grad_weight_ws, ddy, dx_, g.weight_size()),
            ("grad_input", rc.conv2d_grad_input_workspace, rc.repro_conv2d_grad_input_ws, ddy, dw_, g.input_size())):
        code, nbytes = query(g, SLICES)
        if code != 0:
            raise rg.ReproGemmError(code, name + " workspace")
        calls.append((name, fn, a, b, torch.empty(n_out, dtype=torch.float32, device="cuda"),
                      torch.empty(nbytes, dtype=torch.uint8, device="cuda")))
    flush = torch.empty(512 << 20, dtype=torch.uint8, device="cuda")

    def run(call):
        name, fn, a, b, out, ws = call
        code = fn(a, b, out, g, SLICES, ws)
        if code != 0:
            raise rg.ReproGemmError(code, name)

    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        for call in calls:
            run(call)
    torch.cuda.synchronize()
    ms = {}
    for call in calls:
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
        for a, b in ev:
            flush.zero_()
            a.record()
            run(call)
            b.record()
        torch.cuda.synchronize()
        ms[call[0]] = statistics.median(a.elapsed_time(b) for a, b in ev)
    total_ms = sum(ms.values())
    flops = 3 * 2.0 * g.windows() * g.F * g.K()

    use_ref = oracle.ref_conv() is not None
    cpu_fns = (oracle.ref_conv2d, oracle.ref_conv2d_grad_weight, oracle.ref_conv2d_grad_input) if use_ref else \
              (oracle.conv2d, oracle.conv2d_grad_weight, oracle.conv2d_grad_input)
    t0 = time.perf_counter()
    want = [cpu_fns[0](x, w, shape, SLICES), cpu_fns[1](dy, x, shape, SLICES), cpu_fns[2](dy, w, shape, SLICES)]
    cpu_s = time.perf_counter() - t0
    ok = all(rg.fnv1a64(call[4]) == oracle.fnv1a64(ref) for call, ref in zip(calls, want))
    peaks = measured_peaks()
    mma_ops = 2.0 * SLICES * SLICES * g.windows() * g.F * g.K()
    achieved = mma_ops / (ms["forward"] * 1e-3) / 1e12
    print(json.dumps({
        "metric": "bit-exact conv2d forward + both gradients, effective TFLOP/s (3 x 2 x windows x F x K / t), S=3",
        "value": flops / (total_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": total_ms, "higher_is_better": True, "dtype": "int8", "data": "synthetic", "auxiliary": True,
        "output_matches_cpu_reference": ok, "stages": {k + "_ms": v for k, v in ms.items()},
        "config": {"workload": "%s: x[%d,%d,%d,%d], weight[%d,%d,%d,%d], stride (%d,%d), padding (%d,%d); %d windows of %d values"
                               % (args.workload, g.N, g.C, g.H, g.W, g.F, g.C, g.KH, g.KW, g.SY, g.SX, g.PY, g.PX, g.windows(), g.K()),
                   "l2": "512 MiB buffer written between timed iterations (L2 flush)"},
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": 2.0 * peaks["bf16_tflops"], "unit": "TFLOP/s",
                     "frac": achieved / (2.0 * peaks["bf16_tflops"]), "traffic": None,
                     "note": "whole forward call (gather pre-pass + MMA kernel), int8 ops of the slice-pair MMAs on the "
                             "unpadded problem; peak = 2 x the %s dense bf16 cuBLAS rate" % peaks["source"]},
        "cpu_baseline": {"value": flops / cpu_s / 1e12, "unit": "TFLOP/s", "cores": oracle.default_threads(),
                         "kind": "reference" if use_ref else "port",
                         "sample": "the whole layer once: forward, weight gradient, input gradient (%.2f s)" % cpu_s}}), flush=True)


def _max_over_ranks(x, world):
    import torch
    import torch.distributed as dist
    if world == 1:
        return float(x)
    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _all_ranks_true(flag, world):
    import torch
    import torch.distributed as dist
    if world == 1:
        return bool(flag)
    t = torch.tensor([1 if flag else 0], dtype=torch.int32, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    return bool(t.item())


def _barrier(world):
    import torch
    import torch.distributed as dist
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


def timed_loop(step, steps, warmup, flush, world):
    """`warmup` untimed and `steps` timed calls of step(), the L2 flushed before each, one CUDA-event pair per
    call on the current stream, barriers on both sides.  Returns (sum of the step times in ms, maximum over
    ranks; the per-step list of this rank)."""
    import torch
    for _ in range(warmup):
        flush.zero_()
        step()
    _barrier(world)
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for a, b in ev:
        flush.zero_()
        a.record()
        step()
        b.record()
    _barrier(world)
    per_step = [a.elapsed_time(b) for a, b in ev]
    return _max_over_ranks(sum(per_step), world), per_step


def measure_pcie(hA, hB, hC, dA, dB, dC, world, reps=5):
    """What the link allows for one step's bytes: plain cudaMemcpyAsync copies (one per buffer) of A and B to
    the device, of C back, and of both directions at once on two streams; all ranks copy at the same time,
    the slowest rank counts.  Median of `reps`."""
    import torch
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()

    def once(h2d, d2h):
        _barrier(world)
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        cur = torch.cuda.current_stream()
        e0.record(cur)
        s1.wait_event(e0)
        s2.wait_event(e0)
        if h2d:
            with torch.cuda.stream(s1):
                dA.copy_(hA, non_blocking=True)
                dB.copy_(hB, non_blocking=True)
        if d2h:
            with torch.cuda.stream(s2):
                hC.copy_(dC, non_blocking=True)
        e1.record(s1)
        e2.record(s2)
        torch.cuda.synchronize()
        return max(e0.elapsed_time(e1), e0.elapsed_time(e2))

    out = {}
    for key, h2d, d2h in (("h2d_ms", True, False), ("d2h_ms", False, True), ("duplex_ms", True, True)):
        once(h2d, d2h)
        out[key] = _max_over_ranks(statistics.median(once(h2d, d2h) for _ in range(reps)), world)
    nin, nout = (hA.numel() + hB.numel()) * 4, hC.numel() * 4
    out["h2d_gbs"] = nin / (out["h2d_ms"] * 1e-3) / 1e9
    out["d2h_gbs"] = nout / (out["d2h_ms"] * 1e-3) / 1e9
    out["ranks_copying_at_once"] = world
    out["how"] = "plain cudaMemcpyAsync of the step's buffers from/to pinned memory, one copy per buffer; duplex = both directions at once"
    return out


def ksplit_records(args, world, rank, dA, dB, dC, cfg, flush, rows_ms):
    """The 4096 x 4096 x (4096 N) product with one K range per rank, NCCL form and fused form."""
    import torch
    from bit_reproducible_training_b200 import repro_gemm as rg
    from bit_reproducible_training_b200 import sharded
    M = N = K = SIZE
    want = golden_record("c3.4096.kcat%d" % world)["out_hash"] if world in (2, 4, 8) else None
    out = {}
    steps = min(args.steps, 20)
    own = M // world
    for key, fused in (("ksplit", False), ("ksplit_fused", True)):
        ks = sharded.KSplitState(M, N, K, world, cfg, dA, dB, fused=fused)
        dC.fill_(float("nan"))
        total_ms, _ = timed_loop(lambda: ks.step(dC), steps, 3, flush, world)
        ms = total_ms / steps
        ok = None
        if want is not None:
            ok = _all_ranks_true(("%016x" % rg.fnv1a64(dC)) == want, world)
        # bytes this rank sends: its INT64 sums for the other owners' row blocks, then its rounded FP32 rows to the others
        comm = (world - 1) * own * N * 8 + (world - 1) * own * N * 4 + (M + N) * 4
        out[key] = {"ms_per_step": ms, "value": 2.0 * M * N * K * world / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                    "steps": steps, "efficiency_vs_rows": rows_ms / ms, "matches_golden": ok,
                    "comm_bytes_per_rank": comm, "launches_per_step": ks.launches_per_step,
                    "what": ("K ranges; maxima all-reduce, INT64 reduce-scatter by row blocks (NCCL), one rounding per owner, FP32 all-gather"
                             if not fused else
                             "K ranges; maxima all-reduce, MMA epilogue stores INT64 tiles into the row owners over NVLink, one rounding per owner, FP32 all-gather")}
        del ks
        torch.cuda.empty_cache()
    # the fused form leaving C sharded by rows (no FP32 all-gather): each rank's rows must equal the rows of the
    # gathered result just verified
    ks = sharded.KSplitState(M, N, K, world, cfg, dA, dB, fused=True, gather=False)
    C_own = torch.full((own, N), float("nan"), dtype=torch.float32, device="cuda")
    total_ms, _ = timed_loop(lambda: ks.step(C_own), steps, 3, flush, world)
    ms = total_ms / steps
    same = _all_ranks_true(torch.equal(C_own.view(-1).view(torch.int32), dC[rank * own * N:(rank + 1) * own * N].view(torch.int32)), world)
    out["ksplit_fused"]["row_sharded_output"] = {
        "ms_per_step": ms, "value": 2.0 * M * N * K * world / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
        "efficiency_vs_rows": rows_ms / ms, "matches_golden": bool(same and out["ksplit_fused"]["matches_golden"]),
        "comm_bytes_per_rank": (world - 1) * own * N * 8 + (M + N) * 4,
        "what": "as ksplit_fused, but every rank keeps only its M/N rows of C (no FP32 all-gather)"}
    del ks
    torch.cuda.empty_cache()
    return out


def c4_records(args, world, rank, flush):
    """Configuration 4 (16384^3, S = 3) over the ranks: rows of A (no collective) and K ranges (both forms).
    Every rank checks its own 2048-row blocks of the result against the reference's hashes."""
    import torch
    from bit_reproducible_training_b200 import fixtures as fx
    from bit_reproducible_training_b200 import repro_gemm as rg
    from bit_reproducible_training_b200 import sharded
    n = 16384
    rec = golden_record("c4.16384")
    blk = rec["row_block_hashes"]["rows"]
    hashes = rec["row_block_hashes"]["hashes"]
    cfg = rg.Config(slices=SLICES)
    own = n // world
    lo = rank * own
    steps, warm = 5, 3
    flops = 2.0 * n * n * n

    def blocks_match(C_rows, first_row):
        ok = True
        for r0 in range(0, C_rows.shape[0], blk):
            ok = ok and ("%016x" % rg.fnv1a64(C_rows[r0:r0 + blk])) == hashes[(first_row + r0) // blk]
        return _all_ranks_true(ok, world)

    out = {"workload": "C=A.B fp32, M=N=K=16384 in total, S=3, uniform[-1,1) inputs, seed 4", "scaling": "strong"}
    # rows of A
    A_rows, B = fx.config4_device("cuda", n, a_rows=(lo, lo + own))
    rc, plan = rg.make_plan(own, n, n, cfg)
    if rc != 0:
        raise rg.ReproGemmError(rc, "make_plan c4 rows")
    ws = torch.empty(plan.workspace_bytes, dtype=torch.uint8, device="cuda")
    C_rows = torch.full((own, n), float("nan"), dtype=torch.float32, device="cuda")

    def rows_step():
        code = rg.repro_gemm_fp32_ws(A_rows, B, C_rows, own, n, n, cfg, ws)
        if code != 0:
            raise rg.ReproGemmError(code, "c4 rows")
    total_ms, _ = timed_loop(rows_step, steps, warm, flush, world)
    rows_ms = total_ms / steps
    out["rows"] = {"ms_per_step": rows_ms, "value": flops / (rows_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "steps": steps,
                   "matches_golden": blocks_match(C_rows, lo), "comm_bytes_per_rank": 0,
                   "what": "rank r computes rows [r*16384/N, (r+1)*16384/N) against the whole B; no collective"}
    del A_rows, B, ws, C_rows
    torch.cuda.empty_cache()
    if world == 1 or args.no_ksplit:
        return out
    # K ranges
    A_k, B_k = fx.config4_device_k_range("cuda", n, lo, lo + own)
    C_full = torch.full((n, n), float("nan"), dtype=torch.float32, device="cuda")
    for key, fused in (("ksplit", False), ("ksplit_fused", True)):
        ks = sharded.KSplitState(n, n, own, world, cfg, A_k, B_k, fused=fused)
        C_full.fill_(float("nan"))
        total_ms, _ = timed_loop(lambda: ks.step(C_full.view(-1)), steps, warm, flush, world)
        ms = total_ms / steps
        out[key] = {"ms_per_step": ms, "value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "steps": steps,
                    "matches_golden": blocks_match(C_full[lo:lo + own], lo), "efficiency_vs_rows": rows_ms / ms,
                    "comm_bytes_per_rank": (world - 1) * own * n * 12 + 2 * n * 4}
        del ks
        torch.cuda.empty_cache()
    return out


def int8_library_rate():
    """Dense INT8 tensor rate of the vendor library on this GPU (torch._int_mm, 8192^3), as a measured yardstick
    beside the derived peak; None where the call is unavailable."""
    import torch
    try:
        n = 8192
        a = torch.randint(-127, 127, (n, n), dtype=torch.int8, device="cuda")
        b = torch.randint(-127, 127, (n, n), dtype=torch.int8, device="cuda")
        for _ in range(3):
            torch._int_mm(a, b)
        torch.cuda.synchronize()
        best = None
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch._int_mm(a, b)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            best = ms if best is None or ms < best else best
        return 2.0 * n ** 3 / (best * 1e-3) / 1e12
    except Exception:
        return None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-ksplit", action="store_true", help="skip the K-range sub-records of a multi-GPU run")
    ap.add_argument("--no-c4", action="store_true", help="skip the 16384^3 (configuration 4) sub-record")
    ap.add_argument("--int8-library-yardstick", action="store_true",
                    help="also time the vendor library's dense INT8 GEMM (torch._int_mm, 8192^3) after the timed regions and "
                         "report it beside the derived INT8 peak; off by default so that a plain run launches this "
                         "repository's kernels only")
    ap.add_argument("--workload", default="c3", choices=["c1", "c2", "c3", "c4", "c5"] + sorted(CONV_BENCH_SHAPES),
                    help="c3 (default) is the headline 4096^3 workload; c1, c2, c4, c5 time the remaining GEMM configurations "
                         "and conv-* one convolution layer (forward and both gradients) on one GPU, with a reduced line")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        reference_arm(args, rank)
        return
    if args.workload != "c3":
        if rank == 0:
            conv_workload(args) if args.workload in CONV_BENCH_SHAPES else auxiliary_workload(args)
        return

    import torch
    import torch.distributed as dist
    from bit_reproducible_training_b200 import fixtures as fx
    from bit_reproducible_training_b200 import repro_gemm as rg

    args.warmup = max(args.warmup, 3)
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    M = N = K = SIZE
    S = SLICES
    # the same synthetic operands on every rank (generated on the device; same bits as the numpy recipe)
    dA, dB = fx.config3_device("cuda", SIZE)
    golden = golden_record("c3.4096")
    inputs_ok = ("%016x" % rg.fnv1a64(dB, rg.fnv1a64(dA))) == golden["in_hash"]
    hA, hB = dA.cpu().pin_memory(), dB.cpu().pin_memory()
    hC = torch.empty(M * N, dtype=torch.float32).pin_memory()
    dC = torch.full((M * N,), float("nan"), dtype=torch.float32, device="cuda")
    cfg = rg.Config(slices=S)
    rc, plan = rg.make_plan(M, N, K, cfg)
    if rc != 0:
        raise rg.ReproGemmError(rc, "make_plan")
    ws = torch.empty(plan.workspace_bytes, dtype=torch.uint8, device="cuda")
    flush = torch.empty(512 << 20, dtype=torch.uint8, device="cuda")     # 4x the 126 MB L2
    stream = torch.cuda.current_stream()
    stage_ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(args.steps)]
    for evs in stage_ev:
        for e in evs:
            e.record()          # creates the handles the library records into

    def step(events=None):
        rc = rg.repro_gemm_fp32_ws(dA, dB, dC, M, N, K, cfg, ws, stream=stream, stage_events=events)
        if rc != 0:
            raise rg.ReproGemmError(rc, "repro_gemm_fp32_ws")

    for _ in range(args.warmup):
        flush.zero_()
        step()
    _barrier(world)
    if rg.workspace_status(ws) != 0:
        raise RuntimeError("a kernel reported an expired wait (status %d)" % rg.workspace_status(ws))

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    t_ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    _barrier(world)
    for i in range(args.steps):
        flush.zero_()                       # L2 flush between timed iterations, outside the timed brackets
        t_ev[i][0].record()
        step(stage_ev[i])
        t_ev[i][1].record()
    _barrier(world)
    clocks = sampler.stop() if rank == 0 else None
    step_ms = [a.elapsed_time(b) for a, b in t_ev]
    ms_per_step = _max_over_ranks(sum(step_ms), world) / args.steps
    flops_step = 2.0 * M * N * K * world
    value = flops_step / (ms_per_step * 1e-3) / 1e12
    device_ok = _all_ranks_true(("%016x" % rg.fnv1a64(dC)) == golden["out_hash"], world)

    # per-stage durations from the four events the library records inside each call
    pre = [e[0].elapsed_time(e[1]) for e in stage_ev]
    mma = [e[1].elapsed_time(e[2]) for e in stage_ev]
    fin = [e[2].elapsed_time(e[3]) for e in stage_ev]

    def spread(v):      # median [min, p90], the form the reference's stage benchmark prints
        v = sorted(v)
        return {"median": statistics.median(v), "min": v[0], "p90": v[min(len(v) - 1, int(0.9 * len(v)))]}
    stages = {"prepass_ms": statistics.mean(pre), "mma_ms": statistics.mean(mma), "final_ms": statistics.mean(fin),
              "prepass_ms_spread": spread(pre), "mma_ms_spread": spread(mma), "step_ms_spread": spread(step_ms)}

    # ---------------- end to end: host buffers in, host buffer out, copies inside the timed region,
    # through the C ABI's host-buffer entry point
    host_gemm = rg.HostGemm(M, N, K, cfg)
    hC.fill_(float("nan"))
    e2e_total, _ = timed_loop(lambda: host_gemm(hA, hB, hC), args.steps, 2, flush, world)
    e2e_ms = e2e_total / args.steps
    e2e_value = flops_step / (e2e_ms * 1e-3) / 1e12
    e2e_ok = _all_ranks_true(("%016x" % rg.fnv1a64(hC)) == golden["out_hash"] and host_gemm.status() == 0, world)
    pcie = measure_pcie(hA, hB, hC, dA, dB, dC, world)
    e2e_launches = host_gemm.launches
    host_gemm.close()

    sub = {}
    if world > 1 and not args.no_ksplit:
        sub.update(ksplit_records(args, world, rank, dA, dB, dC, cfg, flush, ms_per_step))
    int8_lib = int8_library_rate() if (rank == 0 and args.int8_library_yardstick) else None
    del dA, dB, dC, ws, hA, hB, hC
    torch.cuda.empty_cache()
    if not args.no_c4:
        sub["c4"] = c4_records(args, world, rank, flush)

    all_ok = inputs_ok and device_ok and e2e_ok
    for rec in list(sub.values()):
        for v in ([rec] + [x for x in rec.values() if isinstance(x, dict)]):
            if isinstance(v, dict) and v.get("matches_golden") is False:
                all_ok = False
    if rank == 0:
        peaks = measured_peaks()
        line = {"metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "int8", "data": "synthetic",
                "config": {"workload": WORKLOAD,
                           "sharding": "none" if world == 1 else "rows of A, no collective",
                           "l2": "512 MiB buffer written between timed iterations (L2 flush)"},
                "clocks": clocks,
                "inputs_match_golden": inputs_ok, "output_matches_golden": device_ok,
                "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": 2 * M * K * 4,
                        "d2h_bytes_per_step": M * N * 4, "ms_per_step": e2e_ms, "output_matches_golden": e2e_ok,
                        "through": "rgb200_gemm_fp32_host (C ABI), pinned host buffers", "pcie": pcie,
                        "frac": pcie["duplex_ms"] / e2e_ms,
                        "frac_note": "time of plain copies of the same bytes (both directions at once, all ranks at once) / e2e step"},
                "gpu_launches": 4 * args.steps,
                "e2e_gpu_launches": e2e_launches * args.steps}
        mma_ops = 2.0 * S * S * M * N * K
        achieved = mma_ops / (stages["mma_ms"] * 1e-3) / 1e12
        peak = 2.0 * peaks["bf16_tflops"]
        line["roofline"] = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                            "frac": achieved / peak, "traffic": MMA_DRAM_TRAFFIC_BYTES,
                            "traffic_source": "one ncu capture of this kernel at this workload (dram__bytes_read.sum + "
                                              "dram__bytes_write.sum); a recorded constant, not re-measured by this run",
                            "kernel": "gemm_i8_tcgen05_kernel<3,64>",
                            "note": "int8 ops/s of the slice-pair MMAs (2*S^2*M*N*K per launch); peak = 2 x the %s "
                                    "dense bf16 cuBLAS rate (kind::i8 issues at twice the bf16 rate)" % peaks["source"],
                            "frac_of_nominal_int8_4500": achieved / NOMINAL_INT8_TOPS,
                            "int8_library_tops_measured_here": int8_lib,
                            "frac_of_int8_library": (achieved / int8_lib) if int8_lib else None}
        line["stages"] = stages
        pre_bytes = (4.0 + S) * (M * K + N * K) + 4.0 * (M + N)
        line["prepass_roofline"] = {"bound": "hbm", "achieved": pre_bytes / (stages["prepass_ms"] * 1e-3) / 1e9,
                                    "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                    "frac": pre_bytes / (stages["prepass_ms"] * 1e-3) / 1e9 / peaks["hbm_gbs"]}
        line.update(sub)
        if world == 1 and not args.no_cpu_baseline:
            _, _, info = cpu_reference_run(2, 1, 1024)
            line["cpu_baseline"] = info
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    if not all_ok:
        sys.exit(3)


if __name__ == "__main__":
    main()
