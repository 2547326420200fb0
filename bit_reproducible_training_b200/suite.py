"""The 21 GEMM operations of the reference's GPT-2 conformance suite on this library.

Writes a result file in the reference's format (gpt2_ops_suite/gpt2_ops_suite.cu:654: one
``OP<TAB>name<TAB>shape<TAB>in=<hash><TAB>out=<hash><TAB>ms=..<TAB>base_ms=..`` line per operation after
a ``# ...`` header line), so the reference's ``compare_suite.sh`` can diff it against the result
files the reference commits (gpt2_ops_suite/results/*/cpu.txt).

    python -m bit_reproducible_training_b200.suite [--tokens 1024] [--slices 3] [--reps 10] [--out FILE] [--graph]
"""
import argparse
import statistics
import sys

import torch

from . import fixtures as fx
from . import repro_gemm as rg


def run(tokens=1024, slices=3, reps=10, out=None, graph=False):
    lines = ["# GPU %s tokens=%d S=%d (librgb200)" % (torch.cuda.get_device_name(0), tokens, slices)]
    for op in fx.suite_gemm_ops(tokens):
        name, M, N, K, ta, tb = op[:6]
        A, B = fx.suite_inputs(op)
        hin = rg.fnv1a64(B, rg.fnv1a64(A))
        dA, dB = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
        cfg = rg.Config(slices=slices, trans_a=ta, trans_b=tb)
        rc, plan = rg.make_plan(M, N, K, cfg)
        if rc != 0:
            raise rg.ReproGemmError(rc, "make_plan")
        ws = torch.empty(plan.workspace_bytes, dtype=torch.uint8, device="cuda")
        C = torch.full((M, N), float("nan"), device="cuda")          # poisoned, as the reference does
        times = []
        replay = None
        if graph:
            # time replays of a captured call: what a caller sees whose launches are not paced by Python
            rc = rg.repro_gemm_fp32_ws(dA, dB, C, M, N, K, cfg, ws)
            torch.cuda.synchronize()
            replay = torch.cuda.CUDAGraph()
            with torch.cuda.graph(replay):
                rc = rg.repro_gemm_fp32_ws(dA, dB, C, M, N, K, cfg, ws)
        for i in range(reps + 2):                                     # two warm-ups, then the median
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            if replay is not None:
                replay.replay()
            else:
                rc = rg.repro_gemm_fp32_ws(dA, dB, C, M, N, K, cfg, ws)
            e1.record()
            if rc != 0:
                raise rg.ReproGemmError(rc, name)
            torch.cuda.synchronize()
            if i >= 2:
                times.append(e0.elapsed_time(e1))
        shape = "M=%d N=%d K=%d%s%s" % (M, N, K, " A^T" if ta else "", " B^T" if tb else "")
        lines.append("OP\t%s\t%s\tin=%016x\tout=%016x\tms=%.4f\tbase_ms=%.4f" %
                     (name, shape, hin, rg.fnv1a64(C), statistics.median(times), -1.0))
        print(lines[-1], flush=True)
    if out:
        with open(out, "w") as f:
            f.write("\n".join(lines) + "\n")
    return lines


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=1024)
    ap.add_argument("--slices", type=int, default=3)
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--out", default=None)
    ap.add_argument("--graph", action="store_true", help="time replays of a CUDA graph of the call instead of direct calls")
    a = ap.parse_args()
    run(a.tokens, a.slices, a.reps, a.out, a.graph)
    sys.exit(0)
