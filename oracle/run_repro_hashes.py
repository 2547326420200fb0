"""TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Per-GPU, multi-process hash files, after the reference's repro_gemm_cuda/run_repro.sh:21-28,77-115: for every
visible GPU (one at a time, selected through CUDA_VISIBLE_DEVICES), every shape, input distribution and slice
count, the reference's own hash tool - hash_repro_gemm.cu, unmodified, linked against librgb200.so by
oracle/Makefile - runs in `procs` separate processes; all of them must print the same RESULT line, which goes
into <out>/<host>/gpu<i>.hashes.  Files of different GPUs (or machines) are then compared with a plain diff, as
the reference does (run_repro.sh:11,127-131).

    python oracle/run_repro_hashes.py [--out results] [--procs 3] [--gpus 0,1] [--slices 1,3] [--quick]
"""
import argparse
import os
import socket
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
TOOL = os.path.join(HERE, "_ref", "hash_repro_gemm_rgb200")
DISTS = ("uniform", "normal", "weights", "wide", "stress")          # run_repro.sh:21
SHAPES = (("256", "256", "1024", "1,2,3,4,7,8,16,64"),              # run_repro.sh:23-28
          ("129", "77", "1000", "1,2,3,5,7,13,64"),
          ("64", "64", "7", "1,2,3,7,16"),
          ("1024", "1024", "4096", "1,2,7"))
RUNS, SEED = "5", "12345"


def visible_gpus():
    out = subprocess.run(["nvidia-smi", "--query-gpu=index", "--format=csv,noheader"], capture_output=True, text=True)
    return [x.strip() for x in out.stdout.split() if x.strip()] if out.returncode == 0 else []


def run(out_dir, procs=3, gpus=None, slices=("1", "3"), shapes=SHAPES, dists=DISTS):
    """Returns (list of hash-file paths, failure messages)."""
    if not os.path.exists(TOOL):
        raise RuntimeError("%s has not been built (make -C oracle ref_gpu REF_ROOT=...)" % TOOL)
    host_dir = os.path.join(out_dir, socket.gethostname().split(".")[0])
    os.makedirs(host_dir, exist_ok=True)
    files, failures = [], []
    for g in (gpus if gpus else visible_gpus()):
        env = dict(os.environ, CUDA_DEVICE_ORDER="PCI_BUS_ID", CUDA_VISIBLE_DEVICES=str(g))
        path = os.path.join(host_dir, "gpu%s.hashes" % g)
        lines = []
        for M, N, K, splits in shapes:
            for dist in dists:
                for S in slices:
                    seen = set()
                    line = None
                    for p in range(procs):
                        # "tiled" (the reference's dp4a algorithm) is reported unsupported by this library and skipped by the tool
                        res = subprocess.run([TOOL, M, N, K, RUNS, splits, SEED, dist, "ref,tiled,tc", S], env=env,
                                             capture_output=True, text=True)
                        found = [l for l in res.stdout.splitlines() if l.startswith("RESULT")]
                        line = found[0] if found else "RESULT M=%s N=%s K=%s S=%s seed=%s dist=%s hash=none status=CRASH" % (M, N, K, S, SEED, dist)
                        if res.returncode != 0 or not found:
                            failures.append("gpu %s: %s exited %d" % (g, line, res.returncode))
                        seen.add(line)
                    if len(seen) != 1:
                        failures.append("gpu %s: M=%s N=%s K=%s S=%s dist=%s gave different hashes across processes" % (g, M, N, K, S, dist))
                    lines.append(line)
        with open(path, "w") as f:
            f.write("\n".join(lines) + "\n")
        files.append(path)
    for f in files[1:]:
        if open(f).read() != open(files[0]).read():
            failures.append("%s differs from %s" % (f, files[0]))
    return files, failures


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="results")
    ap.add_argument("--procs", type=int, default=3)
    ap.add_argument("--gpus", default="")
    ap.add_argument("--slices", default="1,3")
    ap.add_argument("--quick", action="store_true", help="leave out the 1024 x 1024 x 4096 shape")
    a = ap.parse_args()
    files, failures = run(a.out, a.procs, [g for g in a.gpus.split(",") if g], tuple(a.slices.split(",")),
                          SHAPES[:3] if a.quick else SHAPES)
    for f in files:
        print(f)
    for m in failures:
        print("FAIL:", m)
    print("OVERALL:", "FAIL" if failures else "PASS")
    sys.exit(2 if failures else 0)
