"""Per-tile cycle breakdown of the MMA kernel (diagnostic).

Builds a copy of the library with -DRGB200_TIMING_STAMPS (CTA 0 then writes clock64 stamps of its first
five tiles into the unused part of the workspace's status block), runs one GEMM and prints, per tile,
the cycles spent issuing the mainloop, the commit-to-epilogue latency and the TMEM drain.

    python -m bit_reproducible_training_b200.tile_timing [M N K [S]]
"""
import os
import subprocess
import sys
import tempfile

from . import build as _build


def main(argv):
    M, N, K = (int(x) for x in argv[:3]) if len(argv) >= 3 else (4096, 4096, 4096)
    S = int(argv[3]) if len(argv) > 3 else 3
    lib = os.path.join(tempfile.mkdtemp(prefix="rgb200_timing_"), "librgb200_timing.so")
    cmd = [_build._nvcc()] + _build.NVCC_FLAGS + ["-DRGB200_TIMING_STAMPS", "-o", lib] + _build.SOURCES
    subprocess.run(cmd, cwd=_build.CSRC, check=True)
    os.environ["RGB200_LIBRARY"] = lib
    import numpy as np
    import torch
    from . import repro_gemm as rg
    A = torch.rand(M * K, device="cuda") - 0.5
    B = torch.rand(K * N, device="cuda") - 0.5
    C = torch.empty(M * N, device="cuda")
    cfg = rg.Config(slices=S)
    rc, plan = rg.make_plan(M, N, K, cfg)
    if rc != 0:
        raise rg.ReproGemmError(rc, "make_plan")
    ws = torch.empty(plan.workspace_bytes, dtype=torch.uint8, device="cuda")
    for _ in range(3):
        rg.repro_gemm_fp32_ws(A, B, C, M, N, K, cfg, ws)
    torch.cuda.synchronize()
    t = ws[:256].cpu().numpy().view(np.int64)
    base = t[1]
    ideal = (K + 127) // 128 * 4 * S * (32 * S * 64 // 64)       # k steps x MMAs x cycles of a 128 x (64 S) x 32 MMA
    print("M=%d N=%d K=%d S=%d   ideal mainloop %d cycles per tile" % (M, N, K, S, ideal))
    for i in range(5):
        s = t[1 + 6 * i:1 + 6 * i + 4] - base
        print("tile %d: start %8d | mainloop issued +%6d | epilogue sees accumulators +%4d | TMEM released +%5d"
              % (i, s[0], s[1] - s[0], s[2] - s[1], s[3] - s[2]))


if __name__ == "__main__":
    main(sys.argv[1:])
