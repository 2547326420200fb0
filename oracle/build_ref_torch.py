"""TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Builds the reference project's PyTorch extension (repro_torch/_backend) with its GEMM and convolution
kernels swapped for librgb200.so, to show that the library drops in behind repro_torch:

  * the reference's extension compiles all of its CUDA code as one unit, src/kernels.cu, which pulls the
    component sources in textually (repro_torch/src/kernels.cu:2-6).  A scratch copy of repro_torch/ is made
    under oracle/_ref/repro_torch_rgb200/ (git-ignored), and in that copy the two lines that include
    repro_gemm.cu and repro_conv.cu are dropped; the remaining includes (exact sums, softmax, pooling, Adam)
    are pointed at the reference checkout, where those sources stay;
  * bindings.cpp is compiled unchanged against the reference's own headers (repro_gemm.cuh, repro_conv.cuh);
    the functions they declare are resolved by -lrgb200, which exports them with the same C++ signatures;
  * the Python package (layers.py, utils.py) is copied as it is.

Nothing of the reference is committed: the copy lives only in the ignored output directory, which travels to
the GPU machine together with the other prebuilt checkers.  Run where the reference sources are present:

    python oracle/build_ref_torch.py            # needs REPRO_REFERENCE_ROOT or ../reference
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
OUT = os.path.join(HERE, "_ref", "repro_torch_rgb200")
LIB_DIR = os.path.join(ROOT, "bit_reproducible_training_b200")

SETUP = r'''
import os, torch
from setuptools import setup
from torch.utils.cpp_extension import BuildExtension, CUDAExtension
ref = os.environ["REF_ROOT"]
lib_dir = os.environ["RGB200_LIB_DIR"]
includes = [os.path.join(ref, d) for d in ("repro_gemm_cuda", "repro_sum_cuda", "repro_math_cuda", "repro_conv_cuda", "repro_nn_cuda")]
includes.append(os.path.join(os.path.dirname(os.path.abspath(__file__)), "src"))
cxx = ["-O2", "-std=c++17", "-fno-fast-math", "-ffp-contract=off"]
nvcc = ["-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "--fmad=false", "-lineinfo"]
link = ["-Wl,-rpath," + os.path.join(os.path.dirname(torch.__file__), "lib"), "-L" + lib_dir, "-lrgb200",
        "-Wl,-rpath,$ORIGIN/../../../../bit_reproducible_training_b200"]
ext = CUDAExtension("repro_torch._backend", ["src/bindings_gpu.cu", "src/kernels.cu"], include_dirs=includes,
                    extra_compile_args={"cxx": cxx, "nvcc": nvcc}, extra_link_args=link)
setup(name="repro_torch", packages=["repro_torch"], ext_modules=[ext], cmdclass={"build_ext": BuildExtension})
'''


def built_module():
    """Path of the built extension module, or None."""
    pkg = os.path.join(OUT, "repro_torch")
    if os.path.isdir(pkg):
        for f in os.listdir(pkg):
            if f.startswith("_backend") and f.endswith(".so"):
                return os.path.join(pkg, f)
    return None


def build(ref_root):
    src = os.path.join(ref_root, "repro_torch")
    if os.path.isdir(OUT):
        shutil.rmtree(OUT)
    os.makedirs(OUT)
    shutil.copytree(os.path.join(src, "repro_torch"), os.path.join(OUT, "repro_torch"))
    shutil.copytree(os.path.join(src, "src"), os.path.join(OUT, "src"))
    kernels = os.path.join(OUT, "src", "kernels.cu")
    lines = []
    for line in open(kernels).read().splitlines():
        if 'repro_gemm.cu"' in line or 'repro_conv.cu"' in line:
            continue                                  # these two come from librgb200.so
        lines.append(line.replace('"../../', '"' + ref_root.rstrip("/") + "/"))
    with open(kernels, "w") as f:
        f.write("\n".join(lines) + "\n")
    with open(os.path.join(OUT, "setup_rgb200.py"), "w") as f:
        f.write(SETUP)
    env = dict(os.environ, REF_ROOT=ref_root, RGB200_LIB_DIR=LIB_DIR, TORCH_CUDA_ARCH_LIST="10.0a", MAX_JOBS="4")
    res = subprocess.run([sys.executable, "setup_rgb200.py", "build_ext", "--inplace"], cwd=OUT, env=env,
                         capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("building the reference's torch extension against librgb200.so failed:\n" +
                           res.stdout[-4000:] + res.stderr[-4000:])
    shutil.rmtree(os.path.join(OUT, "build"), ignore_errors=True)
    return built_module()


if __name__ == "__main__":
    sys.path.insert(0, ROOT)
    import oracle
    root = oracle.reference_root()
    if root is None:
        sys.exit("reference sources not found (set REPRO_REFERENCE_ROOT)")
    print(build(root))
