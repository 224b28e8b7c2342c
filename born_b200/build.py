"""Build libborn_sampler.so (sm_100a only) in-tree with nvcc.

    python -m born_b200.build [--verbose]

nvcc cross-compiles without a GPU.  --fmad=false keeps every fp32 multiply and add
individually rounded; the kernels ask for fused multiply-adds explicitly where they want one.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
SRC = os.path.join(HERE, "csrc", "capi.cu")
DEPS = [os.path.join(HERE, "csrc", f) for f in ("capi.cu", "spec.cuh", "scan_common.cuh", "scan_kernel.cuh", "finish.cuh", "fallback.cuh", "merge_kernel.cuh",
                                                   "prepass.cuh", "spec_kernel.cuh")]
DEPS.append(os.path.join(ROOT, "include", "born_sampler.h"))
OUT = os.path.join(HERE, "libborn_sampler.so")


def nvcc_path():
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def up_to_date():
    if not os.path.exists(OUT):
        return False
    t = os.path.getmtime(OUT)
    return all(os.path.getmtime(d) <= t for d in DEPS)


def build(verbose=False, force=False):
    if not force and up_to_date():
        return OUT
    cmd = [
        nvcc_path(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
        "--fmad=false", "-Xcompiler", "-fPIC", "-shared", "-o", OUT, SRC, "-ldl",
    ]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("nvcc failed")
    if verbose:
        sys.stderr.write(res.stderr)
    return OUT


if __name__ == "__main__":
    print(build(verbose="--verbose" in sys.argv, force=True))
