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
CSRC = os.path.join(HERE, "csrc")
# translation units (compiled side by side: the streaming kernel's instantiations take minutes)
UNITS = ["capi.cu", "scan_f32_pair.cu", "scan_f32_pair_row.cu", "scan_f32_hist.cu", "scan_f32_hist_row.cu", "scan_f32_hist_short_row.cu", "scan_bf16_pair.cu",
         "scan_bf16_pair_row.cu", "scan_bf16.cu", "scan_bf16_row.cu"]
HEADERS = ["spec.cuh", "scan_common.cuh", "scan_kernel.cuh", "scan_inst.cuh", "scan_launch.cuh", "finish.cuh", "fallback.cuh",
           "merge_kernel.cuh", "prepass.cuh", "spec_kernel.cuh"]
DEPS = [os.path.join(CSRC, f) for f in UNITS + HEADERS]
DEPS.append(os.path.join(ROOT, "include", "born_sampler.h"))
OBJ_DIR = os.path.join(HERE, "build")
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
    os.makedirs(OBJ_DIR, exist_ok=True)
    flags = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--fmad=false", "-Xcompiler", "-fPIC"]
    if verbose:
        flags += ["-Xptxas", "-v"]
    procs = []
    for u in UNITS:
        obj = os.path.join(OBJ_DIR, u[:-3] + ".o")
        cmd = [nvcc_path()] + flags + ["-c", os.path.join(CSRC, u), "-o", obj]
        procs.append((u, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)))
    objs, failed = [], False
    for u, obj, p in procs:
        out, err = p.communicate()
        if p.returncode != 0:
            sys.stderr.write("nvcc failed on %s\n" % u + out + err)
            failed = True
        elif verbose:
            sys.stderr.write(err)
        objs.append(obj)
    if failed:
        raise RuntimeError("nvcc failed")
    res = subprocess.run([nvcc_path(), "-shared", "-o", OUT] + objs + ["-ldl"], capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("nvcc link failed")
    return OUT


if __name__ == "__main__":
    print(build(verbose="--verbose" in sys.argv, force=True))
