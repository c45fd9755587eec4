"""Builds libufsm_mx.so in-tree: CUDA sources for sm_100a with nvcc, the C23 host code with gcc, one shared library with a C ABI."""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libufsm_mx.so")
CU = ["runtime.cu", "quant.cu", "norm.cu", "conv_tc.cu", "conv_tcr.cu", "conv_tcp.cu", "conv_stem.cu", "lp_entry.cu", "window.cu", "pred_place.cu", "in_coef_static.cu", "gn_sums.cu", "gn_apply.cu", "mx_ops.cu"]
C = ["unet.c"]
NVCC = os.environ.get("UFSM_NVCC") or shutil.which("nvcc") or os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
GCC = os.environ.get("UFSM_GCC", "gcc")
NVFLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC"] + os.environ.get("UFSM_NVCC_EXTRA", "").split()


def _newer(src, dst):
    return not os.path.exists(dst) or os.path.getmtime(src) > os.path.getmtime(dst)


def build(force=False, verbose=False):
    """Compile what changed and link; returns the library path."""
    objdir = os.path.join(HERE, "..", "build")
    os.makedirs(objdir, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))] + [os.path.join(HERE, "..", "include", "ufsm_mx.h")]
    hdr_time = max(os.path.getmtime(h) for h in headers)
    objs, relink = [], force or not os.path.exists(LIB)
    jobs = []
    for f in CU + C:
        src, obj = os.path.join(CSRC, f), os.path.join(objdir, f + ".o")
        objs.append(obj)
        if force or _newer(src, obj) or os.path.getmtime(obj) < hdr_time:
            if f.endswith(".cu"):
                cmd = [NVCC] + NVFLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
            else:
                cmd = [GCC, "-std=c2x", "-O2", "-fPIC", "-Wall", "-c", src, "-o", obj]
            jobs.append((f, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
            relink = True
    for f, p in jobs:
        out, _ = p.communicate()
        if p.returncode != 0:
            raise RuntimeError("compiling %s failed:\n%s" % (f, out))
        if verbose and out:
            sys.stderr.write(out)
    if relink:
        cmd = [NVCC, "-shared", "-o", LIB] + objs + ["-lcudart_static", "-lpthread", "-ldl", "-lrt"]
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            raise RuntimeError("linking failed:\n" + r.stdout)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
