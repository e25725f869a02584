"""Compile the CUDA library in-tree: simnets_tf_b200/libsimnets_b200.so, sm_100a only.

    python -m simnets_tf_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU.  The library links the CUDA runtime statically and depends on
nothing else (no torch, no cuBLAS): it is the C ABI of include/simnets_b200.h.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
ROOT = os.path.dirname(HERE)
LIB = os.path.join(HERE, "libsimnets_b200.so")
SOURCES = ["api.cu", "host_dims.cpp", "direct_kernels.cu", "mex_tiled.cu", "mex_smallm.cu", "mex_smallk.cu", "mex_tc.cu", "mex_tc_ws.cu", "mex_tc_pair.cu", "sim_tiled.cu", "sim_smallk.cu", "sim_tc.cu", "pool.cu", "loss.cu", "probe.cu", "offsets_norm.cu"]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    raise RuntimeError("nvcc not found")


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    """Compile every translation unit to an object file (in parallel via separate nvcc calls) and link."""
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".hpp", ".h"))]
    headers.append(os.path.join(ROOT, "include", "simnets_b200.h"))
    common = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-fvisibility=hidden", "-I", os.path.join(ROOT, "include"),
              "-I", CSRC] + ARCH
    if verbose:
        common += ["-Xptxas", "-v"]
    procs, objs = [], []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(objdir, os.path.splitext(src)[0] + ".o")
        objs.append(o)
        if force or _stale(o, [s] + headers):
            cmd = [_nvcc(), "-c", s, "-o", o] + common + (["-x", "cu"] if src.endswith(".cpp") else [])
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stderr.write("---- %s\n%s\n" % (src, out))
        failed = failed or p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    if force or procs or _stale(LIB, objs):
        subprocess.check_call([_nvcc(), "-shared", "-o", LIB] + objs + ARCH + ["-cudart", "static"])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
