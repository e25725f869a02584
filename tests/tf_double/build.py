"""Compiles the B200 TensorFlow OpKernels against the test double in this folder and the reference's own kernel
headers (taken from a checkout, never copied), plus the harness that runs them: tests/tf_double/_build/
libtf_opkernels_check.so.  Host compiler only; links libsimnets_b200.so.

    python tests/tf_double/build.py [REFERENCE_DIR]
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
OUT = os.path.join(HERE, "_build", "libtf_opkernels_check.so")


def build(reference_dir="/root/reference", force=False):
    """Returns the path of the built library, or None when no reference checkout is available."""
    common = os.path.join(reference_dir, "include", "kernels", "similarity_kernel_common.hpp")
    if not os.path.exists(common):
        return OUT if os.path.exists(OUT) else None
    pkg = os.path.join(ROOT, "simnets_tf_b200")
    srcs = [os.path.join(HERE, "harness.cc"),
            os.path.join(pkg, "tf_opkernels", "similarity_kernels_b200.cc"),
            os.path.join(pkg, "tf_opkernels", "mex_kernels_b200.cc"),
            os.path.join(reference_dir, "src", "kernels", "mex_kernel_common.cpp")]
    deps = srcs + [os.path.join(HERE, "tensorflow", "core", "framework", f) for f in ("op_kernel.h", "shape_inference.h")]
    deps += [os.path.join(ROOT, "include", "simnets_b200.h"), os.path.join(pkg, "libsimnets_b200.so")]
    if not force and os.path.exists(OUT) and all(os.path.getmtime(d) <= os.path.getmtime(OUT) for d in deps if os.path.exists(d)):
        return OUT
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    cmd = ["g++", "-std=c++14", "-O1", "-shared", "-fPIC", "-Wall", "-Wno-unused-variable", "-Wno-sign-compare", "-Wno-unused-function",
           "-I", HERE, "-I", os.path.join(reference_dir, "include"), "-I", os.path.join(ROOT, "include")] + srcs + \
          ["-L", pkg, "-lsimnets_b200", "-Wl,-rpath,$ORIGIN/../../../simnets_tf_b200", "-o", OUT]
    subprocess.check_call(cmd)
    return OUT


if __name__ == "__main__":
    print(build(sys.argv[1] if len(sys.argv) > 1 else "/root/reference", force=True))
