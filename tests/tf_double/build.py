"""Compiles the B200 TensorFlow OpKernels against the test double in this folder and the reference's own kernel
headers (taken from a checkout, never copied), plus the harness that runs them: tests/tf_double/_build/
libtf_opkernels_check.so.  Host compiler only; links libsimnets_b200.so.

    python tests/tf_double/build.py REFERENCE_DIR
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
OUT = os.path.join(HERE, "_build", "libtf_opkernels_check.so")


def default_reference_dir():
    """SIMNETS_REFERENCE_DIR, else a folder `reference` beside the repository; "" when neither exists."""
    for cand in (os.environ.get("SIMNETS_REFERENCE_DIR"), os.path.join(os.path.dirname(ROOT), "reference")):
        if cand and os.path.isdir(cand):
            return cand
    return ""


def build(reference_dir=None, force=False):
    """Returns the path of the built library, or None when no reference checkout is available (the directory comes from the
    argument or from the environment variable SIMNETS_REFERENCE_DIR)."""
    reference_dir = reference_dir or default_reference_dir()
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


OPS_OUT = os.path.join(HERE, "_build", "libtf_ops_check.so")


def build_ops(reference_dir=None, force=False):
    """The reference's op registrations (src/ops/similarity_op.cpp, src/ops/mex_op.cpp, compiled unchanged where they lie)
    against the double's REGISTER_OP / InferenceContext, plus ops_harness.cc: tests/tf_double/_build/libtf_ops_check.so.
    Returns the path, or None when no reference checkout is available and nothing was built before."""
    reference_dir = reference_dir or default_reference_dir()
    srcs_ref = [os.path.join(reference_dir, "src", "ops", f) for f in ("similarity_op.cpp", "mex_op.cpp")]
    if not reference_dir or not all(os.path.exists(f) for f in srcs_ref):
        return OPS_OUT if os.path.exists(OPS_OUT) else None
    deps = srcs_ref + [os.path.join(HERE, "ops_harness.cc")] + [os.path.join(HERE, "tensorflow", "core", "framework", f) for f in ("op.h", "shape_inference.h")]
    if not force and os.path.exists(OPS_OUT) and all(os.path.getmtime(d) <= os.path.getmtime(OPS_OUT) for d in deps):
        return OPS_OUT
    os.makedirs(os.path.dirname(OPS_OUT), exist_ok=True)
    cmd = ["g++", "-std=c++14", "-O1", "-shared", "-fPIC", "-Wall", "-Wno-unused-variable", "-Wno-sign-compare", "-Wno-unused-function", "-Wno-parentheses", "-Wno-maybe-uninitialized",
           "-I", HERE, "-I", os.path.join(reference_dir, "include"), os.path.join(HERE, "ops_harness.cc")] + srcs_ref + ["-o", OPS_OUT]
    subprocess.check_call(cmd)
    return OPS_OUT


if __name__ == "__main__":
    ref = sys.argv[1] if len(sys.argv) > 1 else None
    print(build(ref, force=True))
    print(build_ops(ref, force=True))
