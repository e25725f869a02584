"""Generates tests/golden/*.npz from the reference project's own CPU templates (oracle/_ref).

    python tests/golden/make_golden.py

Needs oracle/_ref/libsimnets_ref.so, i.e. a checkout of the reference project at build time
(`make -C oracle REFERENCE_DIR=<checkout>`).  Inputs are stored beside the outputs so that the
vectors do not depend on the random generator of whoever reads them.  The `*_quirk` Similarity case
is the only one where the reference's fast op and its SimilarityRef op disagree (constant added
(batch - n) times); it is stored as the fast op computes it.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import cases  # noqa: E402
from oracle import oracle  # noqa: E402
from simnets_tf_b200 import abi  # noqa: E402


def main():
    ref = oracle.load("reference")
    sim = {}
    for c in cases.SIM_SMALL:
        if c["flags"] & abi.FLAG_SIM_L1_SKIP_NAN:
            continue
        # the reference always behaves as the quirk flag says; skip normalised batch>1 cases without it
        if c["norm"] and not c["ignore_nan"] and c["shape"][0] > 1 and not (c["flags"] & abi.FLAG_SIM_BATCH_CONST_QUIRK):
            continue
        d = cases.sim_desc(c)
        x, t, w, dy = cases.sim_inputs(c, ref.sim_out_shape(d))
        y = ref.similarity_forward(d, x, t, w)
        dx = ref.similarity_input_grad(d, x, t, w, dy)
        dt, dw = ref.similarity_params_grad(d, x, t, w, dy)
        for k, v in dict(x=x, t=t, w=w, dy=dy, y=y, dx=dx, dt=dt, dw=dw).items():
            sim["%s/%s" % (c["name"], k)] = v
    np.savez_compressed(os.path.join(HERE, "similarity_small.npz"), **sim)
    mex = {}
    for c in cases.MEX_SMALL:
        d = cases.mex_desc(c)
        x, off, dy = cases.mex_inputs(c, ref.mex_offsets_shape(d), ref.mex_out_shape(d))
        y = ref.mex_forward(d, x, off)
        dx = ref.mex_input_grad(d, x, off, y, dy)
        doff = ref.mex_offsets_grad(d, x, off, y, dy)
        for k, v in dict(x=x, off=off, dy=dy, y=y, dx=dx, doff=doff).items():
            mex["%s/%s" % (c["name"], k)] = v
    np.savez_compressed(os.path.join(HERE, "mex_small.npz"), **mex)
    print("wrote", len(sim), "similarity arrays and", len(mex), "mex arrays")


if __name__ == "__main__":
    main()
