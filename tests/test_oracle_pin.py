"""Pins the CPU oracle: (1) against the committed vectors in tests/golden/, which the reference
project's own CPU templates produced; (2) bit for bit against those templates (oracle/_ref) where
they are built; (3) against the reference's naive second-opinion ops (SimilarityRef / MexRef
restated) at the tolerance the reference's own tests use."""
import os

import numpy as np
import pytest

import cases
from simnets_tf_b200 import abi

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _same(a, b):
    return np.array_equal(a, b, equal_nan=True)


@pytest.fixture(scope="module")
def sim_golden():
    return np.load(os.path.join(GOLDEN, "similarity_small.npz"))


@pytest.fixture(scope="module")
def mex_golden():
    return np.load(os.path.join(GOLDEN, "mex_small.npz"))


def _golden_sim_names(golden):
    return sorted({k.split("/")[0] for k in golden.files})


def test_similarity_port_matches_golden(port, sim_golden):
    names = _golden_sim_names(sim_golden)
    assert len(names) >= 40
    by_name = {c["name"]: c for c in cases.SIM_SMALL}
    for name in names:
        c = by_name[name]
        d = cases.sim_desc(c, flags=c["flags"] | abi.FLAG_SIM_BATCH_CONST_QUIRK)
        g = {k: sim_golden["%s/%s" % (name, k)] for k in ("x", "t", "w", "dy", "y", "dx", "dt", "dw")}
        # same machine + same operation order => identical bits; elsewhere libm may differ in the last ulp
        y = port.similarity_forward(d, g["x"], g["t"], g["w"])
        cases.assert_parity(y, g["y"], tol=1e-6, what=name + " y")
        cases.assert_parity(port.similarity_input_grad(d, g["x"], g["t"], g["w"], g["dy"]), g["dx"], tol=1e-6, what=name + " dx")
        dt, dw = port.similarity_params_grad(d, g["x"], g["t"], g["w"], g["dy"])
        cases.assert_parity(dt, g["dt"], tol=1e-6, what=name + " dt")
        cases.assert_parity(dw, g["dw"], tol=1e-6, what=name + " dw")


def test_mex_port_matches_golden(port, mex_golden):
    names = sorted({k.split("/")[0] for k in mex_golden.files})
    assert len(names) == len(cases.MEX_SMALL)
    by_name = {c["name"]: c for c in cases.MEX_SMALL}
    for name in names:
        d = cases.mex_desc(by_name[name])
        g = {k: mex_golden["%s/%s" % (name, k)] for k in ("x", "off", "dy", "y", "dx", "doff")}
        cases.assert_parity(port.mex_forward(d, g["x"], g["off"]), g["y"], tol=1e-6, what=name + " y")
        cases.assert_parity(port.mex_input_grad(d, g["x"], g["off"], g["y"], g["dy"]), g["dx"], tol=1e-6, what=name + " dx")
        cases.assert_parity(port.mex_offsets_grad(d, g["x"], g["off"], g["y"], g["dy"]), g["doff"], tol=1e-6, what=name + " doff")


def test_similarity_port_bit_exact_with_reference_templates(port, reference):
    for dtype, npdt in ((abi.F32, np.float32), (abi.F64, np.float64)):
        for c in cases.SIM_SMALL:
            if c["flags"] & abi.FLAG_SIM_L1_SKIP_NAN:
                continue
            d = cases.sim_desc(c, dtype=dtype, flags=c["flags"] | abi.FLAG_SIM_BATCH_CONST_QUIRK)
            x, t, w, dy = cases.sim_inputs(c, port.sim_out_shape(d), npdt)
            assert _same(port.similarity_forward(d, x, t, w), reference.similarity_forward(d, x, t, w)), c["name"]
            assert _same(port.similarity_input_grad(d, x, t, w, dy), reference.similarity_input_grad(d, x, t, w, dy)), c["name"]
            a, b = port.similarity_params_grad(d, x, t, w, dy), reference.similarity_params_grad(d, x, t, w, dy)
            assert _same(a[0], b[0]) and _same(a[1], b[1]), c["name"]


def test_mex_port_bit_exact_with_reference_templates(port, reference):
    for dtype, npdt in ((abi.F32, np.float32), (abi.F64, np.float64)):
        for c in cases.MEX_SMALL:
            d = cases.mex_desc(c, dtype=dtype)
            assert port.mex_dims(d).as_dict() == reference.mex_dims(d).as_dict(), c["name"]
            x, off, dy = cases.mex_inputs(c, port.mex_offsets_shape(d), port.mex_out_shape(d), npdt)
            y = port.mex_forward(d, x, off)
            assert _same(y, reference.mex_forward(d, x, off)), c["name"]
            assert _same(port.mex_input_grad(d, x, off, y, dy), reference.mex_input_grad(d, x, off, y, dy)), c["name"]
            assert _same(port.mex_offsets_grad(d, x, off, y, dy), reference.mex_offsets_grad(d, x, off, y, dy)), c["name"]


def test_fast_ops_agree_with_naive_second_opinion(port):
    """The reference's Pattern-A tests: fast op vs SimilarityRef at 1e-2, vs MexRef at 1e-3."""
    for c in cases.SIM_SMALL:
        if c["flags"] or c["shape"][0] == 0:
            continue
        d = cases.sim_desc(c, dtype=abi.F64)
        x, t, w, _ = cases.sim_inputs(c, port.sim_out_shape(d), np.float64)
        fast, naive = port.similarity_forward(d, x, t, w), port.similarity_forward(d, x, t, w, naive=True)
        assert np.array_equal(np.isnan(fast), np.isnan(naive)), c["name"]
        np.testing.assert_allclose(np.nan_to_num(fast), np.nan_to_num(naive), atol=1e-2, err_msg=c["name"])
    for c in cases.MEX_SMALL:
        if c["shape"][0] == 0:
            continue
        d = cases.mex_desc(c, dtype=abi.F64)
        x, off, _ = cases.mex_inputs(c, port.mex_offsets_shape(d), port.mex_out_shape(d), np.float64)
        np.testing.assert_allclose(port.mex_forward(d, x, off), port.mex_forward(d, x, off, naive=True), rtol=1e-3, atol=1e-3,
                                   err_msg=c["name"])


def test_batch_constant_quirk_is_the_only_difference(port):
    """With L2 + normalization_term and no ignore_nan the reference's fast op adds -0.5*K*log(2*pi) to
    sample n (batch - n) times; the default here adds it once.  The two must differ by exactly that."""
    c = next(c for c in cases.SIM_SMALL if c["name"] == "norm_batch3")
    d1, dq = cases.sim_desc(c, dtype=abi.F64, flags=0), cases.sim_desc(c, dtype=abi.F64, flags=abi.FLAG_SIM_BATCH_CONST_QUIRK)
    x, t, w, _ = cases.sim_inputs(c, port.sim_out_shape(d1), np.float64)
    once, quirk = port.similarity_forward(d1, x, t, w), port.similarity_forward(dq, x, t, w)
    B, K = c["shape"][0], c["shape"][1] * c["blocks"][0] * c["blocks"][1]
    const = -0.5 * K * np.log(2 * np.pi)
    for n in range(B):
        np.testing.assert_allclose(quirk[n] - once[n], (B - 1 - n) * const, rtol=0, atol=1e-9)


def test_analytic_gradients_match_numeric(port):
    """The reference's Pattern-B tests (tf.test.compute_gradient) on the float64 oracle: central differences."""
    rng = np.random.default_rng(167)
    h = 1e-6

    def numeric(f, a):
        g = np.zeros_like(a)
        it = np.nditer(a, flags=["multi_index"])
        for _ in it:
            i = it.multi_index
            old = a[i]
            a[i] = old + h; fp = f()
            a[i] = old - h; fm = f()
            a[i] = old
            g[i] = (fp - fm) / (2 * h)
        return g

    for fn, norm, ign in (("L1", False, False), ("L2", True, False), ("L2", True, True), ("L2", False, False)):
        d = abi.make_sim_desc((1, 3, 6, 6), 2, fn, (3, 3), (2, 2), (1, 1), norm, 0.001, ign, 0.0, dtype=abi.F64)
        x = rng.normal(size=(1, 3, 6, 6)); t = rng.normal(size=(2, 3, 3, 3)); w = np.abs(rng.normal(size=t.shape)) + 0.5
        dy = rng.normal(size=port.sim_out_shape(d))
        loss = lambda: float((port.similarity_forward(d, x, t, w) * dy).sum())
        np.testing.assert_allclose(port.similarity_input_grad(d, x, t, w, dy), numeric(loss, x), rtol=1e-4, atol=1e-5)
        dt, dw = port.similarity_params_grad(d, x, t, w, dy)
        np.testing.assert_allclose(dt, numeric(loss, t), rtol=1e-4, atol=1e-5)
        np.testing.assert_allclose(dw, numeric(loss, w), rtol=1e-4, atol=1e-5)
    for eps, unshared in ((1.0, True), (0.5, False), (-1.5, True)):
        d = abi.make_mex_desc((2, 3, 6, 6), 2, True, (0, 1, 1), (1, 2, 2), (3, 3, 3), eps, 0.0, True, unshared, (2,), (2,), dtype=abi.F64)
        x = rng.normal(size=(2, 3, 6, 6)); off = rng.normal(size=port.mex_offsets_shape(d))
        dy = rng.normal(size=port.mex_out_shape(d))
        loss = lambda: float((port.mex_forward(d, x, off) * dy).sum())
        y = port.mex_forward(d, x, off)
        np.testing.assert_allclose(port.mex_input_grad(d, x, off, y, dy), numeric(loss, x), rtol=1e-4, atol=1e-6)
        np.testing.assert_allclose(port.mex_offsets_grad(d, x, off, y, dy), numeric(loss, off), rtol=1e-4, atol=1e-6)
