"""The GEMM + softmax cross-nonlinearity oracle against outputs of the reference's own kernels
(tests/golden/gs_*.npz, made by oracle/ref_harness_gs on a B200): inputs, logits and expected projections bit for bit;
everything behind exp()/log() within 1e-9 (host libm against the device's), decisions equal."""
import glob
import os

import numpy as np
import pytest

from tests import oracle_gs as gs

GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "gs_*.npz")))


def _phase(g, x, m, n, es, ew):
    checks = gs.softmax_checks(x)
    return checks, gs.analyze(es, ew, checks, n)


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p) for p in GOLDEN])
def test_oracle_reproduces_reference_kernels(path):
    g = np.load(path)
    m, n, k = (int(v) for v in g["shape"])
    fault_row, fault_col, fault_value = int(g["fault"][0]), int(g["fault"][1]), float(g["fault"][2])
    a, b = gs.generate(m * k, 17), gs.generate(n * k, 29)  # seeds of src/gemm_softmax_abft.cu:431-432
    np.testing.assert_array_equal(a, g["a"])
    np.testing.assert_array_equal(b, g["b"])
    x = gs.logits(a, b, m, n, k)
    np.testing.assert_array_equal(x.ravel().view(np.uint32), g["logits"].view(np.uint32))
    es, ew = gs.expected(a, b, m, n, k)
    np.testing.assert_array_equal(es.view(np.uint64), g["expected_sum"].view(np.uint64))
    np.testing.assert_array_equal(ew.view(np.uint64), g["expected_weighted"].view(np.uint64))

    def compare(phase, x):
        checks, analysis = _phase(g, x, m, n, es, ew)
        for name in ("actual_sum", "actual_weighted", "probability_sum", "log_z"):
            np.testing.assert_allclose(checks[name], g[f"{name}_{phase}"], rtol=1e-11, atol=1e-9, err_msg=f"{name} {phase}")
        if f"probabilities_{phase}" in g:
            np.testing.assert_allclose(checks["probabilities"].ravel(), g[f"probabilities_{phase}"], rtol=3e-7, atol=0)
        else:
            np.testing.assert_allclose(checks["probabilities"][fault_row], g[f"probabilities_row_{phase}"], rtol=3e-7, atol=0)
        np.testing.assert_array_equal(analysis["detected"], g[f"detected_{phase}"])
        np.testing.assert_array_equal(analysis["estimated_col"], g[f"estimated_col_{phase}"])
        np.testing.assert_array_equal(analysis["counts"], g[f"counts_{phase}"])
        np.testing.assert_allclose(analysis["correction_delta"], g[f"correction_delta_{phase}"], rtol=0, atol=1e-9)
        return analysis

    clean = compare("clean", x)
    assert clean["counts"].tolist() == [0, 0]
    x[fault_row, fault_col] += np.float32(fault_value)
    faulty = compare("fault", x)
    assert faulty["counts"].tolist() == [1, 1] and faulty["estimated_col"][fault_row] == fault_col
    assert faulty["correction_delta"][fault_row] == pytest.approx(fault_value, abs=1e-6)
    recovered = compare("recovered", gs.correct(x, faulty))
    assert recovered["counts"].tolist() == [0, 0]


def test_identities_on_random_logits():
    """sum log P + N logZ = sum x and sum w log P = sum w x for any row; a fault below the tolerance stays invisible."""
    rng = np.random.default_rng(3)
    m, n = 8, 300
    x = rng.standard_normal((m, n)).astype(np.float32)
    checks = gs.softmax_checks(x)
    w = 2.0 * np.arange(n) - (n - 1)
    np.testing.assert_allclose(checks["actual_sum"], x.astype(np.float64).sum(axis=1), atol=1e-9)
    np.testing.assert_allclose(checks["actual_weighted"], (x.astype(np.float64) * w).sum(axis=1), atol=1e-8)
    np.testing.assert_allclose(checks["probability_sum"], 1.0, atol=2e-6)
    es, ew = x.astype(np.float64).sum(axis=1), (x.astype(np.float64) * w).sum(axis=1)
    assert gs.analyze(es, ew, checks, n)["counts"].tolist() == [0, 0]
    y = x.copy()
    y[3, 150] += np.float32(1e-3)  # below abs_tol = 2e-3 in both identities (w_150 = 1)
    assert gs.analyze(es, ew, gs.softmax_checks(y), n)["counts"].tolist() == [0, 0]
    y[3, 17] += np.float32(1e-3)  # w_17 = -265: the weighted identity fires, the unweighted one cannot locate it
    assert gs.analyze(es, ew, gs.softmax_checks(y), n)["counts"].tolist() == [1, 0]
    y = x.copy()
    y[3, 17] += np.float32(0.5)
    out = gs.analyze(es, ew, gs.softmax_checks(y), n)
    assert out["counts"].tolist() == [1, 1] and out["estimated_col"][3] == 17
