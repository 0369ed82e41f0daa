"""GPU parity tests of the GEMM + softmax cross-nonlinearity check (through the C-ABI of include/ft_gemm_softmax.h)
against the CPU oracle: inputs, logits and expected projections bit for bit (the prototype's inputs make every sum
exact), the values behind exp()/log() within 1e-9, decisions and located columns equal."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

from tests import oracle_gs as gs  # noqa: E402

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ftg():
    import ft_gemm_b200
    ft_gemm_b200.load()
    assert torch.cuda.is_available()
    return ft_gemm_b200


@pytest.mark.parametrize("m,n,k,fault", [(64, 64, 64, (32, 32, 1.0)), (96, 200, 128, (5, 199, -0.75)), (128, 1000, 256, (100, 0, 2.5)),
                                         (33, 77, 100, (0, 76, 0.5)), (256, 2048, 512, (255, 1024, -3.0))])
def test_matches_oracle(ftg, m, n, k, fault):
    a = ftg.generate_gs_fp8((m, k), 17)
    b = ftg.generate_gs_fp8((n, k), 29)
    ah, bh = a.cpu().numpy().ravel(), b.cpu().numpy().ravel()
    np.testing.assert_array_equal(ah, gs.generate(m * k, 17))
    np.testing.assert_array_equal(bh, gs.generate(n * k, 29))
    op = ftg.GemmSoftmaxAbft(a, b)
    clean = op.new_output()
    op.run(clean)
    rep = op.report()
    assert (rep.status, rep.detected_rows, rep.located_rows, rep.post_detected_rows, rep.gemm_bad_tiles) == (0, 0, 0, -1, 0)
    x = gs.logits(ah, bh, m, n, k)
    np.testing.assert_array_equal(op.logits().numpy().view(np.uint32), x.view(np.uint32))  # exact products, exact sums
    es, ew = gs.expected(ah, bh, m, n, k)
    got = op.checks()
    np.testing.assert_array_equal(got["expected_sum"].view(np.uint64), es.view(np.uint64))
    np.testing.assert_array_equal(got["expected_weighted"].view(np.uint64), ew.view(np.uint64))
    want = gs.softmax_checks(x)
    for name in ("actual_sum", "actual_weighted", "probability_sum", "log_z"):
        np.testing.assert_allclose(got[name], want[name], rtol=1e-11, atol=1e-9, err_msg=name)
    np.testing.assert_allclose(clean.cpu().numpy(), want["probabilities"], rtol=3e-7, atol=0)
    assert rep.max_projection_residual == pytest.approx(
        max(np.abs(want["actual_sum"] - es).max(), np.abs(want["actual_weighted"] - ew).max()), abs=1e-9)

    row, col, value = fault
    out = op.new_output()
    op.run(out, fault=fault, correct=True)
    rep = op.report()
    xf = x.copy()
    xf[row, col] += np.float32(value)
    analysis = gs.analyze(es, ew, gs.softmax_checks(xf), n)
    assert (rep.detected_rows, rep.located_rows) == tuple(analysis["counts"]) == (1, 1)
    assert rep.records == [(row, col, pytest.approx(analysis["correction_delta"][row], abs=1e-9))]
    assert rep.post_detected_rows == 0
    recovered = gs.softmax_checks(gs.correct(xf, analysis))
    np.testing.assert_allclose(out.cpu().numpy(), recovered["probabilities"], rtol=3e-7, atol=0)
    assert float((out - clean).abs().max()) <= 1e-6  # the reference's recovery criterion (gs:519)
    # without correction the faulty row's probabilities stay wrong and the report says so
    op.run(out, fault=fault, correct=False)
    rep = op.report()
    assert (rep.detected_rows, rep.located_rows, rep.post_detected_rows) == (1, 1, -1)
    assert float((out[row] - clean[row]).abs().max()) > 1e-4
    op.close()


def test_general_inputs(ftg):
    """N(0,1) E4M3 inputs: sums are no longer exact, the logits agree with the FP32 oracle within 1e-5 * K and the
    identities hold within the tolerances."""
    m, n, k = 128, 384, 256
    a = ftg.generate_fp8((m, k), 5, "normal")
    b = ftg.generate_fp8((n, k), 6, "normal")
    ah, bh = a.cpu().numpy().ravel(), b.cpu().numpy().ravel()
    op = ftg.GemmSoftmaxAbft(a, b)
    p = op.new_output()
    op.run(p)
    rep = op.report()
    assert (rep.detected_rows, rep.gemm_bad_tiles) == (0, 0)
    np.testing.assert_allclose(op.logits().numpy(), gs.logits(ah, bh, m, n, k), atol=1e-5 * k, rtol=0)
    truth = torch.softmax(torch.from_numpy(gs.logits(ah, bh, m, n, k)).double(), dim=-1)
    assert float((p.cpu().double() - truth).abs().max()) < 1e-5
    with pytest.raises(ftg.FtGemmError):
        op.run(p, fault=(m, 0, 1.0))
    op.close()
    with pytest.raises(ftg.FtGemmError):
        ftg.GemmSoftmaxAbft(a, b[:1].contiguous())  # N must exceed 1 (gs:121)
