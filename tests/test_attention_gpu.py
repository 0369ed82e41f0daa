"""GPU parity tests of the fault-tolerant attention forward (through the C-ABI)
against the CPU oracle and an FP64 softmax(QK^T/sqrt(D))V.

Tolerances: outputs agree with the oracle within 2e-3 absolute (the products are
exact, the differences come from the accumulation order of the tensor core, from
ex2.approx against libm's exp2f, and from FP16 rounding of probabilities that sit
on a rounding boundary) and with the FP64 truth within 4e-3; counters and
located positions must be equal."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

from tests import oracle_attention as oa  # noqa: E402

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ftg():
    import ft_gemm_b200
    ft_gemm_b200.load()
    assert torch.cuda.is_available()
    return ft_gemm_b200


def _qkv(b, h, n, d=128, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return tuple(torch.randn((b, h, n, d), generator=g).to(torch.float16).cuda() for _ in range(3))


def _np(t):
    return t.cpu().numpy()


@pytest.mark.parametrize("exact_prepare", [False, True])
@pytest.mark.parametrize("b,h,n", [(1, 1, 128), (1, 2, 256), (2, 3, 512), (1, 2, 2176)])
def test_clean_forward(ftg, b, h, n, exact_prepare):
    """exact_prepare=False: score checksums from FP16 pieces of the band sums on the tensor cores; True: CUDA cores."""
    q, k, v = _qkv(b, h, n, seed=n)
    op = ftg.FtAttention(q, k, v, exact_prepare=exact_prepare)
    out = op.new_output()
    op.run(out)
    rep = op.report()
    assert (rep.status, rep.score_detected, rep.pv_detected, rep.failed_rows) == (0, 0, 0, 0)
    assert rep.max_score_noise < 0.1
    want, stats, _ = oa.forward(_np(q), _np(k), _np(v))
    assert stats.score_detected == 0
    np.testing.assert_allclose(_np(out), want, atol=2e-3, rtol=0)
    np.testing.assert_allclose(_np(out), oa.truth_fp64(_np(q), _np(k), _np(v)), atol=4e-3, rtol=0)
    op.close()


@pytest.mark.parametrize("exact_prepare", [False, True])
def test_score_faults_match_oracle(ftg, exact_prepare):
    b, h, n = 1, 2, 512
    q, k, v = _qkv(b, h, n, seed=7)
    op = ftg.FtAttention(q, k, v, exact_prepare=exact_prepare)
    clean = op.new_output()
    op.run(clean)
    assert op.report().score_detected == 0
    out = op.new_output()
    bands = n // 64
    # every TMEM lane quarter of the CTA, both 64-column halves, first / middle / last key tile
    cases = [(0, 0, 0, 3.0), (1, 40, 100, -2.5), (0, 70, 200, 8.0), (1, 100, 511, 1.5), (0, 300, 64, -6.0), (1, 511, 447, 64.0)]
    for head, query, key, value in cases:
        fault = (ftg.FAULT_SCORE, 0, head, query, key, value)
        op.run(out, fault)
        rep = op.report()
        want, stats, records = oa.forward(_np(q), _np(k), _np(v), fault=fault)
        assert stats.min_margin > 1e-3
        assert (rep.score_detected, rep.score_corrected, rep.score_uncorrected) == (1, 1, 0) == \
               (stats.score_detected, stats.score_corrected, stats.score_uncorrected)
        got, exp = rep.records[0], records[0]
        assert (got.tile, got.bad_row, got.bad_col, got.corrected) == (exp.tile, exp.bad_row, exp.bad_col, 1)
        assert got.tile == ((head * bands) + query // 64) * bands + key // 64
        assert got.row_delta == pytest.approx(exp.row_delta, abs=2e-3) and got.col_delta == pytest.approx(exp.col_delta, abs=2e-3)
        assert (rep.pv_detected, rep.failed_rows) == (0, 0)
        np.testing.assert_allclose(_np(out), _np(clean), atol=5e-4, rtol=0)
    op.close()


@pytest.mark.parametrize("protect_softmax", [False, True])
def test_score_tile_with_several_faults_is_replayed(ftg, protect_softmax):
    """Two faults in one 64x64 score tile cannot be located by the row/column intersection: the tile is recomputed on
    the CUDA cores, passes the check the second time and counts as replayed (src/ft_flash_attention_a14.cu:935-959);
    the output equals the clean one.  Patterns: two rows and two columns, one row with two columns, one column with two
    rows; with and without the softmax-stage protection."""
    b, h, n = 1, 2, 512
    q, k, v = _qkv(b, h, n, seed=21)
    op = ftg.FtAttention(q, k, v, protect_softmax=protect_softmax)
    clean = op.new_output()
    op.run(clean)
    assert op.report().score_detected == 0
    out = op.new_output()
    bands = n // 64
    cases = [(0, 70, 200, 8.0, 100, 230, -5.0), (1, 300, 64, -6.0, 300, 100, 9.0), (0, 10, 450, 4.0, 40, 450, 7.0),
             (1, 511, 511, 64.0, 450, 449, -32.0)]
    for head, q1, k1, v1, q2, k2, v2 in cases:
        assert q1 // 64 == q2 // 64 and k1 // 64 == k2 // 64
        fault = (ftg.FAULT_SCORE, 0, head, q1, k1, v1, q2, k2, v2)
        op.run(out, fault)
        rep = op.report()
        want, stats, records = oa.forward(_np(q), _np(k), _np(v), fault=fault, protect_softmax=protect_softmax)
        assert stats.min_margin > 1e-3
        assert (rep.score_detected, rep.score_corrected, rep.score_replayed, rep.score_uncorrected) == (1, 0, 1, 0) == \
               (stats.score_detected, stats.score_corrected, stats.score_replayed, stats.score_uncorrected)
        got, exp = rep.records[0], records[0]
        assert (got.tile, got.bad_row_count, got.bad_col_count, got.corrected) == (exp.tile, exp.bad_row_count, exp.bad_col_count, 0)
        assert got.tile == ((head * bands) + q1 // 64) * bands + k1 // 64
        assert (rep.pv_detected, rep.failed_rows, rep.softmax_detected) == (0, 0, 0)
        np.testing.assert_allclose(_np(out), _np(clean), atol=5e-4, rtol=0)
        np.testing.assert_allclose(_np(out), want, atol=2e-3, rtol=0)
    # faults in two different tiles of one run are two single faults: both located and corrected
    fault = (ftg.FAULT_SCORE, 0, 1, 20, 30, 5.0, 400, 300, -5.0)
    op.run(out, fault)
    rep = op.report()
    assert (rep.score_detected, rep.score_corrected, rep.score_replayed, rep.score_uncorrected) == (2, 2, 0, 0)
    np.testing.assert_allclose(_np(out), _np(clean), atol=5e-4, rtol=0)
    op.close()


def test_stale_cache_tiles_stay_uncorrected_after_replay(ftg):
    # K changes after prepare: the cached checksums are stale, so the replayed tiles disagree with them as well
    b, h, n = 1, 1, 256
    q, k, v = _qkv(b, h, n, seed=9)
    op = ftg.FtAttention(q, k, v)
    k[0, 0, 5, :] += 1.0  # column 5 of every score tile of key band 0 now disagrees with the cached checksums
    out = op.new_output()
    op.run(out)
    rep = op.report()
    assert rep.score_detected >= n // 64 and rep.score_corrected == 0 and rep.score_uncorrected == rep.score_detected
    assert rep.score_replayed == 0
    assert all(r.bad_col_count >= 1 and r.corrected == 0 for r in rep.records)
    op.close()


@pytest.mark.parametrize("n,d", [(256, 128), (333, 128), (512, 64)])
def test_refresh_rebuilds_the_metadata_without_a_new_handle(ftg, n, d):
    """A handle refreshed with new Q, K, V (new pointers, or the old buffers changed in place) gives bit for bit what a fresh
    handle gives; the sequence length that is not a whole tile goes through the handle's padded copies."""
    b, h = 1, 2
    q1, k1, v1 = _qkv(b, h, n, d, seed=21)
    q2, k2, v2 = _qkv(b, h, n, d, seed=22)
    fresh = ftg.FtAttention(q2, k2, v2)
    want = fresh.new_output()
    fresh.run(want)
    assert fresh.report().score_detected == 0
    fresh.close()

    op = ftg.FtAttention(q1, k1, v1)
    out = op.new_output()
    op.run(out)
    assert op.report().score_detected == 0
    op.refresh(q2, k2, v2)  # other buffers
    op.run(out)
    rep = op.report()
    assert (rep.status, rep.score_detected, rep.pv_detected, rep.failed_rows) == (0, 0, 0, 0)
    assert torch.equal(out, want)
    q2.copy_(q1), k2.copy_(k1), v2.copy_(v1)  # the same buffers, new contents: stale until refreshed
    op.refresh(q2, k2, v2)
    op.run(out)
    rep = op.report()
    assert (rep.status, rep.score_detected, rep.pv_detected, rep.failed_rows) == (0, 0, 0, 0)
    np.testing.assert_allclose(_np(out), oa.truth_fp64(_np(q1), _np(k1), _np(v1)), atol=4e-3, rtol=0)
    with pytest.raises(ValueError):
        op.refresh(q2[:, :1], k2[:, :1], v2[:, :1])
    op.close()


def test_output_faults_match_oracle(ftg):
    b, h, n = 2, 2, 256
    q, k, v = _qkv(b, h, n, seed=11)
    op = ftg.FtAttention(q, k, v)
    clean = op.new_output()
    op.run(clean)
    out = op.new_output()
    for batch, head, query, dim, value in [(0, 0, 3, 0, 0.5), (1, 1, 200, 127, -1.0), (0, 1, 64, 64, 0.05), (1, 0, 255, 31, 3.0)]:
        fault = (ftg.FAULT_OUTPUT, batch, head, query, dim, value)
        op.run(out, fault)
        rep = op.report()
        _, stats, _ = oa.forward(_np(q), _np(k), _np(v), fault=fault)
        assert (rep.pv_detected, rep.pv_corrected, rep.failed_rows) == (1, 1, 0) == (stats.pv_detected, stats.pv_corrected, stats.failed_rows)
        assert rep.score_detected == 0
        np.testing.assert_allclose(_np(out), _np(clean), atol=6e-3, rtol=0)
    # under the projection tolerance: invisible, as in the reference
    op.run(out, (ftg.FAULT_OUTPUT, 0, 0, 10, 10, 1e-3))
    assert op.report().pv_detected == 0
    op.close()


def test_repeat_runs_are_bit_identical_and_arguments_checked(ftg):
    q, k, v = _qkv(1, 2, 384, seed=13)
    op = ftg.FtAttention(q, k, v)
    first = op.new_output()
    op.run(first, (ftg.FAULT_SCORE, 0, 1, 100, 300, 5.0))
    for _ in range(5):
        out = op.new_output()
        op.run(out, (ftg.FAULT_SCORE, 0, 1, 100, 300, 5.0))
        assert op.report().score_corrected == 1
        assert torch.equal(out, first)
    with pytest.raises(ftg.FtGemmError):
        op.run(first, (ftg.FAULT_SCORE, 0, 5, 0, 0, 1.0))  # head out of range
    with pytest.raises(ftg.FtGemmError):
        op.run(first, (2, 0, 0, 0, 0, 1.0))  # a softmax-stage fault needs a handle prepared with protect_softmax
    op.close()
    with pytest.raises(ftg.FtGemmError):
        ftg.FtAttention(q[..., :96].contiguous(), k[..., :96].contiguous(), v[..., :96].contiguous())  # D must be 64 or 128


def test_config5_shape_properties(ftg):
    """B=4 H=32 N=4096 D=128: too large for the CPU oracle in full; sampled rows against FP64 and a score fault."""
    b, h, n = 4, 32, 4096
    q, k, v = _qkv(b, h, n, seed=17)
    op = ftg.FtAttention(q, k, v)
    out = op.new_output()
    op.run(out)
    rep = op.report()
    assert (rep.status, rep.score_detected, rep.pv_detected, rep.failed_rows) == (0, 0, 0, 0)
    for batch, head in [(0, 0), (3, 31), (1, 7)]:
        rows = torch.tensor([0, 1, 1000, 2047, 2048, 4095])
        qs = q[batch, head, rows].double()
        s = qs @ k[batch, head].double().T / 128 ** 0.5
        want = torch.softmax(s, dim=-1) @ v[batch, head].double()
        assert float((out[batch, head, rows].double() - want).abs().max()) < 4e-3
    faulty = op.new_output()
    op.run(faulty, (ftg.FAULT_SCORE, 2, 5, 2049, 4000, 12.0))
    rep = op.report()
    assert (rep.score_detected, rep.score_corrected, rep.pv_detected) == (1, 1, 0)
    assert float((faulty - out).abs().max()) < 5e-4
    op.close()


@pytest.mark.parametrize("d", [128, 64])
def test_softmax_stage_protection(ftg, d):
    """protect_softmax adds the reference's third protected stage (a14:964-1099)."""
    b, h, n = 1, 2, 384
    q, k, v = _qkv(b, h, n, d, seed=19)
    plain_op = ftg.FtAttention(q, k, v)
    plain = plain_op.new_output()
    plain_op.run(plain)
    with pytest.raises(ftg.FtGemmError):
        plain_op.run(plain, (ftg.FAULT_SOFTMAX, 0, 0, 1, 1, 0.5))  # needs a handle prepared with the protection
    plain_op.close()
    op = ftg.FtAttention(q, k, v, protect_softmax=True)
    clean = op.new_output()
    op.run(clean)
    rep = op.report()
    assert (rep.softmax_detected, rep.score_detected, rep.pv_detected, rep.failed_rows) == (0, 0, 0, 0)
    assert torch.equal(clean, plain)  # the protection changes nothing when nothing is wrong
    want, _, _ = oa.forward(_np(q), _np(k), _np(v), protect_softmax=True)
    np.testing.assert_allclose(_np(clean), want, atol=2e-3, rtol=0)
    out = op.new_output()
    for head, query, key, value in [(1, 5, 9, 0.25), (0, 200, 383, 0.5), (1, 383, 130, 0.01), (0, 130, 64, 1.0)]:
        fault = (ftg.FAULT_SOFTMAX, 0, head, query, key, value)
        op.run(out, fault)
        rep = op.report()
        _, stats, _ = oa.forward(_np(q), _np(k), _np(v), protect_softmax=True, fault=fault)
        assert (rep.softmax_detected, rep.softmax_corrected, rep.softmax_replayed) == (1, 1, 0) == \
               (stats.softmax_detected, stats.softmax_corrected, stats.softmax_replayed)
        assert (rep.pv_detected, rep.failed_rows, rep.score_detected) == (0, 0, 0)
        assert torch.equal(out, clean)  # the verifier's probability replaces the faulty one exactly
    fault = (ftg.FAULT_SOFTMAX_STATE, 0, 0, 100, 300, 0.75)
    op.run(out, fault)
    rep = op.report()
    _, stats, _ = oa.forward(_np(q), _np(k), _np(v), protect_softmax=True, fault=fault)
    assert (rep.softmax_detected, rep.softmax_corrected, rep.softmax_replayed) == (1, 0, 1) == \
           (stats.softmax_detected, stats.softmax_corrected, stats.softmax_replayed)
    assert torch.equal(out, clean)
    # the other two stages still work under the protection
    op.run(out, (ftg.FAULT_SCORE, 0, 1, 77, 200, 6.0))
    rep = op.report()
    assert (rep.score_corrected, rep.softmax_detected, rep.pv_detected) == (1, 0, 0)
    op.run(out, (ftg.FAULT_OUTPUT, 0, 0, 10, 100 % d, 0.5))
    rep = op.report()
    assert (rep.pv_corrected, rep.softmax_detected, rep.failed_rows) == (1, 0, 0)
    op.close()


def test_whole_row_kernel_when_selected(ftg):
    """FT_ATTENTION_KERNEL=row selects the kernel with one thread per query row (read once per process, hence the child)."""
    import os
    import subprocess
    import sys
    code = """
import numpy as np, torch, ft_gemm_b200 as ftg
from tests import oracle_attention as oa
g = torch.Generator(device='cpu').manual_seed(31)
q, k, v = (torch.randn((1, 2, 384, 128), generator=g).to(torch.float16).cuda() for _ in range(3))
for protect in (False, True):
    op = ftg.FtAttention(q, k, v, protect_softmax=protect)
    clean = op.new_output(); op.run(clean); rep = op.report()
    assert (rep.status, rep.score_detected, rep.pv_detected, rep.failed_rows, rep.softmax_detected) == (0, 0, 0, 0, 0)
    truth = oa.truth_fp64(q.cpu().numpy(), k.cpu().numpy(), v.cpu().numpy())
    np.testing.assert_allclose(clean.cpu().numpy(), truth, atol=4e-3, rtol=0)
    out = op.new_output(); op.run(out, (ftg.FAULT_SCORE, 0, 1, 77, 200, 6.0)); rep = op.report()
    assert (rep.score_detected, rep.score_corrected) == (1, 1)
    assert float((out - clean).abs().max()) < 5e-4
    op.run(out, (ftg.FAULT_SCORE, 0, 0, 70, 200, 8.0, 100, 230, -5.0)); rep = op.report()  # two faults in one tile
    assert (rep.score_detected, rep.score_corrected, rep.score_replayed, rep.score_uncorrected) == (1, 0, 1, 0)
    assert float((out - clean).abs().max()) < 5e-4
    if protect:
        op.run(out, (ftg.FAULT_SOFTMAX, 0, 1, 5, 9, 0.25)); rep = op.report()
        assert (rep.softmax_detected, rep.softmax_corrected, rep.softmax_replayed) == (1, 1, 0)
        assert torch.equal(out, clean)
    op.close()
print('row kernel ok')
"""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, FT_ATTENTION_KERNEL="row", PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""))
    done = subprocess.run([sys.executable, "-c", code], cwd=root, env=env, capture_output=True, text=True, timeout=300)
    assert done.returncode == 0 and "row kernel ok" in done.stdout, done.stdout[-2000:] + done.stderr[-2000:]


@pytest.mark.parametrize("n", [128, 384, 512])
def test_causal_forward_and_faults(ftg, n):
    """causal = key <= query (src/ft_flash_attention_a14.cu:708, 893): key tiles beyond the diagonal are skipped, the
    diagonal tile is verified raw and masked afterwards."""
    b, h = 1, 2
    q, k, v = _qkv(b, h, n, seed=23 + n)
    op = ftg.FtAttention(q, k, v, causal=True)
    clean = op.new_output()
    op.run(clean)
    rep = op.report()
    assert (rep.status, rep.score_detected, rep.pv_detected, rep.failed_rows) == (0, 0, 0, 0)
    want, stats, _ = oa.forward(_np(q), _np(k), _np(v), causal=True)
    assert stats.score_detected == 0
    np.testing.assert_allclose(_np(clean), want, atol=2e-3, rtol=0)
    np.testing.assert_allclose(_np(clean), oa.truth_fp64(_np(q), _np(k), _np(v), causal=True), atol=4e-3, rtol=0)
    assert torch.equal(clean[:, :, 0, :], v[:, :, 0, :].float())  # the first query sees key 0 only
    out = op.new_output()
    for head, query, key, value in [(0, n - 1, 0, 3.0), (1, n // 2, n // 2, -4.0), (0, 100, 64, 6.0), (1, n - 1, n - 2, 2.0)]:
        fault = (ftg.FAULT_SCORE, 0, head, query, key, value)
        op.run(out, fault)
        rep = op.report()
        _, stats, records = oa.forward(_np(q), _np(k), _np(v), causal=True, fault=fault)
        assert (rep.score_detected, rep.score_corrected) == (1, 1) == (stats.score_detected, stats.score_corrected)
        assert (rep.records[0].tile, rep.records[0].bad_row, rep.records[0].bad_col) == (records[0].tile, query % 64, key % 64)
        np.testing.assert_allclose(_np(out), _np(clean), atol=5e-4, rtol=0)
    op.run(out, (ftg.FAULT_OUTPUT, 0, 1, n - 1, 77, 0.5))
    rep = op.report()
    assert (rep.pv_detected, rep.pv_corrected, rep.failed_rows) == (1, 1, 0)
    with pytest.raises(ftg.FtGemmError):
        op.run(out, (ftg.FAULT_SCORE, 0, 0, 10, 11, 1.0))  # a masked score is never computed (a14:278)
    op.close()
    # with the softmax-stage protection
    op = ftg.FtAttention(q, k, v, causal=True, protect_softmax=True)
    protected = op.new_output()
    op.run(protected)
    # the protected form runs in the whole-row kernel, which adds the row sums in another order than the split-row one
    assert float((protected - clean).abs().max()) < 5e-4 and op.report().softmax_detected == 0  # FP16 rounding of the probabilities against different exponent references
    fault = (ftg.FAULT_SOFTMAX, 0, 1, n - 1, n - 3, 0.25)
    op.run(out, fault)
    rep = op.report()
    assert (rep.softmax_detected, rep.softmax_corrected) == (1, 1)
    assert torch.equal(out, protected)
    op.close()


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("exact_prepare", [False, True])
def test_head_dim_64(ftg, causal, exact_prepare):
    """The reference's default head dimension (src/ft_flash_attention_a14.cu:114, 267)."""
    b, h, n, d = 2, 2, 384, 64
    q, k, v = _qkv(b, h, n, d=d, seed=41)
    op = ftg.FtAttention(q, k, v, causal=causal, exact_prepare=exact_prepare)
    clean = op.new_output()
    op.run(clean)
    rep = op.report()
    assert (rep.status, rep.score_detected, rep.pv_detected, rep.failed_rows) == (0, 0, 0, 0)
    want, stats, _ = oa.forward(_np(q), _np(k), _np(v), causal=causal)
    assert stats.score_detected == 0
    np.testing.assert_allclose(_np(clean), want, atol=2e-3, rtol=0)
    np.testing.assert_allclose(_np(clean), oa.truth_fp64(_np(q), _np(k), _np(v), causal=causal), atol=4e-3, rtol=0)
    out = op.new_output()
    for head, query, key, value in [(0, 383, 0, 3.0), (1, 200, 130, -4.0), (0, 64, 63, 6.0)]:
        fault = (ftg.FAULT_SCORE, 1, head, query, key, value)
        op.run(out, fault)
        rep = op.report()
        _, stats, records = oa.forward(_np(q), _np(k), _np(v), causal=causal, fault=fault)
        assert (rep.score_detected, rep.score_corrected) == (1, 1) == (stats.score_detected, stats.score_corrected)
        assert (rep.records[0].tile, rep.records[0].bad_row, rep.records[0].bad_col) == (records[0].tile, query % 64, key % 64)
        np.testing.assert_allclose(_np(out), _np(clean), atol=5e-4, rtol=0)
    for query, dim, value in [(5, 0, 0.5), (300, 63, -1.0), (129, 31, 0.25), (383, 32, 2.0)]:  # both dim halves, both tiles
        fault = (ftg.FAULT_OUTPUT, 0, 1, query, dim, value)
        op.run(out, fault)
        rep = op.report()
        _, stats, _ = oa.forward(_np(q), _np(k), _np(v), causal=causal, fault=fault)
        assert (rep.pv_detected, rep.pv_corrected, rep.failed_rows) == (1, 1, 0) == (stats.pv_detected, stats.pv_corrected, stats.failed_rows)
        np.testing.assert_allclose(_np(out), _np(clean), atol=6e-3, rtol=0)
    op.close()


@pytest.mark.parametrize("n,d,causal", [(384, 64, True), (333, 64, False), (300, 128, True)])
def test_softmax_stage_protection_with_masks(ftg, n, d, causal):
    """The protected forward on causal and padded tiles (masked keys have probability zero in both copies) and with both head
    dimensions: clean runs equal the unprotected ones bit for bit; probability and state faults are detected and repaired,
    on the diagonal tile as well."""
    b, h = 1, 2
    q, k, v = _qkv(b, h, n, d=d, seed=57 + n)
    plain_op = ftg.FtAttention(q, k, v, causal=causal)
    plain = plain_op.new_output()
    plain_op.run(plain)
    plain_op.close()
    op = ftg.FtAttention(q, k, v, causal=causal, protect_softmax=True)
    clean = op.new_output()
    op.run(clean)
    rep = op.report()
    assert (rep.status, rep.softmax_detected, rep.score_detected, rep.pv_detected, rep.failed_rows) == (0, 0, 0, 0, 0)
    assert torch.equal(clean, plain)
    np.testing.assert_allclose(_np(clean), oa.truth_fp64(_np(q), _np(k), _np(v), causal=causal), atol=4e-3, rtol=0)
    out = op.new_output()
    last = n - 1
    for head, query, key, value in [(0, last, last, 0.5), (1, 130, 129, 0.25), (0, 70, 3, 1.0), (1, last, 128, 0.125)]:
        fault = (ftg.FAULT_SOFTMAX, 0, head, query, key, value)  # key <= query: valid under the causal mask too
        op.run(out, fault)
        rep = op.report()
        _, stats, _ = oa.forward(_np(q), _np(k), _np(v), causal=causal, protect_softmax=True, fault=fault)
        assert (rep.softmax_detected, rep.softmax_corrected, rep.softmax_replayed) == (1, 1, 0) == \
               (stats.softmax_detected, stats.softmax_corrected, stats.softmax_replayed)
        assert (rep.pv_detected, rep.failed_rows, rep.score_detected) == (0, 0, 0)
        assert torch.equal(out, clean)
    fault = (ftg.FAULT_SOFTMAX_STATE, 0, 1, last, 5, 0.75)
    op.run(out, fault)
    rep = op.report()
    assert (rep.softmax_detected, rep.softmax_corrected, rep.softmax_replayed) == (1, 0, 1)
    assert torch.equal(out, clean)
    op.close()


@pytest.mark.parametrize("n,d,causal", [(200, 128, False), (333, 64, True), (1, 64, False), (129, 128, True), (2100, 128, False),
                                        (77, 128, True)])
def test_sequence_lengths_that_are_not_whole_tiles(ftg, n, d, causal):
    """Any sequence length (the reference masks by index, src/ft_flash_attention_a14.cu:893): the handle pads Q, K, V to whole
    tiles, padded keys carry no weight, padded queries leave no output row and no counters."""
    b, h = 1, 2
    q, k, v = _qkv(b, h, n, d=d, seed=70 + n)
    op = ftg.FtAttention(q, k, v, causal=causal)
    guard = torch.full((b, h, n + 1, d), 7.0, device="cuda")  # one spare row per head pair: nothing may be written past N
    out = guard.view(-1)[: b * h * n * d].view(b, h, n, d)
    op.run(out)
    rep = op.report()
    assert (rep.status, rep.score_detected, rep.pv_detected, rep.failed_rows) == (0, 0, 0, 0)
    assert torch.all(guard.view(-1)[b * h * n * d:] == 7.0)
    want, stats, _ = oa.forward(_np(q), _np(k), _np(v), causal=causal)
    np.testing.assert_allclose(_np(out), want, atol=2e-3, rtol=0)
    np.testing.assert_allclose(_np(out), oa.truth_fp64(_np(q), _np(k), _np(v), causal=causal), atol=4e-3, rtol=0)
    clean = out.clone()
    last = n - 1
    key = last if causal else max(0, n - 3)
    fault = (ftg.FAULT_SCORE, 0, 1, last, key // 2 if causal else key, 3.0)
    op.run(out, fault)
    rep = op.report()
    _, stats, records = oa.forward(_np(q), _np(k), _np(v), causal=causal, fault=fault)
    assert (rep.score_detected, rep.score_corrected) == (1, 1) == (stats.score_detected, stats.score_corrected)
    assert (rep.records[0].tile, rep.records[0].bad_row, rep.records[0].bad_col) == (records[0].tile, records[0].bad_row, records[0].bad_col)
    np.testing.assert_allclose(_np(out), _np(clean), atol=5e-4, rtol=0)
    fault = (ftg.FAULT_OUTPUT, 0, 0, last, d - 1, 0.5)
    op.run(out, fault)
    rep = op.report()
    assert (rep.pv_detected, rep.pv_corrected, rep.failed_rows) == (1, 1, 0)
    np.testing.assert_allclose(_np(out), _np(clean), atol=6e-3, rtol=0)
    with pytest.raises(ftg.FtGemmError):
        op.run(out, (ftg.FAULT_SCORE, 0, 0, n, 0, 1.0))  # a query in the padding
    op.close()
    if d == 128:
        op = ftg.FtAttention(q, k, v, causal=causal, protect_softmax=True)
        op.run(out, (2, 0, 0, last, key // 2 if causal else key, 0.25))
        rep = op.report()
        assert (rep.softmax_detected, rep.softmax_corrected) == (1, 1)
        # `clean` came from the split-row kernel, this output from the whole-row kernel: FP16 rounding of the probabilities apart
        np.testing.assert_allclose(_np(out), _np(clean), atol=5e-4, rtol=0)
        op.close()


def test_against_reference_a0_fixtures(ftg):
    """The CUDA path on the inputs of the reference's own scalar attention kernel (tests/golden/a0_*.npz): outputs within
    2e-3 of the reference's, the same stage counters for every fault scenario."""
    import glob
    import os
    from tests import oracle_lib
    oracle = oracle_lib.load()
    paths = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "a0_*.npz")))
    assert paths
    for path in paths:
        g = np.load(path)
        b, h, n, d, causal = (int(x) for x in g["shape"])
        q, k, v = (torch.from_numpy(oracle.decode(g[name]).reshape(b, h, n, d)).to(torch.float16).cuda() for name in ("q", "k", "v"))
        ops = {False: ftg.FtAttention(q, k, v, causal=bool(causal))}
        if d == 128:
            ops[True] = ftg.FtAttention(q, k, v, causal=bool(causal), protect_softmax=True)
        out = ops[False].new_output()
        clean = None
        for i, (stage, query, index, value) in enumerate(g["scenarios"]):
            stage, query, index = int(stage), int(query), int(index)
            protect = stage in (2, 3)
            if protect and d != 128:
                continue
            op = ops[protect]
            op.run(out, None if stage == 0 else (stage, 0, 0, query, index, float(value)))
            rep = op.report()
            ref = [int(x) for x in g[f"stats_{i}"]]  # score d/c/replayed, softmax d/c/r, pv d/c, failed rows (a0:35-45)
            assert rep.failed_rows == 0 == ref[8]
            if stage == 0:
                clean = g[f"out_{i}"].astype(np.float32).reshape(b, h, n, d)
                np.testing.assert_allclose(_np(out), clean, atol=2e-3, rtol=0)
                assert (rep.score_detected, rep.pv_detected, rep.softmax_detected) == (0, 0, 0)
                continue
            np.testing.assert_allclose(_np(out)[0, 0, query], g[f"row_{i}"], atol=2e-3, rtol=0)
            np.testing.assert_allclose(_np(out), clean, atol=2e-3, rtol=0)
            if stage == 1:
                assert (rep.score_detected, rep.score_corrected) == (1, 1) == (ref[0], ref[1] + ref[2])
            elif stage == 2:
                assert (rep.softmax_detected, rep.softmax_corrected, rep.softmax_replayed) == (1, 1, 0) == (ref[3], ref[4], ref[5])
            elif stage == 3:
                assert (rep.softmax_detected, rep.softmax_corrected, rep.softmax_replayed) == (1, 0, 1) == (ref[3], ref[4], ref[5])
            else:
                assert (rep.pv_detected, rep.pv_corrected) == (1, 1) == (ref[6], ref[7])
        for op in ops.values():
            op.close()
