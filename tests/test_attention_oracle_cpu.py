"""CPU tests of the attention oracle: FP16 codec against numpy, values against an
FP64 softmax(QK^T/sqrt(D))V, and the two protected stages' decisions."""
import numpy as np
import pytest

from tests import oracle_attention as oa


def _qkv(b, h, n, d, seed=0):
    rng = np.random.default_rng(seed)
    return tuple(rng.standard_normal((b, h, n, d)).astype(np.float16) for _ in range(3))


def test_half_codec_matches_numpy():
    rng = np.random.default_rng(1)
    values = np.concatenate([rng.standard_normal(2000) * 10.0 ** rng.integers(-8, 5, 2000), [0.0, 65504.0, 65519.9, 65520.0, 1e9,
                            6e-8, 2.98e-8, 2.99e-8, 1.0009765625 + 2 ** -12, -3.1415]]).astype(np.float32)
    for x in values:
        bits, back = oa.half_roundtrip(float(x))
        want = np.float32(x).astype(np.float16)
        assert bits == int(want.view(np.uint16)), x
        assert back == float(want) or (np.isinf(want) and np.isinf(back))


def test_clean_forward_matches_fp64():
    q, k, v = _qkv(1, 2, 256, 128)
    out, stats, records = oa.forward(q, k, v)
    assert (stats.score_detected, stats.pv_detected, stats.failed_rows) == (0, 0, 0) and not records
    assert stats.max_score_noise < 0.1
    # FP16 probabilities limit the accuracy: 2^-11 relative per term
    np.testing.assert_allclose(out, oa.truth_fp64(q, k, v), atol=3e-3, rtol=0)


def test_score_fault_is_located_and_corrected():
    q, k, v = _qkv(1, 2, 256, 128, seed=3)
    clean, _, _ = oa.forward(q, k, v)
    for query, key, value in [(0, 0, 2.0), (77, 200, -5.0), (255, 129, 9.0), (128, 63, 1.5)]:
        out, stats, records = oa.forward(q, k, v, fault=(1, 0, 1, query, key, value))
        assert (stats.score_detected, stats.score_corrected, stats.score_uncorrected) == (1, 1, 0)
        rec = records[0]
        bands = 256 // 64
        assert rec.tile == ((1 * bands) + query // 64) * bands + key // 64
        assert (rec.bad_row, rec.bad_col, rec.corrected) == (query % 64, key % 64, 1)
        assert rec.row_delta == pytest.approx(-value, abs=2e-3)
        assert stats.pv_detected == 0
        np.testing.assert_allclose(out, clean, atol=2e-4)


def test_uncorrected_score_fault_corrupts_only_its_row():
    q, k, v = _qkv(1, 1, 128, 128, seed=4)
    clean, _, _ = oa.forward(q, k, v)
    # tolerance so loose that the score checker cannot see the fault: the softmax of that row changes
    out, stats, _ = oa.forward(q, k, v, score_abs=1e3, fault=(1, 0, 0, 5, 9, 40.0))
    assert stats.score_detected == 0
    assert np.abs(out[0, 0, 5] - clean[0, 0, 5]).max() > 1e-2
    mask = np.ones(128, dtype=bool)
    mask[5] = False
    np.testing.assert_array_equal(out[0, 0, mask], clean[0, 0, mask])


def test_output_fault_is_located_and_corrected():
    q, k, v = _qkv(1, 2, 256, 128, seed=5)
    clean, _, _ = oa.forward(q, k, v)
    for query, dim, value in [(3, 0, 0.5), (200, 127, -1.0), (64, 64, 0.05)]:
        out, stats, _ = oa.forward(q, k, v, fault=(4, 0, 0, query, dim, value))
        assert (stats.pv_detected, stats.pv_corrected, stats.failed_rows) == (1, 1, 0)
        np.testing.assert_allclose(out, clean, atol=5e-3)
    # below the projection tolerance (2e-3 + 2e-3 * max(1, |expected|)): invisible, as in the reference
    out, stats, _ = oa.forward(q, k, v, fault=(4, 0, 0, 10, 10, 1e-3))
    assert stats.pv_detected == 0


def test_softmax_stage_protection():
    """The reference's softmax-stage protection (a14:964-1099): a faulty probability is located by the moment
    deltas and replaced, a corrupted running sum is replaced by the verifier's copy."""
    q, k, v = _qkv(1, 2, 384, 128, seed=6)
    clean, stats, _ = oa.forward(q, k, v, protect_softmax=True)
    assert (stats.softmax_detected, stats.score_detected, stats.pv_detected) == (0, 0, 0)
    plain, _, _ = oa.forward(q, k, v)
    np.testing.assert_array_equal(clean, plain)  # protection changes nothing when nothing is wrong
    for query, key, value in [(5, 9, 0.25), (200, 383, 0.5), (383, 130, 0.01)]:
        out, stats, _ = oa.forward(q, k, v, protect_softmax=True, fault=(2, 0, 1, query, key, value))
        assert (stats.softmax_detected, stats.softmax_corrected, stats.softmax_replayed) == (1, 1, 0)
        assert (stats.pv_detected, stats.failed_rows) == (0, 0)
        np.testing.assert_array_equal(out, clean)  # the verifier's probability replaces the faulty one exactly
    out, stats, _ = oa.forward(q, k, v, protect_softmax=True, fault=(3, 0, 0, 100, 300, 0.75))
    assert (stats.softmax_detected, stats.softmax_corrected, stats.softmax_replayed) == (1, 0, 1)
    np.testing.assert_array_equal(out, clean)
    # without the protection a softmax fault cannot even be requested through the operator; in the oracle it is inert
    out, stats, _ = oa.forward(q, k, v, protect_softmax=False, fault=(2, 0, 1, 5, 9, 0.25))
    assert stats.softmax_detected == 0
    np.testing.assert_array_equal(out, plain)


def test_causal_forward():
    """Causal attention (src/ft_flash_attention_a14.cu:708, 893): key <= query only; the checker still sees raw score tiles."""
    q, k, v = _qkv(1, 2, 384, 128, seed=21)
    out, stats, records = oa.forward(q, k, v, causal=True)
    assert (stats.score_detected, stats.pv_detected, stats.failed_rows) == (0, 0, 0) and not records
    np.testing.assert_allclose(out, oa.truth_fp64(q, k, v, causal=True), atol=3e-3, rtol=0)
    # the first query attends to key 0 only
    np.testing.assert_allclose(out[0, :, 0, :], v[0, :, 0, :].astype(np.float32), atol=1e-6, rtol=0)
    # score fault under the diagonal: located, corrected
    for query, key, value in [(300, 5, 4.0), (200, 200, -3.0), (130, 128, 2.0)]:
        got, stats, records = oa.forward(q, k, v, causal=True, fault=(1, 0, 1, query, key, value))
        assert (stats.score_detected, stats.score_corrected) == (1, 1)
        assert (records[0].bad_row, records[0].bad_col) == (query % 64, key % 64)
        np.testing.assert_allclose(got, out, atol=5e-4, rtol=0)
    # softmax and output stages keep working under the mask
    got, stats, _ = oa.forward(q, k, v, causal=True, protect_softmax=True, fault=(2, 0, 0, 260, 257, 0.5))
    assert (stats.softmax_detected, stats.softmax_corrected) == (1, 1)
    np.testing.assert_allclose(got, out, atol=1e-6, rtol=0)
    got, stats, _ = oa.forward(q, k, v, causal=True, fault=(4, 0, 1, 50, 99, 0.75))
    assert (stats.pv_detected, stats.pv_corrected, stats.failed_rows) == (1, 1, 0)


def test_sequence_lengths_that_are_not_whole_tiles():
    """Any sequence length (the reference masks by index, src/ft_flash_attention_a14.cu:893): padded keys carry no weight,
    padded queries leave no row, and faults near the ragged edge are still located."""
    for n, d, causal in [(200, 128, False), (333, 64, True), (1, 64, False), (129, 128, True)]:
        q, k, v = _qkv(1, 2, n, d, seed=50 + n)
        out, stats, records = oa.forward(q, k, v, causal=causal)
        assert out.shape == (1, 2, n, d)
        assert (stats.score_detected, stats.pv_detected, stats.failed_rows) == (0, 0, 0) and not records
        np.testing.assert_allclose(out, oa.truth_fp64(q, k, v, causal=causal), atol=3e-3, rtol=0)
    q, k, v = _qkv(1, 2, 200, 128, seed=61)
    clean, _, _ = oa.forward(q, k, v)
    got, stats, records = oa.forward(q, k, v, fault=(1, 0, 1, 199, 150, 3.0))
    assert (stats.score_detected, stats.score_corrected) == (1, 1)
    assert (records[0].bad_row, records[0].bad_col) == (199 % 64, 150 % 64)
    np.testing.assert_allclose(got, clean, atol=5e-4, rtol=0)
    got, stats, _ = oa.forward(q, k, v, fault=(4, 0, 0, 199, 127, 0.5))
    assert (stats.pv_detected, stats.pv_corrected, stats.failed_rows) == (1, 1, 0)
    np.testing.assert_allclose(got, clean, atol=6e-3, rtol=0)
    got, stats, _ = oa.forward(q, k, v, protect_softmax=True, fault=(2, 0, 0, 130, 199, 0.25))
    assert (stats.softmax_detected, stats.softmax_corrected) == (1, 1)
    np.testing.assert_allclose(got, clean, atol=1e-6, rtol=0)


def test_oracle_replays_a_tile_with_two_faults():
    """Two faults in one 64x64 score tile: not locatable, the tile is recomputed, passes the second check and counts as
    replayed; the output is the clean one bit for bit (the recomputation is the oracle's own score arithmetic)."""
    rng = np.random.default_rng(5)
    q, k, v = (rng.standard_normal((1, 1, 256, 64)).astype(np.float16) for _ in range(3))
    clean, stats0, _ = oa.forward(q, k, v)
    assert (stats0.score_detected, stats0.score_replayed) == (0, 0)
    out, stats, records = oa.forward(q, k, v, fault=(1, 0, 0, 70, 130, 6.0, 100, 180, -4.0))
    assert (stats.score_detected, stats.score_corrected, stats.score_replayed, stats.score_uncorrected) == (1, 0, 1, 0)
    assert (records[0].bad_row_count, records[0].bad_col_count, records[0].corrected) == (2, 2, 0)
    np.testing.assert_array_equal(out, clean)
    # in different tiles they are two single faults
    out, stats, _ = oa.forward(q, k, v, fault=(1, 0, 0, 70, 130, 6.0, 200, 10, -4.0))
    assert (stats.score_detected, stats.score_corrected, stats.score_replayed) == (2, 2, 0)
