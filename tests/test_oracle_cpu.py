"""CPU tests of the oracle itself: codec, generators, GEMM, expected checksums,
checker decisions, campaign RNG and the sampled verifier.  The pins against the
reference's own kernels are in test_golden_cpu.py."""
import os
import subprocess

import numpy as np
import pytest

from tests import oracle_lib
from tests.oracle_lib import B_KN, B_NK, C_COLMAJOR, C_ROWMAJOR


def test_e4m3_codec_matches_cuda_fp8_header():
    subprocess.run(["make", "-C", oracle_lib.ORACLE_DIR, "_build/check_e4m3"], check=True, stdout=subprocess.DEVNULL)
    out = subprocess.run([os.path.join(oracle_lib.ORACLE_DIR, "_build", "check_e4m3")], capture_output=True, text=True)
    assert out.returncode == 0, out.stdout
    assert out.stdout.startswith("e4m3 ok")


def test_e4m3_known_values(oracle):
    # values stated in the E4M3 format definition: max 448, min normal 2^-6, min subnormal 2^-9
    assert oracle.encode(448.0) == 0x7E and oracle.encode(1e9) == 0x7E and oracle.encode(-1e9) == 0xFE
    assert oracle.encode(float("nan")) == 0x7F
    assert oracle.encode(2.0 ** -6) == 0x08 and oracle.encode(2.0 ** -9) == 0x01
    assert oracle.encode(2.0 ** -10) == 0x00  # tie to even -> 0
    assert oracle.encode(0.3) == oracle.encode(0.3125)  # RNE: 0.3 -> 0.3125
    assert oracle.encode(1.0) == 0x38 and oracle.encode(-1.0) == 0xB8
    for v in range(256):
        f = float(oracle.decode([v])[0])
        if not np.isnan(f):
            assert oracle.encode(f) == v or f == 0.0


def test_mix_and_uniform_generator(oracle):
    # python restatement of the hash (src/s0_tiled_abft_fp8_gemm.cu:93-100)
    def mix(x):
        x ^= x >> 16
        x = (x * 0x7FEB352D) & 0xFFFFFFFF
        x ^= x >> 15
        x = (x * 0x846CA68B) & 0xFFFFFFFF
        x ^= x >> 16
        return x
    for x in (0, 1, 0x12345678, 0xFFFFFFFF, 0x9ABCDEF0):
        assert oracle.mix(x) == mix(x)
    seed = 0x12345678
    got = oracle.generate_uniform(4096, seed)
    for i in (0, 1, 17, 4095):
        unit = np.float32(mix((seed + i) & 0xFFFFFFFF) & 0xFFFFFF) / np.float32(16777216.0)
        assert got[i] == oracle.encode(float(np.float32(2.0) * unit - np.float32(1.0)))
    vals = oracle.decode(got)
    assert abs(vals.mean()) < 0.05 and 0.30 < vals.var() < 0.37  # U(-1,1): var 1/3


def test_normal_generator_statistics(oracle):
    vals = oracle.decode(oracle.generate_normal(1 << 16, 0x12345678))
    assert abs(vals.mean()) < 0.02 and 0.95 < vals.var() < 1.05
    llm = oracle.decode(oracle.generate_normal(1 << 16, 7, sigma=0.02, post_scale=1.0 / (5.7 * 0.02)))
    assert np.abs(llm).max() <= 1.25 and 0.15 < llm.std() < 0.2


@pytest.mark.parametrize("m,n,k", [(64, 64, 128), (128, 256, 256), (40, 56, 48)])
def test_gemm_against_float64(oracle, m, n, k):
    a = oracle.generate_uniform(m * k, 1)
    b = oracle.generate_uniform(n * k, 2)
    ref = oracle.decode(a).reshape(m, k).astype(np.float64) @ oracle.decode(b).reshape(n, k).astype(np.float64).T
    c_col = oracle.gemm_f32(a, b, m, n, k, B_NK, C_COLMAJOR)
    np.testing.assert_allclose(c_col.T, ref, atol=1e-5 * k)
    b_kn = np.ascontiguousarray(b.reshape(n, k).T).ravel()
    c_row = oracle.gemm_f32(a, b_kn, m, n, k, B_KN, C_ROWMAJOR)
    np.testing.assert_array_equal(c_row, c_col.T)  # same accumulation order whatever the layouts
    assert oracle.dot_f64(a, b, 3, 5, n, k) == pytest.approx(ref[3, 5], abs=1e-12)


@pytest.mark.parametrize("m,n,k", [(128, 256, 128), (64, 200, 96), (192, 64, 512)])
def test_expected_checksums_against_float64(oracle, m, n, k):
    a = oracle.generate_uniform(m * k, 0x12345678)
    b = oracle.generate_uniform(n * k, 0x9ABCDEF0)
    cache = oracle.expected(a, b, m, n, k)
    af = oracle.decode(a).reshape(m, k).astype(np.float64)
    bf = oracle.decode(b).reshape(n, k).astype(np.float64)
    tr, tc = m // 64, (n + 63) // 64
    for i in range(tr):
        for j in range(tc):
            cols = slice(64 * j, min(n, 64 * j + 64))
            valid = cols.stop - cols.start
            t = i * tc + j
            block = af[64 * i:64 * i + 64] @ bf[cols].T
            np.testing.assert_allclose(cache["expected_rows"][t], block.sum(1), atol=2e-3)
            np.testing.assert_allclose(cache["expected_cols"][t, :valid], block.sum(0), atol=2e-3)
            assert np.all(cache["expected_cols"][t, valid:] == 0) and np.all(cache["col_scales"][t, valid:] == 0)
            scale = np.abs(af[64 * i:64 * i + 64]) @ np.abs(bf[cols]).T
            np.testing.assert_allclose(cache["row_scales"][t], scale.sum(1), rtol=1e-5)
            np.testing.assert_allclose(cache["col_scales"][t, :valid], scale.sum(0), rtol=1e-5)


def test_s0_prepare_equals_band_form_up_to_rounding(oracle):
    m, n, k = 48, 40, 64
    a = oracle.generate_uniform(m * k, 5)
    b_nk = oracle.generate_uniform(n * k, 6)
    b_kn = np.ascontiguousarray(b_nk.reshape(n, k).T).ravel()
    s0 = oracle.s0_prepare(a, b_kn, m, n, k, tile=16)
    af = oracle.decode(a).reshape(m, k).astype(np.float64)
    bf = oracle.decode(b_nk).reshape(n, k).astype(np.float64)
    full = af @ bf.T
    tc = (n + 15) // 16
    for t in range(3 * tc):
        i, j = divmod(t, tc)
        blk = full[16 * i:16 * i + 16, 16 * j:min(n, 16 * j + 16)]
        np.testing.assert_allclose(s0["expected_rows"][t], blk.sum(1), atol=1e-4)
        np.testing.assert_allclose(s0["expected_cols"][t, :blk.shape[1]], blk.sum(0), atol=1e-4)


def _setup(oracle, m=128, n=256, k=256):
    a = oracle.generate_uniform(m * k, 0x12345678)
    b = oracle.generate_uniform(n * k, 0x9ABCDEF0)
    return a, b, oracle.gemm_f32(a, b, m, n, k), oracle.expected(a, b, m, n, k)


def test_checker_clean_and_single_fault(oracle):
    m, n, k = 128, 256, 256
    a, b, c, cache = _setup(oracle, m, n, k)
    after, s, recs = oracle.abft_check(c, m, n, cache)
    assert (s.bad_tiles, s.corrected_tiles, s.multi_fault_tiles) == (0, 0, 0) and s.max_clean_ratio < 0.1
    np.testing.assert_array_equal(after, c)
    # every element of one tile, value well above the threshold
    tile = 5
    for row, col in [(0, 0), (63, 63), (31, 32), (7, 50)]:
        after, s, recs = oracle.abft_check(c, m, n, cache, faults=[(tile, row, col, -7.5)])
        assert (s.bad_tiles, s.corrected_tiles, s.multi_fault_tiles) == (1, 1, 0)
        r = recs[0]
        assert (r.tile, r.bad_row, r.bad_col, r.bad_row_count, r.bad_col_count, r.corrected) == (tile, row, col, 1, 1, 1)
        # delta = expected - actual = -fault (+ checksum noise)
        assert r.row_delta == pytest.approx(7.5, abs=1e-3) and r.col_delta == pytest.approx(7.5, abs=1e-3)
        np.testing.assert_allclose(after, c, atol=1e-3)


def test_checker_below_threshold_is_invisible(oracle):
    m, n, k = 128, 256, 256
    a, b, c, cache = _setup(oracle, m, n, k)
    after, s, _ = oracle.abft_check(c, m, n, cache, abs_tol=1e-2, rel_tol=2e-5, faults=[(0, 1, 1, 5e-3)])
    assert s.bad_tiles == 0 and s.corrected_tiles == 0


def test_checker_multi_fault_rules(oracle):
    m, n, k = 128, 256, 256
    a, b, c, cache = _setup(oracle, m, n, k)
    # two faults, distinct rows and columns -> (2,2): reported, not corrected
    after, s, recs = oracle.abft_check(c, m, n, cache, faults=[(2, 1, 2, 3.0), (2, 5, 7, -2.5)])
    assert (s.bad_tiles, s.corrected_tiles, s.multi_fault_tiles) == (1, 0, 1)
    assert (recs[0].bad_row_count, recs[0].bad_col_count, recs[0].bad_row, recs[0].bad_col) == (2, 2, 1, 2)
    idx = lambda tile, r, col: ((tile % 4) * 64 + col) * m + (tile // 4) * 64 + r
    assert after.ravel()[idx(2, 1, 2)] == pytest.approx(c.ravel()[idx(2, 1, 2)] + 3.0)  # left as injected
    # same row -> (1,2)
    _, s, recs = oracle.abft_check(c, m, n, cache, faults=[(2, 3, 1, 4.0), (2, 3, 9, 6.0)])
    assert (s.bad_tiles, s.corrected_tiles) == (1, 0) and (recs[0].bad_row_count, recs[0].bad_col_count) == (1, 2)
    # cancelling pair in one row -> (0,2): bad under the S1-S4 `||` rule, not under S0's `&&`
    _, s, recs = oracle.abft_check(c, m, n, cache, faults=[(2, 4, 2, 5.0), (2, 4, 11, -5.0)])
    assert (s.bad_tiles, s.corrected_tiles) == (1, 0) and (recs[0].bad_row_count, recs[0].bad_col_count) == (0, 2)
    _, s, _ = oracle.abft_check(c, m, n, cache, faults=[(2, 4, 2, 5.0), (2, 4, 11, -5.0)], or_rule=False)
    assert (s.bad_tiles, s.corrected_tiles) == (0, 0)
    # faults in two different tiles are both corrected
    _, s, recs = oracle.abft_check(c, m, n, cache, faults=[(0, 1, 1, 9.0), (7, 2, 2, -9.0)])
    assert (s.bad_tiles, s.corrected_tiles) == (2, 2) and [r.tile for r in recs] == [0, 7]


def test_checker_ragged_n(oracle):
    m, n, k = 64, 200, 128
    a = oracle.generate_uniform(m * k, 3)
    b = oracle.generate_uniform(n * k, 4)
    c = oracle.gemm_f32(a, b, m, n, k)
    cache = oracle.expected(a, b, m, n, k)
    _, s, _ = oracle.abft_check(c, m, n, cache)
    assert s.bad_tiles == 0
    # injection clamps the column to the last valid one (8 valid columns in tile 3)
    after, s, recs = oracle.abft_check(c, m, n, cache, faults=[(3, 10, 40, 6.0)])
    assert (s.bad_tiles, s.corrected_tiles) == (1, 1) and recs[0].bad_col == 7


def test_campaign_rng(oracle):
    def mix(x):
        x ^= x >> 16
        x = (x * 0x7FEB352D) & 0xFFFFFFFF
        x ^= x >> 15
        x = (x * 0x846CA68B) & 0xFFFFFFFF
        x ^= x >> 16
        return x
    tile_count = 16384
    draws, final = oracle.campaign(12345, 50, tile_count)
    s = 12345
    for trial, (tile, row, col, value, bin_, unit) in enumerate(draws):
        s = mix((s + 0x9E3779B9 + trial) & 0xFFFFFFFF)
        assert tile == s % tile_count
        s = mix(s)
        assert row == s % 64
        s = mix(s)
        assert col == s % 64
        s = mix(s)
        u = np.float32(s & 0xFFFFFF) / np.float32(16777215.0)
        mag = np.float32(1.0) + np.float32(255.0) * u
        assert bin_ == min(3, int(np.float32(4) * u))
        s = mix(s)
        assert value == pytest.approx(float(mag if (s & 1) == 0 else -mag), rel=1e-7)
        assert 1.0 <= abs(value) <= 256.0
    assert final == s
    assert len({d[0] for d in draws}) > 40  # tiles spread out


def test_verify_samples(oracle):
    m, n, k = 128, 256, 128
    a, b, c, _ = _setup(oracle, m, n, k)
    r = oracle.verify_samples(a, b, c, m, n, k)
    assert r.checked == 64 and r.max_tolerance_ratio < 1e-3
    bad = c.copy()
    bad[0, 0] += 1.0  # column 0, row 0 is a sampled entry
    r = oracle.verify_samples(a, b, bad, m, n, k)
    assert r.max_absolute_error == pytest.approx(1.0, abs=1e-3) and r.max_tolerance_ratio > 1.0


def test_full_pass_reports_clean(oracle):
    m, n, k = 128, 256, 256
    a = oracle.generate_uniform(m * k, 0x12345678)
    b = oracle.generate_uniform(n * k, 0x9ABCDEF0)
    c, secs, s = oracle.full_pass(a, b, m, n, k)
    assert s.bad_tiles == 0 and len(secs) == 3 and all(t >= 0 for t in secs)
    np.testing.assert_array_equal(c, oracle.gemm_f32(a, b, m, n, k))


def test_quantize_matches_the_scalar_codec(oracle):
    rng = np.random.default_rng(5)
    src = np.concatenate([rng.standard_normal(4000) * 10.0 ** rng.integers(-4, 3, 4000), [0.0, -0.0, 448.0, 449.0, 1e9, -1e9, 2.0 ** -9,
                          2.0 ** -10, 0.0009765625 * 1.5, 17.0, 18.0, 19.0]]).astype(np.float32)
    for scale in (1.0, 0.37, 8.0):
        got = oracle.quantize(src, scale)
        want = np.array([oracle.encode(float(np.float32(x) * np.float32(scale))) for x in src], dtype=np.uint8)
        np.testing.assert_array_equal(got, want)
    # ties go to the even mantissa: 17 -> 16, 19 -> 20 (step 2 between 16 and 32), and the format saturates at 448
    np.testing.assert_array_equal(oracle.decode(oracle.quantize(np.array([17.0, 18.0, 19.0, 1e9, -1e9], np.float32))),
                                  np.array([16.0, 18.0, 20.0, 448.0, -448.0], np.float32))


def test_ragged_m_is_the_transpose_of_ragged_n(oracle):
    """The reference's cache kernels take a short last band of B (src/s4:203, 240, 284-293) but require M % 128 == 0.
    The oracle treats a short last band of A the same way; this ties the extension to the pinned path: with A and B
    swapped the row arrays of one problem are the column arrays of the other."""
    m, n, k = 200, 136, 96
    a, b = oracle.generate_uniform(m * k, 3), oracle.generate_uniform(n * k, 4)
    ab = oracle.expected(a, b, m, n, k)
    ba = oracle.expected(b, a, n, m, k)
    tr, tc = -(-m // 64), -(-n // 64)
    for rows, cols in (("expected_rows", "expected_cols"), ("row_scales", "col_scales")):
        x = ab[rows].reshape(tr, tc, 64)
        y = ba[cols].reshape(tc, tr, 64).transpose(1, 0, 2)
        np.testing.assert_array_equal(x.view(np.uint32), y.view(np.uint32), err_msg=rows)
        x = ab[cols].reshape(tr, tc, 64)
        y = ba[rows].reshape(tc, tr, 64).transpose(1, 0, 2)
        np.testing.assert_array_equal(x.view(np.uint32), y.view(np.uint32), err_msg=cols)
    assert (ab["expected_rows"].reshape(tr, tc, 64)[-1, :, m - 64 * (tr - 1):] == 0).all()  # rows past M: zeros
