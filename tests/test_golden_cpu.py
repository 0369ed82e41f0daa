"""Pins the oracle against the reference's OWN kernels.

The fixtures in tests/golden/ are outputs of the reference project's kernels
(generator, S0 GEMM / prepare / checker, S2-S4 band-sum and expected-checksum
kernels) launched unmodified on a B200 by oracle/ref_harness_*.cu; see
tests/golden/make_golden.py.  Every comparison here is bit for bit."""
import glob
import os

import numpy as np
import pytest

from tests.oracle_lib import B_KN, C_ROWMAJOR

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
SEED_A, SEED_B = 0x12345678, 0x9ABCDEF0
S4_FILES = sorted(glob.glob(os.path.join(GOLDEN, "s4_prepare_*.npz")))
S0_FILES = sorted(glob.glob(os.path.join(GOLDEN, "s0_path_*.npz")))


def _bits(x):
    return np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)


def test_fixtures_present():
    assert len(S4_FILES) >= 4 and len(S0_FILES) >= 3


@pytest.mark.parametrize("path", S4_FILES, ids=os.path.basename)
def test_s4_prepare_kernels(oracle, path):
    """src/s4_cluster_multicast_abft_fp8_gemm.cu:184-294: generator, band sums, expected checksums and scales."""
    g = np.load(path)
    m, n, k = (int(x) for x in g["shape"])
    a = oracle.generate_uniform(m * k, SEED_A)
    b = oracle.generate_uniform(n * k, SEED_B)
    if "a" in g:
        np.testing.assert_array_equal(a, g["a"])
        np.testing.assert_array_equal(b, g["b"])
    else:
        np.testing.assert_array_equal(a[:256], g["a_head"])
        np.testing.assert_array_equal(b[:256], g["b_head"])
        assert int(a.astype(np.uint64).sum()) == int(g["a_sum"]) and int(b.astype(np.uint64).sum()) == int(g["b_sum"])
    cache = oracle.expected(a, b, m, n, k)
    for mine, theirs in (("a_sums", "a_sums"), ("a_magnitudes", "a_mags"), ("b_sums", "b_sums"), ("b_magnitudes", "b_mags"),
                         ("expected_rows", "expected_rows"), ("row_scales", "row_scales"), ("expected_cols", "expected_cols"),
                         ("col_scales", "col_scales")):
        np.testing.assert_array_equal(_bits(cache[mine]).ravel(), _bits(g[theirs]).ravel(), err_msg=mine)


@pytest.mark.parametrize("path", S0_FILES, ids=os.path.basename)
def test_s0_path(oracle, path):
    """src/s0_tiled_abft_fp8_gemm.cu:102-277: generator, FP32 GEMM, direct-form prepare, checker and corrector
    in five scenarios (clean, the program's own injected fault, and three multi-fault cases)."""
    g = np.load(path)
    m, n, k = (int(x) for x in g["shape"])
    a = oracle.generate_uniform(m * k, SEED_A)
    b = oracle.generate_uniform(k * n, SEED_B)  # S0's B is [K,N]
    if "a" in g:
        np.testing.assert_array_equal(a, g["a"])
        np.testing.assert_array_equal(b, g["b"])
    c = oracle.gemm_f32(a, b, m, n, k, B_KN, C_ROWMAJOR)
    np.testing.assert_array_equal(_bits(c).ravel(), _bits(g["c_gemm"]))
    cache = oracle.s0_prepare(a, b, m, n, k, tile=16)
    for name in ("expected_rows", "expected_cols", "row_scales", "col_scales"):
        np.testing.assert_array_equal(_bits(cache[name]).ravel(), _bits(g[name]), err_msg=name)
    tile_rows, tile_cols = (m + 15) // 16, (n + 15) // 16
    centre_tile = (tile_rows * tile_cols) // 2
    vr = min(16, m - (centre_tile // tile_cols) * 16)
    vc = min(16, n - (centre_tile % tile_cols) * 16)

    def host_faults(entries):  # global (row, col, value) -> (tile, local row, local col, value)
        return [((r // 16) * tile_cols + cc // 16, r % 16, cc % 16, v) for r, cc, v in entries]

    scenarios = {"clean": [], "inject": [(centre_tile, vr // 2, vc // 2, 1.0)],
                 "two_rc": host_faults([(1, 2, 3.0), (5, 7, -2.5)]), "same_row": host_faults([(3, 1, 4.0), (3, 9, 6.0)]),
                 "cancel": host_faults([(4, 2, 5.0), (4, 11, -5.0)])}
    for name, faults in scenarios.items():
        # S0 defaults: abs 5e-2, rel 1e-5 (src/s0:31-32); bad tile needs rows>0 AND cols>0 (src/s0:267)
        after, s, _ = oracle.abft_check(c, m, n, cache, abs_tol=5e-2, rel_tol=1e-5, tile=16, c_layout=C_ROWMAJOR, or_rule=False,
                                        faults=faults)
        assert [s.bad_tiles, s.corrected_tiles] == g["counters_" + name].tolist(), name
        np.testing.assert_array_equal(_bits(after).ravel(), _bits(g["c_" + name]), err_msg=name)
    assert g["counters_inject"].tolist() == [1, 1] and g["counters_clean"].tolist() == [0, 0]
    assert g["counters_two_rc"].tolist() == [1, 0] and g["counters_cancel"].tolist() == [0, 0]
