"""The attention oracle against outputs of the reference's own scalar attention kernel
(src/ft_flash_attention_a0.cu, run unmodified on a B200 by oracle/ref_harness_a0; fixtures tests/golden/a0_*.npz).

The reference takes FP8 inputs and protects the score stage with per-row projections; this build takes FP16 inputs and
protects it with the GEMM's 64x64 tile checksums, so the comparison is: inputs bit for bit (the reference's grid values are
exact in FP16), outputs within 2e-3 (FP16 probabilities here, FP32 there) for clean and for every recovered fault, and the
per-stage counters: detected once, recovered once, no failed rows."""
import glob
import os

import numpy as np
import pytest

from tests import oracle_attention as oa
from tests import oracle_lib

GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "a0_*.npz")))
STATS = ("score_detected", "score_corrected", "score_replayed", "softmax_detected", "softmax_corrected", "softmax_replayed",
         "pv_detected", "pv_corrected", "failed_rows")  # DeviceStats, a0:35-45


def grid_values(count, seed):
    """((mix(seed + i) % 17) - 8) / 16, the attention programs' generator (a0:231-238)."""
    oracle = oracle_lib.load()
    return np.array([(oracle.mix(seed + i) % 17 - 8) / 16.0 for i in range(count)], dtype=np.float32)


@pytest.mark.skipif(not GOLDEN, reason="attention fixtures not generated yet")
@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p) for p in GOLDEN])
def test_oracle_against_reference_a0(path):
    g = np.load(path)
    b, h, n, d, causal = (int(x) for x in g["shape"])
    oracle = oracle_lib.load()
    shape = (b, h, n, d)
    q, k, v = (oracle.decode(g[name]).reshape(shape) for name in ("q", "k", "v"))
    # the generator: the first 4096 values of each tensor, bit for bit (seeds of a0:771-773)
    for t, seed in ((q, 0x12345678), (k, 0x9ABCDEF0), (v, 0x31415926)):
        np.testing.assert_array_equal(t.ravel()[:4096], grid_values(4096, seed))
    q16, k16, v16 = (t.astype(np.float16) for t in (q, k, v))
    assert all((t16.astype(np.float32) == t).all() for t16, t in ((q16, q), (k16, k), (v16, v)))  # exact in FP16
    clean = mine_clean = None
    for i, (stage, query, index, value) in enumerate(g["scenarios"]):
        stage, query, index = int(stage), int(query), int(index)
        ref = dict(zip(STATS, (int(x) for x in g[f"stats_{i}"])))
        fault = None if stage == 0 else (stage, 0, 0, query, index, float(value))
        out, stats, _ = oa.forward(q16, k16, v16, causal=bool(causal), protect_softmax=stage in (2, 3), fault=fault)
        assert ref["failed_rows"] == 0 == stats.failed_rows
        if stage == 0:  # the reference's clean output in full (stored as FP16)
            clean = g[f"out_{i}"].astype(np.float32).reshape(shape)
            np.testing.assert_allclose(out, clean, atol=2e-3, rtol=0)
            mine_clean = out
            assert all(x == 0 for x in ref.values())
            assert (stats.score_detected, stats.pv_detected, stats.softmax_detected) == (0, 0, 0)
            continue
        # of a fault scenario the fixture holds the faulty query's row and how far any other row moved (nowhere)
        np.testing.assert_allclose(out[0, 0, query], g[f"row_{i}"], atol=2e-3, rtol=0, err_msg=f"scenario {i}")
        np.testing.assert_allclose(g[f"row_{i}"], clean[0, 0, query], atol=2e-3, rtol=0)  # the reference recovered as well
        assert float(g[f"others_{i}"]) == 0.0
        rest = np.abs(out - mine_clean)
        rest[0, 0, query] = 0.0
        assert rest.max() < 1e-6
        if stage == 1:
            assert (ref["score_detected"], ref["score_corrected"] + ref["score_replayed"]) == (1, 1)
            assert (stats.score_detected, stats.score_corrected) == (1, 1)
        elif stage in (2, 3):
            assert ref["softmax_detected"] >= 1 and ref["softmax_corrected"] + ref["softmax_replayed"] >= 1
            assert stats.softmax_detected >= 1 and stats.softmax_corrected + stats.softmax_replayed >= 1
            if stage == 3:
                assert ref["softmax_replayed"] >= 1 and stats.softmax_replayed >= 1
        else:
            assert (ref["pv_detected"], ref["pv_corrected"]) == (1, 1) == (stats.pv_detected, stats.pv_corrected)
