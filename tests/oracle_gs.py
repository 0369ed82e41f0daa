"""ctypes wrapper of the GEMM + softmax part of the CPU oracle (oracle/ftq_gemm_softmax.c).
Test infrastructure only."""
import ctypes

import numpy as np

from tests import oracle_lib

DEFAULT_TOLERANCES = dict(abs_tol=2.0e-3, rel_tol=2.0e-5, row_sum_tol=2.0e-6, location_tol=2.5e-1)  # src/gemm_softmax_abft.cu:35-38


def _ptr(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def generate(count, seed):
    out = np.empty(count, dtype=np.uint8)
    oracle_lib.load().lib.ftq_gs_generate(_ptr(out), ctypes.c_size_t(count), ctypes.c_uint32(seed))
    return out


def logits(a, b, m, n, k):
    out = np.empty((m, n), dtype=np.float32)
    oracle_lib.load().lib.ftq_gs_logits(_ptr(a), _ptr(b), _ptr(out), m, n, k)
    return out


def expected(a, b, m, n, k):
    es, ew = np.empty(m, dtype=np.float64), np.empty(m, dtype=np.float64)
    oracle_lib.load().lib.ftq_gs_expected(_ptr(a), _ptr(b), m, n, k, _ptr(es), _ptr(ew))
    return es, ew


def softmax_checks(x):
    """x: float32 [M, N] logits.  Returns a dict with probabilities and the per-row check values."""
    m, n = x.shape
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = {"probabilities": np.empty((m, n), np.float32), "actual_sum": np.empty(m), "actual_weighted": np.empty(m),
           "probability_sum": np.empty(m), "log_z": np.empty(m), "underflow_count": np.empty(m, np.int32)}
    oracle_lib.load().lib.ftq_gs_softmax_checks(_ptr(x), _ptr(out["probabilities"]), _ptr(out["actual_sum"]), _ptr(out["actual_weighted"]),
                                                _ptr(out["probability_sum"]), _ptr(out["log_z"]), _ptr(out["underflow_count"]), m, n)
    return out


def analyze(expected_sum, expected_weighted, checks, n, **tolerances):
    tol = dict(DEFAULT_TOLERANCES, **tolerances)
    m = expected_sum.shape[0]
    out = {"detected": np.empty(m, np.int32), "estimated_col": np.empty(m, np.int32), "correction_delta": np.empty(m),
           "counts": np.empty(2, np.int32)}
    oracle_lib.load().lib.ftq_gs_analyze(_ptr(expected_sum), _ptr(expected_weighted), _ptr(checks["actual_sum"]),
                                         _ptr(checks["actual_weighted"]), _ptr(checks["probability_sum"]), _ptr(out["detected"]),
                                         _ptr(out["estimated_col"]), _ptr(out["correction_delta"]), _ptr(out["counts"]), m, n,
                                         ctypes.c_double(tol["abs_tol"]), ctypes.c_double(tol["rel_tol"]),
                                         ctypes.c_double(tol["row_sum_tol"]), ctypes.c_double(tol["location_tol"]))
    return out


def correct(x, analysis):
    x = np.ascontiguousarray(x, dtype=np.float32).copy()
    m, n = x.shape
    oracle_lib.load().lib.ftq_gs_correct(_ptr(x), _ptr(analysis["detected"]), _ptr(analysis["estimated_col"]),
                                         _ptr(analysis["correction_delta"]), m, n)
    return x
