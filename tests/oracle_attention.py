"""ctypes wrapper of the attention part of the CPU oracle (oracle/ftq_attention.c).
Test infrastructure only."""
import ctypes

import numpy as np

from tests import oracle_lib


class AttnStats(ctypes.Structure):
    _fields_ = [("score_detected", ctypes.c_int), ("score_corrected", ctypes.c_int), ("score_uncorrected", ctypes.c_int),
                ("pv_detected", ctypes.c_int), ("pv_corrected", ctypes.c_int), ("failed_rows", ctypes.c_int),
                ("softmax_detected", ctypes.c_int), ("softmax_corrected", ctypes.c_int), ("softmax_replayed", ctypes.c_int),
                ("n_records", ctypes.c_int), ("max_score_noise", ctypes.c_float), ("min_margin", ctypes.c_float),
                ("score_replayed", ctypes.c_int)]


def forward(q, k, v, score_abs=1e-2, score_rel=2e-5, pv_abs=2e-3, pv_rel=2e-3, fault=None, max_records=64, protect_softmax=False,
            softmax_abs=2e-5, softmax_rel=2e-5, causal=False):
    """q, k, v: numpy float16 arrays [B, H, N, D], any N (zero-padded here to whole 128-row tiles).
    fault = (stage, batch, head, query, index, value[, query2, index2, value2]): a score fault may carry a second one
    in the same head.  Returns (out float32 [B,H,N,D], stats, records)."""
    lib = oracle_lib.load().lib
    b, h, valid, d = q.shape
    n = (valid + 127) // 128 * 128
    if n != valid:
        q, k, v = (np.pad(np.asarray(x, dtype=np.float16), ((0, 0), (0, 0), (0, n - valid), (0, 0))) for x in (q, k, v))
    q16 = np.ascontiguousarray(q, dtype=np.float16).view(np.uint16)
    k16 = np.ascontiguousarray(k, dtype=np.float16).view(np.uint16)
    v16 = np.ascontiguousarray(v, dtype=np.float16).view(np.uint16)
    out = np.empty((b, h, valid, d), dtype=np.float32)
    stats = AttnStats()
    records = (oracle_lib.TileRecord * max_records)()
    stage, fb, fh, fq, fi, fv = fault[:6] if fault is not None else (0, 0, 0, 0, 0, 0.0)
    fq2, fi2, fv2 = fault[6:9] if fault is not None and len(fault) >= 9 else (0, 0, 0.0)
    ptr = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    lib.ftq_attention_forward(ptr(q16), ptr(k16), ptr(v16), b * h, n, valid, d, ctypes.c_float(score_abs), ctypes.c_float(score_rel),
                              ctypes.c_float(pv_abs), ctypes.c_float(pv_rel), ctypes.c_float(softmax_abs), ctypes.c_float(softmax_rel),
                              int(bool(protect_softmax)), int(bool(causal)), int(stage), int(fb * h + fh), int(fq), int(fi),
                              ctypes.c_float(fv), int(fq2), int(fi2), ctypes.c_float(fv2), ptr(out), ctypes.byref(stats), records,
                              max_records)
    return out, stats, list(records[:stats.n_records])


def truth_fp64(q, k, v, causal=False):
    """softmax(Q K^T / sqrt(D)) V in float64; causal keeps key <= query."""
    qd, kd, vd = (np.asarray(x, dtype=np.float64) for x in (q, k, v))
    s = qd @ np.swapaxes(kd, -1, -2) / np.sqrt(q.shape[-1])
    if causal:
        n = q.shape[-2]
        s = np.where(np.arange(n)[None, :] > np.arange(n)[:, None], -np.inf, s)
    s -= s.max(axis=-1, keepdims=True)
    p = np.exp(s)
    p /= p.sum(axis=-1, keepdims=True)
    return p @ vd


def half_roundtrip(x):
    lib = oracle_lib.load().lib
    lib.ftq_float_to_half.restype = ctypes.c_uint16
    lib.ftq_float_to_half.argtypes = [ctypes.c_float]
    lib.ftq_half_to_float.restype = ctypes.c_float
    lib.ftq_half_to_float.argtypes = [ctypes.c_uint16]
    bits = lib.ftq_float_to_half(ctypes.c_float(x))
    return int(bits), float(lib.ftq_half_to_float(ctypes.c_uint16(bits)))
