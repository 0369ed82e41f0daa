"""ctypes wrapper of the CPU oracle (oracle/ftq_oracle.c).  Test infrastructure:
only tests, the smoke run and the benchmark's CPU-baseline leg import this."""
import ctypes
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
SO = os.path.join(ORACLE_DIR, "_build", "libftq_oracle.so")

B_NK, B_KN = 0, 1
C_COLMAJOR, C_ROWMAJOR = 0, 1


class Fault(ctypes.Structure):
    _fields_ = [("tile", ctypes.c_int), ("row", ctypes.c_int), ("col", ctypes.c_int), ("value", ctypes.c_float)]


class TileRecord(ctypes.Structure):
    _fields_ = [("tile", ctypes.c_int), ("bad_row_count", ctypes.c_int), ("bad_col_count", ctypes.c_int),
                ("bad_row", ctypes.c_int), ("bad_col", ctypes.c_int), ("row_delta", ctypes.c_float),
                ("col_delta", ctypes.c_float), ("corrected", ctypes.c_int), ("min_margin", ctypes.c_float)]


class CheckSummary(ctypes.Structure):
    _fields_ = [("bad_tiles", ctypes.c_int), ("corrected_tiles", ctypes.c_int), ("multi_fault_tiles", ctypes.c_int),
                ("n_records", ctypes.c_int), ("max_clean_ratio", ctypes.c_float), ("min_margin", ctypes.c_float)]


class CampaignDraw(ctypes.Structure):
    _fields_ = [("tile", ctypes.c_int), ("row", ctypes.c_int), ("col", ctypes.c_int), ("bin", ctypes.c_int),
                ("magnitude", ctypes.c_float), ("signed_value", ctypes.c_float), ("unit", ctypes.c_float)]


class VerifyResult(ctypes.Structure):
    _fields_ = [("max_absolute_error", ctypes.c_float), ("max_tolerance_ratio", ctypes.c_float), ("checked", ctypes.c_int)]


def build():
    subprocess.run(["make", "-C", ORACLE_DIR, "_build/libftq_oracle.so"], check=True, stdout=subprocess.DEVNULL)


def _ptr(a):
    return a.ctypes.data_as(ctypes.c_void_p)


class Oracle:
    def __init__(self, lib):
        self.lib = lib
        lib.ftq_mix_u32.restype = ctypes.c_uint32
        lib.ftq_mix_u32.argtypes = [ctypes.c_uint32]
        lib.ftq_e4m3_from_float.restype = ctypes.c_uint8
        lib.ftq_e4m3_from_float.argtypes = [ctypes.c_float]
        lib.ftq_e4m3_to_float.restype = ctypes.c_float
        lib.ftq_e4m3_to_float.argtypes = [ctypes.c_uint8]
        lib.ftq_dot_f64.restype = ctypes.c_double
        lib.ftq_num_threads.restype = ctypes.c_int
        self._decode = np.array([lib.ftq_e4m3_to_float(v) for v in range(256)], dtype=np.float32)

    # -- codec / generators
    def mix(self, x):
        return int(self.lib.ftq_mix_u32(ctypes.c_uint32(x & 0xFFFFFFFF)))

    def decode(self, codes):
        return self._decode[np.asarray(codes, dtype=np.uint8)]

    def encode(self, x):
        return int(self.lib.ftq_e4m3_from_float(ctypes.c_float(x)))

    def quantize(self, src, scale=1.0):
        src = np.ascontiguousarray(src, dtype=np.float32)
        out = np.empty(src.size, dtype=np.uint8)
        self.lib.ftq_quantize_f32(_ptr(src), ctypes.c_size_t(src.size), ctypes.c_float(scale), _ptr(out))
        return out

    def generate_uniform(self, count, seed):
        out = np.empty(count, dtype=np.uint8)
        self.lib.ftq_generate_uniform(_ptr(out), ctypes.c_size_t(count), ctypes.c_uint32(seed))
        return out

    def generate_normal(self, count, seed, sigma=1.0, post_scale=1.0):
        out = np.empty(count, dtype=np.uint8)
        self.lib.ftq_generate_normal(_ptr(out), ctypes.c_size_t(count), ctypes.c_uint32(seed), ctypes.c_float(sigma),
                                     ctypes.c_float(post_scale))
        return out

    # -- GEMM
    def gemm_f32(self, a, b, m, n, k, b_layout=B_NK, c_layout=C_COLMAJOR):
        c = np.empty(m * n, dtype=np.float32)
        self.lib.ftq_gemm_f32(_ptr(a), _ptr(b), _ptr(c), m, n, k, b_layout, c_layout)
        return c.reshape((n, m) if c_layout == C_COLMAJOR else (m, n))

    def dot_f64(self, a, b, row, col, n, k, b_layout=B_NK):
        return float(self.lib.ftq_dot_f64(_ptr(a), _ptr(b), row, col, n, k, b_layout))

    # -- expected checksums
    def band_sums(self, a, b, m, n, k, tile=64):
        tr, tc = (m + tile - 1) // tile, (n + tile - 1) // tile
        out = [np.empty((tr, k), np.float32), np.empty((tr, k), np.float32), np.empty((tc, k), np.float32),
               np.empty((tc, k), np.float32)]
        self.lib.ftq_band_sums(_ptr(a), _ptr(b), *[_ptr(x) for x in out], m, n, k, tile)
        return dict(zip(("a_sums", "a_magnitudes", "b_sums", "b_magnitudes"), out))

    def expected(self, a, b, m, n, k, tile=64, bands=None):
        bands = bands or self.band_sums(a, b, m, n, k, tile)
        tiles = ((m + tile - 1) // tile) * ((n + tile - 1) // tile)
        out = {name: np.full((tiles, tile), np.nan, np.float32) for name in
               ("expected_rows", "expected_cols", "row_scales", "col_scales")}
        self.lib.ftq_expected_from_bands(_ptr(a), _ptr(b), _ptr(bands["a_sums"]), _ptr(bands["a_magnitudes"]),
                                         _ptr(bands["b_sums"]), _ptr(bands["b_magnitudes"]), _ptr(out["expected_rows"]),
                                         _ptr(out["expected_cols"]), _ptr(out["row_scales"]), _ptr(out["col_scales"]), m, n, k,
                                         tile)
        out.update(bands)
        return out

    def s0_prepare(self, a, b, m, n, k, tile=16):
        tiles = ((m + tile - 1) // tile) * ((n + tile - 1) // tile)
        out = {name: np.zeros((tiles, tile), np.float32) for name in
               ("expected_rows", "expected_cols", "row_scales", "col_scales")}
        self.lib.ftq_s0_prepare(_ptr(a), _ptr(b), _ptr(out["expected_rows"]), _ptr(out["expected_cols"]),
                                _ptr(out["row_scales"]), _ptr(out["col_scales"]), m, n, k, tile)
        return out

    # -- checker
    def abft_check(self, c, m, n, cache, abs_tol=1e-2, rel_tol=2e-5, tile=64, c_layout=C_COLMAJOR, or_rule=True, faults=(),
                   max_records=256):
        """Checks (and corrects, in place) a copy of c.  Returns (c_after, summary, records)."""
        c = np.ascontiguousarray(c, dtype=np.float32).copy()
        fa = (Fault * max(1, len(faults)))()
        for i, (t, r, col, v) in enumerate(faults):
            fa[i] = Fault(int(t), int(r), int(col), float(v))
        recs = (TileRecord * max_records)()
        summary = CheckSummary()
        self.lib.ftq_abft_check(_ptr(c), m, n, tile, c_layout, _ptr(cache["expected_rows"]), _ptr(cache["expected_cols"]),
                                _ptr(cache["row_scales"]), _ptr(cache["col_scales"]), ctypes.c_float(abs_tol),
                                ctypes.c_float(rel_tol), int(bool(or_rule)), fa, len(faults), recs, max_records,
                                ctypes.byref(summary))
        return c, summary, list(recs[:summary.n_records])

    # -- campaign / verifier
    def campaign(self, seed, trials, tile_count, tile=64, min_value=1.0, max_value=256.0):
        state = ctypes.c_uint32(seed & 0xFFFFFFFF)
        draws = []
        for trial in range(trials):
            d = CampaignDraw()
            self.lib.ftq_campaign_next(ctypes.byref(state), trial, tile_count, tile, ctypes.c_float(min_value),
                                       ctypes.c_float(max_value), ctypes.byref(d))
            draws.append((d.tile, d.row, d.col, d.signed_value, d.bin, d.unit))
        return draws, state.value

    def verify_samples(self, a, b, c, m, n, k, samples=8, abs_tol=0.25, rel_tol=1e-2, b_layout=B_NK, c_layout=C_COLMAJOR):
        out = VerifyResult()
        c = np.ascontiguousarray(c, dtype=np.float32)
        self.lib.ftq_verify_samples(_ptr(a), _ptr(b), _ptr(c), m, n, k, samples, ctypes.c_float(abs_tol), ctypes.c_float(rel_tol),
                                    b_layout, c_layout, ctypes.byref(out))
        return out

    def full_pass(self, a, b, m_rows, n, k, tile=64, abs_tol=1e-2, rel_tol=2e-5):
        c = np.empty(m_rows * n, dtype=np.float32)
        secs = (ctypes.c_double * 3)()
        summary = CheckSummary()
        self.lib.ftq_full_pass(_ptr(a), _ptr(b), _ptr(c), m_rows, n, k, tile, ctypes.c_float(abs_tol), ctypes.c_float(rel_tol),
                               secs, ctypes.byref(summary))
        return c.reshape(n, m_rows), list(secs), summary

    def num_threads(self):
        return int(self.lib.ftq_num_threads())

    def set_num_threads(self, threads):
        self.lib.ftq_set_num_threads(int(threads))


_oracle = None


def load():
    global _oracle
    if _oracle is None:
        if not os.path.exists(SO) or os.path.getmtime(SO) < os.path.getmtime(os.path.join(ORACLE_DIR, "ftq_oracle.c")):
            build()
        _oracle = Oracle(ctypes.CDLL(SO))
    return _oracle
