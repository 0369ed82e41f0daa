"""ctypes view of the C-ABI declared in include/ft_gemm.h.

The shared library is the product; this module only declares its structures and
argument types.  Loading fails loudly when the library has not been built: there
is no fallback path of any kind.
"""
import ctypes
import os

FT_OK = 0
FT_ERR_INVALID = -1
FT_ERR_CUDA = -2
FT_ERR_TIMEOUT = -3
FT_ERR_UNSUPPORTED = -4
FT_ABFT_TILE = 64
FT_MAX_FAULTS = 4
FT_MAX_RECORDS = 64

LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libft_gemm_b200.so")


class FtOptions(ctypes.Structure):
    _fields_ = [("abs_tol", ctypes.c_float), ("rel_tol", ctypes.c_float), ("sm_limit", ctypes.c_int),
                ("single_cta", ctypes.c_int), ("exact_prepare", ctypes.c_int), ("wait_limit_us", ctypes.c_int),
                ("reserved", ctypes.c_int * 2)]


class FtFault(ctypes.Structure):
    _fields_ = [("tile", ctypes.c_int), ("row", ctypes.c_int), ("col", ctypes.c_int), ("value", ctypes.c_float)]


class FtTileRecord(ctypes.Structure):
    _fields_ = [("tile", ctypes.c_int), ("bad_row_count", ctypes.c_int), ("bad_col_count", ctypes.c_int),
                ("bad_row", ctypes.c_int), ("bad_col", ctypes.c_int), ("row_delta", ctypes.c_float),
                ("col_delta", ctypes.c_float), ("corrected", ctypes.c_int)]


class FtReport(ctypes.Structure):
    _fields_ = [("status", ctypes.c_int), ("bad_tiles", ctypes.c_int), ("corrected_tiles", ctypes.c_int),
                ("multi_fault_tiles", ctypes.c_int), ("n_records", ctypes.c_int), ("records_dropped", ctypes.c_int),
                ("max_clean_ratio", ctypes.c_float), ("prepare_ms", ctypes.c_float),
                ("prepare_input_ms", ctypes.c_float), ("prepare_expected_ms", ctypes.c_float),
                ("records", FtTileRecord * FT_MAX_RECORDS)]


class FtCacheView(ctypes.Structure):
    _fields_ = [(name, ctypes.c_void_p) for name in
                ("a_sums", "a_magnitudes", "b_sums", "b_magnitudes", "expected_rows", "expected_cols", "row_scales",
                 "col_scales")] + [("bytes", ctypes.c_size_t)]


_lib = None


def load():
    """Returns the loaded library; raises if it is missing (no fallback exists)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `make lib` (or __graft_entry__.build()). "
            "ft_gemm_b200 has no CPU or PyTorch fallback.")
    lib = ctypes.CDLL(LIB_PATH)
    vp, ci, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    lib.ft_options_default.argtypes = [ctypes.POINTER(FtOptions)]
    lib.ft_options_default.restype = None
    lib.ft_gemm_fp8_abft_prepare.argtypes = [ctypes.POINTER(vp), vp, vp, ci, ci, ci, ctypes.POINTER(FtOptions), vp]
    lib.ft_gemm_fp8_abft_refresh.argtypes = [vp, ci, vp]
    lib.ft_gemm_fp8_abft_quantize_a.argtypes = [vp, vp, ci, cf, vp]
    lib.ft_gemm_fp8_abft_quantize_a.restype = ci
    lib.ft_gemm_fp8_abft_run.argtypes = [vp, vp, ctypes.POINTER(FtFault), ci, vp]
    lib.ft_gemm_fp8_abft_run_window.argtypes = [vp, vp, ctypes.POINTER(FtFault), ci, ci, ci, ci, ci, ci, vp]
    lib.ft_gemm_fp8_abft_run_profiled.argtypes = [vp, vp, vp, ci, ctypes.POINTER(ci), vp]
    lib.ft_gemm_fp8_abft_run_profiled.restype = ci
    lib.ft_gemm_fp8_abft_report.argtypes = [vp, ctypes.POINTER(FtReport)]
    lib.ft_gemm_fp8_abft_destroy.argtypes = [vp]
    lib.ft_gemm_fp8_abft_cache.argtypes = [vp, ctypes.POINTER(FtCacheView)]
    lib.ft_gemm_fp8_abft_cache_read.argtypes = [vp, ci, vp, ctypes.c_size_t]
    lib.ft_gemm_fp8_abft_set_tolerance.argtypes = [vp, cf, cf]
    lib.ft_gemm_fp8_abft_host.argtypes = [ctypes.POINTER(vp), vp, vp, vp, ci, ci, ci, ctypes.POINTER(FtOptions),
                                          ctypes.POINTER(FtFault), ci, ci, ctypes.POINTER(FtReport)]
    lib.ft_gemm_fp8_abft_expected_noalloc.argtypes = [vp, vp, ci, ci, ci, vp, vp, vp, vp, vp]
    lib.ft_gemm_fp8_abft_expected_noalloc.restype = ci
    lib.ft_gemm_generate_fp8.argtypes = [vp, ctypes.c_size_t, ctypes.c_uint32, ci, cf, cf, vp]
    lib.ft_gemm_report_rebase.argtypes = [ctypes.POINTER(FtReport), ci, ci]
    lib.ft_gemm_report_rebase.restype = ci
    lib.ft_gemm_report_merge.argtypes = [ctypes.POINTER(FtReport), ci, ctypes.POINTER(FtReport)]
    lib.ft_gemm_report_merge.restype = ci
    lib.ft_gemm_fp8_abft_selftest_wait.argtypes = [vp, ci, vp]
    lib.ft_gemm_fp8_abft_selftest_wait.restype = ci
    lib.ft_gemm_last_error.argtypes = []
    lib.ft_gemm_last_error.restype = ctypes.c_char_p
    lib.ft_gemm_abi_version.argtypes = []
    for name in ("ft_gemm_fp8_abft_prepare", "ft_gemm_fp8_abft_refresh", "ft_gemm_fp8_abft_run", "ft_gemm_fp8_abft_run_window", "ft_gemm_fp8_abft_report",
                 "ft_gemm_fp8_abft_destroy", "ft_gemm_fp8_abft_cache", "ft_gemm_fp8_abft_cache_read",
                 "ft_gemm_fp8_abft_set_tolerance",
                 "ft_gemm_fp8_abft_host", "ft_gemm_generate_fp8", "ft_gemm_abi_version"):
        getattr(lib, name).restype = ci
    _lib = lib
    return lib


class FtGemmError(RuntimeError):
    def __init__(self, code, message):
        super().__init__(f"ft_gemm error {code}: {message}")
        self.code = code


def check(code):
    if code != FT_OK:
        raise FtGemmError(code, load().ft_gemm_last_error().decode("utf-8", "replace"))
