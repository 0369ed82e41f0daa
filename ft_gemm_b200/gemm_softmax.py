"""Host-side mirror of the reference's GEMM + softmax cross-nonlinearity prototype
(src/gemm_softmax_abft.cu:381-543) over the C-ABI of include/ft_gemm_softmax.h;
torch only supplies device memory and the stream handle."""
import ctypes
from dataclasses import dataclass, field
from typing import List, Optional, Tuple

import torch

from . import _abi
from .operator import _stream_ptr


class FtGsOptions(ctypes.Structure):
    _fields_ = [("abs_tol", ctypes.c_double), ("rel_tol", ctypes.c_double), ("row_sum_tol", ctypes.c_double),
                ("location_tol", ctypes.c_double)]


class FtGsFault(ctypes.Structure):
    _fields_ = [("row", ctypes.c_int), ("col", ctypes.c_int), ("value", ctypes.c_float)]


class FtGsRecord(ctypes.Structure):
    _fields_ = [("row", ctypes.c_int), ("estimated_col", ctypes.c_int), ("correction_delta", ctypes.c_double)]


class FtGsReport(ctypes.Structure):
    _fields_ = [("status", ctypes.c_int), ("detected_rows", ctypes.c_int), ("located_rows", ctypes.c_int),
                ("post_detected_rows", ctypes.c_int), ("n_records", ctypes.c_int), ("gemm_bad_tiles", ctypes.c_int),
                ("gemm_corrected_tiles", ctypes.c_int), ("max_projection_residual", ctypes.c_double),
                ("post_max_projection_residual", ctypes.c_double), ("records", FtGsRecord * 16)]


@dataclass
class GsReport:
    status: int
    detected_rows: int
    located_rows: int
    post_detected_rows: int
    gemm_bad_tiles: int
    gemm_corrected_tiles: int
    max_projection_residual: float
    post_max_projection_residual: float
    records: List[Tuple[int, int, float]] = field(default_factory=list)  # (row, estimated_col, correction_delta)


_bound = False


def _lib():
    global _bound
    lib = _abi.load()
    if not _bound:
        vp, ci = ctypes.c_void_p, ctypes.c_int
        lib.ft_gs_options_default.argtypes = [ctypes.POINTER(FtGsOptions)]
        lib.ft_gs_options_default.restype = None
        lib.ft_gemm_softmax_abft_prepare.argtypes = [ctypes.POINTER(vp), vp, vp, ci, ci, ci, ctypes.POINTER(FtGsOptions), vp]
        lib.ft_gemm_softmax_abft_run.argtypes = [vp, vp, ctypes.POINTER(FtGsFault), ci, vp]
        lib.ft_gemm_softmax_abft_report.argtypes = [vp, ctypes.POINTER(FtGsReport)]
        lib.ft_gemm_softmax_abft_logits.argtypes = [vp, ctypes.POINTER(vp), ctypes.POINTER(ci)]
        lib.ft_gemm_softmax_abft_logits_read.argtypes = [vp, vp]
        lib.ft_gemm_softmax_abft_logits_read.restype = ci
        lib.ft_gemm_softmax_abft_checks.argtypes = [vp, vp, vp, vp, vp, vp, vp]
        lib.ft_gemm_softmax_abft_destroy.argtypes = [vp]
        lib.ft_gemm_softmax_generate_fp8.argtypes = [vp, ctypes.c_size_t, ctypes.c_uint32, vp]
        for name in ("ft_gemm_softmax_abft_prepare", "ft_gemm_softmax_abft_run", "ft_gemm_softmax_abft_report",
                     "ft_gemm_softmax_abft_logits", "ft_gemm_softmax_abft_checks", "ft_gemm_softmax_abft_destroy",
                     "ft_gemm_softmax_generate_fp8"):
            getattr(lib, name).restype = ci
        _bound = True
    return lib


def generate_gs_fp8(shape, seed: int, device="cuda") -> torch.Tensor:
    """The prototype's inputs ((hash(seed + i) % 7) - 3) / 16 as E4M3 bytes."""
    out = torch.empty(shape, dtype=torch.uint8, device=device)
    with torch.cuda.device(out.device):
        _abi.check(_lib().ft_gemm_softmax_generate_fp8(ctypes.c_void_p(out.data_ptr()), out.numel(), seed & 0xFFFFFFFF, _stream_ptr(None)))
    return out


class GemmSoftmaxAbft:
    """logits = A B^T / sqrt(K) on the fault-tolerant tensor-core GEMM, row softmax with the two log-domain identities."""

    def __init__(self, a: torch.Tensor, b: torch.Tensor, abs_tol: float = 2.0e-3, rel_tol: float = 2.0e-5,
                 row_sum_tol: float = 2.0e-6, location_tol: float = 0.25, stream: Optional[torch.cuda.Stream] = None):
        for t, name in ((a, "A"), (b, "B")):
            if not t.is_cuda or t.dtype != torch.uint8 or t.dim() != 2 or not t.is_contiguous():
                raise ValueError(f"{name} must be a contiguous 2-D uint8 (E4M3) CUDA tensor")
        if a.shape[1] != b.shape[1]:
            raise ValueError("A [M,K] and B [N,K] must share K")
        self.lib = _lib()
        self.a, self.b = a, b
        self.m, self.k = a.shape
        self.n = b.shape[0]
        options = FtGsOptions(abs_tol, rel_tol, row_sum_tol, location_tol)
        self.handle = ctypes.c_void_p()
        with torch.cuda.device(a.device):
            _abi.check(self.lib.ft_gemm_softmax_abft_prepare(ctypes.byref(self.handle), ctypes.c_void_p(a.data_ptr()),
                                                             ctypes.c_void_p(b.data_ptr()), self.m, self.n, self.k,
                                                             ctypes.byref(options), _stream_ptr(stream)))

    def new_output(self) -> torch.Tensor:
        return torch.empty((self.m, self.n), dtype=torch.float32, device=self.a.device)

    def run(self, probabilities: torch.Tensor, fault: Optional[Tuple[int, int, float]] = None, correct: bool = False,
            stream: Optional[torch.cuda.Stream] = None):
        if (not probabilities.is_cuda or probabilities.dtype != torch.float32 or not probabilities.is_contiguous() or
                tuple(probabilities.shape) != (self.m, self.n)):
            raise ValueError("probabilities must be a contiguous float32 CUDA tensor of shape [M, N]")
        cf = FtGsFault(*fault) if fault is not None else None
        with torch.cuda.device(self.a.device):
            _abi.check(self.lib.ft_gemm_softmax_abft_run(self.handle, ctypes.c_void_p(probabilities.data_ptr()),
                                                         ctypes.byref(cf) if cf is not None else None, int(correct), _stream_ptr(stream)))

    def report(self) -> GsReport:
        rep = FtGsReport()
        with torch.cuda.device(self.a.device):
            _abi.check(self.lib.ft_gemm_softmax_abft_report(self.handle, ctypes.byref(rep)))
        records = [(r.row, r.estimated_col, r.correction_delta) for r in rep.records[:rep.n_records]]
        return GsReport(rep.status, rep.detected_rows, rep.located_rows, rep.post_detected_rows, rep.gemm_bad_tiles,
                        rep.gemm_corrected_tiles, rep.max_projection_residual, rep.post_max_projection_residual, records)

    def logits(self) -> torch.Tensor:
        """A host copy of the handle's logits, [M, N] float32."""
        out = torch.empty((self.m, self.n), dtype=torch.float32)
        with torch.cuda.device(self.a.device):
            _abi.check(self.lib.ft_gemm_softmax_abft_logits_read(self.handle, ctypes.c_void_p(out.data_ptr())))
        return out

    def checks(self) -> dict:
        import numpy as np
        names = ("expected_sum", "expected_weighted", "actual_sum", "actual_weighted", "probability_sum", "log_z")
        out = {name: np.empty(self.m, dtype=np.float64) for name in names}
        with torch.cuda.device(self.a.device):
            _abi.check(self.lib.ft_gemm_softmax_abft_checks(self.handle, *[out[name].ctypes.data_as(ctypes.c_void_p) for name in names]))
        return out

    def close(self):
        if getattr(self, "handle", None) is not None and self.handle.value:
            self.lib.ft_gemm_softmax_abft_destroy(self.handle)
            self.handle = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
