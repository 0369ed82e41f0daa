"""Host-side mirror of the reference's operator for the ABFT FP8 GEMM path.

The reference drives its kernels from main() in the fixed order prepare ->
GEMM+check+correct -> read counters (src/s4_cluster_multicast_abft_fp8_gemm.cu:
634-714).  `AbftGemm` is that sequence over the C-ABI: it owns a prepared handle
for one (A, B) pair, `run()` launches the fused kernel, `report()` reads the
counters and per-tile records.  torch supplies device memory and streams only.
"""
import ctypes
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import torch

from . import _abi

Fault = Tuple[int, int, int, float]  # (abft_tile, local_row, local_col, value)


@dataclass
class TileRecord:
    tile: int
    bad_row_count: int
    bad_col_count: int
    bad_row: int
    bad_col: int
    row_delta: float
    col_delta: float
    corrected: int


@dataclass
class Report:
    status: int
    bad_tiles: int
    corrected_tiles: int
    multi_fault_tiles: int
    records_dropped: int
    max_clean_ratio: float
    prepare_ms: float
    prepare_input_ms: float
    prepare_expected_ms: float
    records: List[TileRecord] = field(default_factory=list)


def _report_from_c(rep: _abi.FtReport) -> Report:
    records = [TileRecord(r.tile, r.bad_row_count, r.bad_col_count, r.bad_row, r.bad_col, r.row_delta, r.col_delta,
                          r.corrected) for r in rep.records[:rep.n_records]]
    return Report(rep.status, rep.bad_tiles, rep.corrected_tiles, rep.multi_fault_tiles, rep.records_dropped,
                  rep.max_clean_ratio, rep.prepare_ms, rep.prepare_input_ms, rep.prepare_expected_ms, records)


def _fault_array(faults: Optional[Sequence[Fault]]):
    faults = list(faults or [])
    if len(faults) > _abi.FT_MAX_FAULTS:
        raise ValueError(f"at most {_abi.FT_MAX_FAULTS} faults per run")
    arr = (_abi.FtFault * max(1, len(faults)))()
    for i, (tile, row, col, value) in enumerate(faults):
        arr[i] = _abi.FtFault(int(tile), int(row), int(col), float(value))
    return arr, len(faults)


def _stream_ptr(stream: Optional[torch.cuda.Stream]):
    stream = stream if stream is not None else torch.cuda.current_stream()
    return ctypes.c_void_p(stream.cuda_stream)


def _check_operand(t: torch.Tensor, name: str):
    if not t.is_cuda or t.dim() != 2 or not t.is_contiguous() or t.element_size() != 1:
        raise ValueError(f"{name} must be a contiguous 2-D CUDA tensor of 1-byte (FP8 E4M3) elements")


def generate_fp8(count_or_shape, seed: int, dist: str = "uniform", sigma: float = 1.0, post_scale: float = 1.0,
                 device="cuda") -> torch.Tensor:
    """Seeded E4M3 inputs generated on the device; `uniform` is the reference's
    generator (src/s0_tiled_abft_fp8_gemm.cu:102-110), bit for bit."""
    shape = (count_or_shape,) if isinstance(count_or_shape, int) else tuple(count_or_shape)
    out = torch.empty(shape, dtype=torch.uint8, device=device)
    lib = _abi.load()
    _abi.check(lib.ft_gemm_generate_fp8(ctypes.c_void_p(out.data_ptr()), out.numel(), seed & 0xFFFFFFFF,
                                        {"uniform": 0, "normal": 1}[dist], sigma, post_scale, _stream_ptr(None)))
    return out


class AbftGemm:
    """Prepared ABFT FP8 GEMM for one (A[M,K], B[N,K]) pair of E4M3 tensors."""

    def __init__(self, a: torch.Tensor, b: torch.Tensor, abs_tol: float = 1.0e-2, rel_tol: float = 2.0e-5,
                 sm_limit: int = 0, single_cta: bool = False, exact_prepare: bool = False,
                 stream: Optional[torch.cuda.Stream] = None):
        _check_operand(a, "A")
        _check_operand(b, "B")
        if a.shape[1] != b.shape[1]:
            raise ValueError("A[M,K] and B[N,K] disagree on K")
        self.lib = _abi.load()
        self.a, self.b = a, b  # keep the operands alive: the handle holds their addresses
        self.m, self.k = a.shape
        self.n = b.shape[0]
        options = _abi.FtOptions()
        self.lib.ft_options_default(ctypes.byref(options))
        options.abs_tol, options.rel_tol, options.sm_limit = abs_tol, rel_tol, sm_limit
        options.single_cta = int(single_cta)
        options.exact_prepare = int(exact_prepare)
        self.exact_prepare = bool(exact_prepare)
        self.handle = ctypes.c_void_p()
        with torch.cuda.device(a.device):
            _abi.check(self.lib.ft_gemm_fp8_abft_prepare(ctypes.byref(self.handle), ctypes.c_void_p(a.data_ptr()),
                                                         ctypes.c_void_p(b.data_ptr()), self.m, self.n, self.k,
                                                         ctypes.byref(options), _stream_ptr(stream)))

    @property
    def tile_cols(self) -> int:
        return -(-self.n // _abi.FT_ABFT_TILE)  # the last tile column may be short

    @property
    def tile_count(self) -> int:
        return -(-self.m // _abi.FT_ABFT_TILE) * self.tile_cols

    def new_output(self) -> torch.Tensor:
        """C as the reference lays it out: [N, M] with M contiguous (column-major C[M,N])."""
        return torch.empty((self.n, self.m), dtype=torch.float32, device=self.a.device)

    def run(self, c: torch.Tensor, faults: Optional[Sequence[Fault]] = None, stream: Optional[torch.cuda.Stream] = None):
        if not c.is_cuda or c.dtype != torch.float32 or not c.is_contiguous() or tuple(c.shape) != (self.n, self.m):
            raise ValueError("C must be a contiguous float32 CUDA tensor of shape [N, M]")
        arr, count = _fault_array(faults)
        with torch.cuda.device(self.a.device):
            _abi.check(self.lib.ft_gemm_fp8_abft_run(self.handle, ctypes.c_void_p(c.data_ptr()), arr, count,
                                                     _stream_ptr(stream)))

    def run_window(self, c: torch.Tensor, row0: int, rows: int, col0: int, cols: int, faults: Optional[Sequence[Fault]] = None,
                   zero_report: bool = True, stream: Optional[torch.cuda.Stream] = None):
        """The launch restricted to rows [row0, row0+rows) x columns [col0, col0+cols) of the product; `c` is the full [N, M]
        output.  zero_report=False keeps the counters of earlier windows."""
        if not c.is_cuda or c.dtype != torch.float32 or not c.is_contiguous() or tuple(c.shape) != (self.n, self.m):
            raise ValueError("C must be a contiguous float32 CUDA tensor of shape [N, M]")
        arr, count = _fault_array(faults)
        with torch.cuda.device(self.a.device):
            _abi.check(self.lib.ft_gemm_fp8_abft_run_window(self.handle, ctypes.c_void_p(c.data_ptr()), arr, count, row0, rows,
                                                            col0, cols, int(zero_report), _stream_ptr(stream)))

    def run_profiled(self, c: torch.Tensor):
        """Runs once and returns a [ctas, 8] int64 tensor of per-role wait/total cycle counters (see ft_gemm.h)."""
        out = torch.zeros((512, 8), dtype=torch.int64)
        ctas = ctypes.c_int(0)
        with torch.cuda.device(self.a.device):
            _abi.check(self.lib.ft_gemm_fp8_abft_run_profiled(self.handle, ctypes.c_void_p(c.data_ptr()),
                                                              ctypes.c_void_p(out.data_ptr()), 512, ctypes.byref(ctas),
                                                              _stream_ptr(None)))
        return out[:ctas.value]

    def refresh(self, a_changed: bool = True, b_changed: bool = True, stream: Optional[torch.cuda.Stream] = None):
        with torch.cuda.device(self.a.device):
            _abi.check(self.lib.ft_gemm_fp8_abft_refresh(self.handle, int(a_changed) | (int(b_changed) << 1),
                                                         _stream_ptr(stream)))

    def quantize_a(self, src: torch.Tensor, scale: float = 1.0, stream: Optional[torch.cuda.Stream] = None):
        """Overwrites A with E4M3(src * scale) (src: [M, K] float32, bfloat16 or float16 on the device) and refreshes the
        cache, with the band sums of A taken in the same pass over src."""
        dtypes = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}
        if not src.is_cuda or src.dtype not in dtypes or not src.is_contiguous() or tuple(src.shape) != (self.m, self.k):
            raise ValueError("src must be a contiguous [M, K] float32, bfloat16 or float16 CUDA tensor")
        with torch.cuda.device(self.a.device):
            _abi.check(self.lib.ft_gemm_fp8_abft_quantize_a(self.handle, ctypes.c_void_p(src.data_ptr()), dtypes[src.dtype],
                                                            float(scale), _stream_ptr(stream)))

    def set_tolerance(self, abs_tol: float, rel_tol: float):
        _abi.check(self.lib.ft_gemm_fp8_abft_set_tolerance(self.handle, abs_tol, rel_tol))

    def report(self, allow_timeout: bool = False) -> Report:
        rep = _abi.FtReport()
        with torch.cuda.device(self.a.device):
            code = self.lib.ft_gemm_fp8_abft_report(self.handle, ctypes.byref(rep))
        if code != _abi.FT_OK and not (allow_timeout and code == _abi.FT_ERR_TIMEOUT):
            _abi.check(code)
        return _report_from_c(rep)

    def cache(self) -> dict:
        """The expected-checksum cache as torch tensors (copies), for inspection."""
        view = _abi.FtCacheView()
        _abi.check(self.lib.ft_gemm_fp8_abft_cache(self.handle, ctypes.byref(view)))
        tiles = self.tile_count
        kp = -(-self.k // 16) * 16  # the band-sum arrays of a handle with padded operand copies have ceil16(K) columns
        shapes = {"a_sums": (-(-self.m // 64), kp), "a_magnitudes": (-(-self.m // 64), kp),
                  "b_sums": (-(-self.n // 64), kp), "b_magnitudes": (-(-self.n // 64), kp),
                  "expected_rows": (tiles, 64), "expected_cols": (tiles, 64), "row_scales": (tiles, 64),
                  "col_scales": (tiles, 64)}
        out = {}
        for which, (name, shape) in enumerate(shapes.items()):
            host = torch.empty(shape, dtype=torch.float32)
            with torch.cuda.device(self.a.device):
                _abi.check(self.lib.ft_gemm_fp8_abft_cache_read(self.handle, which, ctypes.c_void_p(host.data_ptr()),
                                                                host.numel()))
            out[name] = host[:, :self.k].contiguous() if which < 4 else host
        return out

    def close(self):
        if getattr(self, "handle", None) is not None and self.handle.value:
            self.lib.ft_gemm_fp8_abft_destroy(self.handle)
            self.handle = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class HostAbftGemm:
    """The operator called with HOST buffers (pinned numpy/torch CPU tensors):
    every call copies A and B to the device, runs, and copies C back."""

    def __init__(self, m: int, n: int, k: int, abs_tol: float = 1.0e-2, rel_tol: float = 2.0e-5):
        self.lib = _abi.load()
        self.m, self.n, self.k = m, n, k
        self.options = _abi.FtOptions()
        self.lib.ft_options_default(ctypes.byref(self.options))
        self.options.abs_tol, self.options.rel_tol = abs_tol, rel_tol
        self.handle = ctypes.c_void_p()

    def __call__(self, a_host: torch.Tensor, b_host: torch.Tensor, c_host: torch.Tensor,
                 faults: Optional[Sequence[Fault]] = None, prepare: bool = False) -> Report:
        for t, name in ((a_host, "A"), (b_host, "B"), (c_host, "C")):
            if t.is_cuda or not t.is_contiguous():
                raise ValueError(f"{name} must be a contiguous host tensor")
        arr, count = _fault_array(faults)
        rep = _abi.FtReport()
        _abi.check(self.lib.ft_gemm_fp8_abft_host(ctypes.byref(self.handle), ctypes.c_void_p(a_host.data_ptr()),
                                                  ctypes.c_void_p(b_host.data_ptr()), ctypes.c_void_p(c_host.data_ptr()),
                                                  self.m, self.n, self.k, ctypes.byref(self.options), arr, count,
                                                  int(prepare), ctypes.byref(rep)))
        return _report_from_c(rep)

    def close(self):
        if self.handle.value:
            self.lib.ft_gemm_fp8_abft_destroy(self.handle)
            self.handle = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
