"""Host-side mirror of the reference's fault-tolerant attention operator.

The reference's attention programs prepare K/V metadata, launch the fused forward
with a fault description and read nine counters back
(src/ft_flash_attention_a14.cu:1363-1519).  `FtAttention` is that sequence over
the C-ABI of include/ft_attention.h; torch only supplies device memory and the
stream handle.
"""
import ctypes
from dataclasses import dataclass, field
from typing import List, Optional, Tuple

import torch

from . import _abi
from .operator import TileRecord, _stream_ptr

FAULT_NONE, FAULT_SCORE, FAULT_SOFTMAX, FAULT_SOFTMAX_STATE, FAULT_OUTPUT = 0, 1, 2, 3, 4


class FtAttnOptions(ctypes.Structure):
    _fields_ = [("score_abs_tol", ctypes.c_float), ("score_rel_tol", ctypes.c_float), ("pv_abs_tol", ctypes.c_float),
                ("pv_rel_tol", ctypes.c_float), ("softmax_abs_tol", ctypes.c_float), ("softmax_rel_tol", ctypes.c_float),
                ("protect_softmax", ctypes.c_int), ("causal", ctypes.c_int), ("exact_prepare", ctypes.c_int)]


class FtAttnFault(ctypes.Structure):
    _fields_ = [("stage", ctypes.c_int), ("batch", ctypes.c_int), ("head", ctypes.c_int), ("query", ctypes.c_int),
                ("index", ctypes.c_int), ("value", ctypes.c_float), ("query2", ctypes.c_int), ("index2", ctypes.c_int),
                ("value2", ctypes.c_float)]


class FtAttnReport(ctypes.Structure):
    _fields_ = [("status", ctypes.c_int), ("score_detected", ctypes.c_int), ("score_corrected", ctypes.c_int),
                ("score_uncorrected", ctypes.c_int), ("pv_detected", ctypes.c_int), ("pv_corrected", ctypes.c_int),
                ("failed_rows", ctypes.c_int), ("softmax_detected", ctypes.c_int), ("softmax_corrected", ctypes.c_int),
                ("softmax_replayed", ctypes.c_int), ("score_replayed", ctypes.c_int), ("n_records", ctypes.c_int),
                ("max_score_noise", ctypes.c_float),
                ("prepare_ms", ctypes.c_float), ("records", _abi.FtTileRecord * 16)]


@dataclass
class AttnReport:
    status: int
    score_detected: int
    score_corrected: int
    score_uncorrected: int
    pv_detected: int
    pv_corrected: int
    failed_rows: int
    softmax_detected: int
    softmax_corrected: int
    softmax_replayed: int
    max_score_noise: float
    prepare_ms: float
    records: List[TileRecord] = field(default_factory=list)
    score_replayed: int = 0


_bound = False


def _lib():
    global _bound
    lib = _abi.load()
    if not _bound:
        vp, ci = ctypes.c_void_p, ctypes.c_int
        lib.ft_attn_options_default.argtypes = [ctypes.POINTER(FtAttnOptions)]
        lib.ft_attn_options_default.restype = None
        lib.ft_attention_fp16_abft_prepare.argtypes = [ctypes.POINTER(vp), vp, vp, vp, ci, ci, ci, ci,
                                                       ctypes.POINTER(FtAttnOptions), vp]
        lib.ft_attention_fp16_abft_refresh.argtypes = [vp, vp, vp, vp, vp]
        lib.ft_attention_fp16_abft_run.argtypes = [vp, vp, ctypes.POINTER(FtAttnFault), vp]
        lib.ft_attention_fp16_abft_report.argtypes = [vp, ctypes.POINTER(FtAttnReport)]
        lib.ft_attention_fp16_abft_destroy.argtypes = [vp]
        for name in ("ft_attention_fp16_abft_prepare", "ft_attention_fp16_abft_refresh", "ft_attention_fp16_abft_run",
                     "ft_attention_fp16_abft_report", "ft_attention_fp16_abft_destroy"):
            getattr(lib, name).restype = ci
        _bound = True
    return lib


def shard_heads(batch_heads: int, rank: int, world: int) -> Tuple[int, int]:
    """(first, count) of the (batch, head) pairs rank `rank` owns: attention shards by heads, nothing is exchanged
    except the counters."""
    base, extra = divmod(batch_heads, world)
    count = base + (1 if rank < extra else 0)
    return rank * base + min(rank, extra), count


def gather_attention_reports(report: "AttnReport", first_head: int, heads_per_batch: int, seq: int, group=None,
                             device=None) -> "AttnReport":
    """All-gathers the counters of head-sharded runs (the reference reads back one DeviceStats per run,
    src/ft_flash_attention_a14.cu:1437-1440): counters are added, the noise figure is the maximum, tile ids of the records are
    re-based from the rank's first (batch, head) pair to the whole [B*H] range.  Without a process group: the local report."""
    import torch.distributed as dist
    bands = seq // 64
    per_head = bands * bands
    counters = [report.status, report.score_detected, report.score_corrected, report.score_uncorrected, report.pv_detected,
                report.pv_corrected, report.failed_rows, report.softmax_detected, report.softmax_corrected, report.softmax_replayed,
                report.score_replayed]
    head = len(counters) + 2
    mine = torch.zeros(head + 8 * 16, dtype=torch.float64)
    mine[:11] = torch.tensor(counters, dtype=torch.float64)
    mine[11] = report.max_score_noise
    mine[12] = len(report.records)
    for i, r in enumerate(report.records[:16]):
        mine[head + 8 * i:head + 8 + 8 * i] = torch.tensor([r.tile + first_head * per_head, r.bad_row_count, r.bad_col_count, r.bad_row, r.bad_col,
                                                    r.row_delta, r.col_delta, r.corrected], dtype=torch.float64)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        if device is not None:
            mine = mine.to(device)
        bufs = [torch.empty_like(mine) for _ in range(dist.get_world_size(group))]
        dist.all_gather(bufs, mine, group=group)
        bufs = [b.cpu() for b in bufs]
    else:
        bufs = [mine]
    total = torch.stack(bufs)
    sums = total[:, :11].sum(dim=0)
    records = []
    for b in bufs:
        for i in range(int(b[12].item())):
            f = b[head + 8 * i:head + 8 + 8 * i].tolist()
            records.append(TileRecord(int(f[0]), int(f[1]), int(f[2]), int(f[3]), int(f[4]), f[5], f[6], int(f[7])))
    records.sort(key=lambda r: r.tile)
    status = int(total[:, 0].min().item()) if (total[:, 0] != 0).any() else 0  # any rank's error code (they are negative)
    return AttnReport(status, *(int(x) for x in sums[1:10].tolist()), float(total[:, 11].max().item()), report.prepare_ms, records[:16],
                      int(sums[10].item()))


class FtAttention:
    """Prepared fault-tolerant attention forward for one (Q, K, V) triple of [B, H, N, D] FP16 tensors."""

    def __init__(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, score_abs_tol: float = 1.0e-2,
                 score_rel_tol: float = 2.0e-5, pv_abs_tol: float = 2.0e-3, pv_rel_tol: float = 2.0e-3,
                 protect_softmax: bool = False, causal: bool = False, exact_prepare: bool = False,
                 stream: Optional[torch.cuda.Stream] = None):
        for t, name in ((q, "Q"), (k, "K"), (v, "V")):
            if not t.is_cuda or t.dtype != torch.float16 or t.dim() != 4 or not t.is_contiguous() or t.shape != q.shape:
                raise ValueError(f"{name} must be a contiguous [B, H, N, D] float16 CUDA tensor of the same shape as Q")
        self.lib = _lib()
        self.q, self.k, self.v = q, k, v
        self.batch, self.heads, self.seq, self.dim = q.shape
        options = FtAttnOptions()
        self.lib.ft_attn_options_default(ctypes.byref(options))
        options.score_abs_tol, options.score_rel_tol = score_abs_tol, score_rel_tol
        options.pv_abs_tol, options.pv_rel_tol = pv_abs_tol, pv_rel_tol
        options.protect_softmax = int(protect_softmax)
        options.causal = int(causal)
        options.exact_prepare = int(exact_prepare)
        self.handle = ctypes.c_void_p()
        with torch.cuda.device(q.device):
            _abi.check(self.lib.ft_attention_fp16_abft_prepare(
                ctypes.byref(self.handle), ctypes.c_void_p(q.data_ptr()), ctypes.c_void_p(k.data_ptr()),
                ctypes.c_void_p(v.data_ptr()), self.batch, self.heads, self.seq, self.dim, ctypes.byref(options),
                _stream_ptr(stream)))

    def refresh(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, stream: Optional[torch.cuda.Stream] = None):
        """New Q, K, V of the prepared shape: rebuilds the metadata in the handle's buffers, nothing is allocated."""
        for t, name in ((q, "Q"), (k, "K"), (v, "V")):
            if (not t.is_cuda or t.dtype != torch.float16 or not t.is_contiguous() or t.shape != self.q.shape
                    or t.device != self.q.device):
                raise ValueError(f"{name} must be a contiguous float16 CUDA tensor shaped like the prepared Q, on its device")
        with torch.cuda.device(q.device):
            _abi.check(self.lib.ft_attention_fp16_abft_refresh(self.handle, ctypes.c_void_p(q.data_ptr()),
                                                               ctypes.c_void_p(k.data_ptr()), ctypes.c_void_p(v.data_ptr()),
                                                               _stream_ptr(stream)))
        self.q, self.k, self.v = q, k, v

    def new_output(self) -> torch.Tensor:
        return torch.empty(self.q.shape, dtype=torch.float32, device=self.q.device)

    def run(self, out: torch.Tensor, fault: Optional[Tuple] = None, stream: Optional[torch.cuda.Stream] = None):
        """fault = (stage, batch, head, query, index, value) with the reference's stage numbers (1 score, 4 output); a score
        fault may carry a second one in the same head as three more entries (query2, index2, value2)."""
        if not out.is_cuda or out.dtype != torch.float32 or not out.is_contiguous() or out.shape != self.q.shape:
            raise ValueError("out must be a contiguous float32 CUDA tensor shaped like Q")
        cf = FtAttnFault(*fault) if fault is not None else None
        with torch.cuda.device(self.q.device):
            _abi.check(self.lib.ft_attention_fp16_abft_run(self.handle, ctypes.c_void_p(out.data_ptr()),
                                                           ctypes.byref(cf) if cf is not None else None, _stream_ptr(stream)))

    def report(self, allow_timeout: bool = False) -> AttnReport:
        rep = FtAttnReport()
        with torch.cuda.device(self.q.device):
            code = self.lib.ft_attention_fp16_abft_report(self.handle, ctypes.byref(rep))
        if code != _abi.FT_OK and not (allow_timeout and code == _abi.FT_ERR_TIMEOUT):
            _abi.check(code)
        records = [TileRecord(r.tile, r.bad_row_count, r.bad_col_count, r.bad_row, r.bad_col, r.row_delta, r.col_delta,
                              r.corrected) for r in rep.records[:rep.n_records]]
        return AttnReport(rep.status, rep.score_detected, rep.score_corrected, rep.score_uncorrected, rep.pv_detected,
                          rep.pv_corrected, rep.failed_rows, rep.softmax_detected, rep.softmax_corrected, rep.softmax_replayed,
                          rep.max_score_noise, rep.prepare_ms, records, rep.score_replayed)

    def close(self):
        if getattr(self, "handle", None) is not None and self.handle.value:
            self.lib.ft_attention_fp16_abft_destroy(self.handle)
            self.handle = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
