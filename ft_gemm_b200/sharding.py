"""Row sharding of the ABFT GEMM across the GPUs of one box.

The path partitions by rows of A (and of C): every rank holds its own band of A,
a full copy of B and its own expected-checksum cache, runs the fused kernel on
its band and needs nothing from the other ranks.  The only exchange is the
all-gather of the fixed-size fault reports, so that every rank (and the caller)
sees the faults of the whole product with global tile ids.  One process per GPU;
`torch.distributed` (NCCL on GPUs, gloo in CPU tests) carries the all-gather.
"""
from dataclasses import dataclass
from typing import List

import torch

from ._abi import FT_ABFT_TILE, FT_MAX_RECORDS
from .operator import Report, TileRecord

ROW_ALIGN = 128  # the kernel's M granularity


@dataclass(frozen=True)
class RowShard:
    rank: int
    world: int
    row_begin: int
    rows: int
    n: int

    @property
    def tile_row_offset(self) -> int:
        return self.row_begin // FT_ABFT_TILE

    def global_tile(self, local_tile: int) -> int:
        """ABFT tile id of the whole product for a tile id of this shard
        (tile ids are tile_row * (N/64) + tile_col; only tile_row shifts)."""
        return local_tile + self.tile_row_offset * (-(-self.n // FT_ABFT_TILE))


def shard_rows(m: int, n: int, rank: int, world: int) -> RowShard:
    """Splits M rows into `world` contiguous bands, each a multiple of 128 rows;
    the first (m/128) % world ranks get one extra 128-row block."""
    if m % ROW_ALIGN != 0:
        raise ValueError(f"M must be a multiple of {ROW_ALIGN}")
    blocks = m // ROW_ALIGN
    if blocks < world:
        raise ValueError(f"M={m} has fewer than {world} blocks of {ROW_ALIGN} rows")
    base, extra = divmod(blocks, world)
    mine = base + (1 if rank < extra else 0)
    begin = rank * base + min(rank, extra)
    return RowShard(rank, world, begin * ROW_ALIGN, mine * ROW_ALIGN, n)


_HEADER = 6
_RECORD = 8


def _pack(report: Report, shard: RowShard) -> torch.Tensor:
    buf = torch.zeros(_HEADER + _RECORD * FT_MAX_RECORDS, dtype=torch.float64)
    buf[0:_HEADER] = torch.tensor([report.status, report.bad_tiles, report.corrected_tiles, report.multi_fault_tiles,
                                   report.records_dropped, report.max_clean_ratio], dtype=torch.float64)
    for i, r in enumerate(report.records[:FT_MAX_RECORDS]):
        base = _HEADER + _RECORD * i
        buf[base:base + _RECORD] = torch.tensor(
            [shard.global_tile(r.tile) + 1, r.bad_row_count, r.bad_col_count, r.bad_row, r.bad_col, r.row_delta,
             r.col_delta, r.corrected], dtype=torch.float64)
    return buf


def _unpack(bufs: List[torch.Tensor]) -> Report:
    status = 0
    bad = corrected = multi = dropped = 0
    noise = 0.0
    records: List[TileRecord] = []
    for buf in bufs:
        buf = buf.cpu()
        status = status or int(buf[0])
        bad += int(buf[1])
        corrected += int(buf[2])
        multi += int(buf[3])
        dropped += int(buf[4])
        noise = max(noise, float(buf[5]))
        for i in range(FT_MAX_RECORDS):
            base = _HEADER + _RECORD * i
            if int(buf[base]) == 0:
                break
            v = buf[base:base + _RECORD].tolist()
            records.append(TileRecord(int(v[0]) - 1, int(v[1]), int(v[2]), int(v[3]), int(v[4]), float(v[5]), float(v[6]),
                                      int(v[7])))
    records.sort(key=lambda r: r.tile)
    if len(records) > FT_MAX_RECORDS:
        dropped += len(records) - FT_MAX_RECORDS
        records = records[:FT_MAX_RECORDS]
    return Report(status, bad, corrected, multi, dropped, noise, 0.0, 0.0, 0.0, records)


def gather_reports(report: Report, shard: RowShard, group=None, device=None) -> Report:
    """All-gathers the per-shard reports; returns the report of the whole product
    (records in global tile order).  With world == 1 no collective is issued."""
    import torch.distributed as dist
    if shard.world == 1 or not dist.is_initialized():
        return _unpack([_pack(report, shard)])
    mine = _pack(report, shard)
    if device is not None:
        mine = mine.to(device)
    bufs = [torch.empty_like(mine) for _ in range(shard.world)]
    dist.all_gather(bufs, mine, group=group)
    return _unpack(bufs)
