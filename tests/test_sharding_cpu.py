"""Host-side logic of the row sharding, run as world_size-2 gloo ranks on CPU:
partition arithmetic, global tile ids and the all-gather of fault reports."""
import os
import socket
import sys

import pytest

torch = pytest.importorskip("torch")
import torch.multiprocessing as mp  # noqa: E402

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_rows_partition():
    from ft_gemm_b200 import shard_rows
    for m, world in [(32768, 8), (32768, 4), (8192, 2), (1280, 4), (384, 3), (128, 1)]:
        shards = [shard_rows(m, 8192, r, world) for r in range(world)]
        assert shards[0].row_begin == 0 and sum(s.rows for s in shards) == m
        for prev, nxt in zip(shards, shards[1:]):
            assert prev.row_begin + prev.rows == nxt.row_begin
        assert all(s.rows % 128 == 0 and s.rows > 0 for s in shards)
        assert max(s.rows for s in shards) - min(s.rows for s in shards) <= 128
    with pytest.raises(ValueError):
        shard_rows(100, 256, 0, 1)
    with pytest.raises(ValueError):
        shard_rows(128, 256, 0, 2)
    s = shard_rows(32768, 8192, 3, 8)
    assert (s.row_begin, s.rows) == (12288, 4096)
    # local tile (tile_row 2, tile_col 5) of rank 3 -> global tile_row 2 + 12288/64
    assert s.global_tile(2 * 128 + 5) == (2 + 192) * 128 + 5


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist

    from ft_gemm_b200 import Report, TileRecord, gather_reports, shard_rows
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    shard = shard_rows(512, 256, rank, world)
    recs = [TileRecord(tile=1 + rank, bad_row_count=1, bad_col_count=1, bad_row=3, bad_col=4 + rank, row_delta=-2.0,
                       col_delta=-2.0, corrected=1)]
    if rank == 1:
        recs.append(TileRecord(0, 2, 2, 1, 2, 3.0, 3.0, 0))
    mine = Report(0, len(recs), 1, len(recs) - 1, 0, 0.01 * (rank + 1), 0.0, 0.0, 0.0, recs)
    total = gather_reports(mine, shard)
    out.put((rank, total.bad_tiles, total.corrected_tiles, total.multi_fault_tiles, total.max_clean_ratio,
             [(r.tile, r.bad_col, r.corrected) for r in total.records]))
    dist.destroy_process_group()


def test_report_all_gather_gloo_world2():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(out.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    # rank 1 holds rows 256..511 = tile rows 4..7; tile_cols = 4, so its local tiles 0 and 2 become 16 and 18
    expected_records = [(1, 4, 1), (16, 2, 0), (18, 5, 1)]
    for rank, bad, corrected, multi, noise, records in results:
        assert (bad, corrected, multi) == (3, 2, 1)
        assert noise == pytest.approx(0.02)
        assert records == expected_records


def test_gather_without_process_group_is_local():
    from ft_gemm_b200 import Report, TileRecord, gather_reports, shard_rows
    shard = shard_rows(256, 256, 0, 1)
    rep = Report(0, 1, 1, 0, 0, 0.5, 1.0, 0.5, 0.5, [TileRecord(3, 1, 1, 2, 2, -1.0, -1.0, 1)])
    total = gather_reports(rep, shard)
    assert (total.bad_tiles, total.corrected_tiles, total.records[0].tile) == (1, 1, 3)


def test_shard_heads_partition():
    from ft_gemm_b200 import shard_heads
    for total, world in [(128, 8), (128, 3), (5, 2), (7, 7), (1, 1)]:
        parts = [shard_heads(total, r, world) for r in range(world)]
        assert parts[0][0] == 0 and sum(c for _, c in parts) == total
        for (f0, c0), (f1, _) in zip(parts, parts[1:]):
            assert f0 + c0 == f1
        assert max(c for _, c in parts) - min(c for _, c in parts) <= 1


def _attn_worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist

    from ft_gemm_b200 import AttnReport, TileRecord, gather_attention_reports, shard_heads
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    first, count = shard_heads(6, rank, world)  # 6 (batch, head) pairs over 2 ranks
    seq = 256  # 4 bands: 16 score tiles per head
    recs = [TileRecord(tile=5 + rank, bad_row_count=1, bad_col_count=1, bad_row=2, bad_col=3, row_delta=-1.0, col_delta=-1.0, corrected=1)]
    mine = AttnReport(0, 1, 1, 0, rank, rank, 0, 0, 0, 0, 0.01 * (rank + 1), 0.5, recs, score_replayed=2 * rank + 1)
    total = gather_attention_reports(mine, first, 3, seq)
    out.put((rank, total.score_detected, total.score_corrected, total.pv_detected, total.max_score_noise, [r.tile for r in total.records],
             total.score_replayed))
    dist.destroy_process_group()


def test_attention_counters_all_gather_gloo_world2():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_attn_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(out.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, detected, corrected, pv, noise, tiles, replayed in results:
        assert (detected, corrected, pv, replayed) == (2, 2, 1, 4) and noise == pytest.approx(0.02)
        assert tiles == [5, 3 * 16 + 6]  # rank 1 owns heads 3..5: its local tile 6 is tile 6 of head 3
