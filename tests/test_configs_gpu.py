"""The full-size configurations of the path on a GPU, through the command-line programs and the C-ABI:

* the 1000 + 50 trial fault campaign at M=N=K=8192 with N(0,1) -> E4M3 inputs
  (the reference's campaign program, src/s4_random_fault_campaign.cu:754-809, 858-895,
  driven as its Makefile does, Makefile:9-13, 56-57), at the reference's default
  tolerance and at the tighter relative tolerance the correction rate is quoted on;
* the projection shapes M=32768, K=8192, N=8192 and N=28672 with N(0,0.02)
  inputs scaled to unit max-abs: clean run, sampled FP64 rows, campaign faults;
* shard equivalence: the product computed as row bands, one handle per band,
  equals the unsharded run bit for bit (C, cache, re-based fault records);
* the failure path: a device-side wait that runs out is reported as
  FT_ERR_TIMEOUT and leaves the GPU usable.
"""
import ctypes
import os
import subprocess

import numpy as np
import pytest

torch = pytest.importorskip("torch")

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BUILD = os.path.join(ROOT, "build")


def _run(program, *args, timeout=900):
    exe = os.path.join(BUILD, program)
    if not os.path.exists(exe):
        subprocess.run(["make", "-C", ROOT, "cli"], check=True, stdout=subprocess.DEVNULL)
    out = subprocess.run([exe, *map(str, args)], capture_output=True, text=True, timeout=timeout)
    report = {}
    for line in out.stdout.splitlines():
        key, sep, value = line.partition(": ")
        if sep:
            report.setdefault(key, value)
    return out.returncode, report, out.stderr


CAMPAIGN_8192 = ("--m", 8192, "--n", 8192, "--k", 8192, "--dist", "normal", "--warmup", 1, "--repeat", 3, "--fault-trials", 1000,
                 "--double-trials", 50, "--fault-seed", 12345, "--fault-min-value", 1, "--fault-max-value", 256)


def test_campaign_8192_reference_default_tolerance():
    """abs 1e-2 + rel 2e-5 (src/s4:98-99): with N(0,1) inputs at K = 8192 the threshold is several units, so a few of the
    U[1,256] faults lie below it and pass the reference's checker by design.  Nothing may be corrected wrongly, every
    missed fault must lie below the largest threshold of the run, every fault above it must be caught."""
    rc, rep, err = _run("fault_campaign", *CAMPAIGN_8192)
    assert rc == 0, err
    assert rep["verification"] == "PASS" and rep["bad_tiles"] == "0"
    detected, missed, corrected = (int(rep[f"fault_campaign_{k}"]) for k in ("detected", "missed", "corrected"))
    assert detected + missed == 1000 and rep["fault_campaign_miscorrected"] == "0"
    assert corrected == detected - int(rep["fault_campaign_detected_not_corrected"])
    threshold_max = float(rep["abft_threshold_range"].split("max=")[1])
    assert 1.0 < threshold_max < 20.0
    assert float(rep["fault_campaign_max_missed_magnitude"]) < threshold_max
    assert missed <= 60  # U[1,256]: at most threshold_max / 255 of the trials can hide
    # a double fault whose one half hides below the threshold is indistinguishable from a single fault; none may go unnoticed
    assert int(rep["double_fault_missed"]) == 0
    assert int(rep["double_fault_reported_uncorrected"]) + int(rep["double_fault_silently_corrected"]) == 50


def test_campaign_8192_full_correction_at_stated_tolerance():
    """rel 2e-6: threshold below 1, clean-run noise three orders of magnitude under it -> every one of the 1000 single
    faults is located and corrected, every one of the 50 double faults is reported and left alone."""
    rc, rep, err = _run("fault_campaign", *CAMPAIGN_8192, "--rel-tol", 2e-6)
    assert rc == 0, err
    assert rep["verification"] == "PASS" and rep["bad_tiles"] == "0"
    assert float(rep["abft_threshold_range"].split("max=")[1]) < 1.0
    assert float(rep["clean_checksum_noise_ratio"]) < 0.05
    assert (rep["fault_campaign_detected"], rep["fault_campaign_corrected"]) == ("1000", "1000")
    assert (rep["fault_campaign_missed"], rep["fault_campaign_miscorrected"]) == ("0", "0")
    assert rep["fault_campaign_correction_rate_percent"] == "100.000"
    assert float(rep["fault_campaign_max_post_correction_residual"]) < 5e-3
    assert (rep["double_fault_reported_uncorrected"], rep["double_fault_silently_corrected"], rep["double_fault_missed"]) == ("50", "0", "0")
    assert float(rep["amortized_tflops"]) > 0 and float(rep["fused_gemm_tflops"]) > 0


@pytest.mark.parametrize("n", [8192, 28672])
def test_projection_shapes(n):
    """M = 32768 tokens, K = 8192, N = 8192 and the 28672 up-projection; inputs N(0, 0.02) scaled to unit max-abs.  The
    program verifies 64 sampled rows of dot products in FP64 (src/s4:527-554) and exits 0 only if the clean run is clean."""
    rc, rep, err = _run("fault_campaign", "--m", 32768, "--n", n, "--k", 8192, "--dist", "llm", "--warmup", 1, "--repeat", 3,
                        "--fault-trials", 25, "--double-trials", 5, "--fault-seed", 12345)
    assert rc == 0, err
    assert rep["verification"] == "PASS" and rep["bad_tiles"] == "0" and rep["verification_samples"] == "64"
    # the stated output bound 1e-5 * K * max|a| * max|b| with unit max-abs inputs
    assert float(rep["sampled_max_absolute_error"]) <= 1e-5 * 8192
    assert (rep["fault_campaign_detected"], rep["fault_campaign_corrected"], rep["fault_campaign_miscorrected"]) == ("25", "25", "0")
    assert (rep["double_fault_reported_uncorrected"], rep["double_fault_silently_corrected"]) == ("5", "0")
    assert rep["shape"].startswith(f"M=32768 N={n} K=8192")


@pytest.mark.parametrize("bands", [2, 4])
def test_sharded_equals_unsharded(bands):
    """Row bands with their own handles, caches and tile ids against one handle over the whole product."""
    import ft_gemm_b200 as ftg
    m, n, k = 1024, 512, 256
    a = ftg.generate_fp8((m, k), 0x12345678)
    b = ftg.generate_fp8((n, k), 0x9ABCDEF0)
    tile_cols = n // 64
    # faults by tile id of the whole product: one per band at least, one double
    faults = [(3, 5, 7, 2.5), ((m // 64 - 1) * tile_cols + 2, 63, 0, -4.0), ((m // 128) * tile_cols + 5, 10, 20, 3.0),
              ((m // 128) * tile_cols + 5, 30, 40, 6.0)]
    whole = ftg.AbftGemm(a, b, exact_prepare=True)
    c_whole = whole.new_output()
    whole.run(c_whole, faults)
    rep_whole = whole.report()
    cache_whole = whole.cache()
    c_parts = torch.empty_like(c_whole)
    merged = None
    reports = []
    for rank in range(bands):
        shard = ftg.shard_rows(m, n, rank, bands)
        rows = slice(shard.row_begin, shard.row_begin + shard.rows)
        op = ftg.AbftGemm(a[rows].contiguous(), b, exact_prepare=True)
        mine = [(t - shard.tile_row_offset * tile_cols, r, c, v) for (t, r, c, v) in faults
                if shard.tile_row_offset <= t // tile_cols < shard.tile_row_offset + shard.rows // 64]
        c_band = op.new_output()
        op.run(c_band, mine)
        c_parts[:, rows] = c_band
        reports.append((op.report(), shard))
        cache = op.cache()
        first, count = shard.tile_row_offset * tile_cols, (shard.rows // 64) * tile_cols
        for name in ("expected_rows", "expected_cols", "row_scales", "col_scales"):
            np.testing.assert_array_equal(cache[name].numpy().view(np.uint32),
                                          cache_whole[name].numpy()[first:first + count].view(np.uint32), err_msg=name)
        np.testing.assert_array_equal(cache["a_sums"].numpy(), cache_whole["a_sums"].numpy()[shard.row_begin // 64:(shard.row_begin + shard.rows) // 64])
        op.close()
    assert torch.equal(c_parts.view(torch.int32), c_whole.view(torch.int32))
    # the Python host's merge (world-1 gather per band) ...
    from ft_gemm_b200 import sharding
    merged = sharding._unpack([sharding._pack(rep, shard) for rep, shard in reports])
    # ... and the C-ABI's rebase + merge give the records of the unsharded run
    lib = ftg.load()
    from ft_gemm_b200 import _abi
    carr = (_abi.FtReport * bands)()
    for i, (rep, shard) in enumerate(reports):
        carr[i].status, carr[i].bad_tiles, carr[i].corrected_tiles = rep.status, rep.bad_tiles, rep.corrected_tiles
        carr[i].multi_fault_tiles, carr[i].n_records = rep.multi_fault_tiles, len(rep.records)
        for j, r in enumerate(rep.records):
            carr[i].records[j] = _abi.FtTileRecord(r.tile, r.bad_row_count, r.bad_col_count, r.bad_row, r.bad_col, r.row_delta, r.col_delta, r.corrected)
        assert lib.ft_gemm_report_rebase(ctypes.byref(carr[i]), tile_cols, shard.tile_row_offset) == 0
    total = _abi.FtReport()
    assert lib.ft_gemm_report_merge(carr, bands, ctypes.byref(total)) == 0
    key = lambda r: (r.tile, r.bad_row_count, r.bad_col_count, r.bad_row, r.bad_col, np.float32(r.row_delta).view(np.uint32),
                     np.float32(r.col_delta).view(np.uint32), r.corrected)
    want = [key(r) for r in rep_whole.records]
    assert [key(r) for r in merged.records] == want
    assert [key(total.records[i]) for i in range(total.n_records)] == want
    assert (merged.bad_tiles, merged.corrected_tiles, merged.multi_fault_tiles) == (rep_whole.bad_tiles, rep_whole.corrected_tiles,
                                                                                   rep_whole.multi_fault_tiles) == (3, 2, 1)
    assert (total.bad_tiles, total.corrected_tiles, total.multi_fault_tiles) == (3, 2, 1)
    whole.close()


def test_wait_timeout_is_reported_and_the_gpu_stays_usable():
    """A bounded wait that nothing satisfies gives up after its limit; the kernel leaves normally, _report returns
    FT_ERR_TIMEOUT, and the same handle then runs a clean GEMM.  The waiting kernel is the library's self-test hook: one
    thread, no copies, no tensor memory."""
    import time

    import ft_gemm_b200 as ftg
    from ft_gemm_b200 import _abi
    lib = ftg.load()
    m, n, k = 256, 256, 128
    a = ftg.generate_fp8((m, k), 1)
    b = ftg.generate_fp8((n, k), 2)
    op = ftg.AbftGemm(a, b)
    c = op.new_output()
    op.run(c)
    assert op.report().status == ftg.FT_OK
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    t0 = time.perf_counter()
    assert lib.ft_gemm_fp8_abft_selftest_wait(op.handle, 1000, stream) == ftg.FT_OK  # 1 ms
    rep = _abi.FtReport()
    code = lib.ft_gemm_fp8_abft_report(op.handle, ctypes.byref(rep))
    waited = time.perf_counter() - t0
    assert code == ftg.FT_ERR_TIMEOUT and rep.status == ftg.FT_ERR_TIMEOUT
    assert b"wait expired" in lib.ft_gemm_last_error()
    assert 0.001 <= waited < 1.0
    with pytest.raises(ftg.FtGemmError):
        op.report()  # the host mirror raises unless told that a time-out is expected
    assert op.report(allow_timeout=True).status == ftg.FT_ERR_TIMEOUT
    # the context is intact: the next run starts a clean report and computes the same product as before
    c2 = op.new_output()
    op.run(c2, [(0, 1, 2, 3.0)])
    rep2 = op.report()
    assert (rep2.status, rep2.bad_tiles, rep2.corrected_tiles) == (ftg.FT_OK, 1, 1)
    op.run(c2)
    assert op.report().status == ftg.FT_OK and torch.equal(c, c2)
    assert lib.ft_gemm_fp8_abft_selftest_wait(op.handle, 0, stream) == ftg.FT_ERR_INVALID
    op.close()


def test_wait_limit_option_is_validated_and_accepted():
    import ft_gemm_b200 as ftg
    from ft_gemm_b200 import _abi
    lib = ftg.load()
    a = ftg.generate_fp8((256, 128), 1)
    b = ftg.generate_fp8((256, 128), 2)
    options = _abi.FtOptions()
    lib.ft_options_default(ctypes.byref(options))
    assert options.wait_limit_us == 0
    handle = ctypes.c_void_p()
    options.wait_limit_us = -5
    args = (ctypes.c_void_p(a.data_ptr()), ctypes.c_void_p(b.data_ptr()), 256, 256, 128, ctypes.byref(options), None)
    assert lib.ft_gemm_fp8_abft_prepare(ctypes.byref(handle), *args) == ftg.FT_ERR_INVALID
    options.wait_limit_us = 500000  # half a second: far more than this launch needs
    assert lib.ft_gemm_fp8_abft_prepare(ctypes.byref(handle), *args) == ftg.FT_OK
    c = torch.empty((256, 256), dtype=torch.float32, device="cuda")
    assert lib.ft_gemm_fp8_abft_run(handle, ctypes.c_void_p(c.data_ptr()), None, 0, None) == ftg.FT_OK
    rep = _abi.FtReport()
    assert lib.ft_gemm_fp8_abft_report(handle, ctypes.byref(rep)) == ftg.FT_OK and rep.bad_tiles == 0
    lib.ft_gemm_fp8_abft_destroy(handle)
