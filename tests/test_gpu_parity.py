"""GPU parity tests: the CUDA path, called through the C-ABI, against the CPU
oracle on the same seeded inputs.  Integer/byte results and the expected-checksum
cache are compared bit for bit; the FP32 product within the stated bound
1e-5 * K * max|a| * max|b| of the oracle's FP32 result; checker decisions exactly."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

pytestmark = pytest.mark.gpu

SEED_A, SEED_B = 0x12345678, 0x9ABCDEF0


@pytest.fixture(scope="module")
def ftg():
    import ft_gemm_b200
    ft_gemm_b200.load()  # raises if the CUDA library is missing: no fallback
    assert torch.cuda.is_available()
    return ft_gemm_b200


def _inputs(ftg, oracle, m, n, k, dist="uniform"):
    if dist == "uniform":
        a = ftg.generate_fp8((m, k), SEED_A)
        b = ftg.generate_fp8((n, k), SEED_B)
    else:
        a = ftg.generate_fp8((m, k), SEED_A, "normal")
        b = ftg.generate_fp8((n, k), SEED_B, "normal")
    torch.cuda.synchronize()
    return a, b, a.cpu().numpy().ravel(), b.cpu().numpy().ravel()


def test_generator_bit_exact(ftg, oracle):
    for count, seed in [(1, 0), (1000, SEED_A), (1 << 20, SEED_B), (12345, 0xFFFFFFF0)]:
        got = ftg.generate_fp8(count, seed).cpu().numpy()
        np.testing.assert_array_equal(got, oracle.generate_uniform(count, seed))
    vals = oracle.decode(ftg.generate_fp8(1 << 20, 99, "normal").cpu().numpy())
    assert abs(vals.mean()) < 0.01 and 0.97 < vals.var() < 1.03
    # the normal generator agrees with the oracle's except where libm differs in the last bit
    same = ftg.generate_fp8(1 << 16, 7, "normal").cpu().numpy() == oracle.generate_normal(1 << 16, 7)
    assert same.mean() > 0.999


@pytest.mark.parametrize("m,n,k", [(128, 256, 128), (256, 512, 384), (384, 256, 2048), (1024, 1024, 1024),
                                   (128, 200, 96), (256, 320, 160), (384, 1000, 416), (128, 7, 32),  # boundary tiles in N
                                   (200, 136, 96), (1, 1, 16), (330, 257, 48), (65, 300, 272),  # and in M
                                   (128, 256, 100), (77, 50, 7), (300, 300, 1)])  # any K: zero-padded copies inside the handle
def test_expected_cache_bit_exact(ftg, oracle, m, n, k):
    """exact_prepare: CUDA-core kernels in the reference's summation order."""
    a, b, ah, bh = _inputs(ftg, oracle, m, n, k)
    op = ftg.AbftGemm(a, b, exact_prepare=True)
    got = op.cache()
    want = oracle.expected(ah, bh, m, n, k)
    for name in ("a_sums", "a_magnitudes", "b_sums", "b_magnitudes", "expected_rows", "expected_cols", "row_scales",
                 "col_scales"):
        np.testing.assert_array_equal(got[name].numpy().view(np.uint32), want[name].view(np.uint32), err_msg=name)
    op.close()


@pytest.mark.parametrize("m,n,k,dist", [(128, 256, 128, "uniform"), (256, 512, 384, "normal"), (384, 2304, 2048, "normal"),
                                        (1024, 1024, 1024, "uniform"), (128, 200, 96, "uniform"), (384, 1000, 416, "normal"),
                                        (128, 7, 32, "uniform"), (4352, 64, 160, "normal"), (200, 136, 96, "uniform"), (1, 1, 16, "uniform"),
                                        (330, 257, 48, "normal"), (2500, 300, 272, "uniform")])
def test_expected_cache_tensor_core_prepare(ftg, oracle, m, n, k, dist):
    """Default prepare: band sums as exact E4M3 digit planes times the operand on the tensor cores.  The band sums stay
    bit-exact; the checksums equal the reference's up to FP32 accumulation order (bound: 1e-6 of the magnitude sum)."""
    a, b, ah, bh = _inputs(ftg, oracle, m, n, k, dist)
    op = ftg.AbftGemm(a, b)
    got = op.cache()
    assert op.report().status == 0
    want = oracle.expected(ah, bh, m, n, k)
    for name in ("a_sums", "a_magnitudes", "b_sums", "b_magnitudes"):
        np.testing.assert_array_equal(got[name].numpy().view(np.uint32), want[name].view(np.uint32), err_msg=name)
    for value, scale in (("expected_rows", "row_scales"), ("expected_cols", "col_scales")):
        bound = 1e-6 * want[scale] + 1e-7
        assert (np.abs(got[value].numpy() - want[value]) <= bound).all(), value
        assert (np.abs(got[scale].numpy() - want[scale]) <= bound).all(), scale
    # refreshing one side only reuses the other side's digit planes
    op.refresh(a_changed=True, b_changed=False)
    again = op.cache()
    for name in got:
        np.testing.assert_array_equal(again[name].numpy().view(np.uint32), got[name].numpy().view(np.uint32), err_msg=name)
    op.close()


@pytest.mark.parametrize("m,n,k,dist", [(128, 256, 128, "uniform"), (256, 512, 384, "uniform"), (512, 768, 1024, "normal"),
                                        (1024, 1024, 1024, "normal"), (2048, 256, 4096, "uniform"),
                                        # boundary tiles in N, K not a multiple of the 128-wide K block (src/s3:144-154)
                                        (128, 200, 96, "uniform"), (256, 1000, 416, "normal"), (512, 64, 32, "uniform"),
                                        (384, 320, 2080, "uniform"), (256, 129, 224, "normal"),
                                        # boundary tiles in M as well, K a multiple of 16 only (src/s0:143-144 takes any shape)
                                        (200, 136, 96, "uniform"), (1, 1, 16, "uniform"), (330, 257, 48, "normal"),
                                        (1000, 1000, 1008, "normal"), (257, 64, 16, "uniform"),
                                        (128, 256, 100, "uniform"), (77, 50, 7, "normal"), (300, 300, 1, "uniform")])  # any K
def test_gemm_and_clean_check(ftg, oracle, m, n, k, dist):
    a, b, ah, bh = _inputs(ftg, oracle, m, n, k, dist)
    op = ftg.AbftGemm(a, b)
    c = op.new_output()
    op.run(c)
    rep = op.report()
    want = oracle.gemm_f32(ah, bh, m, n, k)
    bound = 1e-5 * k * float(np.abs(oracle.decode(ah)).max()) * float(np.abs(oracle.decode(bh)).max())
    err = np.abs(c.cpu().numpy() - want).max()
    assert err <= bound, (err, bound)
    assert (rep.status, rep.bad_tiles, rep.corrected_tiles, rep.multi_fault_tiles) == (0, 0, 0, 0)
    assert rep.max_clean_ratio < 0.5
    # the oracle's checker on the GPU's own product agrees that it is clean
    _, s, _ = oracle.abft_check(c.cpu().numpy(), m, n, oracle.expected(ah, bh, m, n, k))
    assert s.bad_tiles == 0
    op.close()


def _compare_decisions(ftg, oracle, op, c_clean, cache, m, n, faults, abs_tol=1e-2, rel_tol=2e-5):
    c = op.new_output()
    op.run(c, faults)
    rep = op.report()
    want_c, s, recs = oracle.abft_check(c_clean, m, n, cache, abs_tol=abs_tol, rel_tol=rel_tol, faults=faults)
    assert s.min_margin > 1e-3, "a decision sits on the threshold; pick another fault"
    assert (rep.bad_tiles, rep.corrected_tiles, rep.multi_fault_tiles) == (s.bad_tiles, s.corrected_tiles, s.multi_fault_tiles)
    assert [r.tile for r in rep.records] == [r.tile for r in recs]
    got_c = c.cpu().numpy()
    corrected_idx = []
    for g, w in zip(rep.records, recs):
        assert (g.bad_row_count, g.bad_col_count, g.corrected) == (w.bad_row_count, w.bad_col_count, w.corrected)
        if w.bad_row_count == 1:
            assert g.bad_row == w.bad_row
            if op.exact_prepare:
                assert g.row_delta == w.row_delta  # row sums use the oracle's order: bit-exact
            else:
                assert g.row_delta == pytest.approx(w.row_delta, abs=2e-3)
        if w.bad_col_count == 1:
            assert g.bad_col == w.bad_col and g.col_delta == pytest.approx(w.col_delta, abs=2e-3)
        if w.corrected:
            tile_cols = -(-n // 64)
            corrected_idx.append(((w.tile % tile_cols) * 64 + w.bad_col, (w.tile // tile_cols) * 64 + w.bad_row))
    mask = np.ones_like(got_c, dtype=bool)
    for col, row in corrected_idx:
        mask[col, row] = False
        assert got_c[col, row] == pytest.approx(want_c[col, row], abs=2e-3)
    np.testing.assert_array_equal(got_c[mask], want_c[mask])  # everything but the corrected elements is bit-identical
    return rep


@pytest.mark.parametrize("exact_prepare", [True, False])
def test_fault_decisions_match_oracle(ftg, oracle, exact_prepare):
    m, n, k = 256, 512, 512
    a, b, ah, bh = _inputs(ftg, oracle, m, n, k)
    op = ftg.AbftGemm(a, b, exact_prepare=exact_prepare)
    c = op.new_output()
    op.run(c)
    assert op.report().bad_tiles == 0
    c_clean = c.cpu().numpy()
    cache = oracle.expected(ah, bh, m, n, k)
    tile_cols = n // 64
    singles = []
    # every TMEM lane quarter (rows 0-31, 32-63 of both row bands), every 64-column group, both halves of a group
    for tile_row in range(4):
        for tile_col in range(tile_cols):
            t = tile_row * tile_cols + tile_col
            singles.append((t, (7 * t) % 64, (11 * t + 3) % 64, 3.0 + t))
    singles += [(0, 0, 0, -1.5), (5, 63, 63, 200.0), (9, 31, 32, -64.0), (31, 32, 31, 0.75)]
    for fault in singles:
        rep = _compare_decisions(ftg, oracle, op, c_clean, cache, m, n, [fault])
        assert (rep.bad_tiles, rep.corrected_tiles) == (1, 1)
        assert (rep.records[0].bad_row, rep.records[0].bad_col) == (fault[1], fault[2])
    # multi-fault tiles are reported and left alone
    multis = [[(2, 1, 2, 3.0), (2, 5, 7, -2.5)], [(2, 3, 1, 4.0), (2, 3, 9, 6.0)], [(2, 4, 2, 5.0), (2, 4, 11, -5.0)],
              [(6, 10, 40, 9.0), (6, 50, 40, 9.0)], [(3, 1, 1, 2.0), (3, 2, 2, 2.0), (3, 3, 3, 2.0), (3, 40, 60, 2.0)]]
    for faults in multis:
        rep = _compare_decisions(ftg, oracle, op, c_clean, cache, m, n, faults)
        assert (rep.bad_tiles, rep.corrected_tiles, rep.multi_fault_tiles) == (1, 0, 1)
    # faults in different tiles are corrected independently
    rep = _compare_decisions(ftg, oracle, op, c_clean, cache, m, n, [(0, 1, 1, 9.0), (17, 2, 2, -9.0), (30, 63, 0, 4.0)])
    assert (rep.bad_tiles, rep.corrected_tiles) == (3, 3)
    # a fault under the threshold is invisible, as in the reference
    rep = _compare_decisions(ftg, oracle, op, c_clean, cache, m, n, [(4, 8, 8, 2e-3)])
    assert rep.bad_tiles == 0
    # row/col beyond 63 are clamped (src/s4_random_fault_campaign.cu:464-465)
    c2 = op.new_output()
    op.run(c2, [(1, 99, 70, 5.0)])
    rec = op.report().records[0]
    assert (rec.bad_row, rec.bad_col, rec.corrected) == (63, 63, 1)
    op.close()


def test_exhaustive_single_fault_sweep_one_tile(ftg, oracle):
    """Every (row, col) of one ABFT tile at 256^3: detected, located, corrected."""
    m = n = k = 256
    a, b, ah, bh = _inputs(ftg, oracle, m, n, k)
    op = ftg.AbftGemm(a, b)
    c_clean = op.new_output()
    op.run(c_clean)
    assert op.report().bad_tiles == 0
    c = op.new_output()
    tile = 6  # tile_row 1, tile_col 2
    worst = 0.0
    for row in range(64):
        for col in range(64):
            value = (1.0 + (row * 64 + col) % 97) * (1.0 if (row + col) % 2 else -1.0)
            op.run(c, [(tile, row, col, value)])
            rep = op.report()
            assert (rep.bad_tiles, rep.corrected_tiles) == (1, 1), (row, col, rep)
            rec = rep.records[0]
            assert (rec.tile, rec.bad_row, rec.bad_col) == (tile, row, col)
            worst = max(worst, float((c - c_clean).abs().max()))
    assert worst < 1e-3
    op.close()


def test_tolerance_is_a_run_time_parameter(ftg, oracle):
    m, n, k = 128, 256, 256
    a, b, ah, bh = _inputs(ftg, oracle, m, n, k)
    op = ftg.AbftGemm(a, b)
    c = op.new_output()
    op.run(c, [(0, 3, 3, 0.5)])
    assert op.report().corrected_tiles == 1
    op.set_tolerance(1.0, 2e-5)  # fault now under the absolute tolerance
    op.run(c, [(0, 3, 3, 0.5)])
    assert op.report().bad_tiles == 0
    op.close()


def test_repeat_runs_are_bit_identical(ftg, oracle):
    m, n, k = 512, 512, 1024
    a, b, _, _ = _inputs(ftg, oracle, m, n, k, "normal")
    op = ftg.AbftGemm(a, b)
    first = op.new_output()
    op.run(first, [(3, 5, 6, 17.0)])
    rep0 = op.report()
    for _ in range(20):
        c = op.new_output()
        op.run(c, [(3, 5, 6, 17.0)])
        rep = op.report()
        assert torch.equal(c, first)
        assert (rep.bad_tiles, rep.corrected_tiles, rep.records[0].row_delta, rep.records[0].col_delta) == \
               (rep0.bad_tiles, rep0.corrected_tiles, rep0.records[0].row_delta, rep0.records[0].col_delta)
    op.close()


def test_small_grid_and_refresh(ftg, oracle):
    """A capped grid walks many tiles per CTA (both TMEM accumulators, ring wrap-around); refresh after A changes."""
    m, n, k = 1024, 1024, 384
    a, b, ah, bh = _inputs(ftg, oracle, m, n, k)
    op = ftg.AbftGemm(a, b, sm_limit=3)
    c = op.new_output()
    op.run(c)
    assert op.report().bad_tiles == 0
    np.testing.assert_allclose(c.cpu().numpy(), oracle.gemm_f32(ah, bh, m, n, k), atol=1e-5 * k)
    a.copy_(ftg.generate_fp8((m, k), 4242))
    op.run(c)
    assert op.report().bad_tiles > 0  # stale cache: the checker notices that A changed
    op.refresh(a_changed=True, b_changed=False)
    op.run(c)
    assert op.report().bad_tiles == 0
    np.testing.assert_allclose(c.cpu().numpy(), oracle.gemm_f32(a.cpu().numpy().ravel(), bh, m, n, k), atol=1e-5 * k)
    op.close()


def test_host_buffer_entry_point(ftg, oracle):
    m, n, k = 256, 256, 256
    ah = oracle.generate_uniform(m * k, SEED_A)
    bh = oracle.generate_uniform(n * k, SEED_B)
    a_pin = torch.from_numpy(ah.reshape(m, k)).pin_memory()
    b_pin = torch.from_numpy(bh.reshape(n, k)).pin_memory()
    c_pin = torch.empty((n, m), dtype=torch.float32).pin_memory()
    host = ftg.HostAbftGemm(m, n, k)
    rep = host(a_pin, b_pin, c_pin)
    assert rep.bad_tiles == 0
    np.testing.assert_allclose(c_pin.numpy(), oracle.gemm_f32(ah, bh, m, n, k), atol=1e-5 * k)
    rep = host(a_pin, b_pin, c_pin, faults=[(1, 2, 3, 8.0)])
    assert (rep.bad_tiles, rep.corrected_tiles) == (1, 1)
    np.testing.assert_allclose(c_pin.numpy(), oracle.gemm_f32(ah, bh, m, n, k), atol=1e-3)
    host.close()


def test_fault_decisions_in_boundary_tiles(ftg, oracle):
    """N = 200: the last tile column holds 8 valid columns; a fault column past them is clamped (campaign:464-466)."""
    for m, n, k in [(256, 200, 160), (128, 449, 96), (200, 200, 80)]:
        a, b, ah, bh = _inputs(ftg, oracle, m, n, k)
        op = ftg.AbftGemm(a, b)
        c = op.new_output()
        op.run(c)
        assert op.report().bad_tiles == 0
        c_clean = c.cpu().numpy()
        cache = oracle.expected(ah, bh, m, n, k)
        tile_cols = -(-n // 64)
        valid_last = n - (tile_cols - 1) * 64
        last = tile_cols - 1
        tile_rows = -(-m // 64)
        valid_rows_last = m - (tile_rows - 1) * 64
        bottom = (tile_rows - 1) * tile_cols  # first tile of the last tile row
        for fault in [(last, 5, 0, 7.0), (tile_cols + last, 40, valid_last - 1, -9.0), (last, 63, 63, 12.0), (1, 2, 3, 4.0),
                      (bottom, 63, 1, 6.0), (bottom + last, 0, 63, -8.0)]:
            rep = _compare_decisions(ftg, oracle, op, c_clean, cache, m, n, [fault])
            assert (rep.bad_tiles, rep.corrected_tiles) == (1, 1)
            want_col = min(fault[2], valid_last - 1) if fault[0] % tile_cols == last else fault[2]
            want_row = min(fault[1], valid_rows_last - 1) if fault[0] // tile_cols == tile_rows - 1 else fault[1]
            assert (rep.records[0].bad_row, rep.records[0].bad_col) == (want_row, want_col)
        rep = _compare_decisions(ftg, oracle, op, c_clean, cache, m, n, [(last, 1, 0, 5.0), (last, 9, 0, 5.0)])
        assert (rep.bad_tiles, rep.corrected_tiles, rep.multi_fault_tiles) == (1, 0, 1)
        # the window form accepts a short last column block
        parts = torch.full_like(c, float("nan"))
        tile_m = 256 if m % 256 == 0 else 128
        op.run_window(parts, 0, min(m, tile_m), 0, n)
        if m > tile_m:
            op.run_window(parts, tile_m, m - tile_m, 0, n, zero_report=False)
        assert torch.equal(parts, c)
        op.close()


def test_windows_cover_the_product(ftg, oracle):
    """Four window launches into one report give the same C, bit for bit, and the same decisions as one full launch."""
    for m, n, k, single in [(1024, 1024, 256, 0), (384, 512, 128, 1)]:
        a = ftg.generate_fp8((m, k), SEED_A)
        b = ftg.generate_fp8((n, k), SEED_B)
        op = ftg.AbftGemm(a, b, single_cta=bool(single))
        whole = op.new_output()
        fault = [((5 * (n // 64)) + 7, 9, 11, 6.0)]  # rows 320.., columns 448..
        op.run(whole, fault)
        want = op.report()
        assert (want.bad_tiles, want.corrected_tiles) == (1, 1)
        parts = torch.full_like(whole, float("nan"))
        rm = 512 if not single else 128
        windows = [(0, rm, 0, 256), (rm, m - rm, 0, 256), (0, rm, 256, n - 256), (rm, m - rm, 256, n - 256)]
        for i, (r0, rows, c0, cols) in enumerate(windows):
            op.run_window(parts, r0, rows, c0, cols, fault, zero_report=(i == 0))
            got = op.report()
            filled = ~torch.isnan(parts)
            assert int(filled.sum()) == sum(w[1] * w[3] for w in windows[:i + 1])  # nothing outside the windows is written
        assert torch.equal(parts, whole)
        assert (got.bad_tiles, got.corrected_tiles, got.multi_fault_tiles) == (1, 1, 0)
        assert (got.records[0].tile, got.records[0].bad_row, got.records[0].bad_col) == (fault[0][0], 9, 11)
        with pytest.raises(ftg.FtGemmError):
            op.run_window(parts, 64, 128, 0, 256)  # not on a tile boundary
        with pytest.raises(ftg.FtGemmError):
            op.run_window(parts, 0, m, 256, n)  # reaches past N
        op.close()


def test_host_entry_point_pipelined(ftg, oracle):
    """Second and later calls on a reused handle take the chunked three-stream form: same C as the device-buffer path."""
    for m, n, k in [(2048, 2048, 256), (1024, 512, 128), (768, 768, 128)]:  # 8, 2 and 1 chunk(s)
        ah = oracle.generate_uniform(m * k, SEED_A)
        bh = oracle.generate_uniform(n * k, SEED_B)
        a_pin = torch.from_numpy(ah.reshape(m, k)).pin_memory()
        b_pin = torch.from_numpy(bh.reshape(n, k)).pin_memory()
        c_first = torch.empty((n, m), dtype=torch.float32).pin_memory()
        c_pipe = torch.full((n, m), float("nan"), dtype=torch.float32).pin_memory()
        host = ftg.HostAbftGemm(m, n, k)
        assert host(a_pin, b_pin, c_first).bad_tiles == 0  # creates the handle: plain form
        rep = host(a_pin, b_pin, c_pipe)  # pipelined form
        assert rep.bad_tiles == 0
        assert torch.equal(c_pipe, c_first)
        tile = (m // 64 - 1) * (n // 64) + 1
        rep = host(a_pin, b_pin, c_pipe, faults=[(tile, 63, 0, -12.0), (0, 0, 0, 5.0)])
        assert (rep.bad_tiles, rep.corrected_tiles, len(rep.records)) == (2, 2, 2)
        assert [r.tile for r in rep.records] == [0, tile]
        np.testing.assert_allclose(c_pipe.numpy(), c_first.numpy(), atol=1e-3)
        dev = ftg.AbftGemm(a_pin.cuda(), b_pin.cuda())
        c_dev = dev.new_output()
        dev.run(c_dev)
        assert torch.equal(c_dev.cpu(), c_first)
        dev.close()
        host.close()


def test_quantize_a_fused_with_band_sums(ftg, oracle):
    """A produced on the device from FP32 / BF16 / FP16 with its band sums in the same pass: the bytes equal the oracle's
    quantiser and the cache equals a fresh prepare on those bytes, bit for bit."""
    m, n, k = 256, 320, 416
    g = torch.Generator(device="cpu").manual_seed(31)
    src32 = torch.randn((m, k), generator=g) * 3.0
    src32[0, :8] = torch.tensor([0.0, -0.0, 1e6, -1e6, 17.0, 19.0, 2.0 ** -10, 447.9])
    b = ftg.generate_fp8((n, k), SEED_B)
    bh = b.cpu().numpy().ravel()
    for dtype, scale in [(torch.float32, 1.0), (torch.bfloat16, 0.5), (torch.float16, 2.0), (torch.float32, 0.013)]:
        src = src32.to(dtype)
        a = torch.zeros((m, k), dtype=torch.uint8, device="cuda")
        op = ftg.AbftGemm(a, b, exact_prepare=True)  # prepared on a placeholder A, as a serving loop would do once
        op.quantize_a(src.cuda(), scale)
        want_a = oracle.quantize(src.float().numpy().ravel(), scale)
        np.testing.assert_array_equal(a.cpu().numpy().ravel(), want_a)
        got = op.cache()
        want = oracle.expected(want_a, bh, m, n, k)
        for name in ("a_sums", "a_magnitudes", "b_sums", "b_magnitudes", "expected_rows", "expected_cols", "row_scales", "col_scales"):
            np.testing.assert_array_equal(got[name].numpy().view(np.uint32), want[name].view(np.uint32), err_msg=name)
        c = op.new_output()
        op.run(c, [(3, 4, 5, 50.0)])
        rep = op.report()
        assert (rep.bad_tiles, rep.corrected_tiles) == (1, 1)
        np.testing.assert_allclose(c.cpu().numpy(), oracle.gemm_f32(want_a, bh, m, n, k), atol=2e-2)
        with pytest.raises(ValueError):
            op.quantize_a(src.cuda()[:128], scale)
        op.close()


def test_padded_k_refresh_and_host_call(ftg, oracle):
    """K = 100: the handle works on zero-padded copies; refresh must re-copy the operand that changed."""
    m, n, k = 128, 192, 100
    a, b, ah, bh = _inputs(ftg, oracle, m, n, k)
    op = ftg.AbftGemm(a, b, exact_prepare=True)
    c = op.new_output()
    a2 = ftg.generate_fp8((m, k), 777)
    a.copy_(a2)
    op.refresh(a_changed=True, b_changed=False)
    a2h = a2.cpu().numpy().ravel()
    want = oracle.expected(a2h, bh, m, n, k)
    got = op.cache()
    for name in want:
        np.testing.assert_array_equal(got[name].numpy().view(np.uint32), want[name].view(np.uint32), err_msg=name)
    op.run(c, [(1, 2, 3, 9.0)])
    rep = op.report()
    assert (rep.bad_tiles, rep.corrected_tiles) == (1, 1)
    np.testing.assert_allclose(c.cpu().numpy(), oracle.gemm_f32(a2h, bh, m, n, k), atol=1e-3)
    with pytest.raises(ftg.FtGemmError):
        op.quantize_a(torch.zeros((m, k), device="cuda"))  # the fused producer needs K % 16 == 0
    op.close()
    a_pin, b_pin = a2.cpu().pin_memory(), b.cpu().pin_memory()
    c_pin = torch.empty((n, m), dtype=torch.float32).pin_memory()
    host = ftg.HostAbftGemm(m, n, k)
    for _ in range(2):  # the second call reuses the handle
        assert host(a_pin, b_pin, c_pin).bad_tiles == 0
        np.testing.assert_allclose(c_pin.numpy(), oracle.gemm_f32(a2h, bh, m, n, k), atol=1e-5 * k)
    a_pin.copy_(ftg.generate_fp8((m, k), 778).cpu())
    assert host(a_pin, b_pin, c_pin, prepare=True).bad_tiles == 0  # new A: prepare again, or the stale cache fires
    np.testing.assert_allclose(c_pin.numpy(), oracle.gemm_f32(a_pin.numpy().ravel(), bh, m, n, k), atol=1e-5 * k)
    host.close()


def test_invalid_arguments_are_rejected(ftg):
    a = torch.zeros((128, 128), dtype=torch.uint8, device="cuda")
    b = torch.zeros((256, 128), dtype=torch.uint8, device="cuda")
    with pytest.raises(ftg.FtGemmError) as e:
        ftg.AbftGemm(a[:0].contiguous(), b)  # an empty operand: the shape must be positive
    assert e.value.code == ftg.FT_ERR_INVALID
    op = ftg.AbftGemm(a, b)
    c = op.new_output()
    with pytest.raises(ftg.FtGemmError):
        op.run(c, [(10 ** 6, 0, 0, 1.0)])  # tile id out of range
    op.close()


def test_campaign_config1_normal_1024(ftg, oracle):
    """The 1024^3 configuration: N(0,1) inputs, one fault U[1,256] per trial from the campaign chain."""
    m = n = k = 1024
    a, b, ah, bh = _inputs(ftg, oracle, m, n, k, "normal")
    op = ftg.AbftGemm(a, b)
    c_clean = op.new_output()
    op.run(c_clean)
    assert op.report().bad_tiles == 0
    cache = oracle.expected(ah, bh, m, n, k)
    clean_np = c_clean.cpu().numpy()
    draws, _ = oracle.campaign(12345, 40, op.tile_count)
    c = op.new_output()
    for tile, row, col, value, _, _ in draws:
        rep = _compare_decisions(ftg, oracle, op, clean_np, cache, m, n, [(tile, row, col, value)])
        assert (rep.bad_tiles, rep.corrected_tiles) == (1, 1)
    op.close()


def test_full_size_properties_4096(ftg, oracle):
    """Size-independent properties at 4096^3 (README headline shape): sampled FP64 check, clean checker,
    tile sums of C equal the sums of the cached expected checksums (linearity), campaign faults corrected."""
    m = n = k = 4096
    a, b, _, _ = _inputs(ftg, oracle, m, n, k, "normal")
    op = ftg.AbftGemm(a, b)
    c = op.new_output()
    op.run(c)
    rep = op.report()
    assert rep.bad_tiles == 0 and rep.max_clean_ratio < 0.5
    # sampled rows/cols against FP64 on the host
    rows = list(range(0, m, m // 8))
    cols = list(range(0, n, n // 8))
    af = torch.from_numpy(oracle.decode(a[rows].cpu().numpy())).double()
    bf = torch.from_numpy(oracle.decode(b[cols].cpu().numpy())).double()
    ref = af @ bf.T
    got = c[cols][:, rows].T.cpu().double()
    bound = 1e-5 * k * float(af.abs().max()) * float(bf.abs().max())
    assert float((got - ref).abs().max()) <= bound
    # checksum of checksums per ABFT tile
    cache = op.cache()
    tiles = c.view(n // 64, 64, m // 64, 64).double().sum(dim=(1, 3)).T.reshape(-1).cpu()  # [tile_row, tile_col]
    np.testing.assert_allclose(tiles.numpy(), cache["expected_rows"].double().sum(1).numpy(), atol=0.5)
    np.testing.assert_allclose(tiles.numpy(), cache["expected_cols"].double().sum(1).numpy(), atol=0.5)
    c_fault = op.new_output()
    draws, _ = oracle.campaign(12345, 25, op.tile_count)
    tile_cols = n // 64
    for tile, row, col, value, _, _ in draws:
        op.run(c_fault, [(tile, row, col, value)])
        rep = op.report()
        gr, gc = (tile // tile_cols) * 64 + row, (tile % tile_cols) * 64 + col
        if abs(value) > 8.0:  # above the default threshold at this K
            assert (rep.bad_tiles, rep.corrected_tiles) == (1, 1)
            assert abs(float(c_fault[gc, gr] - c[gc, gr])) < 0.05
    op.close()
