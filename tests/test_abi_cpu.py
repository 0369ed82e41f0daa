"""CPU checks of the drop-in boundary: the shared library loads without a GPU,
exports every symbol include/ft_gemm.h declares, and rejects bad arguments
before touching CUDA.  No compute is launched here."""
import ctypes
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADERS = [os.path.join(ROOT, "include", name) for name in ("ft_gemm.h", "ft_attention.h", "ft_gemm_softmax.h")]


def declared_functions():
    names = set()
    for header in HEADERS:
        text = re.sub(r"/\*.*?\*/", "", open(header).read(), flags=re.S)
        names.update(re.findall(r"\b(ft_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_header_declares_the_north_star_entry_points():
    names = declared_functions()
    for required in ("ft_gemm_fp8_abft_prepare", "ft_gemm_fp8_abft_run", "ft_gemm_fp8_abft_report", "ft_gemm_fp8_abft_destroy",
                     "ft_attention_fp16_abft_prepare", "ft_attention_fp16_abft_run", "ft_attention_fp16_abft_report"):
        assert required in names


def test_library_exports_every_declared_symbol(lib_path):
    lib = ctypes.CDLL(lib_path)
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} is declared in ft_gemm.h but not exported"
    out = subprocess.run(["nm", "-D", "--defined-only", lib_path], capture_output=True, text=True, check=True).stdout
    for name in declared_functions():
        assert re.search(rf"\bT {name}\b", out), name


def test_header_compiles_as_c(tmp_path):
    src = tmp_path / "t.c"
    src.write_text('#include "ft_gemm.h"\n#include "ft_attention.h"\n#include "ft_gemm_softmax.h"\nint main(void){ft_options o; ft_report r; ft_attn_report a; ft_gs_report g; (void)o; (void)r; (void)a; (void)g; return FT_OK;}\n')
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), "-c", str(src), "-o",
                    str(tmp_path / "t.o")], check=True)


def test_python_struct_sizes_match_the_header(tmp_path, lib_path):
    src = tmp_path / "s.c"
    src.write_text('#include <stdio.h>\n#include "ft_gemm.h"\nint main(void){printf("%zu %zu %zu %zu %zu\\n", sizeof(ft_options),'
                   ' sizeof(ft_fault), sizeof(ft_tile_record), sizeof(ft_report), sizeof(ft_cache_view)); return 0;}\n')
    exe = tmp_path / "s"
    subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)], check=True)
    sizes = [int(x) for x in subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split()]
    from ft_gemm_b200 import _abi
    assert sizes == [ctypes.sizeof(_abi.FtOptions), ctypes.sizeof(_abi.FtFault), ctypes.sizeof(_abi.FtTileRecord),
                     ctypes.sizeof(_abi.FtReport), ctypes.sizeof(_abi.FtCacheView)]


def test_argument_errors_without_a_gpu():
    import ft_gemm_b200 as ftg
    from ft_gemm_b200 import _abi
    lib = ftg.load()
    assert lib.ft_gemm_abi_version() == 1
    opts = _abi.FtOptions()
    lib.ft_options_default(ctypes.byref(opts))
    assert opts.abs_tol == pytest.approx(1e-2) and opts.rel_tol == pytest.approx(2e-5)  # src/s4:98-99
    handle = ctypes.c_void_p()
    fake = ctypes.c_void_p(0x1000)
    # the shape rule (any positive shape), checked before any CUDA call
    for m, n, k in [(0, 256, 128), (128, 0, 128), (-128, 256, 128), (128, 256, 0)]:
        rc = lib.ft_gemm_fp8_abft_prepare(ctypes.byref(handle), fake, fake, m, n, k, None, None)
        assert rc == ftg.FT_ERR_INVALID and b"positive shape" in lib.ft_gemm_last_error()
    assert lib.ft_gemm_fp8_abft_prepare(ctypes.byref(handle), None, fake, 128, 256, 128, None, None) == ftg.FT_ERR_INVALID
    assert lib.ft_gemm_fp8_abft_run(None, fake, None, 0, None) == ftg.FT_ERR_INVALID
    assert lib.ft_gemm_fp8_abft_report(None, None) == ftg.FT_ERR_INVALID
    assert lib.ft_gemm_fp8_abft_destroy(None) == ftg.FT_OK
    assert lib.ft_gemm_generate_fp8(fake, 16, 1, 7, 1.0, 1.0, None) == ftg.FT_ERR_INVALID


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from ft_gemm_b200 import _abi
    monkeypatch.setattr(_abi, "_lib", None)
    monkeypatch.setattr(_abi, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _abi.load()


def test_report_rebase_and_merge_are_host_functions():
    """The multi-GPU report plumbing of the C-ABI needs no device: tile ids of a band become ids of the whole product,
    the union keeps rank order, adds the counters and counts what does not fit."""
    import ft_gemm_b200 as ftg
    from ft_gemm_b200 import _abi
    lib = ftg.load()
    tile_cols = 8
    shards = (_abi.FtReport * 3)()
    for rank in range(3):
        r = shards[rank]
        r.bad_tiles, r.corrected_tiles, r.multi_fault_tiles = rank + 1, rank, 1
        r.n_records = 30
        r.max_clean_ratio = 0.1 * (rank + 1)
        r.prepare_ms = 1.0 + rank
        for i in range(30):
            r.records[i] = _abi.FtTileRecord(i, 1, 1, i, i + 1, 0.5, 0.25, 1)
        assert lib.ft_gemm_report_rebase(ctypes.byref(r), tile_cols, 4 * rank) == ftg.FT_OK
        assert [r.records[i].tile for i in range(3)] == [32 * rank + i for i in range(3)]
    shards[1].status = ftg.FT_ERR_TIMEOUT
    total = _abi.FtReport()
    assert lib.ft_gemm_report_merge(shards, 3, ctypes.byref(total)) == ftg.FT_OK
    assert (total.status, total.bad_tiles, total.corrected_tiles, total.multi_fault_tiles) == (ftg.FT_ERR_TIMEOUT, 6, 3, 3)
    assert total.n_records == _abi.FT_MAX_RECORDS and total.records_dropped == 90 - _abi.FT_MAX_RECORDS
    assert [total.records[i].tile for i in (0, 29, 30, 59, 60, 63)] == [0, 29, 32, 61, 64, 67]
    assert abs(total.max_clean_ratio - 0.3) < 1e-6 and total.prepare_ms == 3.0
    assert lib.ft_gemm_report_merge(shards, 0, ctypes.byref(total)) == ftg.FT_ERR_INVALID
    assert lib.ft_gemm_report_rebase(None, tile_cols, 0) == ftg.FT_ERR_INVALID
