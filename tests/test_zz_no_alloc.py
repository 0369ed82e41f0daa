"""The allocation-free prepare entry point against the allocating one.

ft_gemm_fp8_abft_expected_noalloc serves callers that cannot call cudaMalloc when
they need fresh expected checksums (a serving loop under a framework allocator
that owns the device memory).  Its four outputs must equal, bit for bit, the cache
that ft_gemm_fp8_abft_prepare builds for the same operands -- on two calls in a
row, because the calls share one built-in scratch array that keeps the previous
call's contents.  Ragged shapes (M or N not a multiple of 64) size their outputs
with whole boundary tiles, ceil(M/64) * ceil(N/64) * 64 floats each."""
import ctypes

import numpy as np
import pytest

torch = pytest.importorskip("torch")

pytestmark = pytest.mark.gpu


def _noalloc(ftg, a, b):
    lib = ftg.load()
    m, k = a.shape
    n = b.shape[0]
    checks = ((m + 63) // 64) * ((n + 63) // 64) * 64
    guard = 256  # floats past the documented size: must stay untouched
    outs = [torch.full((checks + guard,), float("nan"), dtype=torch.float32, device="cuda") for _ in range(4)]
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.ft_gemm_fp8_abft_expected_noalloc(ctypes.c_void_p(a.data_ptr()), ctypes.c_void_p(b.data_ptr()), m, n, k,
                                               *[ctypes.c_void_p(t.data_ptr()) for t in outs], stream)
    assert rc == ftg.FT_OK, lib.ft_gemm_last_error()
    torch.cuda.synchronize()
    for t in outs:
        assert bool(torch.isnan(t[checks:]).all()), "the entry point wrote past ceil(M/64)*ceil(N/64)*64 floats"
    return dict(zip(("expected_rows", "expected_cols", "row_scales", "col_scales"), (t[:checks].cpu().numpy() for t in outs)))


def test_noalloc_prepare_matches_prepare_twice_in_a_row():
    import ft_gemm_b200 as ftg
    lib = ftg.load()
    assert torch.cuda.is_available()
    # two different shapes back to back: the second call finds the first call's band sums in the scratch
    # ragged shapes in between: boundary tiles in M, in N and in both
    shapes = [((512, 768, 1024), (11, 12)), ((256, 256, 384), (21, 22)), ((200, 136, 96), (41, 42)), ((100, 256, 128), (51, 52)),
              ((512, 768, 1024), (31, 32))]
    for (m, n, k), seeds in shapes:
        a = ftg.generate_fp8((m, k), seeds[0])
        b = ftg.generate_fp8((n, k), seeds[1])
        got = _noalloc(ftg, a, b)
        op = ftg.AbftGemm(a, b, exact_prepare=True)
        want = op.cache()
        for name, value in got.items():
            np.testing.assert_array_equal(value.view(np.uint32), want[name].numpy().ravel().view(np.uint32), err_msg=name)
        op.close()
    # one step beyond the largest shape the built-in scratch takes (8192^3: band sums = 16 MiB) is refused
    fake = ctypes.c_void_p(0x10000)
    rc = lib.ft_gemm_fp8_abft_expected_noalloc(fake, fake, 8192 + 128, 8192, 8192, fake, fake, fake, fake, None)
    assert rc == ftg.FT_ERR_INVALID and b"built-in array" in lib.ft_gemm_last_error()
    rc = lib.ft_gemm_fp8_abft_expected_noalloc(fake, fake, 100, 256, 120, fake, fake, fake, fake, None)
    assert rc == ftg.FT_ERR_INVALID


def test_noalloc_accepts_the_largest_shape():
    """8192^3 needs exactly the 16 MiB of built-in scratch: the call is accepted and its output equals the cache of the
    allocating entry point."""
    import ft_gemm_b200 as ftg
    m = n = k = 8192
    a = ftg.generate_fp8((m, k), 61)
    b = ftg.generate_fp8((n, k), 62)
    got = _noalloc(ftg, a, b)
    op = ftg.AbftGemm(a, b, exact_prepare=True)
    want = op.cache()
    for name, value in got.items():
        np.testing.assert_array_equal(value.view(np.uint32), want[name].numpy().ravel().view(np.uint32), err_msg=name)
    op.close()
