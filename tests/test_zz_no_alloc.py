"""The allocation-free column sum, called through its exported C symbol, matches the regular entry point."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from superscaler_b200.ops import native
    native.ext()
    lib = ctypes.CDLL(native.ext().__file__)
    fn = lib.ssb_colsum_bf16_static
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                   ctypes.c_void_p]
    lib.ssb_colsum_static_strerror.restype = ctypes.c_char_p
    lib.ssb_colsum_static_strerror.argtypes = [ctypes.c_int]
    return lib, fn


def test_static_colsum_matches_regular_two_calls_in_a_row():
    from superscaler_b200.ops import native
    ext = native.ext()
    lib, fn = _lib()
    torch.manual_seed(7)
    stream = torch.cuda.current_stream().cuda_stream
    for rows, n in [(4096, 2048), (1000, 514)]:           # second call in a row reuses the shared array
        a = torch.randn(rows, n, device="cuda").bfloat16()
        want = torch.empty(n, device="cuda", dtype=torch.float32)
        ext.colsum(a, want, False)
        got = torch.full((n,), 123.0, device="cuda", dtype=torch.float32)
        mem_before = torch.cuda.memory_allocated()
        rc = fn(a.data_ptr(), a.stride(0), got.data_ptr(), 0, rows, n, stream)
        assert rc == 0, lib.ssb_colsum_static_strerror(rc)
        assert torch.cuda.memory_allocated() == mem_before
        torch.cuda.synchronize()
        ref = a.float().sum(0)
        torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-4)
        torch.testing.assert_close(got, ref, rtol=1e-3, atol=5e-2)
        # accumulate on top of the previous result
        rc = fn(a.data_ptr(), a.stride(0), got.data_ptr(), 1, rows, n, stream)
        assert rc == 0
        torch.cuda.synchronize()
        torch.testing.assert_close(got, 2 * want, rtol=1e-5, atol=2e-4)


def test_static_colsum_rejects_oversize_and_bad_arguments():
    lib, fn = _lib()
    a = torch.zeros(8, 16, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros(16, device="cuda")
    assert fn(a.data_ptr(), 8194, out.data_ptr(), 0, 8, 8194, None) == 2       # beyond the fixed maximum
    assert b"8192" in lib.ssb_colsum_static_strerror(2)
    assert fn(a.data_ptr(), 16, out.data_ptr(), 0, 8, 15, None) == 1           # odd n
    assert fn(None, 16, out.data_ptr(), 0, 8, 16, None) == 1
    # a view that starts on an odd bf16 element (2-byte aligned) or an `out` off a 4-byte boundary: refused on the
    # host, nothing launched, `out` untouched
    out.fill_(5.0)
    assert fn(a.data_ptr() + 2, 16, out.data_ptr(), 0, 7, 14, None) == 1
    assert fn(a.data_ptr(), 16, out.data_ptr() + 2, 0, 8, 14, None) == 1
    assert b"aligned" in lib.ssb_colsum_static_strerror(1)
    torch.cuda.synchronize()
    assert bool((out == 5.0).all())
