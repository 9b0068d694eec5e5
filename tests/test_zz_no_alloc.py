"""The allocation-free entry point, called through its exported C symbol.

Some users of this library cannot allocate device memory where they need the
codec (plain C / ctypes callers without a tensor library, code inside regions
where the driver allocator must not be touched), so `lbc_no_alloc_roundtrip`
keeps its intermediate payload in a fixed array inside the library.  This test
loads the shared object with ctypes, exactly as such a caller would, and checks
two consecutive calls against the regular tensor-allocating path bit for bit
(the comparison the other codec tests use).  It lives in the file pytest
collects last so that a `-x` run has already exercised everything else.
"""

import ctypes

import pytest
import torch

from lowbit_comm_b200.config import CompressionConfig
from lowbit_comm_b200.ops import codec
from lowbit_comm_b200.ops.build import extension_path

pytestmark = pytest.mark.gpu

_DTYPE_CODE = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}


def _library():
    lib = ctypes.CDLL(str(extension_path()))
    lib.lbc_no_alloc_roundtrip.restype = ctypes.c_int
    lib.lbc_no_alloc_roundtrip.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
                                           ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong,
                                           ctypes.c_void_p]
    lib.lbc_no_alloc_error_string.restype = ctypes.c_char_p
    lib.lbc_no_alloc_error_string.argtypes = [ctypes.c_int]
    lib.lbc_no_alloc_max_numel.restype = ctypes.c_longlong
    lib.lbc_no_alloc_scratch_bytes.restype = ctypes.c_longlong
    return lib


def _existing_path(x, residual, cfg):
    """The regular entry points: payload in a torch-allocated buffer."""

    res = residual.clone()
    payload = codec.quantize_tensor(x, cfg, residual=res, prepared_out=res)
    out = torch.empty_like(x)
    assert codec.inplace_dequantize_reduce_mean_update_error_feedback([payload], res, out, res, cfg, reduce="mean")
    return out, res


def _call(lib, x, residual_in, out, residual_out, cfg):
    stream = torch.cuda.current_stream().cuda_stream
    return lib.lbc_no_alloc_roundtrip(
        _DTYPE_CODE[x.dtype], cfg.group_size, cfg.bit, x.data_ptr(),
        None if residual_in is None else residual_in.data_ptr(), out.data_ptr(),
        None if residual_out is None else residual_out.data_ptr(), x.numel(), ctypes.c_void_p(stream))


@pytest.mark.parametrize("dtype,group,bit", [(torch.bfloat16, 64, 8), (torch.float32, 16, 8), (torch.float16, 32, 4)])
def test_two_calls_in_a_row_match_the_allocating_path(ext, dtype, group, bit):
    lib = _library()
    cfg = CompressionConfig(bit=bit, group_size=group, allow_experimental=True)
    gen = torch.Generator().manual_seed(5)
    # second call is smaller than the first: stale payload bytes of call one must not leak into call two
    for n in (3 * 64 * 1000 + 37, 64 * 100 + 5):
        x = (torch.randn(n, generator=gen) * 1e-2).to(dtype).cuda()
        residual = (torch.randn(n, generator=gen) * 1e-4).to(dtype).cuda()
        want_out, want_res = _existing_path(x, residual, cfg)
        out = torch.empty_like(x)
        res = residual.clone()
        before = torch.cuda.memory_allocated()
        code = _call(lib, x, res, out, res, cfg)
        assert code == 0, lib.lbc_no_alloc_error_string(code)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert torch.equal(out.view(torch.uint8), want_out.view(torch.uint8)), n
        assert torch.equal(res.view(torch.uint8), want_res.view(torch.uint8)), n


@pytest.mark.parametrize("dtype,group,bit", [(torch.float32, 16, 8), (torch.bfloat16, 64, 8)])
def test_the_largest_accepted_size_fits_the_fixed_array(ext, dtype, group, bit):
    """`numel == lbc_no_alloc_max_numel()`: for fp32 / groups of 16 / 8 bit the payload fills the array to its last
    byte.  Bit-for-bit agreement with the allocating path shows that neither region is cut short."""

    lib = _library()
    cfg = CompressionConfig(bit=bit, group_size=group, allow_experimental=True)
    n = lib.lbc_no_alloc_max_numel()
    gen = torch.Generator().manual_seed(9)
    x = (torch.randn(n, generator=gen) * 1e-2).to(dtype).cuda()
    residual = (torch.randn(n, generator=gen) * 1e-4).to(dtype).cuda()
    want_out, want_res = _existing_path(x, residual, cfg)
    out, res = torch.empty_like(x), residual.clone()
    for _ in range(2):                      # two calls in a row, the second on the first one's leftovers
        res.copy_(residual)
        code = _call(lib, x, res, out, res, cfg)
        assert code == 0, lib.lbc_no_alloc_error_string(code)
        torch.cuda.synchronize()
        assert torch.equal(out.view(torch.uint8), want_out.view(torch.uint8))
        assert torch.equal(res.view(torch.uint8), want_res.view(torch.uint8))
    # one element more, with valid pointers: refused before anything is launched
    big = torch.zeros(n + 1, dtype=dtype, device="cuda")
    sentinel = torch.full((n + 1,), 3.0, dtype=dtype, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    code = lib.lbc_no_alloc_roundtrip(_DTYPE_CODE[dtype], group, bit, big.data_ptr(), None, sentinel.data_ptr(), None,
                                      n + 1, stream)
    torch.cuda.synchronize()
    assert code == -2 and bool((sentinel == 3.0).all())


def test_without_error_feedback_and_limits(ext):
    lib = _library()
    cfg = CompressionConfig()
    x = (torch.randn(10_000) * 1e-2).to(torch.bfloat16).cuda()
    out = torch.empty_like(x)
    assert _call(lib, x, None, out, None, cfg) == 0
    torch.cuda.synchronize()
    want = codec.dequantize_tensor(codec.quantize_tensor(x, cfg), x.shape, cfg, dtype="bf16")
    assert torch.equal(out.view(torch.uint8), want.view(torch.uint8))
    assert lib.lbc_no_alloc_scratch_bytes() == lib.lbc_no_alloc_max_numel() // 16 * 20
    # beyond the stated maximum: a clear error, nothing launched (the pointers are never touched)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    code = lib.lbc_no_alloc_roundtrip(1, 64, 8, x.data_ptr(), None, out.data_ptr(), None,
                                      lib.lbc_no_alloc_max_numel() + 1, stream)
    assert code == -2 and b"split" in lib.lbc_no_alloc_error_string(code)
    assert lib.lbc_no_alloc_roundtrip(1, 48, 8, x.data_ptr(), None, out.data_ptr(), None, 10, stream) == -1
    assert lib.lbc_no_alloc_roundtrip(1, 64, 8, x.data_ptr(), x.data_ptr(), out.data_ptr(), None, 10, stream) == -1
