"""sm_100a codec kernels against the bit-exact torch oracle (plain fp32 math on CPU).

Mirrors the intent of the reference's tests/cuda/test_fused_quant_pack.py and
tests/test_cuda_extension_smoke.py: uneven lengths, every dtype x bit x group
size, residual add, unaligned views, empty tensors, zero steady-state
allocation.
"""

import itertools

import pytest
import torch

from lowbit_comm_b200.config import CompressionConfig
from lowbit_comm_b200.ops import codec, oracle

pytestmark = pytest.mark.gpu

DTYPES = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}


def _cfg(**kw):
    return CompressionConfig(allow_experimental=True, **kw)


def _data(n, dtype, seed=0, outliers=True):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(n, generator=g) * 1e-2
    if outliers and n > 10:
        idx = torch.randint(0, n, (max(1, n // 100),), generator=g)
        x[idx] *= 50
    return x.to(dtype)


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("bit,group", list(itertools.product((8, 4), (16, 32, 64))))
@pytest.mark.parametrize("compact", (False, True))
def test_fast_quantize_matches_oracle(ext, dtype, bit, group, compact):
    cfg = _cfg(bit=bit, group_size=group, compact=compact)
    for n in (group + 7, 1, group, 5 * group - 1, 4096 + 3 * group + 5):
        x = _data(n, DTYPES[dtype], seed=n)
        r = _data(n, DTYPES[dtype], seed=n + 1, outliers=False)
        for residual in (None, r):
            want = oracle.encode(x, cfg, residual=residual)
            got = codec.quantize_tensor(x.cuda(), cfg, residual=None if residual is None else residual.cuda())
            assert got.dtype == torch.uint8 and got.numel() == want.numel()
            assert torch.equal(got.cpu(), want), (dtype, bit, group, compact, n, residual is not None)
            back = codec.dequantize_tensor(got, (n,), cfg, dtype=dtype)
            assert torch.equal(back.cpu().view(torch.uint8), oracle.decode(want, n, cfg, dtype).view(torch.uint8))


def test_unaligned_views_and_prepared_out(ext):
    cfg = _cfg()
    base = _data(10_000, torch.bfloat16).cuda()
    rbase = _data(10_000, torch.bfloat16, seed=3, outliers=False).cuda()
    for off in (1, 3, 8, 17):
        x, r = base[off:off + 4099], rbase[off:off + 4099]
        prepared = torch.empty_like(x)
        got = codec.quantize_tensor(x, cfg, residual=r, prepared_out=prepared)
        assert torch.equal(got.cpu(), oracle.encode(x.cpu(), cfg, residual=r.cpu()))
        assert torch.equal(prepared.cpu(), oracle.prepare(x.cpu(), r.cpu()))


def test_empty_and_zero_tensors(ext):
    cfg = _cfg()
    empty = torch.empty(0, dtype=torch.bfloat16, device="cuda")
    assert codec.quantize_tensor(empty, cfg).numel() == 0
    zeros = torch.zeros(256, dtype=torch.float16, device="cuda")
    p = codec.quantize_tensor(zeros, cfg)
    assert torch.equal(p.cpu(), oracle.encode(zeros.cpu(), cfg))
    assert codec.dequantize_tensor(p, (256,), cfg, dtype="fp16").abs().max().item() == 0


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("bit,group,compact", [(8, 64, False), (8, 64, True), (8, 16, False), (4, 32, False), (4, 64, True)])
@pytest.mark.parametrize("world", (1, 2, 8, 16))
def test_fused_reduce_mean_and_error_feedback(ext, dtype, bit, group, compact, world):
    cfg = _cfg(bit=bit, group_size=group, compact=compact)
    n = 9 * group + 11
    xs = [_data(n, DTYPES[dtype], seed=10 + r) for r in range(world)]
    payloads = [oracle.encode(x, cfg) for x in xs]
    want, want32 = oracle.reduce_mean(payloads, n, cfg, dtype)
    dev = [p.cuda() for p in payloads]
    out = torch.empty(n, dtype=DTYPES[dtype], device="cuda")
    assert codec.inplace_dequantize_reduce_mean(dev, out, cfg, reduce="mean")
    assert torch.equal(out.cpu().view(torch.uint8), want.view(torch.uint8))
    total = codec.dequantize_reduce_tensors(dev, (n,), cfg, dtype=dtype, reduce="sum")
    assert torch.equal(total.cpu().view(torch.uint8), oracle.reduce_mean(payloads, n, cfg, dtype, 1.0)[0].view(torch.uint8))
    prepared = xs[0].cuda()
    restored = torch.empty_like(prepared)
    residual = torch.zeros_like(prepared)
    assert codec.inplace_dequantize_reduce_mean_update_error_feedback(dev, prepared, restored, residual, cfg, reduce="mean")
    assert torch.equal(restored.cpu().view(torch.uint8), want.view(torch.uint8))
    assert torch.equal(residual.cpu().view(torch.uint8), oracle.residual_update(xs[0], want32).view(torch.uint8))
    # in-place form used by the DDP hook: `prepared` lives in the residual buffer
    alias = xs[0].cuda().clone()
    assert codec.inplace_dequantize_reduce_mean_update_error_feedback(dev, alias, restored, alias, cfg, reduce="mean")
    assert torch.equal(alias.cpu().view(torch.uint8), oracle.residual_update(xs[0], want32).view(torch.uint8))


def test_unfused_sum_accumulates_in_source_dtype(ext):
    cfg = _cfg()
    n = 1000
    a, b = _data(n, torch.bfloat16, 1), _data(n, torch.bfloat16, 2)
    pa, pb = oracle.encode(a, cfg), oracle.encode(b, cfg)
    out = codec.dequantize_tensor(pa.cuda(), (n,), cfg, dtype="bf16")
    codec.dequantize_tensor(pb.cuda(), (n,), cfg, dtype="bf16", output=out, reduce_op="sum")
    want = oracle.decode_accumulate(pb, oracle.decode(pa, n, cfg, "bf16"), cfg)
    assert torch.equal(out.cpu().view(torch.uint8), want.view(torch.uint8))


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("group", (16, 32, 64))
@pytest.mark.parametrize("bit,quant_type,topk", [(8, "linear", 1), (8, "linear", 2), (4, "linear", 2), (4, "normal", 0),
                                                  (4, "uniform", 1), (4, "e3m0", 0), (4, "e2m1", 2)])
@pytest.mark.parametrize("compact", (False, True))
def test_general_kernels_match_oracle(ext, dtype, group, bit, quant_type, topk, compact):
    cfg = _cfg(bit=bit, group_size=group, topk=topk, quant_type=quant_type, compact=compact)
    for n in (group + 7, 7 * group, 2048 + 5):
        x = _data(n, DTYPES[dtype], seed=n + topk)
        x[:group] = 0  # an all-zero group exercises the top-k fall-backs
        if n > 2 * group:
            x[group:group + 4] = x[group]  # ties
        r = _data(n, DTYPES[dtype], seed=n + 9, outliers=False)
        want = oracle.encode(x, cfg, residual=r)
        got = codec.quantize_tensor(x.cuda(), cfg, residual=r.cuda())
        assert torch.equal(got.cpu(), want), (dtype, group, bit, quant_type, topk, compact, n)
        back = codec.dequantize_tensor(got, (n,), cfg, dtype=dtype)
        assert torch.equal(back.cpu().view(torch.uint8), oracle.decode(want, n, cfg, dtype).view(torch.uint8))
        both = codec.dequantize_reduce_tensors([got, got], (n,), cfg, dtype=dtype, reduce="sum")
        want2 = oracle.decode_accumulate(want, oracle.decode(want, n, cfg, dtype), cfg)
        assert torch.equal(both.cpu().view(torch.uint8), want2.view(torch.uint8))


def test_stochastic_rounding_is_unbiased(ext):
    cfg = _cfg(stochastic=True)
    x = torch.full((64 * 4096,), 0.3, dtype=torch.float32)
    x[::64] = 1.0  # scale 1.0 -> 0.3 * 127 = 38.1: rounds up 10 % of the time
    got = codec.dequantize_tensor(codec.quantize_tensor(x.cuda(), cfg), x.shape, cfg, dtype="fp32").cpu()
    body = got.reshape(-1, 64)[:, 1:]
    assert set(torch.unique(torch.round(body * 127)).tolist()) <= {38.0, 39.0}
    assert abs(body.double().mean().item() - 0.3) < 2e-4
    det = codec.dequantize_tensor(codec.quantize_tensor(x.cuda(), _cfg()), x.shape, _cfg(), dtype="fp32").cpu()
    assert abs(det.reshape(-1, 64)[:, 1:].double().mean().item() - 38 / 127) < 1e-6


def test_round_trip_error_envelope(ext):
    cfg = _cfg()
    x = torch.randn(1 << 20, dtype=torch.float16)
    y = codec.dequantize_tensor(codec.quantize_tensor(x.cuda(), cfg), x.shape, cfg, dtype="fp16").cpu()
    rel = ((y.float() - x.float()).norm() / x.float().norm()).item()
    assert rel < 0.02 and (y.float() - x.float()).abs().max().item() <= 0.0235


def test_error_feedback_update_and_scale(ext):
    a, b = _data(5001, torch.bfloat16, 1).cuda(), _data(5001, torch.bfloat16, 2).cuda()
    res = torch.empty_like(a)
    codec.update_error_feedback_residual(a, b, res)
    assert torch.equal(res.cpu(), oracle.residual_update_from_restored(a.cpu(), b.cpu()))


def test_zero_steady_state_allocation(ext):
    cfg = _cfg()
    x = _data(1 << 16, torch.bfloat16).cuda()
    r = torch.zeros_like(x)
    out = codec.allocate_quantized_buffer(x, cfg)
    restored = torch.empty_like(x)
    codec.quantize_tensor(x, cfg, output=out, residual=r)
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    ptr = out.data_ptr()
    for _ in range(100):
        codec.quantize_tensor(x, cfg, output=out, residual=r)
        codec.inplace_dequantize_reduce_mean_update_error_feedback([out], x, restored, r, cfg, reduce="mean")
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before and out.data_ptr() == ptr


def test_payload_size_is_validated(ext):
    cfg = _cfg()
    x = _data(640, torch.bfloat16).cuda()
    with pytest.raises(ValueError):
        codec.quantize_tensor(x, cfg, output=torch.empty(10, dtype=torch.uint8, device="cuda"))
    with pytest.raises(ValueError):
        codec.dequantize_tensor(torch.empty(10, dtype=torch.uint8, device="cuda"), (640,), cfg, dtype="bf16")
