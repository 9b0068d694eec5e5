"""Wire-format oracle and codec facade on CPU: hand-computed vectors, layouts, byte order, round trips."""

import itertools

import pytest
import torch

from lowbit_comm_b200 import CompressionConfig, Quantizer
from lowbit_comm_b200.ops import codec, oracle
from lowbit_comm_b200.ops.torch_fallback import dequantize_tensor_fallback, quantize_tensor_fallback


def cfg(**kw):
    return CompressionConfig(allow_experimental=True, **kw)


def test_hand_computed_payload_bf16():
    x = torch.tensor([1.0, -2.0, 3.0, 0.5] * 16, dtype=torch.bfloat16)
    p = oracle.encode(x, cfg())
    assert p.numel() == 66
    # scale 3.0: codes 42, -85, 127, 21; 16-bit words hold (even << 8) | odd, little endian in memory
    assert p[:4].tolist() == [171, 42, 21, 127]
    assert p[64:].tolist() == [0x40, 0x40]  # bf16(3.0) = 0x4040: the stored scale is the abs-max itself
    compact = oracle.encode(torch.cat([x, x * 2]), cfg(compact=True))
    assert compact[:4].tolist() == [171, 42, 21, 127] and compact[64:66].tolist() == [0x40, 0x40]
    assert compact[66:70].tolist() == [171, 42, 21, 127] and compact[130:132].tolist() == [0xC0, 0x40]  # bf16(6.0)


def test_hand_computed_payload_fp32_and_int4():
    x = torch.tensor([1.0, -2.0, 3.0, 0.5] * 4, dtype=torch.float32)
    p = oracle.encode(x, cfg(group_size=16))
    assert p[:4].tolist() == [21, 127, 171, 42]  # 32-bit words: element 0 in the most significant byte
    assert p[16:].view(torch.float32).item() == 3.0
    q = oracle.encode(x.to(torch.float16), cfg(group_size=16, bit=4))
    # codes round(v*7/3) = 2, -5, 7, 1 -> nibbles 2, b, 7, 1 -> word 0x2b71 -> bytes 71 2b
    assert q[:2].tolist() == [0x71, 0x2B] and q.numel() == 8 + 2


def test_rounding_is_half_to_even_and_scale_is_rounded_first():
    x = torch.zeros(64, dtype=torch.float32)
    x[0], x[1], x[2], x[3] = 127.0, 0.5, 1.5, -2.5
    back = oracle.decode(oracle.encode(x, cfg()), 64, cfg(), "fp32")
    assert back[:4].tolist() == [127.0, 0.0, 2.0, -2.0]
    y = torch.zeros(64, dtype=torch.float32)
    y[0] = 1.00390625  # not representable in bf16: the stored scale rounds to 1.0 and the code saturates at 127
    p = oracle.encode(y.to(torch.bfloat16), cfg())
    assert p[64:].tolist() == [0x80, 0x3F]


def test_zero_group_and_tail_padding():
    x = torch.zeros(70, dtype=torch.float16)
    x[65] = 2.0
    c = cfg()
    p = oracle.encode(x, c)
    assert p.numel() == 2 * 66
    back = oracle.decode(p, 70, c, "fp16")
    assert back.abs().sum().item() == 2.0 and back[65].item() == 2.0


@pytest.mark.parametrize("dtype", ["bf16", "fp16", "fp32"])
@pytest.mark.parametrize("bit,group,topk", list(itertools.product((8, 4), (16, 64), (0, 1, 2))))
@pytest.mark.parametrize("compact", (False, True))
def test_round_trip_through_facade(dtype, bit, group, topk, compact):
    c = cfg(bit=bit, group_size=group, topk=topk, compact=compact)
    x = (torch.randn(5 * group + 3) * 0.1).to(oracle.TORCH_DTYPES[dtype])
    payload = codec.quantize_tensor(x, c)
    assert payload.numel() == codec.allocate_quantized_buffer(x, c).numel()
    back = codec.dequantize_tensor(payload, x.shape, c, dtype=dtype)
    rel = ((back.float() - x.float()).norm() / x.float().norm()).item()
    assert rel < (0.02 if bit == 8 else 0.2)
    if topk:  # the largest magnitudes survive verbatim
        g0 = x[:group].float().abs()
        keep = torch.topk(g0, topk).indices
        assert torch.equal(back[:group][keep], x[:group][keep])


@pytest.mark.parametrize("quant_type", ["normal", "uniform", "e3m0", "e2m1"])
def test_codebook_quantization(quant_type):
    c = cfg(bit=4, quant_type=quant_type)
    x = torch.linspace(-1, 1, 64, dtype=torch.float32)
    back = oracle.decode(oracle.encode(x, c), 64, c, "fp32")
    table = oracle.codebook(quant_type)[:15]
    assert all(torch.isclose(table, v, atol=1e-6).any() for v in back)  # outputs are code-book entries (scale 1.0)
    assert back[0].item() == -1.0 and back[-1].item() == 1.0
    nearest = table[(x[:, None] - table[None, :]).abs().argmin(dim=1)]
    assert (back - x).abs().max() <= (nearest - x).abs().max() + 1e-6


def test_reduce_and_error_feedback_semantics():
    c = cfg()
    gen = torch.Generator().manual_seed(17)
    xs = [(torch.randn(300, generator=gen) * 0.01).to(torch.bfloat16) for _ in range(4)]
    payloads = [codec.quantize_tensor(x, c) for x in xs]
    mean = codec.dequantize_reduce_tensors(payloads, (300,), c, dtype="bf16", reduce="mean")
    exact = torch.stack([codec.dequantize_tensor(p, (300,), c, dtype="bf16").float() for p in payloads]).mean(0)
    half_ulp = exact.abs().max().item() * 2.0 ** -8          # one rounding of the fp32 mean to bf16
    assert (mean.float() - exact).abs().max() <= half_ulp
    prepared, restored, residual = xs[0].clone(), torch.empty(300, dtype=torch.bfloat16), torch.zeros(300, dtype=torch.bfloat16)
    assert codec.inplace_dequantize_reduce_mean_update_error_feedback(payloads, prepared, restored, residual, c, reduce="mean")
    assert torch.equal(restored, mean)
    assert (residual.float() - (prepared.float() - exact)).abs().max() <= 2 * half_ulp
    assert not codec.inplace_dequantize_reduce_mean([], restored, c)
    assert not codec.inplace_quantize_pack(xs[0], payloads[0], None, cfg(topk=1))
    assert codec.inplace_quantize_pack(xs[0], payloads[0].clone(), xs[1], c)
    with pytest.raises(ValueError):
        codec.dequantize_reduce_tensors(payloads, (300,), c, dtype="bf16", reduce="max")


def test_int8_envelope_matches_published_value():
    torch.manual_seed(0)
    x = torch.randn(1 << 16, dtype=torch.float16)
    c = cfg()
    back = codec.dequantize_tensor(codec.quantize_tensor(x, c), x.shape, c, dtype="fp16")
    err = (back.float() - x.float()).abs().max().item()
    assert err <= 0.02 and ((back.float() - x.float()).norm() / x.float().norm()).item() < 0.01


def test_quantizer_facade_and_fallback_codec():
    q = Quantizer(cfg(), dtype="bf16")
    x = torch.randn(130, dtype=torch.bfloat16)
    p = q.quantize(x)
    assert Quantizer.is_quantized(p) and not Quantizer.is_quantized(x) and q.allocate_q(x).numel() == p.numel()
    assert q.dequantize(p, x.shape).shape == x.shape
    assert Quantizer.from_dict(q.to_dict()).config == q.config
    with pytest.raises(ValueError):
        Quantizer().dequantize(p, x.shape)
    assert q.is_quantized() and q.is_quantized(p) and not q.is_quantized(x)
    assert q.wire_bytes(130) == p.numel() and q.roundtrip(x).dtype == x.dtype
    err = q.error(x)
    assert 0 < err["relative_rms"] < 0.02 and err["rms"] <= err["max_abs"]
    calls = []
    spy = Quantizer(cfg(), dtype="bf16", quantize_fn=lambda t, c, **kw: calls.append(sorted(kw)) or p)
    assert spy.quantize(x) is p and calls == [["extension_status", "output"]]
    payload = quantize_tensor_fallback(x.float(), cfg())
    assert payload.buffer.dtype == torch.int8 and payload.metadata["scales"].dtype == torch.float32
    assert payload.metadata["original_numel"] == 130 and payload.buffer.numel() == 192
    back = dequantize_tensor_fallback(payload, x.shape, cfg(), "fp32")
    assert (back - x.float()).abs().max() <= payload.metadata["scales"].max() / 2 + 1e-6
    with pytest.raises(ValueError):
        quantize_tensor_fallback(x, cfg(bit=4))


def test_facade_rejects_bad_payloads():
    c = cfg()
    x = torch.randn(128, dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        codec.quantize_tensor(x, c, output=torch.empty(7, dtype=torch.uint8))
    with pytest.raises(TypeError):
        codec.dequantize_tensor(torch.empty(132, dtype=torch.int8), (128,), c, dtype="bf16")
    with pytest.raises(ValueError):
        codec.dequantize_tensor(codec.quantize_tensor(x, c), (128,), c, dtype="bf16", reduce_op="sum")


def test_codec_corners_on_cpu():
    from lowbit_comm_b200.ops import oracle

    c = cfg()
    x = torch.randn(4, 50, dtype=torch.bfloat16) * 0.1
    meta = {}
    payload = codec.quantize_tensor(x.t(), c, metadata=meta)                   # a non-contiguous view
    assert meta == {"original_numel": 200, "padded_numel": 256, "num_groups": 4, "dtype": "bf16", "compact": False}
    assert torch.equal(payload, oracle.encode(x.t().contiguous().reshape(-1), c))
    empty = codec.quantize_tensor(torch.empty(0, dtype=torch.bfloat16), c)
    assert empty.numel() == 0 and codec.dequantize_tensor(empty, (0,), c, dtype="bf16").numel() == 0

    # stochastic rounding has no host-codec twin: the oracle serves it, with the prepared value on request
    noisy = CompressionConfig(stochastic=True)
    residual = torch.randn(200, dtype=torch.bfloat16) * 0.01
    prepared = torch.empty(200, dtype=torch.bfloat16)
    torch.manual_seed(5)
    a = codec.quantize_tensor(x.reshape(-1), noisy, residual=residual, prepared_out=prepared)
    torch.manual_seed(5)
    b = codec.quantize_tensor(x.reshape(-1), noisy, residual=residual)
    assert torch.equal(a, b) and torch.equal(prepared, oracle.prepare(x.reshape(-1), residual))
    back = codec.dequantize_tensor(a, (200,), noisy, dtype="bf16")
    assert (back.float() - prepared.float()).abs().max() <= prepared.float().abs().max() / 127 * 1.01 + 1e-6

    # top-k payloads decode through the oracle as well, with and without accumulation
    topk = CompressionConfig(topk=2)
    p = codec.quantize_tensor(x.reshape(-1), topk)
    once = codec.dequantize_tensor(p, (200,), topk, dtype="bf16")
    twice = codec.dequantize_tensor(p, (200,), topk, dtype="bf16", output=once.clone(), reduce_op="sum")
    assert torch.equal(twice, (once.float() + once.float()).to(torch.bfloat16))

    good = codec.quantize_tensor(x.reshape(-1), c)
    with pytest.raises(ValueError, match="unsupported reduce_op"):
        codec.dequantize_tensor(good, (200,), c, dtype="bf16", reduce_op="max")
    with pytest.raises(ValueError, match="wrong number of elements"):
        codec.dequantize_tensor(good, (200,), c, dtype="bf16", output=torch.empty(199, dtype=torch.bfloat16))
    with pytest.raises(TypeError, match="wrong dtype"):
        codec.dequantize_tensor(good, (200,), c, dtype="bf16", output=torch.empty(200, dtype=torch.float16))
    with pytest.raises(ValueError, match="contiguous"):
        codec.dequantize_tensor(good, (200,), c, dtype="bf16", output=torch.empty(400, dtype=torch.bfloat16)[::2])
    with pytest.raises(ValueError, match="expected"):
        codec.quantize_tensor(x.reshape(-1), c, output=torch.empty(good.numel() + 1, dtype=torch.uint8))
    with pytest.raises(TypeError, match="uint8"):
        codec.quantize_tensor(x.reshape(-1), c, output=torch.empty(good.numel(), dtype=torch.int8))
    with pytest.raises(ValueError, match="contiguous"):
        codec.quantize_tensor(x.reshape(-1), c, output=torch.empty(2 * good.numel(), dtype=torch.uint8)[::2])
    with pytest.raises(ValueError, match="unsupported dtype"):
        codec.resolve_dtype("fp64")
    with pytest.raises(ValueError, match="needs a tensor"):
        codec.resolve_dtype("auto")
    with pytest.raises(ValueError, match="at least one payload"):
        codec.dequantize_reduce_tensors([], (200,), c, dtype="bf16")
    with pytest.raises(ValueError, match="unsupported reduce"):
        codec.dequantize_reduce_tensors([good], (200,), c, dtype="bf16", reduce="max")
