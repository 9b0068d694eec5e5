"""The C++ host codec against the torch oracle: two independently written statements of the wire
format have to agree bit for bit (conversions, encode, decode, accumulate, fused reduce + residual)."""

import ctypes
import struct

import pytest
import torch

from lowbit_comm_b200.config import CompressionConfig
from lowbit_comm_b200.ops import codec, host_codec, oracle
from lowbit_comm_b200.ops.build import build_host_library

DT = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}


@pytest.fixture(scope="module", autouse=True)
def host_library():
    build_host_library()
    host_codec._tried = False          # pick up a library built after the first import
    lib = host_codec.library()
    assert lib is not None, "g++ build of csrc/host_codec.cpp failed"
    return lib


def _bits(t: torch.Tensor) -> torch.Tensor:
    return t.contiguous().view(torch.uint8)


def _inputs(n, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(n, generator=g) * 10 ** torch.empty(n).uniform_(-9, 3, generator=g)
    x[::7] = 0
    if n > 40:
        x[5], x[11], x[23], x[37] = 3.0e4, -6.1e-5, 5.9e-8, 3.0e37 if dtype != "fp16" else 2.0e4   # sums stay finite
    return x.to(DT[dtype])


def test_half_conversions_are_exact(host_library):
    lib = host_library
    halves = torch.arange(0, 65536, dtype=torch.int32).to(torch.uint16).view(torch.float16).float()
    for h in range(0, 65536):
        want = halves[h].item()
        got = lib.lbc_host_half_to_float(h)
        assert (got != got and want != want) or struct.pack("f", got) == struct.pack("f", want), h
    g = torch.Generator().manual_seed(3)
    raw = torch.randint(-2 ** 31, 2 ** 31 - 1, (60_000,), generator=g, dtype=torch.int64).to(torch.int32)
    edge = torch.tensor([0x33000000, 0x33000001, 0x32FFFFFF, 0x387FE000, 0x387FF000, 0x38800000, 0x477FEFFF, 0x477FF000,
                         0x3F801000, 0x3F803000, 0x3F801001, 0x7F800000, 0x00000001, 0x38000000], dtype=torch.int32)
    raw = torch.cat([raw, edge, edge | torch.tensor(-2 ** 31, dtype=torch.int32)])
    floats = raw.view(torch.float32)
    want_h = floats.to(torch.float16).view(torch.int16).to(torch.int32) & 0xFFFF
    want_b = floats.to(torch.bfloat16).view(torch.int16).to(torch.int32) & 0xFFFF
    for i in range(floats.numel()):
        f = floats[i].item()
        if f != f:
            continue  # NaN payloads are not part of the contract
        assert lib.lbc_host_float_to_half(ctypes.c_float(f)) == want_h[i].item(), hex(raw[i].item() & 0xFFFFFFFF)
        assert lib.lbc_host_float_to_bf16(ctypes.c_float(f)) == want_b[i].item(), hex(raw[i].item() & 0xFFFFFFFF)


@pytest.mark.parametrize("dtype", ("bf16", "fp16", "fp32"))
@pytest.mark.parametrize("bit,group", [(8, 64), (8, 16), (4, 32), (4, 64)])
@pytest.mark.parametrize("compact", (False, True))
def test_encode_decode_match_the_oracle(dtype, bit, group, compact):
    cfg = CompressionConfig(bit=bit, group_size=group, compact=compact, allow_experimental=True)
    for seed, n in enumerate((1, group - 1, group, group + 7, 1000, 64 * 129 + 5)):
        x = _inputs(n, dtype, seed)
        r = (_inputs(n, dtype, 100 + seed).float() * 1e-2).to(DT[dtype])
        for residual in (None, r):
            want = oracle.encode(x, cfg, residual=residual)
            out = torch.empty_like(want)
            prepared = torch.empty_like(x)
            host_codec.quantize(x, cfg, dtype, out, residual, prepared)
            assert torch.equal(out, want), (n, residual is not None)
            assert torch.equal(_bits(prepared), _bits(oracle.prepare(x, residual))), n
            dec = torch.empty(n, dtype=DT[dtype])
            host_codec.dequantize(want, n, cfg, dtype, dec)
            assert torch.equal(_bits(dec), _bits(oracle.decode(want, n, cfg, dtype))), n
            acc = _inputs(n, dtype, 200 + seed)
            expect = oracle.decode_accumulate(want, acc.clone(), cfg)
            host_codec.dequantize(want, n, cfg, dtype, acc, accumulate=True)
            assert torch.equal(_bits(acc), _bits(expect)), n


@pytest.mark.parametrize("dtype", ("bf16", "fp16", "fp32"))
@pytest.mark.parametrize("bit,group,count", [(8, 64, 1), (8, 64, 2), (8, 32, 8), (4, 16, 3)])
def test_fused_reduce_matches_the_oracle(dtype, bit, group, count):
    cfg = CompressionConfig(bit=bit, group_size=group, allow_experimental=True)
    for seed, n in enumerate((1, group + 3, 4097)):
        xs = [(_inputs(n, dtype, 10 * seed + r).float().clamp(-1e3, 1e3) * 1e-2).to(DT[dtype]) for r in range(count)]
        payloads = [oracle.encode(x, cfg) for x in xs]
        for divisor in (None, 1.0, 3.0):
            y, y32 = oracle.reduce_mean(payloads, n, cfg, dtype, divisor)
            div = float(count) if divisor is None else divisor
            inv = float(torch.tensor(1.0) / torch.tensor(div))
            out = torch.empty(n, dtype=DT[dtype])
            residual = xs[0].clone()            # prepared and residual alias, as in the hook
            host_codec.reduce(payloads, n, cfg, dtype, inv, out, residual, residual)
            assert torch.equal(_bits(out), _bits(y)), (n, divisor)
            assert torch.equal(_bits(residual), _bits(oracle.residual_update(xs[0], y32))), (n, divisor)


@pytest.mark.parametrize("dtype", ("bf16", "fp16", "fp32"))
@pytest.mark.parametrize("topk", (0, 1, 2))
@pytest.mark.parametrize("bit,group,quant", [(8, 64, "linear"), (4, 32, "linear"), (4, 16, "normal"), (4, 64, "uniform"),
                                             (4, 32, "e3m0"), (4, 64, "e2m1")])
@pytest.mark.parametrize("compact", (False, True))
def test_general_profiles_match_the_oracle(dtype, topk, bit, group, quant, compact):
    if topk == 0 and quant == "linear":
        pytest.skip("covered by the fast-path test")
    cfg = CompressionConfig(bit=bit, group_size=group, topk=topk, quant_type=quant, compact=compact,
                            allow_experimental=True)
    for seed, n in enumerate((group, group * 9, group * 31 + 5)):
        x = _inputs(n, dtype, seed)
        if n > 8:
            x[3] = x[2]                      # equal magnitudes inside a group: the tie rule of the top-k scan matters
            x[6] = -x[2]
        r = (_inputs(n, dtype, 300 + seed).float() * 1e-2).to(DT[dtype])
        for residual in (None, r):
            want = oracle.encode(x, cfg, residual=residual)
            out = torch.empty_like(want)
            prepared = torch.empty_like(x)
            host_codec.quantize(x, cfg, dtype, out, residual, prepared)
            assert torch.equal(out, want), (n, residual is not None)
            assert torch.equal(_bits(prepared), _bits(oracle.prepare(x, residual)))
            dec = torch.empty(n, dtype=DT[dtype])
            host_codec.dequantize(want, n, cfg, dtype, dec)
            assert torch.equal(_bits(dec), _bits(oracle.decode(want, n, cfg, dtype))), n
            acc = (_inputs(n, dtype, 400 + seed).float() * 1e-3).to(DT[dtype])
            expect = oracle.decode_accumulate(want, acc.clone(), cfg)
            host_codec.dequantize(want, n, cfg, dtype, acc, accumulate=True)
            assert torch.equal(_bits(acc), _bits(expect)), n


def test_facade_uses_the_host_library_on_cpu():
    cfg = CompressionConfig()
    x = _inputs(5000, "bf16", 1)
    assert host_codec.serves(cfg)
    payload = codec.quantize_tensor(x, cfg)
    assert torch.equal(payload, oracle.encode(x, cfg))
    back = codec.dequantize_tensor(payload, x.shape, cfg, dtype="bf16")
    assert torch.equal(_bits(back), _bits(oracle.decode(payload, x.numel(), cfg, "bf16")))
    assert host_codec.serves(CompressionConfig(topk=1))
    assert not host_codec.serves(CompressionConfig(stochastic=True))  # the oracle keeps stochastic rounding
    with pytest.raises(ValueError):
        host_codec.reduce([payload], x.numel(), CompressionConfig(topk=1), "bf16", 1.0, torch.empty_like(x))


def test_arguments_are_validated():
    cfg = CompressionConfig()
    x = torch.zeros(128, dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        host_codec.quantize(x, cfg, "bf16", torch.empty(10, dtype=torch.uint8))
    with pytest.raises(ValueError):
        host_codec.quantize(x.float(), cfg, "bf16", torch.empty(132, dtype=torch.uint8))
    with pytest.raises(ValueError):
        host_codec.dequantize(torch.empty(132, dtype=torch.uint8), 128, cfg, "bf16", torch.empty(64, dtype=torch.bfloat16))


def test_large_tensors_split_over_threads_give_the_same_bytes():
    """Above 8192 groups per thread the host codec splits its group loops over threads; ranges are disjoint,
    so the bytes must equal the oracle's whatever the split (odd sizes put a ragged range at the end)."""

    import torch

    from lowbit_comm_b200.config import CompressionConfig
    from lowbit_comm_b200.ops import codec, oracle

    cfg = CompressionConfig()
    n = 64 * 8192 * 3 + 37
    g = torch.Generator().manual_seed(21)
    x = (torch.randn(n, generator=g) * 0.02).to(torch.bfloat16)
    r = (torch.randn(n, generator=g) * 0.002).to(torch.bfloat16)
    prepared = torch.empty_like(x)
    payload = codec.quantize_tensor(x, cfg, residual=r, prepared_out=prepared)
    assert torch.equal(payload, oracle.encode(x, cfg, residual=r)) and torch.equal(prepared, oracle.prepare(x, r))
    assert torch.equal(codec.dequantize_tensor(payload, (n,), cfg, dtype="bf16"), oracle.decode(payload, n, cfg, "bf16"))
    other = codec.quantize_tensor(-x, cfg)
    out, residual = torch.empty_like(x), torch.empty_like(x)
    assert codec.inplace_dequantize_reduce_mean_update_error_feedback([payload, other], prepared, out, residual, cfg,
                                                                       reduce="mean")
    y, y32 = oracle.reduce_mean([payload, other], n, cfg, "bf16")
    assert torch.equal(out, y) and torch.equal(residual, oracle.residual_update(prepared, y32))
