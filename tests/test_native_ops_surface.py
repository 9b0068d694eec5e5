"""The reference's pybind op surface (`ccdl_cuda_ops`) re-exposed over this library's codec: same call
shapes, same bytes as the oracle.  CPU tensors here; the CUDA path is the codec's, covered by its own tests."""

import pytest
import torch

from lowbit_comm_b200.config import CompressionConfig
from lowbit_comm_b200.ops import native_ops as ops
from lowbit_comm_b200.ops import oracle

DT = {ops.FP16: torch.float16, ops.BF16: torch.bfloat16, ops.FP32: torch.float32}


def _x(n, dtype, seed=0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(n, generator=g) * 0.05).to(dtype)


def test_module_exports_the_reference_names():
    for name in ("quantize", "dequantize", "inplace_quantize", "inplace_quantize_pack", "inplace_dequantize",
                 "dequantize_reduce", "inplace_dequantize_reduce", "inplace_dequantize_reduce_mean",
                 "inplace_error_feedback_update", "dequantize_reduce_update_error_feedback",
                 "inplace_dequantize_reduce_mean_update_error_feedback"):
        assert callable(getattr(ops, name)), name
    assert ops.NATIVE_WORK_ABI_VERSION == 1
    assert {m.name for m in ops.ReduceOP} == {"SUM", "NONE", "MIN", "MAX"}
    assert [m.name for m in ops.QuantType] == ["Linear", "Normal", "Uniform", "E3M0", "E2M1"]
    assert [m.name for m in ops.DType] == ["FP16", "BF16", "FP32"] and ops.SUM is ops.ReduceOP.SUM


@pytest.mark.parametrize("dtype", (ops.FP16, ops.BF16, ops.FP32))
@pytest.mark.parametrize("bit,group,compact", [(8, 64, False), (8, 16, True), (4, 32, True)])
def test_quantize_matches_the_oracle_and_round_trips(dtype, bit, group, compact):
    x = _x(group * 5 + 7, DT[dtype])
    cfg = CompressionConfig(bit=bit, group_size=group, compact=compact, allow_experimental=True)
    payload = ops.quantize(x, group, 0, False, bit, ops.Linear, compact)
    assert torch.equal(payload, oracle.encode(x, cfg))
    again = torch.empty_like(payload)
    ops.inplace_quantize(x, again, group, 0, False, bit, ops.Linear, compact)
    assert torch.equal(again, payload)
    back = ops.dequantize(payload, group, 0, bit, ops.NONE, ops.Linear, dtype, compact)
    assert back.dtype == DT[dtype] and back.numel() == group * 6            # whole groups, padding included
    assert torch.equal(back[: x.numel()], oracle.decode(payload, x.numel(), cfg, oracle.dtype_name(x)))
    into = torch.zeros(x.numel(), dtype=DT[dtype])
    ops.inplace_dequantize(payload, into, group, 0, bit, ops.NONE, ops.Linear, compact)
    ops.inplace_dequantize(payload, into, group, 0, bit, ops.SUM, ops.Linear, compact)
    twice = oracle.decode_accumulate(payload, oracle.decode(payload, x.numel(), cfg, oracle.dtype_name(x)), cfg)
    assert torch.equal(into, twice)
    with pytest.raises(ValueError):
        ops.inplace_dequantize(payload, into, group, 0, bit, ops.MAX, ops.Linear, compact)


def test_pack_reads_the_residual_and_declines_general_profiles():
    x, r = _x(300, torch.bfloat16, 1), _x(300, torch.bfloat16, 2)
    cfg = CompressionConfig(compact=True)
    kept = r.clone()
    out = torch.empty(oracle.encode(x, cfg).numel(), dtype=torch.uint8)
    assert ops.inplace_quantize_pack(x, out, r, 64, 0, False, 8, ops.Linear, True) is True
    assert torch.equal(out, oracle.encode(x, cfg, residual=kept)) and torch.equal(r, kept)
    assert ops.inplace_quantize_pack(x, out, None, 64, 1, False, 8, ops.Linear, True) is False      # top-k
    assert ops.inplace_quantize_pack(x, out, None, 64, 0, False, 4, ops.Normal, True) is False      # code-book


def test_fused_reduce_and_error_feedback_forms_agree():
    n, w = 64 * 9 + 5, 4
    xs = [_x(n, torch.float16, 10 + i) for i in range(w)]
    cfg = CompressionConfig()
    payloads = [ops.quantize(x, 64, 0, False, 8) for x in xs]
    y, y32 = oracle.reduce_mean(payloads, n, cfg, "fp16", float(w))
    out = torch.empty(n, dtype=torch.float16)
    assert ops.inplace_dequantize_reduce_mean(payloads, out, 64, 0, 8, ops.Linear, False, w) is True
    assert torch.equal(out, y)
    summed = ops.dequantize_reduce(payloads, 64, 0, 8, ops.Linear, ops.FP16, False)
    direct = torch.empty(n, dtype=torch.float16)
    ops.inplace_dequantize_reduce(payloads, direct, 64, 0, 8)
    assert torch.equal(summed[:n], direct)
    prepared = xs[0]
    residual, restored = torch.zeros_like(prepared), torch.empty_like(prepared)
    assert ops.inplace_dequantize_reduce_mean_update_error_feedback(payloads, prepared, restored, residual, 64, 0, 8,
                                                                     ops.Linear, False, w)
    assert torch.equal(restored, y) and torch.equal(residual, oracle.residual_update(prepared, y32))
    padded_prepared = torch.cat([prepared, torch.zeros(64 * 10 - n, dtype=torch.float16)])
    residual2 = torch.zeros_like(padded_prepared)
    restored2 = ops.dequantize_reduce_update_error_feedback(payloads, padded_prepared, residual2, 64, 0, 8, ops.Linear,
                                                            ops.FP16, False, w)
    assert torch.equal(restored2[:n], y) and torch.equal(residual2[:n], residual)
    plain = torch.zeros_like(prepared)
    ops.inplace_error_feedback_update(prepared, restored, plain)
    assert torch.equal(plain, oracle.residual_update_from_restored(prepared, restored))
    with pytest.raises(ValueError):
        ops.inplace_dequantize_reduce_mean(payloads, out, 64, 0, 8, ops.Linear, False, 0)
    assert ops.inplace_dequantize_reduce_mean(payloads, out, 64, 2, 8, ops.Linear, False, w) is False


@pytest.mark.gpu
def test_cuda_tensors_give_the_cpu_bytes(ext):
    x, r = _x(64 * 33 + 9, torch.bfloat16, 5), _x(64 * 33 + 9, torch.bfloat16, 6)
    cpu = torch.empty(oracle.encode(x, CompressionConfig(compact=True)).numel(), dtype=torch.uint8)
    gpu = torch.empty_like(cpu, device="cuda")
    assert ops.inplace_quantize_pack(x, cpu, r, 64, 0, False, 8) and ops.inplace_quantize_pack(x.cuda(), gpu, r.cuda(), 64, 0, False, 8)
    assert torch.equal(gpu.cpu(), cpu)
    back_cpu = ops.dequantize(cpu, 64, 0, 8, ops.NONE, ops.Linear, ops.BF16, True)
    back_gpu = ops.dequantize(gpu, 64, 0, 8, ops.NONE, ops.Linear, ops.BF16, True)
    assert torch.equal(back_gpu.cpu().view(torch.uint8), back_cpu.view(torch.uint8))
    out_cpu, out_gpu = torch.empty_like(x), torch.empty_like(x, device="cuda")
    assert ops.inplace_dequantize_reduce_mean([cpu, cpu], out_cpu, 64, 0, 8, ops.Linear, True, 2)
    assert ops.inplace_dequantize_reduce_mean([gpu, gpu], out_gpu, 64, 0, 8, ops.Linear, True, 2)
    assert torch.equal(out_gpu.cpu().view(torch.uint8), out_cpu.view(torch.uint8))
