"""Wire compatibility with the unmodified reference, checked directly: the payload bytes of this library's
kernels must equal the bytes of the reference's own CUDA extension for the same input, and each side must
decode the other's payload to the same values.  Needs the reference install under baseline/_ref (skipped
without it); runs both extensions in one process on one GPU."""

import os
import sys

import pytest
import torch

from lowbit_comm_b200.config import CompressionConfig
from lowbit_comm_b200.ops import codec

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DT = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}


@pytest.fixture(scope="module")
def reference():
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    try:
        import reference_env

        ok, why = reference_env.reference_available()
        if not ok:
            pytest.skip(why)
        _, status = reference_env.activate(need_cuda_extension=True)
        from ccdl_comm.config import CompressionConfig as RefConfig
        from ccdl_comm.quantization import codec as ref_codec
    except ImportError as exc:
        pytest.skip(f"reference not importable: {exc}")
    return ref_codec, RefConfig, status


def _input(n, dtype, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(n, generator=g, device="cuda") * 10 ** torch.empty(n, device="cuda").uniform_(-4, 1, generator=g)
    return x.to(DT[dtype])


@pytest.mark.parametrize("dtype", ("bf16", "fp16", "fp32"))
@pytest.mark.parametrize("bit,group", [(8, 64), (8, 32), (4, 16)])
@pytest.mark.parametrize("compact", (False, True))
@pytest.mark.parametrize("topk", (0, 1, 2))
def test_payload_bytes_and_cross_decoding(ext, reference, dtype, bit, group, compact, topk):
    ref_codec, RefConfig, status = reference
    kw = dict(bit=bit, group_size=group, topk=topk, compact=compact, allow_experimental=True)
    ours_cfg, ref_cfg = CompressionConfig(**kw), RefConfig(**kw)
    # ragged tails only without top-k: in a zero-padded group the top-k index among equal zeros is arbitrary
    n = group * 37 + (7 if topk == 0 else 0)
    x = _input(n, dtype, seed=bit * 100 + group + topk)
    mine = codec.quantize_tensor(x, ours_cfg)
    theirs = ref_codec.quantize_tensor(x.clone(), ref_cfg, extension_status=status)
    torch.cuda.synchronize()
    assert mine.dtype == theirs.dtype == torch.uint8 and mine.numel() == theirs.numel()
    assert torch.equal(mine, theirs.reshape(-1)), "payload bytes differ"
    a = codec.dequantize_tensor(theirs.reshape(-1).contiguous(), x.shape, ours_cfg, dtype=dtype)
    b = ref_codec.dequantize_tensor(mine, tuple(x.shape), ref_cfg, dtype=dtype, extension_status=status)
    torch.cuda.synchronize()
    if topk > 0 and bit == 4 and group == 16 and not compact:
        # Measured on B200: for this corner (planar layout, 4-bit, groups of 16, top-k outliers) the reference's
        # decoder returns values unrelated to the input in the tail of the tensor, although its encoder's bytes
        # equal ours and its compact-layout decoder agrees with ours.  Our decoder is held to the oracle here.
        from lowbit_comm_b200.ops import oracle

        want = oracle.decode(theirs.reshape(-1).cpu(), n, ours_cfg, dtype)
        assert torch.equal(a.cpu().view(torch.uint8), want.view(torch.uint8)), "our decode differs from the oracle"
        close = (a.float() - x.float()).abs().max().item() <= x.float().abs().max().item() / 7 + 1e-6
        assert close, "our decode is not within one 4-bit step of the input"
        return
    assert torch.equal(a.view(torch.uint8), b.reshape(x.shape).view(torch.uint8)), "decoded values differ"


@pytest.mark.parametrize("dtype", ("bf16", "fp16"))
@pytest.mark.parametrize("count", (2, 8))
def test_fused_mean_of_payloads_agrees(ext, reference, dtype, count):
    ref_codec, RefConfig, status = reference
    ours_cfg, ref_cfg = CompressionConfig(), RefConfig()
    n = 64 * 129 + 5
    xs = [_input(n, dtype, seed=50 + r) for r in range(count)]
    payloads = [codec.quantize_tensor(x, ours_cfg) for x in xs]
    mine = codec.dequantize_reduce_tensors(payloads, xs[0].shape, ours_cfg, dtype=dtype, reduce="mean")
    theirs = ref_codec.dequantize_reduce_tensors([p.clone() for p in payloads], tuple(xs[0].shape), ref_cfg,
                                                 dtype=dtype, extension_status=status, reduce="mean")
    torch.cuda.synchronize()
    # same payloads, fp32 accumulation on both sides; the last rounding may differ by one unit of the source dtype
    # where the two kernels contract multiply-adds differently
    assert torch.allclose(mine.float(), theirs.reshape(mine.shape).float(), rtol=2 ** -7, atol=1e-9)
    same = (mine.view(torch.int16) == theirs.reshape(mine.shape).view(torch.int16)).float().mean().item()
    assert same > 0.99, same
