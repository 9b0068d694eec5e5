"""Benchmark models (tiny instances on CPU, parameter counts of the named configurations on the meta device)
and the small utilities around the benchmarks."""

import pytest
import torch

from lowbit_comm_b200.models import GPT2, GPT2Config, Llama, LlamaConfig
from lowbit_comm_b200.utils import roofline, tracing


def _params(model) -> int:
    return sum(p.numel() for p in model.parameters())


@pytest.mark.parametrize("cls,cfg", [(GPT2, GPT2Config.tiny()), (Llama, LlamaConfig.tiny())])
def test_tiny_models_train_one_step(cls, cfg):
    torch.manual_seed(0)
    model = cls(cfg)
    tok = torch.randint(0, cfg.vocab_size, (2, cfg.seq_len + 1))
    loss = model(tok[:, :-1], tok[:, 1:])
    assert loss.ndim == 0 and torch.isfinite(loss)
    assert abs(loss.item() - torch.log(torch.tensor(float(cfg.vocab_size))).item()) < 1.0    # near uniform at init
    loss.backward()
    grads = [p.grad for p in model.parameters()]
    assert all(g is not None and torch.isfinite(g).all() for g in grads)
    logits = model(tok[:, :-1])
    assert logits.shape == (2, cfg.seq_len, cfg.vocab_size)


def test_named_configurations_have_the_advertised_size():
    with torch.device("meta"):
        gpt2 = GPT2(GPT2Config())
        llama = Llama(LlamaConfig())
    assert _params(gpt2) == 124_439_808                       # GPT-2 small with tied embeddings
    assert 3.0e9 < _params(llama) < 3.7e9                     # "Llama-style 3B": 28 layers, d 3072, 24 / 8 heads
    c = LlamaConfig()
    assert (c.n_layer, c.d_model, c.n_head, c.n_kv_head, c.d_ff, c.vocab_size, c.seq_len) == \
        (28, 3072, 24, 8, 8192, 128256, 2048)
    g = GPT2Config()
    assert (g.n_layer, g.d_model, g.n_head, g.vocab_size, g.seq_len) == (12, 768, 12, 50257, 1024)


def test_roofline_model():
    assert roofline.payload_factor() == pytest.approx(66 / 128)
    assert roofline.payload_factor(group_size=16, bit=4, element_bytes=4) == pytest.approx((8 + 4) / 64)
    nbytes = 64 << 20
    two = roofline.fused_all_reduce_roofline(nbytes, 8, stages=2, hbm_gbs=6552.3)
    one = roofline.fused_all_reduce_roofline(nbytes, 8, stages=1, hbm_gbs=6552.3)
    payload = nbytes * 66 / 128
    assert two["link_bytes"] == pytest.approx(2 * payload * 7 / 8) and one["link_bytes"] == pytest.approx(7 * payload)
    assert two["bound"] == "hbm" and one["bound"] == "nvlink"
    assert two["roofline_us"] == max(two["t_hbm_us"], two["t_link_us"])
    no_ef = roofline.fused_all_reduce_roofline(nbytes, 8, stages=2, error_feedback=False, hbm_gbs=6552.3)
    assert no_ef["hbm_bytes"] == pytest.approx(2 * nbytes + 4 * payload) and no_ef["bound"] == "nvlink"
    gbs, kind = roofline.measured_hbm_gbs("/nonexistent")
    assert (gbs, kind) == (roofline.FALLBACK_HBM_GBS, "fallback")


def test_tracing_is_a_no_op_unless_enabled(monkeypatch):
    monkeypatch.setattr(tracing, "ENABLED", False)
    with tracing.nvtx_range("phase"):
        pass                                           # must not touch torch.cuda on a CPU box
    timer = tracing.PhaseTimer()
    timer.flush()                                      # nothing marked: nothing to do
    assert timer.summary() == {}


def test_kernel_names_is_empty_without_a_gpu_and_counts_device_events_with_a_fake():
    import types

    import torch

    from lowbit_comm_b200.utils.tracing import kernel_names

    if not torch.cuda.is_available():
        assert kernel_names(lambda: torch.ones(4) + 1) == {}

    class Profile:
        def __init__(self, activities):
            self.activities = activities

        def __enter__(self):
            return self

        def __exit__(self, *exc):
            return False

        def events(self):
            make = types.SimpleNamespace
            return [make(name="quant_push_tiled_kernel", device_type="DeviceType.CUDA"),
                    make(name="aten::add", device_type="DeviceType.CPU"),
                    make(name="quant_push_tiled_kernel", device_type="DeviceType.CUDA"),
                    make(name="reduce_kernel", device_type="DeviceType.CUDA")]

    ran = []
    fake = types.SimpleNamespace(
        profiler=types.SimpleNamespace(profile=lambda activities: Profile(activities),
                                       ProfilerActivity=types.SimpleNamespace(CPU="cpu", CUDA="cuda")),
        cuda=types.SimpleNamespace(is_available=lambda: True, synchronize=lambda: ran.append("sync")))
    counts = kernel_names(lambda: ran.append("fn"), torch_module=fake)
    assert counts == {"quant_push_tiled_kernel": 2, "reduce_kernel": 1} and ran == ["fn", "sync"]


def test_trace_switch_puts_one_nvtx_range_around_every_bucket(monkeypatch):
    """LBC_TRACE=1: the hook wraps each bucket in a named NVTX range on the host timeline; off, it calls nothing."""

    import torch

    from lowbit_comm_b200.parallel.ddp_hook import DDPCommHook
    from lowbit_comm_b200.utils import tracing

    calls = []
    monkeypatch.setattr(torch.cuda.nvtx, "range_push", lambda name: calls.append(("push", name)))
    monkeypatch.setattr(torch.cuda.nvtx, "range_pop", lambda: calls.append(("pop",)))

    class Bucket:
        def index(self):
            return 3

        def buffer(self):
            return torch.zeros(4)

    hook = DDPCommHook(lambda bucket: calls.append(("bucket",)) or bucket.buffer(), torch.futures.Future)
    monkeypatch.setattr(tracing, "ENABLED", False)
    hook(None, Bucket())
    assert calls == [("bucket",)]
    calls.clear()
    monkeypatch.setattr(tracing, "ENABLED", True)
    assert hook(None, Bucket()).wait().numel() == 4
    assert calls == [("push", "lbc.ddp_bucket[3]"), ("bucket",), ("pop",)]
