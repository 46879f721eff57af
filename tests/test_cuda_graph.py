"""`CompileConfig.enabled` -> CUDA-graph replay of the DiT forward: same numbers as the eager forward, one graph per
call signature, eager fallback where a call cannot be captured."""

import pytest
import torch

from telefuser_b200.core.config import CompileConfig
from telefuser_b200.core.cuda_graph import GraphRunner, _signature
from telefuser_b200.models.wan_dit import WanModel


def test_signature_tells_shapes_dtypes_and_scalars_apart():
    a, b = torch.zeros(2, 3), torch.zeros(2, 3)
    assert _signature(((a,), {"k": 1})) == _signature(((b,), {"k": 1}))
    assert _signature(((a,), {"k": 1})) != _signature(((a,), {"k": 2}))
    assert _signature(((a,), {})) != _signature(((a.bfloat16(),), {}))
    assert _signature(((a,), {})) != _signature(((torch.zeros(3, 2),), {}))


def test_cpu_calls_run_eagerly_and_the_switch_follows_the_model_state():
    model = WanModel(dim=64, ffn_dim=128, num_heads=2, num_layers=1, text_dim=32).eval()
    x, t, ctx = torch.randn(1, 16, 1, 8, 8), torch.tensor([500.0]), torch.randn(1, 4, 32)
    want = model(x, t, ctx)
    model.compile(CompileConfig(enabled=True))
    assert model.graph_capture and model.graph_capturable()
    assert torch.equal(model(x, t, ctx), want) and model._graph_runner.stats()["eager_calls"] == 1
    model.usp_flag = True
    assert not model.graph_capturable()
    model.usp_flag = False
    model.compile(CompileConfig(enabled=False))
    assert not model.graph_capture and model._graph_runner is None


@pytest.mark.gpu
def test_graph_replay_matches_the_eager_forward():
    torch.manual_seed(0)
    model = WanModel(dim=256, ffn_dim=512, num_heads=2, num_layers=2, text_dim=256).cuda().bfloat16().eval()
    xs = [torch.randn(1, 16, 3, 16, 16, device="cuda", dtype=torch.bfloat16) for _ in range(3)]
    ts = [torch.tensor([t], device="cuda") for t in (900.0, 500.0, 100.0)]
    ctx = torch.randn(1, 32, 256, device="cuda", dtype=torch.bfloat16)
    want = [model(x, t, ctx) for x, t in zip(xs, ts)]
    model.compile(CompileConfig(enabled=True))
    got = [model(x, t, ctx) for x, t in zip(xs, ts)]
    for g, w in zip(got, want):
        assert torch.equal(g, w)
    st = model._graph_runner.stats()
    assert st == {"graphs": 1, "replays": 3, "eager_calls": 0}
    model(torch.randn(1, 16, 2, 16, 16, device="cuda", dtype=torch.bfloat16), ts[0], ctx)  # another shape: second graph
    assert model._graph_runner.stats()["graphs"] == 2
    from telefuser_b200.ops import native

    assert native.last_status() == 0


@pytest.mark.gpu
def test_runner_falls_back_when_too_many_shapes_are_seen():
    r = GraphRunner(lambda x: x * 2 + 1, warmup=1, max_graphs=2)
    for n in (4, 8, 16, 32):
        x = torch.arange(n, device="cuda", dtype=torch.float32)
        assert torch.equal(r(x), x * 2 + 1)
    assert r.stats()["graphs"] == 2 and r.stats()["eager_calls"] == 2
