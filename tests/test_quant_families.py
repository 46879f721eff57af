"""Every quantised weight format through `enable_quant` of every DiT family that has linears worth quantising: the
converted model still runs and stays close to its full-precision output (CPU: the fp32 evaluation of each format)."""

import importlib.util
import sys
from pathlib import Path

import pytest
import torch

HERE = Path(__file__).resolve().parent
LIMITS = {"fp8": 0.12, "int8": 0.06, "mxfp8": 0.12, "nvfp4": 0.45, "nf4": 0.40}
WEIGHT_DTYPE = {"fp8": torch.float8_e4m3fn, "mxfp8": torch.float8_e4m3fn, "int8": torch.int8, "nvfp4": torch.uint8, "nf4": torch.uint8}


def load_test_module(name: str):
    spec = importlib.util.spec_from_file_location(f"_family_{name}", HERE / f"{name}.py")
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod
    spec.loader.exec_module(mod)
    return mod


def flux2_case():
    t = load_test_module("test_flux2")
    m = t.small(head_dim=64, heads=2, in_channels=64)
    x, e, ts = torch.randn(1, 8 * 8, 64), torch.randn(1, 6, 48), torch.tensor([0.7])
    ids, tids = t.P.latent_ids(8, 8), t.P.text_ids(6)
    return m, lambda mm: mm(x, e, ts, ids, tids), "transformer_blocks"


def qwen_case():
    t = load_test_module("test_qwen_image")
    m = t.small(head_dim=64, axes=(16, 24, 24))
    lat, ts, emb = torch.randn(1, 16, 16, 16), torch.tensor([700.0]), torch.randn(1, 7, 48)
    return m, lambda mm: mm(lat, ts, emb), "transformer_blocks"


def z_image_case():
    t = load_test_module("test_z_image")
    m = t.small(head_dim=64, axes=(16, 24, 24))
    x, caps, ts = [torch.randn(16, 1, 16, 16)], [torch.randn(9, 24)], torch.tensor([0.4])
    return m, lambda mm: mm(x, ts, caps)[0], "layers"


def lingbot_video_case():  # no `enable_quant` of its own: the BaseModel default over its block list
    from telefuser_b200.testing.lingbot_video_checks import make_inputs, make_model

    m = make_model("tiny", hidden_size=128, num_attention_heads=2, intermediate_size=256)
    x, ts, txt = make_inputs(text_dim=m.config.text_dim, size=8)
    return m, lambda mm: mm(x, ts, txt), "blocks"


def wan_case():
    t = load_test_module("test_wan_dit")
    m = t._tiny()
    x, ctx, ts = torch.randn(1, 16, 3, 8, 8), torch.randn(1, 16, 256), torch.tensor([500.0])
    return m, lambda mm: mm(x, ts, ctx), "blocks"


def hunyuan_case():  # BaseModel default; its attention keeps METHODS named like cache slots of other families
    t = load_test_module("test_hunyuan_video")
    m = t.small(head_dim=64, axes=(16, 24, 24))
    x, ts = torch.randn(1, 9, 2, 4, 4), torch.tensor([600.0])
    txt, mask = torch.randn(1, 7, 24), torch.tensor([[1, 1, 1, 1, 1, 0, 0]])
    return m, lambda mm: mm(x, ts, txt, None, mask), "double_blocks"


def longcat_case():  # BaseModel default
    t = load_test_module("test_longcat")
    m = t.small(head_dim=64)
    x, y = torch.randn(1, 16, 3, 8, 8), torch.randn(1, 1, 6, 24)
    mask, ts = torch.tensor([[1, 1, 1, 1, 0, 0]]), torch.tensor([[600.0, 600.0, 600.0]])
    return m, lambda mm: mm(x, ts, y, mask), "blocks"


def ltx_case():
    from telefuser_b200.models import ltx_dit as D

    net = D.LTXVideoTransformer({"transformer": dict(num_attention_heads=2, attention_head_dim=64, num_layers=1, cross_attention_dim=128,
                                                      audio_num_attention_heads=2, audio_attention_head_dim=32, audio_cross_attention_dim=64)},
                                D.LTXModelType.VideoOnly)  # fmt: skip
    for p in net.parameters():
        torch.nn.init.normal_(p, std=0.05)
    net = net.float().eval()
    mod = D.Modality(latent=torch.randn(1, 6, 128), sigma=torch.tensor([0.5]), timesteps=torch.full((1, 6, 1), 0.5),
                     positions=torch.rand(1, 3, 6, 2), context=torch.randn(1, 4, 128))  # fmt: skip
    return net, lambda mm: mm(mod, None)[0], "velocity_model.transformer_blocks"


def liveact_case():  # BaseModel default; driven through its denoising stage (KV caches, audio conditioning)
    from telefuser_b200.core.config import ModelRuntimeConfig

    t = load_test_module("test_liveact")
    dit = t.small_dit(head_dim=64)
    noise, y = torch.randn(16, 6, 8, 8), torch.randn(1, 20, 14, 8, 8)
    ctx, clip, audio = torch.randn(1, 4, 24), torch.randn(1, 257, 20), torch.randn(1, 1 + 4 * 13, 5, 2, 32)

    def run(model):
        stage = t.LiveActDenoisingStage("denoise", None, ModelRuntimeConfig(device_type="cpu", torch_dtype=torch.float32), dit=model)
        stage.onload_models_flag = True
        return stage.process(noise.clone(), ctx, clip, audio, y, 16)

    return dit, run, "blocks"


CASES = {"wan": wan_case, "ltx": ltx_case, "flux2": flux2_case, "qwen_image": qwen_case, "z_image": z_image_case,
         "lingbot_video": lingbot_video_case, "hunyuan_video": hunyuan_case, "longcat": longcat_case,
         "liveact": liveact_case}  # fmt: skip


@pytest.mark.parametrize("kind", list(LIMITS))
@pytest.mark.parametrize("family", list(CASES))
def test_every_format_on_every_family(family, kind):
    torch.manual_seed(0)
    model, run, block_list = CASES[family]()
    with torch.no_grad():
        ref = run(model)
        n = model.enable_quant(kind)
        assert n > 0
        blocks = model.get_submodule(block_list)
        dtypes = {m.weight.dtype for m in blocks.modules() if isinstance(m, torch.nn.Linear)}
        assert WEIGHT_DTYPE[kind] in dtypes, (dtypes, kind)
        out = run(model)
    assert out.shape == ref.shape and torch.isfinite(out).all()
    err = ((out.float() - ref.float()).norm() / ref.float().norm()).item()
    assert err < LIMITS[kind], (family, kind, err)


def test_resolve_quant_kind_reads_configs_types_and_names():
    from telefuser_b200.core.config import QuantConfig, QuantType
    from telefuser_b200.ops.quant import resolve_quant_kind

    assert resolve_quant_kind(None) == "fp8" and resolve_quant_kind("FP8") == "fp8" and resolve_quant_kind(torch.int8) == "int8"
    assert resolve_quant_kind(QuantType.MXFP8) == "mxfp8" and resolve_quant_kind(QuantType.NVFP4) == "nvfp4"
    assert resolve_quant_kind(QuantType.BNB_NF4) == "nf4" and resolve_quant_kind("nf4") == "nf4"
    assert resolve_quant_kind(QuantConfig(enabled=True, quant_type=QuantType.INT8)) == "int8"
    assert resolve_quant_kind(QuantType.TORCHAO_FP8) == "fp8"
    assert resolve_quant_kind(QuantType.MXFP4) == "nvfp4" and resolve_quant_kind(QuantType.MXFP6) == "mxfp8"  # nearest run-time formats


@pytest.mark.parametrize("family", list(CASES))
def test_every_family_builds_without_weight_storage_and_adopts_a_checkpoint(family):
    """What `ModuleManager` does for every checkpoint: construct with parameters on the meta device (constructor constants
    and buffers stay real), adopt the tensors, run. The result must equal the model the tensors came from, bit for bit."""
    from telefuser_b200.utils.model_weight import init_weights_on_device

    torch.manual_seed(0)
    model, run, _ = CASES[family]()
    state = {k: v.detach().clone() for k, v in model.state_dict().items()}
    moves = torch.nn.Module.to
    torch.nn.Module.to = lambda self, *a, **k: self  # the test builders cast / move; the loader does that after adopting
    try:
        with init_weights_on_device("meta"):
            empty, _, _ = CASES[family]()
    finally:
        torch.nn.Module.to = moves
    params = list(empty.parameters())
    assert params and all(p.is_meta for p in params), [n for n, p in empty.named_parameters() if not p.is_meta][:3]
    assert not any(b.is_meta for b in empty.buffers())
    missing, unexpected = empty.load_state_dict(state, assign=True, strict=False)
    assert not unexpected and not [k for k in missing if k in dict(empty.named_parameters())]
    assert not any(p.is_meta for p in empty.parameters())
    with torch.no_grad():
        want, got = run(model), run(empty)  # the same inputs for both
    assert torch.equal(got, want)
