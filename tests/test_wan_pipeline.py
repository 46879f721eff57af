"""Wan2.1 pipeline end to end on CPU with tiny random-init components."""
import torch

from telefuser_b200.core.config import ModelRuntimeConfig
from telefuser_b200.core.module_manager import ModuleManager
from telefuser_b200.models.umt5 import WanTextEncoder
from telefuser_b200.models.wan_dit import WanModel
from telefuser_b200.models.wan_vae import WanVideoVAE
from telefuser_b200.pipelines.wan.stages import TextEncodingStage
from telefuser_b200.pipelines.wan.wan21_video import Wan21VideoPipeline, Wan21VideoPipelineConfig, discover_wan_components
from telefuser_b200.testing.synthetic import HashTokenizer, random_init_


def tiny_pipeline():
    torch.manual_seed(0)
    dit = random_init_(WanModel(dim=64, ffn_dim=128, num_heads=2, num_layers=1, text_dim=32).float())
    dit.dtype = torch.float32
    vae = random_init_(WanVideoVAE(dim=8).float(), std=0.05)
    te = random_init_(WanTextEncoder(vocab=128, dim=32, dim_attn=32, dim_ffn=64, num_heads=2, num_layers=1).float())
    mm = ModuleManager(torch_dtype=torch.float32, device="cpu")
    mm.add_module(dit.eval(), "wan_video_dit")
    mm.add_module(vae.eval(), "wan_video_vae")
    mm.add_module(te.eval(), "wan_video_text_encoder")
    rc = lambda: ModelRuntimeConfig(device_type="cpu", torch_dtype=torch.float32)  # noqa: E731
    cfg = Wan21VideoPipelineConfig(vae_config=rc(), dit_config=rc(), clip_config=rc(), text_encoding_config=rc())
    pipe = Wan21VideoPipeline(device="cpu", torch_dtype=torch.float32)
    ts = TextEncodingStage("text", mm, rc(), text_encoder=te, tokenizer=HashTokenizer(128, 16))
    pipe.init(mm, cfg, text_stage=ts)
    return pipe


def test_t2v_call_returns_frames_and_is_seeded():
    pipe = tiny_pipeline()
    frames = pipe("a cat on a skateboard", num_frames=5, height=32, width=32, num_inference_steps=2, seed=3)
    assert len(frames) == 5 and frames[0].size == (32, 32)
    a = pipe("a cat on a skateboard", num_frames=5, height=32, width=32, num_inference_steps=2, seed=3, output_type="pt")
    b = pipe("a cat on a skateboard", num_frames=5, height=32, width=32, num_inference_steps=2, seed=3, output_type="pt")
    c = pipe("a dog", num_frames=5, height=32, width=32, num_inference_steps=2, seed=3, output_type="pt")
    assert a.shape == (1, 3, 5, 32, 32) and torch.equal(a, b) and not torch.equal(a, c)
    assert pipe.last_call_seconds is not None
    assert pipe.dump_config()["pipeline"] == "Wan21VideoPipeline"


def test_num_frames_rounding_and_size_check():
    pipe = tiny_pipeline()
    out = pipe("x", num_frames=6, height=30, width=32, num_inference_steps=1, seed=0, cfg_scale=1.0, output_type="pt")
    assert out.shape == (1, 3, 9, 32, 32)


def test_component_discovery(tmp_path):
    for f in ("diffusion_pytorch_model-00001-of-00002.safetensors", "diffusion_pytorch_model-00002-of-00002.safetensors",
              "models_t5_umt5-xxl-enc-bf16.pth", "Wan2.1_VAE.pth"):
        (tmp_path / f).write_bytes(b"")
    c = discover_wan_components(str(tmp_path))
    assert len(c["dit"]) == 2 and c["vae"].endswith("Wan2.1_VAE.pth") and "t5" in c["text_encoder"]


def test_from_pretrained_on_a_model_folder_end_to_end(tmp_path, monkeypatch):
    """`Wan21VideoPipeline.from_pretrained(folder)(prompt, num_frames, height, width)` on real files in the published
    layout (tiny widths): component discovery, meta-device construction with adopted weights (constants a constructor
    computes, such as the VAE's latent statistics, must stay real tensors), text encode, denoise, decode."""
    import telefuser_b200.models.umt5 as U
    from telefuser_b200.models.umt5 import WanTextEncoder
    from telefuser_b200.models.wan_dit import WanModel, WanModelConfig
    from telefuser_b200.models.wan_vae import WanVideoVAE
    from telefuser_b200.pipelines.wan.wan21_video import Wan21VideoPipeline
    from telefuser_b200.testing.synthetic import HashTokenizer, random_init_
    from telefuser_b200.utils.model_weight import init_weights_on_device, save_state_dict

    torch.manual_seed(0)
    cfg = WanModelConfig.preset("tiny")
    dit = random_init_(WanModel.from_config(cfg).float())
    vae = random_init_(WanVideoVAE(dim=8).float(), std=0.05)
    te = random_init_(WanTextEncoder(vocab=4096, dim=cfg.text_dim, dim_attn=cfg.text_dim, dim_ffn=2 * cfg.text_dim,
                                     num_heads=max(1, cfg.text_dim // 64), num_layers=2).float())  # fmt: skip
    save_state_dict(dit.state_dict(), str(tmp_path / "diffusion_pytorch_model.safetensors"))
    torch.save(vae.state_dict(), tmp_path / "Wan2.1_VAE.pth")
    torch.save(te.state_dict(), tmp_path / "models_t5_umt5-xxl-enc-bf16.pth")
    monkeypatch.setattr(U, "HuggingfaceTokenizer", lambda *a, **k: HashTokenizer(4096, 32))  # no tokenizer files offline

    pipe = Wan21VideoPipeline.from_pretrained(str(tmp_path), device="cpu", torch_dtype=torch.float32)
    loaded_vae = pipe.vae_stage.vae
    assert loaded_vae.mean.device.type == "cpu" and torch.equal(loaded_vae.mean, vae.mean) and not any(p.is_meta for p in loaded_vae.parameters())
    assert torch.equal(pipe.denoise_stage.dit.blocks[0].self_attn.q.weight, dit.blocks[0].self_attn.q.weight)
    frames = pipe("a red fox", num_frames=5, height=32, width=32, num_inference_steps=2, seed=1)
    assert len(frames) == 5 and frames[0].size == (32, 32)
    again = pipe("a red fox", num_frames=5, height=32, width=32, num_inference_steps=2, seed=1)
    assert all(a.tobytes() == b.tobytes() for a, b in zip(frames, again))
    pipe.close()

    # the construction context on its own: parameters without storage, everything else real, no initialiser run
    class WithConstants(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.lin = torch.nn.Linear(64, 64)
            self.table = torch.arange(4.0)  # a plain attribute
            self.register_buffer("freqs", torch.ones(3), persistent=False)

    calls = []
    real = torch.nn.init.kaiming_uniform_
    monkeypatch.setattr(torch.nn.init, "kaiming_uniform_", lambda t, *a, **k: calls.append(1) or real(t, *a, **k))
    with init_weights_on_device("meta"):
        m = WithConstants()
    assert m.lin.weight.is_meta and m.lin.bias.is_meta and m.lin.weight.requires_grad
    assert not m.table.is_meta and m.table.tolist() == [0.0, 1.0, 2.0, 3.0] and not m.freqs.is_meta and calls == []
    torch.nn.Linear(4, 4)
    assert calls == [1] and torch.nn.Module.register_parameter.__name__ == "register_parameter"  # everything restored
    with init_weights_on_device("meta", include_buffers=True):
        assert WithConstants().freqs.is_meta
