"""`from_pretrained` of the Wan2.2 pipelines: component discovery in both folder layouts, expert order, module names
and runtime configuration. Checkpoint reading is replaced by tiny random models (the loaders' file handling is
covered by tests/test_module_manager.py and tests/test_hf_model_analyzer.py)."""

import json

import pytest
import torch

from telefuser_b200.core.module_manager import ModuleManager
from telefuser_b200.models.wan_dit import WanModel
from telefuser_b200.pipelines.wan import wan22_video as W
from telefuser_b200.testing.synthetic import HashTokenizer


def _touch(path):
    path.parent.mkdir(parents=True, exist_ok=True)
    path.write_bytes(b"\0" * 8)


class _TinyVAE(torch.nn.Module):
    z_dim, upsampling_factor = 48, 16


class _TinyText(torch.nn.Module):
    def forward(self, ids, mask):
        return torch.zeros(ids.shape[0], ids.shape[1], 64)


@pytest.fixture
def fake_loading(monkeypatch):
    calls = []

    def load_model(self, file_path, device=None, torch_dtype=None, low_cpu_mem_usage=False, name=None, model_class=None,
                   model_resource="official", converter_kwargs=None, quant_config=None):  # fmt: skip
        calls.append((name, model_class.__name__, model_resource, file_path))
        if model_class is WanModel:
            module = WanModel(dim=64, ffn_dim=128, num_heads=2, num_layers=1, text_dim=64)
        elif "VAE" in model_class.__name__:
            module = _TinyVAE()
        else:
            module = _TinyText()
        self.add_module(module, name, path=file_path)
        return True

    monkeypatch.setattr(ModuleManager, "load_model", load_model)
    monkeypatch.setattr("telefuser_b200.models.umt5.HuggingfaceTokenizer", lambda *a, **k: HashTokenizer(4096, 32))
    return calls


def test_wan22_a14b_official_layout(tmp_path, fake_loading):
    root = tmp_path / "Wan2.2-T2V-A14B"
    for expert in ("high_noise_model", "low_noise_model"):
        for i in (1, 2):
            _touch(root / expert / f"diffusion_pytorch_model-0000{i}-of-00002.safetensors")
        (root / expert / "config.json").write_text(json.dumps({"_class_name": "WanModel"}))
    _touch(root / "models_t5_umt5-xxl-enc-bf16.pth")
    _touch(root / "Wan2.1_VAE.pth")
    pipe = W.Wan22VideoPipeline.from_pretrained(str(root), device="cpu", torch_dtype=torch.float32, sample_solver="mix-euler",
                                                parallel_devices=[0, 1, 2, 3], enable_vfi=False)  # fmt: skip
    names = [(n, c, r) for n, c, r, _ in fake_loading]
    assert names == [("wan_video_dit", "WanModel", "official"), ("wan_video_dit", "WanModel", "official"),
                     ("wan_video_vae", "WanVideoVAE", "official"), ("wan_video_text_encoder", "WanTextEncoder", "official")]
    assert "high_noise_model" in fake_loading[0][3][0] and "low_noise_model" in fake_loading[1][3][0]  # high-noise expert first
    assert len(fake_loading[0][3]) == 2
    cfg = pipe.config
    assert cfg.sample_solver == "mix-euler" and cfg.enable_denoising_parallel
    pc = cfg.dit_high_config.parallel_config
    assert (pc.cfg_degree, pc.sp_ulysses_degree, pc.device_ids) == (2, 2, [0, 1, 2, 3])
    pipe.close()


def test_wan22_ti2v_diffusers_layout_and_missing_parts(tmp_path, fake_loading):
    root = tmp_path / "Wan2.2-TI2V-5B-Diffusers"
    (root).mkdir()
    (root / "model_index.json").write_text(json.dumps({
        "transformer": ["diffusers", "WanTransformer3DModel"], "vae": ["diffusers", "AutoencoderKLWan"],
        "text_encoder": ["transformers", "UMT5EncoderModel"], "tokenizer": ["transformers", "T5TokenizerFast"]}))
    _touch(root / "transformer" / "diffusion_pytorch_model.safetensors")
    _touch(root / "vae" / "diffusion_pytorch_model.safetensors")
    _touch(root / "text_encoder" / "model.safetensors")
    (root / "tokenizer").mkdir()
    (root / "tokenizer" / "tokenizer_config.json").write_text("{}")
    pipe = W.Wan22TI2VPipeline.from_pretrained(str(root), device="cpu", torch_dtype=torch.float32)
    assert [(n, c, r) for n, c, r, _ in fake_loading] == [
        ("wan_video_dit", "WanModel", "diffusers"), ("wan22_video_vae", "Wan22VideoVAE", "official"),
        ("wan_video_text_encoder", "WanTextEncoder", "official")]
    assert pipe.z_dim == 48 and not pipe.config.enable_denoising_parallel
    assert isinstance(pipe.text_encoding_stage.tokenizer, HashTokenizer)  # built from the `tokenizer/` folder
    (root / "vae" / "diffusion_pytorch_model.safetensors").unlink()
    with pytest.raises(FileNotFoundError, match="a VAE"):
        W.Wan22TI2VPipeline.from_pretrained(str(root), device="cpu")
    with pytest.raises(FileNotFoundError, match="low-noise"):
        (root / "vae").rmdir()
        _touch(root / "vae" / "diffusion_pytorch_model.safetensors")
        W.Wan22VideoPipeline.from_pretrained(str(root), device="cpu")


def test_wan22_a14b_real_files_end_to_end(tmp_path, monkeypatch):
    """No stand-in for the loader: two expert checkpoints, VAE and text encoder as real (tiny) files in the official layout,
    loaded through `ModuleManager`, then one seeded generation across the expert boundary."""
    import telefuser_b200.models.umt5 as U
    from telefuser_b200.models.umt5 import WanTextEncoder
    from telefuser_b200.models.wan_dit import WanModelConfig
    from telefuser_b200.models.wan_vae import WanVideoVAE
    from telefuser_b200.testing.synthetic import random_init_
    from telefuser_b200.utils.model_weight import save_state_dict

    cfg = WanModelConfig.preset("tiny")
    experts = []
    for i, sub in enumerate(("high_noise_model", "low_noise_model")):
        (tmp_path / sub).mkdir()
        experts.append(random_init_(WanModel.from_config(cfg).float(), seed=i))
        save_state_dict(experts[-1].state_dict(), str(tmp_path / sub / "diffusion_pytorch_model.safetensors"))
    torch.save(random_init_(WanVideoVAE(dim=8).float(), std=0.05).state_dict(), tmp_path / "Wan2.1_VAE.pth")
    te = WanTextEncoder(vocab=4096, dim=cfg.text_dim, dim_attn=cfg.text_dim, dim_ffn=2 * cfg.text_dim, num_heads=max(1, cfg.text_dim // 64), num_layers=2)
    torch.save(random_init_(te.float()).state_dict(), tmp_path / "models_t5_umt5-xxl-enc-bf16.pth")
    monkeypatch.setattr(U, "HuggingfaceTokenizer", lambda *a, **k: HashTokenizer(4096, 32))
    pipe = W.Wan22VideoPipeline.from_pretrained(str(tmp_path), device="cpu", torch_dtype=torch.float32)
    stage = pipe.denoise_stage
    high, low = stage.dit_high, stage.dit_low
    assert torch.equal(high.blocks[0].ffn[0].weight, experts[0].blocks[0].ffn[0].weight)  # the high-noise expert runs first
    assert torch.equal(low.blocks[0].ffn[0].weight, experts[1].blocks[0].ffn[0].weight)
    frames = pipe("a red fox", num_frames=5, height=32, width=32, num_inference_steps=3, seed=1)
    assert len(frames) == 5 and frames[0].size == (32, 32)
    pipe.close()
