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
