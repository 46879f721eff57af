"""Checkpoint loading: fingerprints, auto-detection, diffusers key renaming, sharded files."""
import json
import os

import torch

from telefuser_b200.core.model_registry import ModelRegistry
from telefuser_b200.core.module_manager import ModuleManager
from telefuser_b200.models.wan_dit import WanModel, WanModelConfig
from telefuser_b200.models.wan_dit_convert import infer_wan_config, rename_diffusers_key
from telefuser_b200.utils.model_weight import hash_state_dict_keys, load_state_dict, save_state_dict


def test_preset_fingerprints_equal_published_checkpoint_hashes():
    # The published Wan2.1 checkpoints are identified by these key+shape hashes.
    want = {"wan2.1-t2v-1.3b": "9269f8db9040a9d860eaca435be61814", "wan2.1-t2v-14b": "aafcfd9672c3a2456dc46e1cb6e52c70"}
    for name, h in want.items():
        with torch.device("meta"):
            m = WanModel.from_config(WanModelConfig.preset(name))
        assert hash_state_dict_keys(m.state_dict()) == h
    hashes = {e.keys_hash_with_shape for e in ModelRegistry.instance().entries()}
    assert set(want.values()) <= hashes


def _small():
    torch.manual_seed(0)
    return WanModel(dim=128, ffn_dim=256, num_heads=1, num_layers=2, text_dim=64)


def test_load_explicit_class_roundtrip_and_sharded(tmp_path):
    m = _small()
    sd = m.state_dict()
    keys = sorted(sd)
    a, b = {k: sd[k] for k in keys[::2]}, {k: sd[k] for k in keys[1::2]}
    save_state_dict(a, str(tmp_path / "model-00001-of-00002.safetensors"))
    save_state_dict(b, str(tmp_path / "model-00002-of-00002.safetensors"))
    wm = {k: "model-00001-of-00002.safetensors" for k in a} | {k: "model-00002-of-00002.safetensors" for k in b}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
    loaded = load_state_dict(str(tmp_path))
    assert set(loaded) == set(sd)
    mm = ModuleManager(torch_dtype=torch.float32, device="cpu")
    assert mm.load_model(str(tmp_path / "model.safetensors.index.json"), model_class=WanModel, name="wan_video_dit")
    got = mm.fetch_module("wan_video_dit")
    assert isinstance(got, WanModel) and got.num_layers == 2 and got.dim == 128
    for k, v in got.state_dict().items():
        assert torch.equal(v, sd[k]), k
    x, ctx, t = torch.randn(1, 16, 1, 4, 4), torch.randn(1, 4, 64), torch.tensor([10.0])
    got.dtype = m.dtype = torch.float32
    assert torch.equal(got(x, t, ctx), m(x, t, ctx))
    assert mm.get_model_info()[0]["class"] == "WanModel"
    assert mm.remove_module("wan_video_dit") and mm.fetch_module("wan_video_dit") is None


def test_unknown_checkpoint_is_not_loaded(tmp_path):
    save_state_dict({"foo.weight": torch.zeros(2, 2)}, str(tmp_path / "x.safetensors"))
    mm = ModuleManager(torch_dtype=torch.float32, device="cpu")
    assert mm.load_model(str(tmp_path / "x.safetensors")) is False


def test_diffusers_key_renaming_and_shape_inference():
    assert rename_diffusers_key("blocks.3.attn1.to_out.0.weight") == "blocks.3.self_attn.o.weight"
    assert rename_diffusers_key("blocks.0.attn2.add_k_proj.bias") == "blocks.0.cross_attn.k_img.bias"
    assert rename_diffusers_key("blocks.7.ffn.net.0.proj.weight") == "blocks.7.ffn.0.weight"
    assert rename_diffusers_key("blocks.7.norm2.weight") == "blocks.7.norm3.weight"
    assert rename_diffusers_key("condition_embedder.time_proj.bias") == "time_projection.1.bias"
    assert rename_diffusers_key("scale_shift_table") == "head.modulation"
    cfg = infer_wan_config(_small().state_dict())
    assert (cfg["dim"], cfg["ffn_dim"], cfg["num_layers"], cfg["num_heads"], cfg["text_dim"]) == (128, 256, 2, 1, 64)
    assert cfg["patch_size"] == (1, 2, 2) and cfg["out_dim"] == 16 and not cfg["has_image_input"]
