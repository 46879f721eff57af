"""Checkpoint converter / quantiser, LoRA extraction, video and audio file helpers, artefact save stage."""

import json
import wave

import numpy as np
import pytest
import torch
from PIL import Image

from telefuser_b200.models.wan_dit import WanModel, WanModelConfig
from telefuser_b200.orchestrator.artifact_save import ArtifactSaveConfig, ArtifactSaveStage
from telefuser_b200.tools import convert, lora_extract
from telefuser_b200.utils import video as V
from telefuser_b200.utils.lora import LoRALoader
from telefuser_b200.utils.model_weight import load_state_dict, save_state_dict


def test_convert_key_mapping_round_trip_and_quantise(tmp_path):
    torch.manual_seed(0)
    model = WanModel.from_config(WanModelConfig.preset("tiny"))
    sd = {k: v.detach().clone() for k, v in model.state_dict().items()}
    src = tmp_path / "native.safetensors"
    save_state_dict(sd, str(src))
    r = convert.main(["-s", str(src), "-o", str(tmp_path / "d"), "-d", "backward", "-t", "wan_dit"])
    assert r["tensors"] == len(sd)
    other = load_state_dict(str(tmp_path / "d" / "converted.safetensors"))
    assert "blocks.0.attn1.to_q.weight" in other and "blocks.0.ffn.net.0.proj.weight" in other
    assert "scale_shift_table" in other and not any(".self_attn." in k for k in other)
    convert.main(["-s", str(tmp_path / "d" / "converted.safetensors"), "-o", str(tmp_path / "n"), "-d", "forward",
                  "-t", "wan_dit"])  # fmt: skip
    back = load_state_dict(str(tmp_path / "n" / "converted.safetensors"))
    assert set(back) == set(sd) and all(torch.equal(back[k], sd[k]) for k in sd)
    # fp8 quantisation of attention / ffn linears, saved block by block
    r = convert.main(["-s", str(src), "-o", str(tmp_path / "q"), "--quantized", "--linear_dtype", "fp8", "-b"])
    assert r["quantized"] > 0
    index = json.loads((tmp_path / "q" / "converted.safetensors.index.json").read_text())
    q = load_state_dict(str(tmp_path / "q" / index["weight_map"]["blocks.0.self_attn.q.weight"]))
    w8, s = q["blocks.0.self_attn.q.weight"], q["blocks.0.self_attn.q.weight_scale"]
    assert w8.dtype == torch.float8_e4m3fn and s.shape == (w8.shape[0], 1)
    w = sd["blocks.0.self_attn.q.weight"]
    assert (w8.float() * s - w).abs().max() <= w.abs().max() * 0.07
    assert q["blocks.0.norm3.weight"].dtype == w.dtype  # norms untouched
    # mxfp8 payload + UE8M0 scales
    convert.main(["-s", str(src), "-o", str(tmp_path / "m"), "--quantized", "--linear_dtype", "mxfp8"])
    m = load_state_dict(str(tmp_path / "m" / "converted.safetensors"))
    assert m["blocks.0.ffn.0.weight_sf"].shape == (512, 128 // 32) and m["blocks.0.ffn.0.weight_sf"].dtype == torch.uint8
    # int8 per output channel; NVFP4 codes with block and tensor scales (both read back and de-quantised)
    convert.main(["-s", str(src), "-o", str(tmp_path / "i"), "--quantized", "--linear_dtype", "int8"])
    i8 = load_state_dict(str(tmp_path / "i" / "converted.safetensors"))
    assert i8["blocks.0.self_attn.q.weight"].dtype == torch.int8
    assert (i8["blocks.0.self_attn.q.weight"].float() * i8["blocks.0.self_attn.q.weight_scale"] - w).abs().max() <= w.abs().max() / 127
    convert.main(["-s", str(src), "-o", str(tmp_path / "f4"), "--quantized", "--linear_dtype", "nvfp4"])
    f4 = load_state_dict(str(tmp_path / "f4" / "converted.safetensors"))
    from telefuser_b200.ops.nvfp4 import dequantize_nvfp4

    key = "blocks.0.self_attn.q"
    assert f4[key + ".weight"].dtype == torch.uint8 and f4[key + ".weight"].shape == (w.shape[0], w.shape[1] // 2)
    back4 = dequantize_nvfp4(f4[key + ".weight"], f4[key + ".weight_scale"], f4[key + ".weight_global_scale"])
    assert ((back4 - w.float()).norm() / w.float().norm()).item() < 0.13


def test_lora_extract_then_merge_recovers_the_tuned_weights(tmp_path):
    torch.manual_seed(0)
    base = {"blocks.0.q.weight": torch.randn(32, 32), "blocks.0.q.bias": torch.randn(32), "head.modulation": torch.randn(1, 2, 32)}
    tuned = {k: v.clone() for k, v in base.items()}
    tuned["blocks.0.q.weight"] += torch.randn(32, 4) @ torch.randn(4, 32) * 0.1  # rank-4 update
    tuned["blocks.0.q.bias"] += 0.5
    lora = lora_extract.extract_lora(base, tuned, rank=8)
    assert lora["blocks.0.q.lora_up.weight"].shape == (32, 8) and "blocks.0.q.diff_b" in lora
    assert "head.diff_m" not in lora  # unchanged tensors are skipped
    save_state_dict(base, str(tmp_path / "b.safetensors"))
    save_state_dict(lora, str(tmp_path / "l.safetensors"))
    convert.main(["-s", str(tmp_path / "b.safetensors"), "-o", str(tmp_path / "o"), "--lora_path", str(tmp_path / "l.safetensors")])
    merged = load_state_dict(str(tmp_path / "o" / "converted.safetensors"))
    assert torch.allclose(merged["blocks.0.q.weight"], tuned["blocks.0.q.weight"], atol=1e-4)
    assert torch.allclose(merged["blocks.0.q.bias"], tuned["blocks.0.q.bias"], atol=1e-6)
    assert LoRALoader().extract_lora_pairs(lora)["blocks.0.q.weight"]["alpha"] == 8.0


def test_video_round_trip_sizes_and_wav(tmp_path):
    assert V.get_target_video_size_from_ratio("720p", "16:9") == (720, 1280)
    assert V.get_target_video_size_from_ratio("480p", "9:16") == (848, 480)
    im = Image.fromarray(np.random.randint(0, 255, (60, 100, 3), dtype=np.uint8))
    assert V.crop_and_resize(im, 32, 32).size == (32, 32)
    assert V.get_target_image_size(im, 32 * 32 * 4) == (48, 80)
    frames = torch.rand(3, 6, 32, 48) * 2 - 1
    path = V.save_video(frames, str(tmp_path / "v" / "a.mp4"), fps=8)
    vd = V.VideoData(video_file=path)
    assert len(vd) == 6 and vd.shape() == (32, 48) and abs(vd.fps() - 8) < 0.5
    t = V.VideoData(video_file=path, height=16, width=16, length=4).to_tensor()
    assert t.shape == (3, 4, 16, 16) and t.min() >= -1 and t.max() <= 1
    V.save_frames(frames, str(tmp_path / "f"))
    folder = V.VideoData(image_folder=str(tmp_path / "f"))
    assert len(folder) == 6 and V.search_for_images(str(tmp_path / "f"))[:3] == ["0.png", "1.png", "2.png"]
    want = ((frames[:, 0] + 1) * 127.5).round().clamp(0, 255).permute(1, 2, 0).numpy().astype(np.uint8)
    assert np.array_equal(np.asarray(folder[0]), want)
    assert len(V.images_to_base_64([im])[0]) > 100
    wav = V.save_wav(torch.sin(torch.linspace(0, 100, 1600)), str(tmp_path / "a.wav"), 16000)
    with wave.open(wav) as w:
        assert (w.getnchannels(), w.getframerate(), w.getnframes()) == (1, 16000, 1600)


def test_artifact_save_stage(tmp_path):
    stage = ArtifactSaveStage()
    cfg = ArtifactSaveConfig(output_root=tmp_path, run_name="run/../x", fps=12)
    meta = stage.process(torch.rand(3, 5, 16, 16) * 2 - 1, request_id="../../evil id", config=cfg, make_date_subdir=False)
    assert meta["num_frames"] == 5 and meta["fps"] == 12
    p = tmp_path / "run_.._x" / "evil_id.mp4"
    assert str(p) == meta["path"] and p.is_file() and (tmp_path / "run_.._x" / "evil_id.json").is_file()
    meta2 = stage.process([Image.new("RGB", (8, 8))] * 2, request_id="frames", config=cfg, file_ext=".png",
                          make_date_subdir=False)  # fmt: skip
    assert (tmp_path / "run_.._x" / "frames" / "1.png").is_file() and meta2["num_frames"] == 2


@pytest.mark.parametrize("kind", ["fp8", "int8", "mxfp8", "nvfp4", "mxfp4"])
def test_offline_quantised_checkpoint_loads_with_its_stored_payloads(tmp_path, kind):
    """convert --quantized -> ModuleManager.load_model: the model class is recognised from the dense form of the checkpoint,
    the layers come back in their stored format with the stored values (formats without a run-time path stay dense)."""
    from telefuser_b200.core.module_manager import ModuleManager
    from telefuser_b200.models.wan_dit import WanModel
    from telefuser_b200.ops.quant import dense_weight, stored_format
    from telefuser_b200.testing.distributed_checks import make_tiny_inputs, make_tiny_model
    from telefuser_b200.tools import convert
    from telefuser_b200.utils.model_weight import load_state_dict, save_state_dict

    src = make_tiny_model()
    save_state_dict(src.state_dict(), str(tmp_path / "dit.safetensors"))
    convert.main(["-s", str(tmp_path / "dit.safetensors"), "-o", str(tmp_path / "q"), "--quantized", "--linear_dtype", kind,
                  "--quantize_modules", "self_attn", "cross_attn", "ffn"])  # fmt: skip
    mm = ModuleManager(torch_dtype=torch.float32, device="cpu")
    assert mm.load_model(str(tmp_path / "q" / "converted.safetensors"), model_class=WanModel, name="wan_video_dit")
    dit = mm.fetch_module("wan_video_dit")
    lin = dit.blocks[0].ffn[0]
    assert stored_format(lin) == ("dense" if kind == "mxfp4" else kind) and stored_format(dit.head.head) == "dense"
    stored = load_state_dict(str(tmp_path / "q" / "converted.safetensors"))
    if kind not in ("mxfp4",):
        assert torch.equal(lin.weight.data.view(torch.uint8), stored["blocks.0.ffn.0.weight"].view(torch.uint8))  # not re-quantised
    want = convert.dequantize_model(stored, torch.float32)[0]["blocks.0.ffn.0.weight"]
    assert torch.allclose(dense_weight(lin), want, atol=1e-2 * want.abs().max().item())
    lat, ctx, _ = make_tiny_inputs()
    t = torch.tensor([500.0])
    with torch.no_grad():
        ref, out = src(lat, t, ctx), dit(lat, t, ctx)
    assert torch.isfinite(out).all() and ((out - ref).norm() / ref.norm()).item() < (0.3 if kind == "mxfp4" else 0.1)
