"""Component discovery in model folders: diffusers layout with `model_index.json`, sub-folder configs only,
and a flat folder of official single-file checkpoints (with a sharded DiT)."""

import json

from telefuser_b200.utils.hf_model_analyzer import HFModelAnalyzer, discover_model_components


def _touch(path, size=8):
    path.parent.mkdir(parents=True, exist_ok=True)
    path.write_bytes(b"\0" * size)


def test_diffusers_layout_with_two_experts_and_sharded_weights(tmp_path):
    root = tmp_path / "Wan2.2-T2V-A14B-Diffusers"
    (root).mkdir()
    (root / "model_index.json").write_text(json.dumps({
        "_class_name": "WanPipeline", "transformer": ["diffusers", "WanTransformer3DModel"],
        "transformer_2": ["diffusers", "WanTransformer3DModel"], "vae": ["diffusers", "AutoencoderKLWan"],
        "text_encoder": ["transformers", "UMT5EncoderModel"], "tokenizer": ["transformers", "T5TokenizerFast"],
        "scheduler": ["diffusers", "UniPCMultistepScheduler"], "image_encoder": [None, None]}))
    for name in ("transformer", "transformer_2"):
        for i in (1, 2):
            _touch(root / name / f"diffusion_pytorch_model-0000{i}-of-00002.safetensors", 16)
        _touch(root / name / "stray_copy.safetensors", 99)  # not in the index: must not be loaded
        (root / name / "diffusion_pytorch_model.safetensors.index.json").write_text(json.dumps({"weight_map": {
            "a": "diffusion_pytorch_model-00001-of-00002.safetensors", "b": "diffusion_pytorch_model-00002-of-00002.safetensors"}}))
        (root / name / "config.json").write_text(json.dumps({"_class_name": "WanTransformer3DModel", "in_dim": 16}))
    _touch(root / "vae" / "diffusion_pytorch_model.safetensors")
    _touch(root / "text_encoder" / "model.safetensors")
    (root / "tokenizer").mkdir()
    (root / "tokenizer" / "tokenizer_config.json").write_text(json.dumps({"tokenizer_class": "T5TokenizerFast"}))
    (root / "scheduler").mkdir()
    (root / "scheduler" / "scheduler_config.json").write_text(json.dumps({"_class_name": "UniPCMultistepScheduler"}))
    a = HFModelAnalyzer(str(root))
    comps = a.analyze()
    assert set(comps) == {"transformer", "transformer_2", "vae", "text_encoder", "tokenizer", "scheduler"}
    assert [p.rsplit("/", 1)[1] for p in a.get_transformer_path()] == [
        "diffusion_pytorch_model-00001-of-00002.safetensors", "diffusion_pytorch_model-00002-of-00002.safetensors"]
    assert a.get_transformer_2_path()[0].startswith(str(root / "transformer_2"))
    assert a.get_vae_path().endswith("vae/diffusion_pytorch_model.safetensors")
    assert a.get_tokenizer_path() == str(root / "tokenizer") and a.get_image_encoder_path() is None
    assert comps["transformer"].class_name == "WanTransformer3DModel" and comps["transformer"].size_bytes == 32
    assert comps["text_encoder"].library == "transformers"
    assert "transformer_2" in a.describe()


def test_subfolder_configs_without_an_index_and_second_text_encoder(tmp_path):
    root = tmp_path / "model"
    _touch(root / "dit" / "model.safetensors")
    (root / "dit" / "config.json").write_text(json.dumps({"_class_name": "QwenImageTransformer2DModel"}))
    _touch(root / "llm" / "model-00001-of-00001.safetensors")
    (root / "llm" / "config.json").write_text(json.dumps({"architectures": ["Qwen2_5_VLForConditionalGeneration"]}))
    _touch(root / "byt5" / "pytorch_model.bin")
    _touch(root / "first_stage" / "model.pth")
    (root / "first_stage" / "config.json").write_text(json.dumps({"_class_name": "AutoencoderKLQwenImage"}))
    found = discover_model_components(str(root))
    assert found["transformer"].endswith("dit/model.safetensors")
    assert found["text_encoder"].endswith("llm/model-00001-of-00001.safetensors")
    assert found["text_encoder_2"].endswith("byt5/pytorch_model.bin")
    assert found["vae"].endswith("first_stage/model.pth")  # classified by its declared class, not its folder name


def test_flat_official_release(tmp_path):
    root = tmp_path / "Wan2.1-T2V-14B"
    for i in range(1, 4):
        _touch(root / f"diffusion_pytorch_model-0000{i}-of-00003.safetensors")
    _touch(root / "models_t5_umt5-xxl-enc-bf16.pth")
    _touch(root / "Wan2.1_VAE.pth")
    _touch(root / "models_clip_open-clip-xlm-roberta-large-vit-huge-14.pth")
    (root / "config.json").write_text(json.dumps({"_class_name": "WanModel", "model_type": "t2v"}))
    a = HFModelAnalyzer(str(root))
    assert len(a.get_transformer_path()) == 3 and a.analyze()["transformer"].class_name == "WanModel"
    assert a.get_text_encoder_path().endswith("umt5-xxl-enc-bf16.pth")
    assert a.get_vae_path().endswith("Wan2.1_VAE.pth") and a.get_image_encoder_path().endswith("vit-huge-14.pth")
    assert a.task() == "t2v"
