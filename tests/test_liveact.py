"""LiveAct: memory compression of the KV cache, audio windows, the fixed three-step denoiser with audio guidance,
and the block-by-block pipeline with tiny random components on CPU; bf16 forward on GPUs."""

import pytest
import torch
from transformers import Wav2Vec2Config

from telefuser_b200.cache.kv_cache import KVCache
from telefuser_b200.core.config import ModelRuntimeConfig
from telefuser_b200.core.module_manager import ModuleManager
from telefuser_b200.models.liveact_dit import AudioProjModel, LiveActDiT, MemorySelfAttention, rope_tables
from telefuser_b200.models.wan_vae import WanVideoVAE
from telefuser_b200.models.wav2vec2 import Wav2Vec2Model
from telefuser_b200.pipelines.liveact import (AudioEncodingStage, LiveActDenoisingStage, LiveActPipeline, LiveActPipelineConfig,
                                              resample_to_16k)  # fmt: skip


def small_dit(dtype=torch.float32, device="cpu", head_dim=48):
    torch.manual_seed(0)
    m = LiveActDiT(in_dim=36, dim=2 * head_dim, ffn_dim=128, text_dim=24, out_dim=16, num_heads=2, num_layers=2, text_len=6,
                   intermediate_dim=16, output_dim=24, context_tokens=4, clip_dim=20)  # fmt: skip
    m.audio_proj = AudioProjModel(seq_len=5, seq_len_vf=8, blocks=2, channels=32, intermediate_dim=16, output_dim=24,
                                  context_tokens=4, norm_output_audio=True)  # fmt: skip
    for n, p in m.named_parameters():
        if "memory_proj" not in n:
            torch.nn.init.normal_(p, std=0.05)
    m = m.to(dtype).to(device).eval()
    m.dtype = dtype
    return m


def test_memory_compression_and_rope():
    att = MemorySelfAttention(32, 2)
    att.post_init()
    t = torch.randn(1, 10, 2, 16)
    assert torch.allclose(att._compress(t, 2, att.memory_proj_k), t.view(1, 2, 5, 2, 16).mean(2), atol=1e-6)  # starts as a mean
    torch.nn.init.normal_(att.memory_proj_k.weight)
    conv = att.memory_proj_k(t.view(1, 10, 32).transpose(1, 2)).view(1, 2, 16, 2).permute(0, 3, 1, 2)
    assert torch.allclose(att._compress(t, 2, att.memory_proj_k), conv, atol=1e-5)
    tpf = 2
    k_full, v_full = torch.randn(1, 14 * tpf, 2, 16), torch.randn(1, 14 * tpf, 2, 16)
    kc, vc = torch.zeros(1, 6 * tpf, 2, 16), torch.zeros(1, 6 * tpf, 2, 16)
    att.compress_cache(k_full, v_full, kc, vc, tpf)
    assert kc[:, : 2 * tpf].abs().max() == 0 and torch.equal(kc[:, 4 * tpf :], k_full[:, 12 * tpf :])  # anchors untouched here
    cos, sin = rope_tables(48, 2, 3, 4, 5, "cpu")
    assert cos.shape == (24, 24) and torch.allclose(sin[0, 0], torch.sin(torch.tensor(5.0)))  # frame offset


def test_audio_stage_windows_and_resampling():
    torch.manual_seed(0)
    cfg = Wav2Vec2Config(hidden_size=32, num_hidden_layers=2, num_attention_heads=2, intermediate_size=64, conv_dim=(16, 16),
                         conv_stride=(5, 2), conv_kernel=(10, 3), num_conv_pos_embeddings=16, num_conv_pos_embedding_groups=2)  # fmt: skip
    enc = Wav2Vec2Model(cfg).eval()
    stage = AudioEncodingStage("audio", None, ModelRuntimeConfig(device_type="cpu", torch_dtype=torch.float32), 5, encoder=enc)
    stage.onload_models_flag = True
    assert resample_to_16k(torch.ones(1, 800), 8000).shape == (1, 1600)
    wave = torch.randn(1, 24000)  # 1 s at 24 kHz
    emb, dur = stage.process(audio=wave, sr=24000, fps=24, stream_audio=False)
    assert emb.shape == (24, 2, 32) and abs(dur - 1.0) < 1e-6
    win = stage.process_pre_encoded_segment(0, 5)
    assert win.shape == (1, 5, 5, 2, 32) and torch.equal(win[0, 0, 0], emb[0]) and torch.equal(win[0, 0, 4], emb[2])
    stage.process(audio=wave, sr=24000, fps=24, stream_audio=True)
    seg = stage.process_stream_audio_segment(0, 12, 24, 12)
    assert seg.shape == (1, 12, 5, 2, 32)


def _inputs(f, h=8, w=8):
    return ([torch.randn(16, f, h, w)], [torch.randn(20, f, h, w)], [torch.randn(4, 24)], torch.randn(1, 257, 20),
            torch.randn(1, 1 + 4 * 13, 5, 2, 32))  # fmt: skip


def test_denoiser_blocks_and_audio_guidance():
    dit = small_dit()
    cfg = ModelRuntimeConfig(device_type="cpu", torch_dtype=torch.float32)
    stage = LiveActDenoisingStage("denoise", None, cfg, dit=dit)
    stage.onload_models_flag = True
    tpf = 16
    y = torch.randn(1, 20, 14, 8, 8)
    ctx, clip, audio = torch.randn(1, 4, 24), torch.randn(1, 257, 20), torch.randn(1, 1 + 4 * 13, 5, 2, 32)
    first = stage.process(torch.randn(16, 6, 8, 8), ctx, clip, audio, y, tpf)
    assert first.shape == (16, 6, 8, 8) and stage.kv_cache_manager.get_cache(2, 1).k.shape == (1, 6 * tpf, 2, 48)
    anchors = stage.kv_cache_manager.get_cache(0, 0).k[:, : 2 * tpf].clone()
    nxt = stage.process(torch.randn(16, 8, 8, 8), ctx, clip, audio, y, tpf)
    assert nxt.shape == (16, 8, 8, 8) and torch.equal(stage.kv_cache_manager.get_cache(0, 0).k[:, : 2 * tpf], anchors)
    noise = torch.randn(16, 8, 8, 8)
    plain = stage.process(noise, ctx, clip, audio, y, tpf)
    stage2 = LiveActDenoisingStage("denoise", None, cfg, dit=dit)
    stage2.onload_models_flag = True
    stage2.process(torch.randn(16, 6, 8, 8), ctx, clip, audio, y, tpf, audio_cfg=2.0)
    guided = stage2.process(noise, ctx, clip, audio, y, tpf, audio_cfg=2.0)
    assert stage2._null_audio_manager is not None and torch.isfinite(guided).all() and not torch.allclose(guided, plain)


def test_pipeline_generates_block_by_block():
    torch.manual_seed(0)
    dit = small_dit()
    vae = WanVideoVAE(z_dim=16, dim=8).eval()
    cfg = Wav2Vec2Config(hidden_size=32, num_hidden_layers=2, num_attention_heads=2, intermediate_size=64, conv_dim=(16, 16),
                         conv_stride=(5, 2), conv_kernel=(10, 3), num_conv_pos_embeddings=16, num_conv_pos_embedding_groups=2)  # fmt: skip
    mm = ModuleManager(torch_dtype=torch.float32, device="cpu")
    mm.add_module(dit, "liveact_dit")
    mm.add_module(vae, "wan_video_vae")
    mm.add_module(Wav2Vec2Model(cfg).eval(), "wav2vec2")
    rc = lambda: ModelRuntimeConfig(device_type="cpu", torch_dtype=torch.float32)  # noqa: E731

    class Fixed:
        def __init__(self, value):
            self.value = value

        def process(self, *a, **k):
            return self.value

    pipe = LiveActPipeline(device="cpu", torch_dtype=torch.float32)
    pipe.init(mm, LiveActPipelineConfig(vae_config=rc(), dit_config=rc(), clip_config=rc(), text_encoding_config=rc(), audio_config=rc()),
              text_stage=Fixed([torch.randn(1, 4, 24)]), clip_stage=Fixed(torch.randn(1, 257, 20)))  # fmt: skip
    image = torch.rand(1, 3, 64, 64) * 2 - 1
    video = pipe("a person talking", image, audio=torch.randn(1, 16000 * 2), audio_sr=16000, seed=0, height=64, width=64,
                 fps=24, output_type="pt")  # fmt: skip
    # 2 s of audio -> 2 blocks: 6 latents (21 frames) + 8 latents (32 frames)
    assert video.shape == (3, 21 + 32, 64, 64) and torch.isfinite(video).all()


@pytest.mark.gpu
def test_gpu_bf16_forward_tracks_cpu_fp32():
    ref_m = small_dit(head_dim=128)
    x, y, ctx, clip, audio = _inputs(6, 16, 16)
    def caches(dtype, dev):
        out = []
        for _ in range(2):
            c = KVCache()
            c.allocate((1, 6 * 64, 2, 128), dtype, dev)
            out.append(c)
        return out
    t = torch.tensor([937.5])
    ref = ref_m(x, t, ctx, clip_fea=clip, y=y, audio=audio, kv_cache=caches(torch.float32, "cpu"), start_idx=0)
    gpu_m = small_dit(torch.bfloat16, "cuda", head_dim=128)
    got = gpu_m([x[0].cuda()], t.cuda(), [ctx[0].cuda()], clip_fea=clip.cuda(), y=[y[0].cuda()], audio=audio.cuda(),
                kv_cache=caches(torch.bfloat16, "cuda"), start_idx=0).float().cpu()  # fmt: skip
    err = ((got - ref).norm() / ref.norm()).item()
    assert err < 3e-2, err
