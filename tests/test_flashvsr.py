"""FlashVSR: window partition, local / draft block masks, sparse attention with its cache, the tiny conditional
decoder's chunked streaming, the causal LQ projector, the DiT clip by clip and the streaming pipeline."""

import torch
from PIL import Image

from telefuser_b200.core.config import ModelRuntimeConfig
from telefuser_b200.core.module_manager import ModuleManager
from telefuser_b200.models.flashvsr_dit import FlashVSRModel
from telefuser_b200.models.tc_decoder import TAEHV, pixel_unshuffle_3d
from telefuser_b200.models.video_projector import Causal_LQ4x_Proj
from telefuser_b200.ops import functional as TF
from telefuser_b200.ops import local_sparse_attention as LSA
from telefuser_b200.pipelines.flashvsr import FlashVSRPipelineConfig, FlashVSRStreamPipeline, prepare_input_tensor


def test_windows_and_masks():
    x = torch.arange(2 * 4 * 16 * 16 * 3, dtype=torch.float32).view(2, 4, 16, 16, 3)
    w = LSA.window_partition(x, (2, 8, 8))
    assert w.shape == (2 * 2 * 2 * 2, 128, 3) and torch.equal(LSA.window_reverse(w, (2, 8, 8), (4, 16, 16)), x)
    assert torch.equal(w[3, 0], x[0, 0, 8, 8])  # window order: frame group, row, column
    m = LSA.build_local_block_mask(4, 5, 3, 3)
    assert m.shape == (20, 20) and m[0].sum() == 4 and m[6].sum() == 9 and m[6, 0] and not m[6, 3]
    torch.manual_seed(0)
    q_w, k_w = torch.randn(8, 128, 32), torch.randn(12, 128, 32)  # 2 query groups, 3 key groups of 4 windows
    mask = LSA.draft_block_mask(q_w, k_w, 2, 2, topk=10, local_mask=torch.ones(4, 4, dtype=torch.bool))
    assert mask.shape == (1, 2, 8, 12) and (mask.view(2, 2, -1).sum(-1) == 10).all()  # per (head, query group)
    none = LSA.draft_block_mask(q_w, k_w, 2, 2, topk=0, local_mask=torch.ones(4, 4, dtype=torch.bool))
    assert not none.any()


def test_sparse_attention_dense_limit_and_cache():
    torch.manual_seed(0)
    f, h, w, heads, hd = 2, 16, 16, 2, 16
    D = heads * hd
    q, k, v = (torch.randn(1, f * h * w, D) for _ in range(3))
    out, ck, cv = LSA.local_sparse_attention(q, k, v, 1, f, h, w, D, topk=10**6, local_range=99, num_heads=heads, kv_len=1)
    dense = TF.attention_reference(q.view(1, -1, heads, hd), k.view(1, -1, heads, hd), v.view(1, -1, heads, hd)).reshape(1, -1, D)
    # the draft keeps the pairs strictly above the weakest one: per head all but one (query window, key window) pair equal dense
    assert ((out - dense).abs().amax(-1) > 1e-5).sum() <= 128 * heads
    assert ck.shape == (4, 128, D) and torch.equal(ck, LSA.window_partition(k.view(1, f, h, w, D), (2, 8, 8)))
    out2, ck2, _ = LSA.local_sparse_attention(q, k, v, 1, f, h, w, D, 10**6, 99, heads, 1, ck, cv)
    assert ck2.shape == (4, 128, D) and torch.equal(ck2, ck)  # two groups present, the older one is dropped
    both = TF.attention_reference(q.view(1, -1, heads, hd), torch.cat([k, k], 1).view(1, -1, heads, hd),
                                  torch.cat([v, v], 1).view(1, -1, heads, hd)).reshape(1, -1, D)  # fmt: skip
    assert ((out2 - both).abs().amax(-1) > 1e-5).sum() <= 128 * heads
    sparse, _, _ = LSA.local_sparse_attention(q, k, v, 1, f, h, w, D, topk=3, local_range=1, num_heads=heads, kv_len=1)
    assert torch.isfinite(sparse).all() and not torch.allclose(sparse, dense, atol=1e-3)


def _small_parts():
    torch.manual_seed(0)
    dit = FlashVSRModel(dim=64, in_dim=16, ffn_dim=128, out_dim=16, text_dim=32, freq_dim=32, num_heads=2, num_layers=2,
                        lq_layers=1, ctx_len=8)  # fmt: skip
    dec = TAEHV(channels=(16, 8, 8, 8), latent_channels=16 + 768)
    for p in list(dit.parameters()) + list(dec.parameters()):
        torch.nn.init.normal_(p, std=0.05)
    dit, dec = dit.float().eval(), dec.float().eval()
    dit.dtype = torch.float32
    return dit, dec


def test_decoder_and_projector_stream_in_chunks():
    _, dec = _small_parts()
    lat, cond = torch.randn(1, 5, 16, 4, 4), torch.rand(1, 3, 20, 32, 32)
    assert pixel_unshuffle_3d(cond, 4, 8, 8).shape == (1, 5, 768, 4, 4)
    whole = dec.decode(lat, cond=cond)
    assert whole.shape == (1, 5 * 4 - 3, 3, 32, 32)
    dec.clean_mem()
    parts = torch.cat([dec.decode(lat[:, :3], cond=cond[:, :, :12]), dec.decode(lat[:, 3:], cond=cond[:, :, 12:])], 1)
    assert torch.allclose(parts, whole, atol=1e-5)
    proj = Causal_LQ4x_Proj(3, 8, layer_num=2, hidden_dim1=16, hidden_dim2=24).eval()
    video = torch.rand(1, 3, 9, 32, 48)
    with torch.no_grad():
        full = proj(video)
        proj.clear_cache()
        assert proj.stream_forward(video[:, :, :1]) is None
        chunks = [proj.stream_forward(video[:, :, 1:5]), proj.stream_forward(video[:, :, 5:9])]
    assert full[0].shape == (1, 2 * 2 * 3, 8)
    assert torch.allclose(torch.cat([c[1] for c in chunks], 1), full[1], atol=1e-6)


def test_dit_clips_and_pipeline_stream():
    dit, dec = _small_parts()
    x = torch.randn(1, 16, 6, 32, 32)
    out = dit(x, LQ_latents=[torch.zeros(1, 6 * 256, 64)], topk_ratio=0.5, kv_ratio=2)
    assert out.shape == x.shape and dit.kv_cache[0][0].shape == (2 * 4, 128, 64)  # 3 groups, the oldest dropped
    nxt = dit(torch.randn(1, 16, 2, 32, 32), topk_ratio=0.5, kv_ratio=2, cur_process_idx=1)
    assert nxt.shape == (1, 16, 2, 32, 32) and dit.kv_cache[0][0].shape == (2 * 4, 128, 64)
    keys = set(dit.state_dict())
    assert {"LQ_proj_in.linear_layers.0.weight", "ctx", "blocks.1.cross_attn.norm_k.weight", "head.modulation"} <= keys
    dit.clear_kv_cache()
    dit.clean_LQ_proj_in_cache()
    mm = ModuleManager(torch_dtype=torch.float32, device="cpu")
    mm.add_module(dit, "flashvsr_dit")
    mm.add_module(dec, "wan_video_decoder")
    rc = lambda: ModelRuntimeConfig(device_type="cpu", torch_dtype=torch.float32)  # noqa: E731
    pipe = FlashVSRStreamPipeline(device="cpu", torch_dtype=torch.float32)
    pipe.init(mm, FlashVSRPipelineConfig(vae_config=rc(), dit_config=rc()))
    frames = [Image.new("RGB", (64, 64), (8 * i, 100, 200 - 8 * i)) for i in range(33)]
    vid, tH, tW, sH, sW = prepare_input_tensor(frames[:2], scale=4, dtype=torch.float32)
    assert vid.shape == (1, 3, 2, 256, 256) and (tH, tW, sH, sW) == (256, 256, 256, 256) and vid.abs().max() <= 1.01
    first = pipe(seed=0, LQ_video=frames, scale=4, sparse_ratio=2.0, output_type="pt")
    assert first.shape == (3, 29, 256, 256) and torch.isfinite(first).all()  # 25 + 8 frames in -> 8 latent frames -> 29 frames
    more = pipe(seed=1, LQ_video=frames[:16], scale=4, output_type="pt")  # continues the stream: 16 new frames
    assert more.shape == (3, 12, 256, 256) and pipe.process_chunk_idx == 4 + 2
