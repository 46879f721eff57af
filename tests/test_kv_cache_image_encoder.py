"""fp8 / offloaded KV cache round trips and the CLIP image tower's shapes and checkpoint naming."""

import torch

from telefuser_b200.cache.kv_cache import KVCache, KVCacheManager, fp8_kv_quant_reference
from telefuser_b200.models.wan_image_encoder import WanImageEncoder


def test_kv_cache_plain_fp8_offload():
    torch.manual_seed(0)
    k, v = torch.randn(1, 10, 4, 16), torch.randn(1, 10, 4, 16) * 3
    c = KVCache()
    c.store(k, v)
    k2, v2 = c.load("cpu", torch.float32)
    assert torch.equal(k, k2) and torch.equal(v, v2)
    c8 = KVCache(fp8_kv_cache=True, offload_cache=True)
    c8.store(k, v)
    assert c8.k.dtype == torch.float8_e4m3fn and c8.k_scale.shape == (1, 10, 4, 1)
    k8, v8 = c8.load("cpu", torch.float32)
    assert (k8 - k).abs().max() <= k.abs().amax() * 0.07 and (v8 - v).abs().max() <= v.abs().amax() * 0.07
    assert c8.nbytes() < c.nbytes() / 2
    q, s = fp8_kv_quant_reference(torch.zeros(2, 3, 8))
    assert torch.isfinite(q.float()).all() and (s > 0).all()
    c9 = KVCache.from_dict(c8.to_dict())
    assert c9.fp8_kv_cache and torch.equal(c9.load("cpu", torch.float32)[0], k8)


def test_kv_cache_manager_grid():
    m = KVCacheManager(num_timesteps=3, num_layers=2, fp8_kv_cache=True)
    assert not m.is_allocated
    m.allocate((1, 6, 2, 8), torch.bfloat16, "cpu")
    assert m.is_allocated and m.shape == (1, 6, 2, 8)
    m.get_cache(2, 1).store(torch.ones(1, 6, 2, 8), torch.ones(1, 6, 2, 8) * 2)
    k, v = m.get_cache(2, 1).load("cpu", torch.float32)
    assert torch.allclose(k, torch.ones_like(k)) and torch.allclose(v, 2 * torch.ones_like(v))
    assert len(m.get_timestep_caches(0)) == 2
    m2 = KVCacheManager.from_dict(m.to_dict())
    assert m2.num_timesteps == 3 and m2.num_layers == 2 and m2.fp8_kv_cache
    try:
        m.get_cache(3, 0)
        raise AssertionError("expected IndexError")
    except IndexError:
        pass
    m.clear()
    assert not m.is_allocated


def test_image_encoder_penultimate_states_and_converter():
    torch.manual_seed(0)
    enc = WanImageEncoder(image_size=56, patch_size=14, dim=64, out_dim=32, num_heads=4, num_layers=3).eval()
    img = torch.rand(1, 3, 80, 100) * 2 - 1
    out = enc.encode_image([img, img.flip(-1)])
    assert out.shape == (2, 17, 64) and torch.isfinite(out).all()
    full = enc.model.visual(torch.randn(1, 3, 56, 56))
    pen = enc.model.visual(torch.randn(1, 3, 56, 56), use_31_block=True)
    assert full.shape == pen.shape
    sd = {"visual.pos_embedding": 1, "textual.token_embedding.weight": 2, "log_scale": 3}
    conv, _ = enc.state_dict_converter().from_official(sd)
    assert conv == {"model.visual.pos_embedding": 1}
    assert all(k.startswith("model.visual.") for k in enc.state_dict())
