"""Wan DiT on CPU: shapes, state-dict layout, fused-projection views, scheduler loop."""
import torch

from telefuser_b200.models.wan_dit import WanModel, WanModelConfig, rope_tables_3d
from telefuser_b200.ops import functional as TF


def _tiny():
    torch.manual_seed(0)
    m = WanModel.from_config(WanModelConfig.preset("tiny")).float().eval()
    m.dtype = torch.float32
    return m


def test_forward_shape_and_determinism():
    m = _tiny()
    x, ctx, t = torch.randn(2, 16, 3, 8, 8), torch.randn(2, 16, 256), torch.tensor([500.0, 250.0])
    y1, y2 = m(x, t, ctx), m(x, t, ctx)
    assert y1.shape == x.shape and torch.equal(y1, y2) and torch.isfinite(y1).all()


def test_state_dict_keys_follow_checkpoint_layout():
    keys = set(_tiny().state_dict().keys())
    for k in ("patch_embedding.weight", "text_embedding.0.weight", "time_embedding.2.bias", "time_projection.1.weight",
              "blocks.0.self_attn.q.weight", "blocks.0.self_attn.norm_k.weight", "blocks.1.cross_attn.o.bias",
              "blocks.0.norm3.weight", "blocks.0.ffn.2.weight", "blocks.0.modulation", "head.head.weight",
              "head.modulation"):
        assert k in keys, k


def test_fused_qkv_views_track_loaded_weights():
    m = _tiny()
    x, ctx, t = torch.randn(1, 16, 3, 8, 8), torch.randn(1, 16, 256), torch.tensor([500.0])
    y0 = m(x, t, ctx)
    sa = m.blocks[0].self_attn
    W, _ = sa.fused_qkv()
    assert sa.q.weight.data_ptr() == W.data_ptr()
    sd = {k: v.clone() for k, v in m.state_dict().items()}
    sd["blocks.0.self_attn.k.weight"] = sd["blocks.0.self_attn.k.weight"] * 2
    m.load_state_dict(sd)
    assert torch.equal(sa.fused_qkv()[0][128:256], sd["blocks.0.self_attn.k.weight"])
    assert not torch.equal(m(x, t, ctx), y0)


def test_per_token_timestep_matches_scalar_when_constant():
    m = _tiny()
    x, ctx = torch.randn(1, 16, 3, 8, 8), torch.randn(1, 16, 256)
    y_scalar = m(x, torch.tensor([300.0]), ctx)
    y_token = m(x, torch.full((1, 48), 300.0), ctx)
    assert (y_scalar - y_token).abs().max() < 1e-5


def test_rope_tables_split():
    cos, sin = rope_tables_3d(32, (3, 4, 4), "cpu")
    assert cos.shape == (48, 16) and torch.allclose(cos**2 + sin**2, torch.ones_like(cos), atol=1e-6)
    # frame part (first 12 - 2*(32//3)//... ) is constant across h,w within a frame
    d_f = (32 - 2 * (32 // 3)) // 2
    assert torch.equal(cos[0, :d_f], cos[15, :d_f]) and not torch.equal(cos[0, :d_f], cos[16, :d_f])


def test_merge_attn_states_equals_full_attention():
    q, k, v = torch.randn(1, 8, 2, 16), torch.randn(1, 12, 2, 16), torch.randn(1, 12, 2, 16)
    full = TF.attention_reference(q, k, v)
    o1, l1 = TF.attention_reference(q, k[:, :5], v[:, :5], return_lse=True)
    o2, l2 = TF.attention_reference(q, k[:, 5:], v[:, 5:], return_lse=True)
    merged, _ = TF.merge_attn_states(o1, l1, o2, l2)
    assert (merged - full).abs().max() < 1e-5
