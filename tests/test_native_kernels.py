"""GPU numerics: every native kernel against the fp32 PyTorch reference of the same op."""
import math

import pytest
import torch

from telefuser_b200.ops import functional as TF
from telefuser_b200.ops import native

pytestmark = pytest.mark.gpu


def rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


@pytest.fixture(autouse=True)
def _lib():
    native.load()
    yield
    torch.cuda.synchronize()
    assert native.last_status() == 0


@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (300, 512, 512), (128, 64, 64), (1000, 1536, 1536),
                                     (4099, 5120, 5120), (777, 8960, 1536)])
@pytest.mark.parametrize("mode", ["plain", "gelu", "gate_res", "res"])
def test_gemm(M, N, K, mode):
    torch.manual_seed(0)
    x = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
    b = torch.randn(N, device="cuda").bfloat16()
    res = torch.randn(M, N, device="cuda").bfloat16() if mode in ("gate_res", "res") else None
    gate = torch.randn(1, N, device="cuda") if mode == "gate_res" else None
    act = "gelu_tanh" if mode == "gelu" else None
    got = TF.linear(x, w, b, act=act, residual=res, gate=gate)
    ref = TF.linear_reference(x, w, b, act=act, residual=res, gate=gate)
    assert rel(got, ref) < 6e-3


def test_gemm_per_row_gate_and_batched():
    torch.manual_seed(0)
    x = torch.randn(2, 130, 256, device="cuda").bfloat16()
    w = (torch.randn(512, 256, device="cuda") * 0.05).bfloat16()
    res = torch.randn(2, 130, 512, device="cuda").bfloat16()
    gate = torch.randn(2, 1, 512, device="cuda")
    assert rel(TF.linear(x, w, None, residual=res, gate=gate), TF.linear_reference(x, w, None, residual=res, gate=gate)) < 6e-3
    gate_tok = torch.randn(2, 130, 512, device="cuda")
    assert rel(TF.linear(x, w, None, residual=res, gate=gate_tok),
               TF.linear_reference(x, w, None, residual=res, gate=gate_tok)) < 6e-3


@pytest.mark.parametrize("B,Sq,Skv,H", [(1, 128, 128, 1), (1, 256, 384, 2), (2, 300, 500, 3), (1, 1000, 77, 2),
                                         (1, 515, 1029, 2), (1, 4096, 4096, 4)])
def test_attention(B, Sq, Skv, H):
    torch.manual_seed(0)
    q = torch.randn(B, Sq, H, 128, device="cuda").bfloat16()
    k = torch.randn(B, Skv, H, 128, device="cuda").bfloat16()
    v = torch.randn(B, Skv, H, 128, device="cuda").bfloat16()
    got, lse = TF.attention(q, k, v, return_lse=True)
    ref, lse_ref = TF.attention_reference(q, k, v, return_lse=True)
    assert rel(got, ref) < 1e-2
    assert rel(lse, lse_ref) < 1e-4


def test_attention_strided_fused_qkv_and_peaked_scores():
    torch.manual_seed(0)
    S, H = 700, 2
    qkv = torch.randn(1, S, 3 * H * 128, device="cuda").bfloat16()
    q, k, v = (qkv[..., i * H * 128:(i + 1) * H * 128].unflatten(-1, (H, 128)) for i in range(3))
    assert rel(TF.attention(q, k, v), TF.attention_reference(q, k, v)) < 1e-2
    # large-magnitude scores exercise the lazy rescale of the accumulator
    q2 = (q.float() * 6).bfloat16()
    assert rel(TF.attention(q2, k, v), TF.attention_reference(q2, k, v)) < 2e-2


@pytest.mark.parametrize("C", [256, 1536, 5120])
def test_layernorm_modulate(C):
    torch.manual_seed(0)
    x = torch.randn(2, 333, C, device="cuda").bfloat16()
    shift, scale = torch.randn(2, 1, C, device="cuda"), torch.randn(2, 1, C, device="cuda") * 0.1
    assert rel(TF.layernorm_modulate(x, shift, scale), TF.layernorm_modulate_reference(x, shift, scale)) < 6e-3
    w, b = torch.randn(C, device="cuda").bfloat16(), torch.randn(C, device="cuda").bfloat16()
    assert rel(TF.layernorm_modulate(x, weight=w, bias=b), TF.layernorm_modulate_reference(x, weight=w, bias=b)) < 6e-3
    sh_t, sc_t = torch.randn(2, 333, C, device="cuda"), torch.randn(2, 333, C, device="cuda") * 0.1
    assert rel(TF.layernorm_modulate(x, sh_t, sc_t), TF.layernorm_modulate_reference(x, sh_t, sc_t)) < 6e-3
    # strided modulation rows (slices of a [B, 1, 6, C] table)
    tab = torch.randn(2, 1, 6, C, device="cuda")
    assert rel(TF.layernorm_modulate(x, tab[:, :, 3], tab[:, :, 4]),
               TF.layernorm_modulate_reference(x, tab[:, :, 3], tab[:, :, 4])) < 6e-3


@pytest.mark.parametrize("H", [2, 12, 40])
def test_rmsnorm_rope_fused_buffer(H):
    torch.manual_seed(0)
    C, S = H * 128, 257
    qkv = torch.randn(1, S, 3 * C, device="cuda").bfloat16()
    ref_in = qkv.clone()
    wq, wk = torch.randn(C, device="cuda").bfloat16(), torch.randn(C, device="cuda").bfloat16()
    ang = torch.randn(S, 64, device="cuda")
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    TF.rmsnorm_rope_(qkv[..., :C], wq, H, cos, sin, x2=qkv[..., C:2 * C], weight2=wk)
    for i, w in enumerate((wq, wk)):
        y = TF.rmsnorm_reference(ref_in[..., i * C:(i + 1) * C].float(), w)
        y = TF.rope_reference(y.reshape(1, S, H, 128), cos, sin).reshape(1, S, C)
        assert rel(qkv[..., i * C:(i + 1) * C], y) < 6e-3
    assert torch.equal(qkv[..., 2 * C:], ref_in[..., 2 * C:])


def test_elementwise_ops():
    torch.manual_seed(0)
    x, y = torch.randn(3, 100, 1536, device="cuda").bfloat16(), torch.randn(3, 100, 1536, device="cuda").bfloat16()
    g = torch.randn(3, 1, 1536, device="cuda")
    assert rel(TF.gated_residual(x, y, g), x.float() + g * y.float()) < 6e-3
    xx = torch.randn(77, 2 * 768, device="cuda").bfloat16()
    for act in ("silu", "gelu_tanh", "gelu"):
        assert rel(TF.act_mul(xx, act), TF.act_mul_reference(xx, act)) < 6e-3
    lat = torch.randn(1, 16, 5, 30, 52, device="cuda")
    c, u = torch.randn_like(lat).bfloat16(), torch.randn_like(lat).bfloat16()
    ref, _ = TF.cfg_euler_step_reference(lat, c, u, 5.0, -0.03)
    assert rel(TF.cfg_euler_step(lat, c, u, 5.0, -0.03), ref) < 1e-6
    ref1, _ = TF.cfg_euler_step_reference(lat, c, None, 1.0, -0.03)
    assert rel(TF.cfg_euler_step(lat, c, None, 1.0, -0.03), ref1) < 1e-6


def test_quant_mxfp8_roundtrip():
    torch.manual_seed(0)
    x = (torch.randn(300, 1536, device="cuda") * torch.logspace(-3, 2, 1536, device="cuda")).bfloat16()
    q, sf = TF.quant_mxfp8(x)
    assert rel(TF.dequant_mxfp8(q, sf), x) < 4e-2
    q_ref, sf_ref = TF.quant_mxfp8_reference(x)
    assert (sf.int() - sf_ref.int()).abs().max() <= 1


def test_wan_block_native_matches_reference_path():
    from telefuser_b200.models.wan_dit import WanModel

    torch.manual_seed(0)
    m = WanModel(dim=256, ffn_dim=512, num_heads=2, num_layers=2, text_dim=256).cuda().bfloat16().eval()
    x = torch.randn(1, 16, 3, 16, 16, device="cuda").bfloat16()
    ctx = torch.randn(1, 32, 256, device="cuda").bfloat16()
    t = torch.tensor([500.0], device="cuda")
    got = m(x, t, ctx)
    TF.set_force_reference(True)
    try:
        ref = m(x, t, ctx)
    finally:
        TF.set_force_reference(False)
    assert rel(got, ref) < 3e-2
