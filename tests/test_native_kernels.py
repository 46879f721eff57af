"""GPU numerics: every native kernel against the fp32 PyTorch reference of the same op."""
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


@pytest.mark.parametrize("variant", [0, 21, 30, 31])  # default by shape / one thread per row / two threads per row
@pytest.mark.parametrize("B,Sq,Skv,H", [(1, 128, 128, 1), (1, 256, 384, 2), (2, 300, 500, 3), (1, 1000, 77, 2),
                                         (1, 515, 1029, 2), (1, 4096, 4096, 4)])
def test_attention(B, Sq, Skv, H, variant):
    torch.manual_seed(0)
    q = torch.randn(B, Sq, H, 128, device="cuda").bfloat16()
    k = torch.randn(B, Skv, H, 128, device="cuda").bfloat16()
    v = torch.randn(B, Skv, H, 128, device="cuda").bfloat16()
    got, lse = TF.attention(q, k, v, return_lse=True, variant=variant)
    ref, lse_ref = TF.attention_reference(q, k, v, return_lse=True)
    assert rel(got, ref) < 1e-2
    assert rel(lse, lse_ref) < 1e-4
    again = TF.attention(q, k, v, variant=variant)
    assert torch.equal(got, again)  # no atomics, fixed order: bitwise reproducible


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("B,Sq,Skv,H", [(1, 256, 256, 2), (2, 300, 300, 3), (1, 200, 777, 2), (1, 1031, 1031, 1)])
def test_attention_causal_and_head_dim_64(B, Sq, Skv, H, D):
    torch.manual_seed(0)
    q = torch.randn(B, Sq, H, D, device="cuda").bfloat16()
    k = torch.randn(B, Skv, H, D, device="cuda").bfloat16()
    v = torch.randn(B, Skv, H, D, device="cuda").bfloat16()
    for causal in (False, True):
        got, lse = TF.attention(q, k, v, return_lse=True, causal=causal)
        ref, lse_ref = TF.attention_reference(q, k, v, return_lse=True, causal=causal)
        assert rel(got, ref) < 1e-2, (causal, D)
        assert rel(lse, lse_ref) < 1e-4, (causal, D)


@pytest.mark.parametrize("D,dtype", [(80, torch.bfloat16), (40, torch.float16), (96, torch.bfloat16)])
def test_attention_pads_other_head_dims(D, dtype):
    torch.manual_seed(0)
    q, k, v = (torch.randn(2, 257, 4, D, device="cuda").to(dtype) for _ in range(3))
    launches = TF.native.launch_count()
    got = TF.attention(q, k, v)
    assert TF.native.launch_count() == launches + 1 and got.dtype == dtype and got.shape == q.shape
    assert rel(got, TF.attention_reference(q, k, v)) < 1e-2


def test_attention_masked_and_wide_heads_take_the_blocked_fp32_path():
    torch.manual_seed(0)
    q, k, v = (torch.randn(1, 300, 2, 384, device="cuda").bfloat16() for _ in range(3))
    want = TF.attention_reference(q, k, v)
    assert rel(TF.attention(q, k, v), want) < 1e-6
    assert rel(TF.attention_reference(q, k, v, q_block=64), want) < 1e-6
    q, k, v = (torch.randn(2, 100, 2, 64, device="cuda").bfloat16() for _ in range(3))
    mask = torch.rand(2, 1, 100, 100, device="cuda") > 0.3
    mask[..., 0] = True
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float()) / 8
    want = torch.einsum("bhqk,bkhd->bqhd", s.masked_fill(~mask, float("-inf")).softmax(-1), v.float())
    assert rel(TF.attention(q, k, v, mask=mask), want) < 1e-2
    assert rel(TF.attention_reference(q, k, v, mask=mask, q_block=32), want) < 1e-2


def test_attention_long_sequence_and_layer_like_magnitudes():
    """32k keys with inputs shaped like a DiT layer's: RMS-normed, RoPE-rotated q / k with a learned gain and a few
    outlier channels, so the running maximum moves and the lazy rescale fires many times over 256 key tiles."""
    torch.manual_seed(0)
    S, H = 32768, 2
    q = torch.randn(1, S, H, 128, device="cuda")
    k = torch.randn(1, S, H, 128, device="cuda")
    gain = 1 + 0.5 * torch.randn(128, device="cuda").abs()
    gain[::17] *= 4
    ramp = torch.linspace(0.2, 3.0, S, device="cuda").reshape(1, S, 1, 1)  # later keys score higher
    q = (q / q.pow(2).mean(-1, keepdim=True).sqrt() * gain).bfloat16()
    k = (k / k.pow(2).mean(-1, keepdim=True).sqrt() * gain * ramp).bfloat16()
    v = torch.randn(1, S, H, 128, device="cuda").bfloat16()
    for variant in (0, 20, 30):
        got, lse = TF.attention(q[:, :2048], k, v, return_lse=True, variant=variant)
        ref, lse_ref = TF.attention_reference(q[:, :2048], k, v, return_lse=True)
        assert rel(got, ref) < 1.5e-2, variant
        assert rel(lse, lse_ref) < 1e-4, variant


def test_attention_strided_fused_qkv_and_peaked_scores():
    torch.manual_seed(0)
    S, H = 700, 2
    qkv = torch.randn(1, S, 3 * H * 128, device="cuda").bfloat16()
    q, k, v = (qkv[..., i * H * 128:(i + 1) * H * 128].unflatten(-1, (H, 128)) for i in range(3))
    assert rel(TF.attention(q, k, v), TF.attention_reference(q, k, v)) < 1e-2
    # large-magnitude scores exercise the lazy rescale of the accumulator 
    for scale_up, variant in ((6, 0), (6, 30), (20, 30), (20, 21)):
        q2 = (q.float() * scale_up).bfloat16()
        got, lse = TF.attention(q2, k, v, return_lse=True, variant=variant)
        ref, lse_ref = TF.attention_reference(q2, k, v, return_lse=True)
        assert rel(got, ref) < 2e-2, (scale_up, variant)
        assert rel(lse, lse_ref) < 1e-4, (scale_up, variant)


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


def test_attention_int8_scores():
    """Quantisers against their PyTorch statement, then the int8-score kernel against (a) the fp32 evaluation of the
    same quantised operands (kernel arithmetic) and (b) full-precision attention (what the quantisation costs)."""
    torch.manual_seed(0)
    B, Sq, Skv, H = 2, 300, 515, 3
    q = (torch.randn(B, Sq, H, 128, device="cuda") * 1.5).bfloat16()
    k = (torch.randn(B, Skv, H, 128, device="cuda") + 0.7).bfloat16()  # a common offset: what the mean removal is for
    v = torch.randn(B, Skv, H, 128, device="cuda").bfloat16()
    q8, qs, k8, ks, mean = TF.quantize_qk_int8(q, k)
    rq8, rqs, rk8, rks, rmean = TF.quantize_qk_int8_reference(q, k)
    assert torch.allclose(qs, rqs, rtol=1e-5) and torch.allclose(ks, rks, rtol=1e-4) and torch.allclose(mean, rmean, atol=2e-3)
    assert (q8.int() - rq8.int()).abs().max() <= 1 and (q8 != rq8).float().mean() < 1e-3
    assert (k8.int() - rk8.int()).abs().max() <= 1 and (k8 != rk8).float().mean() < 2e-2
    for causal in (False, True):
        kk, vv = (k, v) if not causal else (k[:, :Sq], v[:, :Sq])
        got = TF.attention(q, kk, vv, quant="int8", causal=causal)
        g8, gs, gk8, gks, _ = TF.quantize_qk_int8(q, kk)
        s = torch.einsum("bqhd,bkhd->bhqk", g8.float(), gk8.float()) * gs.unsqueeze(-1) * gks[:, :, None, None] / 128**0.5
        if causal:
            s = s.masked_fill(torch.ones(Sq, Sq, device="cuda", dtype=torch.bool).triu(1), float("-inf"))
        same_operands = torch.einsum("bhqk,bkhd->bqhd", s.softmax(-1), vv.float())
        assert rel(got, same_operands) < 1e-2, causal
        assert rel(got, TF.attention_reference(q, kk, vv, causal=causal)) < 4e-2, causal
    cpu = TF.attention_int8(q.cpu().float(), k.cpu().float(), v.cpu().float())
    assert rel(cpu, TF.attention_reference(q.cpu().float(), k.cpu().float(), v.cpu().float())) < 4e-2


@pytest.mark.gpu
@pytest.mark.parametrize("rows,C,scale", [(37, 64, 1.0), (130, 3000, 0.05), (5, 14400, 0.051)])
def test_softmax_rows_in_place_matches_fp32(rows, C, scale):
    torch.manual_seed(0)
    x = (torch.randn(rows, C, device="cuda") * 6).bfloat16()
    want = torch.softmax(x.float() * scale, dim=-1)
    got = TF.softmax_rows_(x.clone(), scale).float()
    assert (got - want).abs().max().item() <= 4e-3 * want.max().item() + 1e-6
    assert (got.sum(-1) - 1).abs().max().item() < 2e-2


@pytest.mark.gpu
@pytest.mark.parametrize("S,D", [(1560, 384), (200, 512), (333, 384)])
def test_wide_single_head_attention_runs_as_gemm_softmax_gemm(S, D):
    """The VAE mid-block attention (one head, D = 384 / 512): tensor-core GEMMs around the row softmax when the key
    count is a multiple of 8, the blocked fp32 evaluation otherwise; both against the fp32 oracle."""
    torch.manual_seed(0)
    q, k, v = (torch.randn(2, S, 1, D, device="cuda").bfloat16() for _ in range(3))
    before = native.launch_count()
    got = TF.attention(q, k, v).float()
    if S % 8 == 0 and S >= 1024:
        assert native.launch_count() > before
    want = TF.attention_reference(q.float(), k.float(), v.float())
    assert ((got - want).norm() / want.norm()).item() < 3e-2


@pytest.mark.gpu
def test_attention_with_additive_bias_matches_torch():
    torch.manual_seed(0)
    q, k, v = (torch.randn(2, 77, 4, 64, device="cuda").bfloat16() for _ in range(3))
    bias = torch.randn(1, 4, 77, 77, device="cuda")
    got = TF.attention(q, k, v, scale=1.0, bias=bias).float()
    want = torch.nn.functional.scaled_dot_product_attention(
        q.float().transpose(1, 2), k.float().transpose(1, 2), v.float().transpose(1, 2), attn_mask=bias, scale=1.0).transpose(1, 2)
    assert (got - want).abs().max().item() < 3e-2

