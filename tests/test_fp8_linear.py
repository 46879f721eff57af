"""W8A8 FP8 linear: quantisation helpers, in-place model conversion, and on GPUs the tcgen05 FP8 GEMM
with all epilogue options against an fp32 evaluation of the same quantised operands."""

import pytest
import torch
from torch import nn

from telefuser_b200.ops import functional as TF
from telefuser_b200.ops.quant import LinearFP8, quantize_linear_fp8_, quantize_weight_fp8
from telefuser_b200.testing.distributed_checks import make_tiny_inputs, make_tiny_model


def test_weight_and_row_quantisation_round_trip():
    torch.manual_seed(0)
    w = torch.randn(48, 64)
    q, s = quantize_weight_fp8(w)
    assert q.dtype == torch.float8_e4m3fn and s.shape == (48, 1)
    assert (q.float() * s - w).abs().max() <= w.abs().max() * 0.07
    x = torch.randn(5, 64)
    xq, xs = TF.quant_fp8_rowwise(x)
    assert xs.shape == (5, 1) and (xq.float() * xs - x).abs().max() <= x.abs().max() * 0.07
    lin = nn.Linear(64, 48)
    ref = lin(x)
    m = LinearFP8.from_linear(lin)
    assert (m(x) - ref).abs().max() <= 0.15 * ref.abs().max()
    sd = m.state_dict()
    assert set(sd) == {"weight", "weight_scale", "bias"}
    m2 = LinearFP8(64, 48)
    m2.load_state_dict(sd)
    assert torch.equal(m2(x), m(x))
    quantize_linear_fp8_(lin)
    assert lin.weight.dtype == torch.float8_e4m3fn and torch.equal(lin.weight.tfb_scale, lin.weight_scale)
    assert torch.allclose(TF.linear(x, lin.weight, lin.bias), m(x).to(x.dtype), atol=2e-3)  # m holds a bf16 bias


def test_wan_enable_quant_stays_close_and_keeps_fused_views():
    model = make_tiny_model()
    latents, ctx, _ = make_tiny_inputs()
    t = torch.tensor([500.0])
    ref = model(latents, t, ctx)
    n = model.enable_quant()
    assert n == 2 * 10  # per block: 4 + 4 attention projections and 2 FFN layers
    blk = model.blocks[0]
    assert blk.ffn[0].weight.dtype == torch.float8_e4m3fn and model.head.head.weight.dtype == torch.float32
    W, _ = blk.self_attn.fused_qkv()
    assert W.dtype == torch.float8_e4m3fn and W.tfb_scale.shape == (3 * 128,)
    out = model(latents, t, ctx)
    assert torch.isfinite(out).all()
    assert ((out - ref).norm() / ref.norm()).item() < 0.1


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", [(300, 256, 512), (1024, 1536, 5120), (77, 72, 144)])
def test_fp8_gemm_matches_fp32_product_of_the_quantised_operands(M, N, K):
    torch.manual_seed(0)
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = torch.randn(N, K, device="cuda") / K**0.5
    bias = torch.randn(N, device="cuda").bfloat16()
    res = torch.randn(M, N, device="cuda").bfloat16()
    gate = torch.randn(1, N, device="cuda")
    q, ws = quantize_weight_fp8(w)
    xq, xs = TF.quant_fp8_rowwise(x)
    rq, rs = TF.quant_fp8_rowwise(x.float().cpu())
    assert (xq.view(torch.uint8).cpu() != rq.view(torch.uint8)).float().mean() < 2e-3
    assert torch.allclose(xs.cpu(), rs, rtol=1e-6, atol=0)
    base = (xq.float() @ q.float().t()) * xs * ws.reshape(1, -1)
    for kw in (dict(), dict(bias=bias), dict(bias=bias, act="gelu_tanh"), dict(bias=bias, residual=res, gate=gate)):
        got = TF.linear_fp8(x, q, ws, **kw).float()
        want = base.clone()
        if "bias" in kw:
            want = want + bias.float()
        if kw.get("act"):
            want = torch.nn.functional.gelu(want, approximate="tanh")
        if "gate" in kw:
            want = want * gate
        if "residual" in kw:
            want = want + res.float()
        err = ((got - want).abs() / (1 + want.abs())).max().item()
        assert err <= 1.5e-2, (kw.keys(), err)


@pytest.mark.gpu
def test_fp8_wan_block_on_gpu_tracks_bf16():
    model = make_tiny_model(dtype=torch.bfloat16, preset="native-small").cuda()
    latents, ctx, _ = make_tiny_inputs()
    t = torch.tensor([500.0], device="cuda")
    ref = model(latents.cuda().bfloat16(), t, ctx.cuda().bfloat16()).float()
    assert model.enable_quant() == 20
    out = model(latents.cuda().bfloat16(), t, ctx.cuda().bfloat16()).float()
    assert ((out - ref).norm() / ref.norm()).item() < 0.1


def test_scale_follows_the_module_across_moves_copies_and_pickling():
    import copy
    import io

    def round_trip(m):
        buf = io.BytesIO()
        torch.save(m, buf)
        buf.seek(0)
        return torch.load(buf, weights_only=False)

    torch.manual_seed(0)
    x = torch.randn(5, 64)
    for make in (lambda: quantize_linear_fp8_(nn.Linear(64, 48)), lambda: LinearFP8.from_linear(nn.Linear(64, 48))):
        lin = make()
        want = TF.linear(x, lin.weight, lin.bias)
        old = lin.weight_scale
        lin._apply(lambda t: t.clone())  # what .to() / .cuda() do: new buffer object, same Parameter object
        assert lin.weight_scale is not old and lin.weight.tfb_scale is lin.weight_scale
        assert TF.fp8_weight_scale(lin.weight) is lin.weight_scale
        for other in (copy.deepcopy(lin), round_trip(lin)):
            assert other.weight.tfb_scale is other.weight_scale
            assert torch.equal(TF.linear(x, other.weight, other.bias), want)
    model = make_tiny_model()
    model.enable_quant()
    model._apply(lambda t: t.clone())
    blk = model.blocks[0]
    W, _ = blk.self_attn.fused_qkv()
    live = torch.cat([m.weight_scale.reshape(-1) for m in (blk.self_attn.q, blk.self_attn.k, blk.self_attn.v)])
    assert torch.equal(W.tfb_scale, live)
    assert all(m.weight.tfb_scale is m.weight_scale for m in (blk.self_attn.q, blk.ffn[0]))


@pytest.mark.gpu
def test_model_quantised_on_the_host_then_moved_runs_on_the_device():
    torch.manual_seed(0)
    lin = nn.Linear(256, 128).bfloat16()
    x = torch.randn(64, 256).bfloat16()
    ref = lin(x).float()
    quantize_linear_fp8_(lin)
    lin.cuda()
    assert lin.weight.tfb_scale.is_cuda and lin.weight.tfb_scale is lin.weight_scale
    got = TF.linear(x.cuda(), lin.weight, lin.bias).float().cpu()
    assert ((got - ref).norm() / ref.norm()).item() < 0.06
    from telefuser_b200.ops import native

    with pytest.raises(native.NativeLibraryError):
        TF.linear_fp8(x.cuda(), lin.weight, lin.weight_scale, lin.bias.cpu())


def test_mxfp8_linear_reference_path_and_model_conversion():
    torch.manual_seed(0)
    x, w = torch.randn(70, 256), torch.randn(64, 256)
    wq, wsf = TF.quantize_weight_mxfp8(w)
    assert wq.dtype == torch.float8_e4m3fn and wsf.shape == (1, 2, 512) and wsf.dtype == torch.uint8
    want = x @ w.t()
    assert ((TF.linear_mxfp8(x, wq, wsf) - want).norm() / want.norm()).item() < 0.05
    sf = torch.randint(0, 255, (300, 8), dtype=torch.uint8)
    tiled = TF.mx_tile_scales(sf)
    assert torch.equal(TF.mx_untile_scales(tiled, 300), sf)
    r, b = 137, 5  # row 137, 32-element block 5: tile (1, 1), inside it (r%32)*16 + (r/32)*4 + b%4
    assert tiled.view(-1)[((r >> 7) * 2 + (b >> 2)) * 512 + (r & 31) * 16 + ((r >> 5) & 3) * 4 + (b & 3)] == sf[r, b]

    model = make_tiny_model()
    latents, ctx, _ = make_tiny_inputs()
    t = torch.tensor([500.0])
    ref = model(latents, t, ctx)
    assert model.enable_quant("mxfp8") == 20
    blk = model.blocks[0]
    assert blk.ffn[0].weight.tfb_mx_sf is blk.ffn[0].weight_scale_mx
    W, _ = blk.self_attn.fused_qkv()
    assert W.dtype == torch.float8_e4m3fn and W.tfb_mx_sf.shape == (3, 1, 512)
    out = model(latents, t, ctx)
    assert ((out - ref).norm() / ref.norm()).item() < 0.1
    model._apply(lambda t_: t_.clone())
    assert blk.ffn[0].weight.tfb_mx_sf is blk.ffn[0].weight_scale_mx


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", [(256, 256, 256), (300, 200, 512), (1024, 1536, 5120), (77, 72, 128), (512, 960, 256)])
def test_mxfp8_gemm_matches_fp32_product_of_the_dequantised_operands(M, N, K):
    torch.manual_seed(0)
    x = (torch.randn(M, K, device="cuda") * torch.rand(M, 1, device="cuda") * 4).bfloat16()
    # every weight row gets its own power-of-two magnitude: a scale factor read from the wrong row shows as a 2x error
    w = (torch.randn(N, K, device="cuda") / K**0.5 * torch.exp2(torch.randint(-3, 4, (N, 1), device="cuda"))).bfloat16()
    bias = torch.randn(N, device="cuda").bfloat16()
    res = torch.randn(M, N, device="cuda").bfloat16()
    gate = torch.randn(1, N, device="cuda")
    wq, wsf = TF.quantize_weight_mxfp8(w)
    xq, xsf_t = TF.quant_mxfp8(x, tiled=True)
    xq_r, xsf_r = TF.quant_mxfp8(x)
    assert torch.equal(xq, xq_r) and torch.equal(TF.mx_untile_scales(xsf_t, M), xsf_r)  # tiled order written right
    base = TF.dequant_mxfp8(xq, xsf_r) @ TF.dequant_mxfp8(wq.view(torch.uint8), TF.mx_untile_scales(wsf, N)).t()
    for kw in (dict(), dict(bias=bias), dict(bias=bias, act="gelu_tanh"), dict(bias=bias, residual=res, gate=gate)):
        got = TF.linear_mxfp8(x, wq, wsf, **kw).float()
        want = base.clone()
        if "bias" in kw:
            want = want + bias.float()
        if kw.get("act"):
            want = torch.nn.functional.gelu(want, approximate="tanh")
        if "gate" in kw:
            want = want * gate
        if "residual" in kw:
            want = want + res.float()
        err = ((got - want).abs() / (1 + want.abs())).max().item()
        assert err <= 1.5e-2, (kw.keys(), err)
    full = (x.float() @ w.float().t())
    assert ((TF.linear_mxfp8(x, wq, wsf).float() - full).norm() / full.norm()).item() < 0.05


@pytest.mark.parametrize("kind", ["fp8", "mxfp8", "int8", "nvfp4"])
def test_quantised_sidecar_round_trip(tmp_path, kind):
    from telefuser_b200.ops.quant import load_quantized_sidecar, save_quantized_sidecar

    latents, ctx, _ = make_tiny_inputs()
    t = torch.tensor([500.0])
    model = make_tiny_model()
    model.enable_quant(kind)
    want = model(latents, t, ctx)
    path = str(tmp_path / "dit.quant.safetensors")
    assert save_quantized_sidecar(model, path) == 20
    fresh = make_tiny_model()  # same seed: identical bf16 weights, not quantised
    assert fresh.blocks[0].ffn[0].weight.dtype != torch.float8_e4m3fn
    assert load_quantized_sidecar(fresh, path) == 20
    lin = fresh.blocks[0].ffn[0]
    assert lin.weight.dtype == {"int8": torch.int8, "nvfp4": torch.uint8}.get(kind, torch.float8_e4m3fn)
    if kind == "mxfp8":
        assert lin.weight.tfb_mx_sf is lin.weight_scale_mx
    elif kind == "nvfp4":
        assert lin.weight.tfb_nvfp4_sf is lin.weight_scale and lin.weight_scale.dtype == torch.float8_e4m3fn
    else:
        assert lin.weight.tfb_scale is lin.weight_scale
    assert torch.equal(fresh(latents, t, ctx), want)  # no second quantisation: bit-identical weights and scales
    with pytest.raises(ValueError, match="not a quantised side-car"):
        from safetensors.torch import save_file

        save_file({"x": torch.zeros(1)}, str(tmp_path / "other.safetensors"))
        load_quantized_sidecar(fresh, str(tmp_path / "other.safetensors"))


def test_int8_linear_and_per_tensor_quantisation_reference_paths():
    torch.manual_seed(0)
    x, w = torch.randn(9, 64), torch.randn(48, 64) / 8
    q, s = TF.quantize_weight_int8(w)
    assert q.dtype == torch.int8 and s.shape == (48,) and int(q.abs().max()) == 127
    xq, xs = TF.quant_int8_rowwise(x)
    assert xq.dtype == torch.int8 and (xq.float() * xs - x).abs().max() <= x.abs().max() / 127 * 0.51
    full = x @ w.t()
    got = TF.linear_int8(x, q, s)
    assert ((got - full).norm() / full.norm()).item() < 0.02
    q.tfb_scale = s
    assert torch.equal(TF.linear(x, q), got)  # the functional linear dispatches on the int8 weight
    from telefuser_b200.ops.quant import QuantizedLinearInt8, quantize_linear_int8_

    lin = nn.Linear(64, 48)
    ref = lin(x)
    quantize_linear_int8_(lin)
    assert isinstance(lin, QuantizedLinearInt8) and lin.weight.dtype == torch.int8
    assert ((lin(x) - ref).norm() / ref.norm()).item() < 0.02
    model = make_tiny_model()
    latents, ctx, _ = make_tiny_inputs()
    t = torch.tensor([500.0])
    ref = model(latents, t, ctx)
    assert model.enable_quant("int8") == 20 and model.blocks[0].ffn[0].weight.dtype == torch.int8
    out = model(latents, t, ctx)
    assert ((out - ref).norm() / ref.norm()).item() < 0.05
    # per-tensor: dynamic scale = amax / 448, static scale used as given
    pq, ps = TF.quant_fp8_per_tensor(x)
    assert ps.shape == (1,) and torch.allclose(ps, x.abs().amax().reshape(1) / 448)
    assert (pq.float() * ps - x).abs().max() <= x.abs().max() * 0.07
    pq2, ps2 = TF.quant_fp8_per_tensor(x, scale=torch.tensor([0.05]))
    assert float(ps2) == pytest.approx(0.05) and torch.equal(pq2, (x / 0.05).clamp(-448, 448).to(torch.float8_e4m3fn))


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", [(300, 256, 512), (1024, 1536, 5120), (77, 72, 144)])
def test_int8_gemm_is_exact_on_the_integer_product(M, N, K):
    torch.manual_seed(0)
    x = (torch.randn(M, K, device="cuda") * torch.rand(M, 1, device="cuda") * 4).bfloat16()
    w = torch.randn(N, K, device="cuda") / K**0.5
    bias = torch.randn(N, device="cuda").bfloat16()
    res = torch.randn(M, N, device="cuda").bfloat16()
    gate = torch.randn(1, N, device="cuda")
    wq, ws = TF.quantize_weight_int8(w)
    xq, xs = TF.quant_int8_rowwise(x)
    xq_r = torch.round(x.float() / xs).clamp(-127, 127).to(torch.int8)
    assert torch.allclose(xs, (x.float().abs().amax(-1, keepdim=True) / 127).clamp_min(1e-12), rtol=1e-6)
    assert (xq.int() - xq_r.int()).abs().max().item() <= 1 and (xq != xq_r).float().mean().item() < 1e-3
    prod = (xq.double() @ wq.double().t()).float()  # exact: |sum| < 2^24 * 127 fits a double easily
    base = prod * xs * ws
    for kw in (dict(), dict(bias=bias), dict(bias=bias, act="gelu_tanh"), dict(bias=bias, residual=res, gate=gate)):
        got = TF.linear_int8(x, wq, ws, **kw).float()
        want = base.clone()
        if "bias" in kw:
            want = want + bias.float()
        if kw.get("act"):
            want = torch.nn.functional.gelu(want, approximate="tanh")
        if "gate" in kw:
            want = want * gate
        if "residual" in kw:
            want = want + res.float()
        err = ((got - want).abs() / (1 + want.abs())).max().item()
        assert err <= 1e-2, (kw.keys(), err)  # bf16 rounding of the output only
    full = x.float() @ w.t()
    assert ((TF.linear_int8(x, wq, ws).float() - full).norm() / full.norm()).item() < 0.02


@pytest.mark.gpu
@pytest.mark.parametrize("C", [64, 5120, 13824, 20480])
def test_row_and_tensor_quantisers_match_their_references_at_every_width(C):
    torch.manual_seed(0)
    x = (torch.randn(37, C, device="cuda") * torch.rand(37, 1, device="cuda") * 3).bfloat16()
    q, s = TF.quant_fp8_rowwise(x)
    s_ref = (x.float().abs().amax(-1, keepdim=True) / 448).clamp_min(1e-12)
    assert torch.allclose(s, s_ref, rtol=1e-6)
    assert torch.equal(q.float(), (x.float() * (1 / s_ref)).to(torch.float8_e4m3fn).float()) or \
        ((q.float() - (x.float() / s_ref).to(torch.float8_e4m3fn).float()).abs() > 0).float().mean().item() < 1e-3
    q8, s8 = TF.quant_int8_rowwise(x)
    assert (q8.float() * s8 - x.float()).abs().max().item() <= (s8.max().item() * 0.51 + 1e-6)
    pq, ps = TF.quant_fp8_per_tensor(x)
    assert torch.allclose(ps, x.float().abs().amax().reshape(1) / 448, rtol=1e-6)
    want = (x.float() / ps).to(torch.float8_e4m3fn).float()
    assert ((pq.float() - want).abs() > 0).float().mean().item() < 1e-3
    pq2, ps2 = TF.quant_fp8_per_tensor(x, scale=torch.tensor([0.02], device="cuda"))
    assert float(ps2) == pytest.approx(0.02)
    assert ((pq2.float() - (x.float() / 0.02).clamp(-448, 448).to(torch.float8_e4m3fn).float()).abs() > 0).float().mean().item() < 1e-3


def test_bmm_fp8_reference_path():
    torch.manual_seed(0)
    a = (torch.randn(3, 5, 32) * 4).to(torch.float8_e4m3fn)
    b = (torch.randn(3, 7, 32) * 4).to(torch.float8_e4m3fn).transpose(1, 2)  # [B, K, N] with K contiguous
    sa, sb = torch.tensor([0.25]), torch.tensor(0.5)
    got = TF.bmm_fp8(a, b, sa, sb, torch.float32)
    assert got.shape == (3, 5, 7) and torch.allclose(got, torch.bmm(a.float(), b.float()) * 0.125)
    out = torch.empty(3, 5, 7, dtype=torch.bfloat16)
    assert TF.bmm_fp8(a, b, sa, sb, out=out) is out and torch.allclose(out.float(), got, rtol=1e-2, atol=1e-2)
    with pytest.raises(ValueError):
        TF.bmm_fp8(a, b[:, :16], sa, sb)


@pytest.mark.gpu
@pytest.mark.parametrize("B,M,N,K", [(2, 300, 256, 512), (3, 77, 72, 144)])
def test_bmm_fp8_runs_every_batch_entry_on_the_fp8_gemm(B, M, N, K):
    torch.manual_seed(0)
    a = torch.randn(B, M, K, device="cuda").to(torch.float8_e4m3fn)
    b = torch.randn(B, N, K, device="cuda").to(torch.float8_e4m3fn).transpose(1, 2)
    sa, sb = torch.tensor([0.02], device="cuda"), torch.tensor([3.0], device="cuda")
    from telefuser_b200.ops import native

    before = native.launch_count()
    got = TF.bmm_fp8(a, b, sa, sb).float()
    assert native.launch_count() - before == B
    want = torch.bmm(a.float(), b.float()) * 0.06
    assert ((got - want).abs() / (1 + want.abs())).max().item() <= 1e-2  # bf16 rounding of the output only
    f32 = TF.bmm_fp8(a, b, sa, sb, torch.float32)
    assert f32.dtype == torch.float32 and torch.allclose(f32, got, atol=1e-6)
