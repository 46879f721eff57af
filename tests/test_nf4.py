"""NF4 weight-only quantisation: codebook round trip, packed layout, in-place model conversion, GPU expansion kernel."""

import pytest
import torch
from torch import nn

from telefuser_b200.ops import functional as TF
from telefuser_b200.ops import nf4


def test_quantise_round_trip_and_layout():
    torch.manual_seed(0)
    w = torch.randn(32, 128)
    packed, absmax = nf4.quantize_nf4(w)
    assert packed.shape == (32 * 128 // 2,) and packed.dtype == torch.uint8 and absmax.shape == (64,)
    deq = nf4.dequantize_nf4_reference(packed, absmax, w.shape)
    # every value lands on the nearest level of its block: error below half the widest level gap times the block maximum
    gap = (nf4.NF4_LEVELS[1:] - nf4.NF4_LEVELS[:-1]).max() / 2
    assert ((deq - w).abs().view(-1, 64) <= gap * absmax[:, None] + 1e-6).all()
    assert (deq - w).pow(2).mean().sqrt() < 0.12
    # exact levels survive; first value of a pair sits in the high nibble
    exact = (nf4.NF4_LEVELS[torch.randint(0, 16, (64,))] * 3.0).clone()
    exact[0] = 3.0
    p2, a2 = nf4.quantize_nf4(exact)
    assert torch.allclose(nf4.dequantize_nf4_reference(p2, a2, (64,)), exact, atol=1e-6) and float(a2) == 3.0 and int(p2[0]) >> 4 == 15
    with pytest.raises(ValueError):
        nf4.quantize_nf4(torch.randn(10, 10))


def test_linear_module_and_in_place_model():
    torch.manual_seed(0)
    lin = nn.Linear(128, 64)
    x = torch.randn(3, 128)
    q = nf4.LinearNF4.from_linear(lin, compute_dtype=torch.float32)
    ref = lin(x)
    assert (q(x) - ref).abs().max() < 0.25 * ref.abs().max() and set(q.state_dict()) == {"weight", "absmax", "bias"}
    model = nn.Sequential(nn.Linear(128, 256), nn.GELU(), nn.Linear(256, 128), nn.Linear(128, 8))
    dense = [m.weight.detach().clone() for m in model if isinstance(m, nn.Linear)]
    assert nf4.quantize_model_nf4_(model, exclude_names=("3",)) == 2
    assert model[0].weight.dtype == torch.uint8 and model[0].weight.shape == (256, 64) and model[3].weight.dtype == torch.float32
    y = TF.linear(x, model[0].weight, model[0].bias)  # the functional path expands tagged packed weights
    assert (y - torch.nn.functional.linear(x, dense[0], model[0].bias)).abs().max() < 0.3
    assert "0.absmax" in model.state_dict() and nf4.quantize_model_nf4_(model, exclude_names=("3",)) == 2  # idempotent
    fresh = nn.Sequential(nn.Linear(128, 64), nn.Linear(64, 128))
    assert nf4.replace_linear_layers_with_nf4(fresh, torch.float32, exclude_names=["1"]) == 1 and isinstance(fresh[0], nf4.LinearNF4)


def test_ltx_transformer_nf4():
    from telefuser_b200.core.config import QuantConfig, QuantType
    from telefuser_b200.models import ltx_dit as D

    torch.manual_seed(0)
    net = D.LTXVideoTransformer({"transformer": dict(num_attention_heads=2, attention_head_dim=32, num_layers=1, cross_attention_dim=64,
                                                      audio_num_attention_heads=2, audio_attention_head_dim=32, audio_cross_attention_dim=64)},
                                D.LTXModelType.VideoOnly)  # fmt: skip
    for p in net.parameters():
        torch.nn.init.normal_(p, std=0.05)
    net = net.float().eval()
    pos = torch.rand(1, 3, 6, 2)
    mod = D.Modality(latent=torch.randn(1, 6, 128), sigma=torch.tensor([0.5]), timesteps=torch.full((1, 6, 1), 0.5), positions=pos,
                     context=torch.randn(1, 4, 64))  # fmt: skip
    ref, _ = net(mod, None)
    n = net.enable_quant(QuantConfig(enabled=True, quant_type=QuantType.BNB_NF4))
    assert n == 10 and net.velocity_model.transformer_blocks[0].attn1.to_q.weight.dtype == torch.uint8
    out, _ = net(mod, None)
    assert torch.isfinite(out).all() and (out - ref).norm() / ref.norm() < 0.35


@pytest.mark.gpu
def test_gpu_dequant_kernel_and_linear():
    torch.manual_seed(0)
    w = torch.randn(512, 1024)
    packed, absmax = nf4.quantize_nf4(w)
    ref = nf4.dequantize_nf4_reference(packed, absmax, w.shape)
    got = nf4.dequantize_nf4(packed.cuda(), absmax.cuda(), w.shape)
    assert got.dtype == torch.bfloat16 and (got.float().cpu() - ref).abs().max() <= ref.abs().max() * 2**-8
    lin = nn.Linear(1024, 512).to("cuda", torch.bfloat16)
    x = torch.randn(64, 1024, device="cuda", dtype=torch.bfloat16)
    dense = lin(x).float()
    nf4.quantize_linear_nf4_(lin)
    y = TF.linear(x, lin.weight, lin.bias).float()
    w_deq = nf4.dequantize_nf4_reference(lin.weight.data.reshape(-1).cpu(), lin.absmax.cpu(), (512, 1024))
    oracle = x.float().cpu() @ w_deq.T + lin.bias.float().cpu()
    assert (y.cpu() - oracle).abs().max() < 0.05 * oracle.abs().max() and (y - dense).norm() / dense.norm() < 0.2
