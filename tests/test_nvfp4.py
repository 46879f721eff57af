"""NVFP4 storage format: rounding on the e2m1 grid, block / tensor scales, the tiled scale layout, the weight-only
linear and the in-place model conversion."""

import pytest
import torch
from torch import nn

from telefuser_b200.ops import functional as TF
from telefuser_b200.ops import nvfp4 as F4
from telefuser_b200.testing.distributed_checks import make_tiny_inputs, make_tiny_model


def decode(codes):
    return F4.E2M1_VALUES[(codes & 7).long()] * torch.where((codes & 8) > 0, -1.0, 1.0)


def test_rounding_to_the_e2m1_grid_is_nearest_even_and_saturates():
    x = torch.tensor([0.0, 0.24, 0.25, 0.26, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 5.1, 7.0, -0.75, -6.5])
    want = torch.tensor([0.0, 0.0, 0.0, 0.5, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0, 6.0, 6.0, -1.0, -6.0])
    assert torch.equal(decode(F4.e2m1_codes(x)), want)
    g = torch.Generator().manual_seed(0)
    y = torch.rand(4096, generator=g) * 7 - 3.5
    got = decode(F4.e2m1_codes(y))
    grid = torch.cat([-F4.E2M1_VALUES.flip(0), F4.E2M1_VALUES])
    nearest = grid[(y[:, None] - grid[None]).abs().argmin(1)]
    assert torch.equal(got.abs(), nearest.abs())  # away from exact ties the nearest grid point is unique


def test_round_trip_scales_and_tiled_layout():
    torch.manual_seed(0)
    w = torch.randn(300, 256) * 0.02
    w[7] *= 40  # one loud row must not wreck the others: scales are per block of 16
    packed, sf, gs = F4.quantize_nvfp4(w)
    assert packed.shape == (300, 128) and packed.dtype == torch.uint8 and sf.shape == (300, 16) and sf.dtype == torch.float8_e4m3fn
    assert gs.shape == (1,) and torch.allclose(gs, 448 * 6 / w.abs().amax())
    back = F4.dequantize_nvfp4(packed, sf, gs)
    rel_rows = (back - w).norm(dim=1) / w.norm(dim=1)
    assert rel_rows.max().item() < 0.16 and ((back - w).norm() / w.norm()).item() < 0.12
    assert (back.abs().amax(1) <= w.abs().amax(1) * 1.13).all()  # block maxima are kept up to the scale's own rounding
    tiled = F4.swizzle_block_scales(sf)
    assert tiled.shape == (3 * 4, 512)
    raw, t = sf.view(torch.uint8), tiled.view(torch.uint8)
    for r, c in ((0, 0), (31, 3), (32, 0), (130, 5), (299, 15)):  # the documented address of a scale inside its tile
        tile = (r // 128) * 4 + c // 4
        assert t[tile, (r % 32) * 16 + ((r % 128) // 32) * 4 + c % 4] == raw[r, c]
    assert torch.equal(F4.unswizzle_block_scales(tiled, 300, 16).view(torch.uint8), raw)
    p2, sf2, gs2 = F4.quantize_nvfp4(w, swizzle=True)
    assert torch.equal(F4.dequantize_nvfp4(p2, sf2, gs2, swizzled_rows=300), back)
    p3, sf3, gs3 = F4.quantize_nvfp4(w, global_scale=1000.0)  # a calibrated scale is used as given
    assert float(gs3) == 1000.0 and ((F4.dequantize_nvfp4(p3, sf3, gs3) - w).norm() / w.norm()).item() < 0.13
    with pytest.raises(ValueError):
        F4.quantize_nvfp4(torch.randn(4, 24))
    assert torch.equal(F4.dequantize_nvfp4(*F4.quantize_nvfp4(torch.zeros(2, 32))), torch.zeros(2, 32))


def test_weight_only_linear_and_model_conversion():
    torch.manual_seed(0)
    lin = nn.Linear(256, 96)
    x = torch.randn(5, 256)
    ref = lin(x)
    F4.quantize_linear_nvfp4_(lin)
    assert isinstance(lin, F4.QuantizedLinearNVFP4) and lin.weight.dtype == torch.uint8 and lin.weight.shape == (96, 128)
    assert set(lin.state_dict()) == {"weight", "bias", "weight_scale", "weight_global_scale"}
    got = lin(x)
    assert ((got - ref).norm() / ref.norm()).item() < 0.12
    assert torch.equal(TF.linear(x, lin.weight, lin.bias), got)  # the functional linear dispatches on the tagged weight
    twin = nn.Linear(256, 96)
    F4.quantize_linear_nvfp4_(twin)
    twin.load_state_dict(lin.state_dict())
    assert torch.equal(twin(x), got)
    model = make_tiny_model()
    latents, ctx, _ = make_tiny_inputs()
    t = torch.tensor([500.0])
    ref = model(latents, t, ctx)
    assert model.enable_quant("nvfp4") == 20
    blk = model.blocks[0]
    W, _ = blk.self_attn.fused_qkv()  # the fused view carries one global scale per output row
    assert W.dtype == torch.uint8 and W.tfb_nvfp4_global.shape == (W.shape[0],) and W.tfb_nvfp4_sf.shape[0] == W.shape[0]
    out = model(latents, t, ctx)
    assert torch.isfinite(out).all() and ((out - ref).norm() / ref.norm()).item() < 0.25
