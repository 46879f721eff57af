"""MXFP4 / MXFP6 weight storage: code tables, rounding, packing, block scales, converter round trip."""

import pytest
import torch

from telefuser_b200.ops import mxfp


def test_code_tables_are_the_ocp_element_formats():
    v4 = mxfp.mx_code_values("mxfp4")
    assert v4[:8].tolist() == [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0] and torch.equal(v4[8:], -v4[:8])
    e2m3, e3m2 = mxfp.mx_code_values("mxfp6_e2m3")[:32], mxfp.mx_code_values("mxfp6_e3m2")[:32]
    assert e2m3[1] == 0.125 and e2m3[8] == 1.0 and e2m3[-1] == 7.5 and (e2m3[1:] > e2m3[:-1]).all()
    assert e3m2[1] == 0.0625 and e3m2[4] == 0.25 and e3m2[-1] == 28.0 and (e3m2[1:] > e3m2[:-1]).all()
    assert mxfp.mx_format("mxfp6") is mxfp.MX_FORMATS["mxfp6_e3m2"] and mxfp.bits_per_weight("mxfp4") == 4.25
    assert mxfp.bits_per_weight("mxfp6") == 6.25
    with pytest.raises(ValueError, match="unknown MX element format"):
        mxfp.mx_format("mxfp5")


@pytest.mark.parametrize("bits", [4, 6])
def test_packing_round_trip_and_bit_order(bits):
    g = torch.Generator().manual_seed(bits)
    codes = torch.randint(0, 1 << bits, (5, 64), generator=g, dtype=torch.uint8)
    packed = mxfp.pack_codes(codes, bits)
    assert packed.shape == (5, 64 * bits // 8) and torch.equal(mxfp.unpack_codes(packed, bits), codes)
    first = torch.zeros(1, 4, dtype=torch.uint8)
    first[0, 1] = (1 << bits) - 1  # all ones in the second element only
    raw = mxfp.pack_codes(first, bits)[0].tolist()
    assert raw == ([0xF0, 0x00] if bits == 4 else [0xC0, 0x0F, 0x00])
    with pytest.raises(ValueError, match="packing needs"):
        mxfp.pack_codes(codes[:, :3], bits)


@pytest.mark.parametrize("fmt", ["mxfp4", "mxfp6_e2m3", "mxfp6_e3m2"])
def test_every_representable_value_survives_and_ties_go_to_even(fmt):
    f = mxfp.mx_format(fmt)
    mags = mxfp.mx_code_values(f)[: 1 << (f.bits - 1)]
    n = mags.numel()
    row = torch.zeros(2 * ((n + 31) // 32) * 32)
    row[:n], row[n : 2 * n] = mags, -mags
    row[2 * n - 1] = -mags[-1]
    blocks = row.reshape(-1, 32)
    blocks[:, -1] = torch.where(blocks.abs().amax(1) < mags[-1], mags[-1], blocks[:, -1])  # every block spans the full range
    packed, sf = mxfp.quantize_mx(blocks.reshape(1, -1), f)
    assert (sf == 127).all()  # amax = largest value -> scale 2^0
    assert torch.equal(mxfp.dequantize_mx(packed, sf, f), blocks.reshape(1, -1))
    mids = (mags[:-1] + mags[1:]) / 2
    x = torch.full((1, 32 * ((mids.numel() + 30) // 31)), 0.0)
    pos = [i for i in range(x.shape[1]) if i % 32 != 31][: mids.numel()]
    x[0, pos] = mids
    x[0, 31::32] = mags[-1]
    got = mxfp.dequantize_mx(*mxfp.quantize_mx(x, f), f)[0, pos]
    even = torch.where(torch.arange(mids.numel()) % 2 == 0, mags[:-1], mags[1:])  # the neighbour with an even code
    assert torch.equal(got, even)
    big = torch.full((1, 32), 1.0)
    big[0, 0] = 2.0 ** (f.emax + 1) * 0.999  # just below the next power of two: the scale stays 2^0 and the value saturates
    packed, sf = mxfp.quantize_mx(big, f)
    assert sf[0, 0] == 127 and mxfp.dequantize_mx(packed, sf, f)[0, 0] == mags[-1]


@pytest.mark.parametrize("fmt,bound", [("mxfp4", 0.17), ("mxfp6_e2m3", 0.045), ("mxfp6_e3m2", 0.08)])
def test_block_scales_and_error_on_weights(fmt, bound):
    torch.manual_seed(0)
    w = torch.randn(96, 256) * torch.logspace(-3, 1, 96).unsqueeze(1)  # rows four decades apart
    w[5] = 0
    packed, sf = mxfp.quantize_mx(w, fmt)
    f = mxfp.mx_format(fmt)
    assert packed.shape == (96, 256 * f.bits // 8) and sf.shape == (96, 8) and sf.dtype == torch.uint8
    amax = w.reshape(96, 8, 32).abs().amax(-1)
    want = torch.floor(torch.log2(amax.clamp_min(2.0**-126))) - f.emax + 127
    assert torch.equal(sf[amax > 0].float(), want[amax > 0]) and (sf[5] == 0).all()
    deq = mxfp.dequantize_mx(packed, sf, fmt)
    assert (deq[5] == 0).all() and ((deq - w).norm() / w.norm()).item() < bound
    assert ((deq - w).abs() <= amax.repeat_interleave(32, 1).reshape(96, 256) * 0.26).all()  # no element off by more than a step
    with pytest.raises(ValueError, match="blocks of 32"):
        mxfp.quantize_mx(w[:, :40], fmt)


@pytest.mark.parametrize("kind", ["mxfp4", "mxfp6", "mxfp6_e2m3", "mxfp8", "fp8", "int8", "nvfp4"])
def test_converter_writes_and_expands_every_format(tmp_path, kind):
    from telefuser_b200.tools import convert
    from telefuser_b200.utils.model_weight import load_state_dict, save_state_dict

    torch.manual_seed(1)
    sd = {"blocks.0.attn.q.weight": torch.randn(128, 256).bfloat16() * 0.05, "blocks.0.attn.q.bias": torch.randn(128).bfloat16(),
          "blocks.0.ffn.0.weight": torch.randn(256, 128).bfloat16() * 0.05, "head.weight": torch.randn(64, 128).bfloat16()}  # fmt: skip
    save_state_dict(sd, str(tmp_path / "src.safetensors"))
    r = convert.main(["-s", str(tmp_path / "src.safetensors"), "-o", str(tmp_path / "q"), "--quantized", "--linear_dtype", kind])
    assert r["quantized"] == 2
    q = load_state_dict(str(tmp_path / "q" / "converted.safetensors"))
    assert torch.equal(q["head.weight"], sd["head.weight"]) and q["blocks.0.attn.q.weight"].dtype != torch.bfloat16
    if kind.startswith("mxfp") and kind != "mxfp8":
        f = mxfp.mx_format(kind)
        assert q["blocks.0.attn.q.weight"].shape == (128, 256 * f.bits // 8) and q["blocks.0.attn.q.weight_sf"].shape == (128, 8)
        assert q["blocks.0.attn.q.weight_mx_format"].tolist() == [f.exp_bits, f.man_bits]
    r = convert.main(["-s", str(tmp_path / "q" / "converted.safetensors"), "-o", str(tmp_path / "d"), "--dequantize"])
    assert r["quantized"] == 2
    d = load_state_dict(str(tmp_path / "d" / "converted.safetensors"))
    assert set(d) == set(sd) and all(d[k].dtype == torch.bfloat16 and d[k].shape == sd[k].shape for k in sd)
    limit = {"mxfp4": 0.18, "nvfp4": 0.14, "mxfp6": 0.09, "mxfp6_e2m3": 0.05}.get(kind, 0.05)
    for k in ("blocks.0.attn.q.weight", "blocks.0.ffn.0.weight"):
        assert ((d[k].float() - sd[k].float()).norm() / sd[k].float().norm()).item() < limit, (k, kind)
