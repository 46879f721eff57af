"""Property tests (hypothesis) of small pieces whose inputs vary widely in production: tensor packing for weight sharding
and offload, sequence padding, the flow-match sampler's exactness on straight paths, MX / NVFP4 codecs, frame-count rules."""

import math

import torch
from hypothesis import given, settings
from hypothesis import strategies as st
from torch import nn

from telefuser_b200.utils.packing import ALIGN, PackedBlock

FAST = settings(max_examples=40, deadline=None, derandomize=True, database=None)  # the same cases on every run


@FAST
@given(st.lists(st.tuples(st.integers(1, 9), st.integers(1, 9)), min_size=1, max_size=5), st.booleans(), st.integers(0, 2**31 - 1))
def test_packing_keeps_values_views_and_alignment(shapes, fuse_first_two, seed):
    torch.manual_seed(seed)
    layers = [nn.Linear(i * 8, o * 8, bias=True) for o, i in shapes]
    if fuse_first_two and len(layers) >= 2 and layers[0].in_features == layers[1].in_features:
        # two weights re-homed as row slices of one buffer (a fused projection): they must stay adjacent after packing
        both = torch.cat([layers[0].weight.data, layers[1].weight.data])
        layers[0].weight.data, layers[1].weight.data = both[: layers[0].out_features], both[layers[0].out_features :]
    block = nn.ModuleList(layers)
    want = {n: p.detach().clone() for n, p in block.named_parameters()}
    packed = PackedBlock(block, min_numel=1)
    flat = torch.full((packed.numel,), float("nan"))
    packed.pack_into(flat)
    packed.bind(flat)
    for n, p in block.named_parameters():
        assert torch.equal(p.data, want[n])
        if p.dim() == 2:
            assert p.data.untyped_storage().data_ptr() == flat.untyped_storage().data_ptr()  # a view into the slot
    offsets = sorted({o for t, o, _, _ in packed.entries if t.dim() == 2 and t.storage_offset() % ALIGN == 0})
    assert all(o % ALIGN == 0 for o in offsets) and packed.numel % ALIGN == 0
    if fuse_first_two and len(layers) >= 2 and layers[0].in_features == layers[1].in_features:
        a, b = layers[0].weight.data, layers[1].weight.data
        assert b.data_ptr() == a.data_ptr() + a.numel() * a.element_size()
    # a second slot: re-binding moves every packed tensor, and writes through the views land in the new slot
    other = flat.clone()
    packed.bind(other)
    layers[0].weight.data.zero_()
    assert not torch.equal(other, flat) or layers[0].weight.numel() == 0


@FAST
@given(st.integers(1, 5000), st.integers(1, 16))
def test_padded_length_is_the_smallest_multiple(n, parts):
    from telefuser_b200.parallel.shard import padded_len

    p = padded_len(n, parts)
    assert p % parts == 0 and n <= p < n + parts


@FAST
@given(st.integers(2, 60), st.floats(0.5, 12.0), st.integers(0, 2**31 - 1))
def test_flow_match_euler_is_exact_on_straight_paths(steps, shift, seed):
    """With the true velocity x1 - x0 of a straight noise -> data path, Euler over any shifted schedule lands on the data."""
    from telefuser_b200.schedulers.flow_match import FlowMatchScheduler

    g = torch.Generator().manual_seed(seed)
    data, noise = torch.randn(2, 3, generator=g, dtype=torch.float64), torch.randn(2, 3, generator=g, dtype=torch.float64)
    sch = FlowMatchScheduler("Wan")
    sch.set_timesteps(steps, shift=shift)
    sig = sch.sigmas.double()
    assert sig[0] <= 1.0 + 1e-6 and (sig[1:] < sig[:-1]).all() and sig[-1] > 0
    x = sch.add_noise(data, noise, sch.timesteps[0])
    assert torch.allclose(x, (1 - sig[0]) * data + sig[0] * noise, atol=1e-6)
    for i, t in enumerate(sch.timesteps):
        x = sch.step(noise - data, t, x, to_final=i == steps - 1)
    assert torch.allclose(x, data, atol=1e-5)


@FAST
@given(st.sampled_from(["mxfp4", "mxfp6_e2m3", "mxfp6_e3m2"]), st.integers(1, 6), st.integers(1, 4), st.floats(-12, 12), st.integers(0, 2**31 - 1))
def test_mx_codecs_are_idempotent_and_bounded(fmt, rows, blocks, log_scale, seed):
    from telefuser_b200.ops import mxfp

    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, blocks * 32, generator=g) * 2.0**log_scale
    packed, sf = mxfp.quantize_mx(x, fmt)
    deq = mxfp.dequantize_mx(packed, sf, fmt)
    again = mxfp.quantize_mx(deq, fmt)
    assert torch.equal(again[0], packed) and torch.equal(again[1], sf)  # representable values survive a second pass
    f = mxfp.mx_format(fmt)
    step = torch.exp2(sf.float() - 127 + f.emax - f.man_bits).repeat_interleave(32, 1)  # spacing at the top binade
    sat = torch.exp2(sf.float() - 127).repeat_interleave(32, 1) * float(mxfp.mx_code_values(f).max())
    inside = x.abs() <= sat
    assert ((deq - x).abs()[inside] <= step[inside] / 2 + 1e-30).all() and (torch.sign(deq) * torch.sign(x) >= 0).all()


@FAST
@given(st.integers(1, 4), st.integers(1, 4), st.floats(-8, 8), st.integers(0, 2**31 - 1))
def test_nvfp4_round_trip_is_stable(rows, blocks, log_scale, seed):
    from telefuser_b200.ops.nvfp4 import dequantize_nvfp4, quantize_nvfp4

    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows * 8, blocks * 16, generator=g) * 2.0**log_scale
    packed, sf, gs = quantize_nvfp4(x)
    deq = dequantize_nvfp4(packed, sf, gs, torch.float32)
    assert torch.isfinite(deq).all() and ((deq - x).norm() / x.norm()).item() < 0.2
    p2, sf2, _ = quantize_nvfp4(deq, global_scale=gs)
    assert torch.equal(dequantize_nvfp4(p2, sf2, gs, torch.float32), deq)  # a fixed point after one pass


@FAST
@given(st.integers(0, 60), st.integers(1, 8), st.sampled_from(["strict", "truncate"]))
def test_frame_count_rule_is_consistent(n, chunk, policy):
    from telefuser_b200.pipelines.lingbot_world.session import resolve_lingbot_frame_count

    frames = 4 * n + 1
    latent = n + 1
    try:
        eff, lat = resolve_lingbot_frame_count(frames, chunk, policy)
    except ValueError:
        assert latent < chunk or (policy == "strict" and latent % chunk)
        return
    assert lat % chunk == 0 and lat >= chunk and eff == 4 * (lat - 1) + 1 and eff <= frames
    assert (lat == latent) if policy == "strict" else (latent - lat < chunk)


@FAST
@given(st.floats(0.0, 30.0), st.sampled_from([8, 16, 24, 30]))
def test_duration_to_frames_covers_the_duration(duration, fps):
    from telefuser_b200.pipelines.lingbot_video.data import num_frames_from_duration, validate_frame_count

    n = num_frames_from_duration(duration, fps)
    assert validate_frame_count(n) == n and n >= int(duration * fps) and n - int(duration * fps) <= 4
    assert math.isclose(num_frames_from_duration(0, fps), 1)
