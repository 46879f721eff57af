"""RIFE frame interpolation and Real-ESRGAN upscaling: timing of the resampled frames, warp identity, batched
synthesis equals per-pair synthesis, architecture detection from checkpoints, the shared stages."""

import torch
from PIL import Image

from telefuser_b200.core.config import ModelRuntimeConfig
from telefuser_b200.models.realesrgan import RRDBNet, RealESRGAN, SRVGGNetCompact, build_net_from_state_dict
from telefuser_b200.models.rife import IFNet, target_frame_positions, warp
from telefuser_b200.pipelines.common import RealESRGANStage, RiftVFIStage


def test_frame_positions_and_warp():
    pos = target_frame_positions(16, 32, 3)
    assert [p[:2] for p in pos] == [(0, 1), (0, 1), (1, 2), (1, 2), (2, 2)]
    assert [round(p[2], 3) for p in pos] == [0.0, 0.5, 0.0, 0.5, 0.0]
    img = torch.rand(1, 3, 8, 10)
    assert torch.allclose(warp(img, torch.zeros(1, 2, 8, 10)), img, atol=1e-6)
    shifted = warp(img, torch.cat([torch.ones(1, 1, 8, 10), torch.zeros(1, 1, 8, 10)], 1))  # sample one pixel to the right
    assert torch.allclose(shifted[..., :-1], img[..., 1:], atol=1e-5)


def test_rife_batched_interpolation_equals_per_pair():
    torch.manual_seed(0)
    net = IFNet().eval()
    for p in net.parameters():
        torch.nn.init.normal_(p, std=0.02)
    keys = set(net.state_dict())
    assert {"block0.conv0.0.0.weight", "block4.convblock.7.beta", "block2.lastconv.0.weight", "encode.cnn3.weight"} <= keys
    clip = torch.rand(3, 40, 56, 3)
    out = net.interpolate_frames(clip, 8, 20, device="cpu", batch=3)
    pos = target_frame_positions(8, 20, 3)
    assert out.shape == (len(pos), 40, 56, 3)
    pad = torch.nn.functional.pad(clip.permute(0, 3, 1, 2), (0, 128 - 56, 0, 128 - 40))
    for k, (i0, i1, f) in enumerate(pos):
        if f == 0.0:
            assert torch.equal(out[k], clip[i0])
        else:
            with torch.no_grad():
                one = net.interpolate_frame(pad[i0 : i0 + 1], pad[i1 : i1 + 1], f)[0, :, :40, :56].permute(1, 2, 0)
            assert torch.allclose(out[k], one, atol=1e-5)
    stage = RiftVFIStage("vfi", None, ModelRuntimeConfig(device_type="cpu", torch_dtype=torch.float32), model=net)
    stage.onload_models_flag = True
    frames = stage.process([Image.new("RGB", (32, 24), (10 * i, 0, 0)) for i in range(3)], 8, 16)
    assert len(frames) == 5 and frames[0].size == (32, 24)


def test_realesrgan_architectures_and_stage(tmp_path):
    torch.manual_seed(0)
    compact = SRVGGNetCompact(num_feat=8, num_conv=2, upscale=2)
    rebuilt = build_net_from_state_dict(compact.state_dict())
    assert isinstance(rebuilt, SRVGGNetCompact) and rebuilt.upscale == 2 and len(rebuilt.body) == len(compact.body)
    rrdb = RRDBNet(num_feat=8, num_block=2, num_grow_ch=4)
    again = build_net_from_state_dict(rrdb.state_dict())
    assert isinstance(again, RRDBNet) and len(again.body) == 2
    assert rrdb(torch.rand(1, 3, 6, 6)).shape == (1, 3, 24, 24)
    path = tmp_path / "w.pth"
    torch.save({"params_ema": compact.state_dict()}, path)
    model = RealESRGAN(str(path), scale=3)
    up = model.upscale_frames(torch.rand(3, 6, 8, 3), device="cpu", batch=2)
    assert up.shape == (3, 18, 24, 3) and model.native_scale == 2 and 0 <= up.min() and up.max() <= 1
    stage = RealESRGANStage("up", None, ModelRuntimeConfig(device_type="cpu", torch_dtype=torch.float32), model=model)
    stage.onload_models_flag = True
    assert stage.process([Image.new("RGB", (8, 6))])[0].size == (24, 18)
    assert stage.process_tensor(torch.rand(1, 6, 8, 3)).shape == (1, 18, 24, 3)
