"""VAE kernels: the implicit-GEMM causal convolution, the fused pixel norm + SiLU and the 2x upsample against their
fp32 statements, and the whole decoder on the native path (bf16, channels-last) against the fp32 evaluation."""

import pytest
import torch
import torch.nn.functional as F

from telefuser_b200.ops import functional as TF


def rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


def test_reference_conv_chunks_with_prev_equal_the_whole_clip():
    torch.manual_seed(0)
    x, w, b = torch.randn(1, 8, 7, 6, 5), torch.randn(4, 8, 3, 3, 3), torch.randn(4)
    whole = TF.conv3d_causal(x, w, b)
    parts = [TF.conv3d_causal(x[:, :, :3], w, b), TF.conv3d_causal(x[:, :, 3:4], w, b, prev=x[:, :, 1:3]),
             TF.conv3d_causal(x[:, :, 4:], w, b, prev=x[:, :, 3:4])]  # one frame of history: the other is zeros
    assert torch.allclose(torch.cat(parts[:2], 2), whole[:, :, :4], atol=1e-5)
    assert torch.equal(TF.conv_weight_taps(w)[2, 5], w[2, :, 0, 1, 2].bfloat16())
    lib = F.conv3d(F.pad(x, (1, 1, 1, 1, 2, 0)), w, b)
    assert torch.allclose(whole, lib, atol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("cin,cout,k,T,H,W", [(16, 96, (3, 3, 3), 3, 13, 21), (96, 96, (3, 3, 3), 2, 16, 32),
                                               (192, 96, (1, 1, 1), 3, 9, 17), (96, 3, (3, 3, 3), 2, 24, 40),
                                               (96, 192, (3, 1, 1), 4, 8, 16), (384, 384, (3, 3, 3), 2, 8, 20),
                                               (192, 96, (1, 3, 3), 3, 10, 18)])
def test_conv3d_kernel_matches_fp32(cin, cout, k, T, H, W):
    torch.manual_seed(0)
    x = torch.randn(2, cin, T, H, W, device="cuda").bfloat16()
    w = (torch.randn(cout, cin, *k, device="cuda") / (cin * k[0] * k[1] * k[2]) ** 0.5).bfloat16()
    b = torch.randn(cout, device="cuda").bfloat16()
    res = torch.randn(2, cout, T, H, W, device="cuda").bfloat16()
    pad_t = k[0] - 1
    launches = TF.native.launch_count()
    got = TF.conv3d_causal(x, w, b, pad_t=pad_t)
    assert TF.native.launch_count() == launches + 1
    assert got.shape == (2, cout, T, H, W) and got.permute(0, 2, 3, 4, 1).is_contiguous()
    assert rel(got, TF.conv3d_causal_reference(x.float(), w.float(), b.float(), pad_t=pad_t)) < 6e-3
    got = TF.conv3d_causal(x, w, b, residual=res, pad_t=pad_t)
    assert rel(got, TF.conv3d_causal_reference(x.float(), w.float(), b.float(), residual=res.float(), pad_t=pad_t)) < 6e-3
    if pad_t:
        for n_prev in (1, 2):
            prev = torch.randn(2, cin, n_prev, H, W, device="cuda").bfloat16()
            got = TF.conv3d_causal(x, w, b, prev=prev, pad_t=pad_t)
            want = TF.conv3d_causal_reference(x.float(), w.float(), b.float(), prev=prev.float(), pad_t=pad_t)
            assert rel(got, want) < 6e-3, n_prev
    assert torch.equal(got, TF.conv3d_causal(x, w, b, prev=prev, pad_t=pad_t)) if pad_t else True  # fixed order: bitwise
    assert TF.native.last_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("C", [16, 96, 192, 384, 128])
def test_pixel_norm_act_and_upsample(C):
    torch.manual_seed(0)
    x = (torch.randn(1, C, 3, 11, 7, device="cuda") * 3).bfloat16()
    g = torch.rand(C, 1, 1, 1, device="cuda") + 0.5
    for silu in (True, False):
        want = F.normalize(x.float(), dim=1) * C**0.5 * g
        want = F.silu(want) if silu else want
        got = TF.pixel_norm_act(x, g, silu)
        assert got.permute(0, 2, 3, 4, 1).is_contiguous() and rel(got, want) < 6e-3
    img = torch.randn(3, C, 5, 9, device="cuda").bfloat16()
    up = TF.upsample2x_nearest(img)
    assert torch.equal(up, F.interpolate(img.float(), scale_factor=2.0, mode="nearest-exact").bfloat16())
    assert up.is_contiguous(memory_format=torch.channels_last)


@pytest.mark.gpu
def test_vae_decode_native_path_tracks_fp32_and_streams():
    from telefuser_b200.models.wan_vae import WanVideoVAE
    from telefuser_b200.testing.synthetic import random_init_

    torch.manual_seed(0)
    vae = random_init_(WanVideoVAE(dim=32).float(), 0, std=0.05).eval()  # widths 32 .. 128: every kernel instance small
    z = torch.randn(1, 16, 3, 10, 12)
    with torch.no_grad():
        want = vae.model.decode(z, vae.scale).clamp(-1, 1)
        gpu = vae.cuda().bfloat16()
        launches = TF.native.launch_count()
        got = gpu.model.decode(z.cuda().bfloat16(), gpu.scale).clamp(-1, 1).float().cpu()
        assert TF.native.launch_count() - launches > 40  # convolutions, norms and upsamples ran on the native kernels
        assert got.shape == want.shape == (1, 3, 9, 80, 96)
        assert rel(got, want) < 5e-2
        TF.set_force_reference(True)
        try:
            lib = gpu.model.decode(z.cuda().bfloat16(), gpu.scale).clamp(-1, 1).float().cpu()  # cuDNN / torch path, bf16
        finally:
            TF.set_force_reference(False)
        assert rel(got, want) <= rel(lib, want) * 1.5 + 1e-3  # no less accurate than the library path in bf16
        stream = gpu.new_stream("decode")
        parts = [gpu.cached_decode(z[:, :, i : i + 1].cuda().bfloat16(), stream) for i in range(3)]
        chunks = torch.cat(parts, dim=2).clamp(-1, 1).float().cpu()
        assert rel(chunks, got) < 1e-2  # frame-by-frame decode with carried history == whole-clip decode
    assert TF.native.last_status() == 0
