"""RIFE (IFNet v4 family) video frame interpolation.

A small shared encoder produces 8 feature channels per frame; five coarse-to-fine blocks (strided convs, eight
scaled residual convs, transposed conv + pixel shuffle) refine a bidirectional flow, a blend mask and a feature
carry at scales 16, 8, 4, 2, 1; the frames warped by the final flows are blended with the sigmoid of the mask.
`interpolate_frames` resamples a clip to another frame rate; unlike a per-pair loop it gathers all frame pairs
that need synthesis and runs them through the network in batches that stay on the device.
Role parity: telefuser/models/rift_hdv3.py:14-353.
"""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from telefuser_b200.core.base_model import BaseModel


def target_frame_positions(source_fps: float, target_fps: float, total_source_frames: int) -> list[tuple[int, int, float]]:
    """For every output frame: (left source frame, right source frame, position between them in [0, 1))."""
    duration = (total_source_frames - 1) / source_fps
    out = []
    for k in range(int(duration * target_fps) + 1):
        pos = k / target_fps * source_fps
        i0 = int(pos)
        i1 = min(i0 + 1, total_source_frames - 1)
        out.append((i0, i1, 0.0 if i0 == i1 else pos - i0))
    return out


def warp(image: torch.Tensor, flow: torch.Tensor) -> torch.Tensor:
    """Backward warp: samples `image` at pixel + flow (bilinear, border padding)."""
    B, _, H, W = flow.shape
    gx = torch.linspace(-1.0, 1.0, W, device=flow.device, dtype=flow.dtype).view(1, 1, 1, W).expand(B, 1, H, W)
    gy = torch.linspace(-1.0, 1.0, H, device=flow.device, dtype=flow.dtype).view(1, 1, H, 1).expand(B, 1, H, W)
    norm = torch.cat([flow[:, 0:1] / ((image.shape[3] - 1.0) / 2.0), flow[:, 1:2] / ((image.shape[2] - 1.0) / 2.0)], 1)
    grid = (torch.cat([gx, gy], 1) + norm).permute(0, 2, 3, 1)
    return F.grid_sample(image, grid, mode="bilinear", padding_mode="border", align_corners=True)


def conv(cin: int, cout: int, k: int = 3, stride: int = 1, padding: int = 1):
    return nn.Sequential(nn.Conv2d(cin, cout, k, stride, padding), nn.LeakyReLU(0.2, True))


class Head(nn.Module):
    def __init__(self) -> None:
        super().__init__()
        self.cnn0 = nn.Conv2d(3, 16, 3, 2, 1)
        self.cnn1 = nn.Conv2d(16, 16, 3, 1, 1)
        self.cnn2 = nn.Conv2d(16, 16, 3, 1, 1)
        self.cnn3 = nn.ConvTranspose2d(16, 4, 4, 2, 1)
        self.relu = nn.LeakyReLU(0.2, True)

    def forward(self, x):
        x = self.relu(self.cnn0(x))
        x = self.relu(self.cnn1(x))
        return self.cnn3(self.relu(self.cnn2(x)))


class ResConv(nn.Module):
    def __init__(self, c: int, dilation: int = 1) -> None:
        super().__init__()
        self.conv = nn.Conv2d(c, c, 3, 1, dilation, dilation=dilation)
        self.beta = nn.Parameter(torch.ones(1, c, 1, 1))
        self.relu = nn.LeakyReLU(0.2, True)

    def forward(self, x):
        return self.relu(self.conv(x) * self.beta + x)


class IFBlock(nn.Module):
    def __init__(self, in_planes: int, c: int = 64) -> None:
        super().__init__()
        self.conv0 = nn.Sequential(conv(in_planes, c // 2, 3, 2, 1), conv(c // 2, c, 3, 2, 1))
        self.convblock = nn.Sequential(*[ResConv(c) for _ in range(8)])
        self.lastconv = nn.Sequential(nn.ConvTranspose2d(c, 4 * 13, 4, 2, 1), nn.PixelShuffle(2))

    def forward(self, x, flow=None, scale: float = 1):
        x = F.interpolate(x, scale_factor=1.0 / scale, mode="bilinear", align_corners=False)
        if flow is not None:
            flow = F.interpolate(flow, scale_factor=1.0 / scale, mode="bilinear", align_corners=False) / scale
            x = torch.cat((x, flow), 1)
        out = self.lastconv(self.convblock(self.conv0(x)))
        out = F.interpolate(out, scale_factor=scale, mode="bilinear", align_corners=False)
        return out[:, :4] * scale, out[:, 4:5], out[:, 5:]


class IFNet(BaseModel):
    def __init__(self) -> None:
        super().__init__()
        self.block0 = IFBlock(7 + 8, c=192)
        self.block1 = IFBlock(8 + 4 + 8 + 8, c=128)
        self.block2 = IFBlock(8 + 4 + 8 + 8, c=96)
        self.block3 = IFBlock(8 + 4 + 8 + 8, c=64)
        self.block4 = IFBlock(8 + 4 + 8 + 8, c=32)
        self.encode = Head()

    def forward(self, x, timestep=0.5, scale_list=(16, 8, 4, 2, 1)):
        """x: [B, 6, H, W] (two RGB frames in [0, 1]); timestep: float or [B, 1, 1, 1] -> (flows, mask, merged)."""
        img0, img1 = x[:, :3], x[:, 3:6]
        if not torch.is_tensor(timestep):
            t = torch.full_like(x[:, :1], float(timestep))
        else:
            t = timestep.to(x).reshape(-1, 1, 1, 1).expand(x.shape[0], 1, x.shape[2], x.shape[3])
        f0, f1 = self.encode(img0), self.encode(img1)
        flows, merged = [], []
        w0, w1, flow, mask, feat = img0, img1, None, None, None
        for blk, s in zip((self.block0, self.block1, self.block2, self.block3, self.block4), scale_list):
            if flow is None:
                flow, mask, feat = blk(torch.cat((img0, img1, f0, f1, t), 1), None, scale=s)
            else:
                inp = torch.cat((w0, w1, warp(f0, flow[:, :2]), warp(f1, flow[:, 2:4]), t, mask, feat), 1)
                fd, mask, feat = blk(inp, flow, scale=s)
                flow = flow + fd
            flows.append(flow)
            w0, w1 = warp(img0, flow[:, :2]), warp(img1, flow[:, 2:4])
            merged.append((w0, w1))
        m = torch.sigmoid(mask)
        merged[-1] = w0 * m + w1 * (1 - m)
        return flows, mask, merged

    def interpolate_frame(self, img0, img1, timestep=0.5, scale: float = 1.0):
        return self(torch.cat((img0, img1), 1), timestep, [16 / scale, 8 / scale, 4 / scale, 2 / scale, 1 / scale])[2][-1]

    @torch.no_grad()
    def interpolate_frames(self, images: torch.Tensor, source_fps: float, target_fps: float, scale: float = 1.0,
                           device="cuda", batch: int = 8) -> torch.Tensor:  # fmt: skip
        """images: [N, H, W, 3] in [0, 1] -> the clip resampled to `target_fps` ([M, H, W, 3], on the host)."""
        if images.dim() != 4 or images.shape[-1] != 3:
            raise ValueError("input must be [N, H, W, 3]")
        if source_fps == target_fps:
            return images
        n, h, w = images.shape[:3]
        mult = max(128, int(128 / scale))
        pad = (0, ((w - 1) // mult + 1) * mult - w, 0, ((h - 1) // mult + 1) * mult - h)
        positions = target_frame_positions(source_fps, target_fps, n)
        p = next(self.parameters())
        frames = F.pad(images.permute(0, 3, 1, 2).to(device=device, dtype=p.dtype), pad)  # whole clip on the device once
        out = torch.empty(len(positions), h, w, 3, dtype=images.dtype)
        todo = [(k, i0, i1, f) for k, (i0, i1, f) in enumerate(positions) if f != 0.0 and i0 != i1]
        for k, (i0, _, f) in enumerate(positions):
            if f == 0.0:
                out[k] = images[i0]
        for s in range(0, len(todo), batch):
            part = todo[s : s + batch]
            a = frames[[q[1] for q in part]]
            b = frames[[q[2] for q in part]]
            t = torch.tensor([q[3] for q in part], device=frames.device, dtype=frames.dtype)
            mid = self.interpolate_frame(a, b, t, scale)[:, :, :h, :w].permute(0, 2, 3, 1).to(images.dtype).cpu()
            for j, q in enumerate(part):
                out[q[0]] = mid[j]
        return out

    @staticmethod
    def state_dict_converter():
        return IFNetStateDictConverter()


class IFNetStateDictConverter:
    def from_official(self, sd: dict):
        keep = {k.replace("module.", ""): v for k, v in sd.items()
                if "module." in k and "teacher" not in k and "caltime" not in k}  # fmt: skip
        return (keep or dict(sd)), {}


def _register() -> None:
    from telefuser_b200.core.model_registry import register_architecture

    register_architecture("vfi_model", IFNet, lambda: IFNet())


_register()
