"""Real-ESRGAN upscalers: the RRDB network (23 residual-in-residual dense blocks, two nearest 2x stages) and the
compact VGG-style network (conv + PReLU stack, pixel shuffle, nearest-upsampled skip). The architecture is
read off the checkpoint's keys and shapes; frames are processed in batches on the device and resized with
bicubic interpolation when the requested scale is not the network's own.
Role parity: telefuser/models/realesrgan.py:22-356.
"""

from __future__ import annotations

import math
import os

import torch
import torch.nn as nn
import torch.nn.functional as F

from telefuser_b200.core.base_model import BaseModel


class SRVGGNetCompact(nn.Module):
    def __init__(self, num_in_ch=3, num_out_ch=3, num_feat=64, num_conv=16, upscale=4, act_type="prelu") -> None:
        super().__init__()
        self.upscale = upscale

        def act():
            if act_type == "relu":
                return nn.ReLU(inplace=True)
            if act_type == "prelu":
                return nn.PReLU(num_parameters=num_feat)
            if act_type == "leakyrelu":
                return nn.LeakyReLU(0.1, inplace=True)
            raise ValueError(f"unsupported activation {act_type}")

        layers = [nn.Conv2d(num_in_ch, num_feat, 3, 1, 1), act()]
        for _ in range(num_conv):
            layers += [nn.Conv2d(num_feat, num_feat, 3, 1, 1), act()]
        layers.append(nn.Conv2d(num_feat, num_out_ch * upscale * upscale, 3, 1, 1))
        self.body = nn.ModuleList(layers)
        self.upsampler = nn.PixelShuffle(upscale)

    def forward(self, x):
        out = x
        for layer in self.body:
            out = layer(out)
        return self.upsampler(out) + F.interpolate(x, scale_factor=self.upscale, mode="nearest")


class ResidualDenseBlock(nn.Module):
    def __init__(self, num_feat=64, num_grow_ch=32) -> None:
        super().__init__()
        for i in range(1, 5):
            setattr(self, f"conv{i}", nn.Conv2d(num_feat + (i - 1) * num_grow_ch, num_grow_ch, 3, 1, 1))
        self.conv5 = nn.Conv2d(num_feat + 4 * num_grow_ch, num_feat, 3, 1, 1)
        self.lrelu = nn.LeakyReLU(0.2, inplace=True)

    def forward(self, x):
        feats = [x]
        for i in range(1, 5):
            feats.append(self.lrelu(getattr(self, f"conv{i}")(torch.cat(feats, 1))))
        return self.conv5(torch.cat(feats, 1)) * 0.2 + x


class RRDB(nn.Module):
    def __init__(self, num_feat: int, num_grow_ch: int = 32) -> None:
        super().__init__()
        self.rdb1, self.rdb2, self.rdb3 = (ResidualDenseBlock(num_feat, num_grow_ch) for _ in range(3))

    def forward(self, x):
        return self.rdb3(self.rdb2(self.rdb1(x))) * 0.2 + x


class RRDBNet(nn.Module):
    def __init__(self, num_in_ch=3, num_out_ch=3, scale=4, num_feat=64, num_block=23, num_grow_ch=32) -> None:
        super().__init__()
        self.scale = scale
        in_ch = num_in_ch * {4: 1, 2: 4, 1: 16}[scale]
        self.conv_first = nn.Conv2d(in_ch, num_feat, 3, 1, 1)
        self.body = nn.Sequential(*[RRDB(num_feat, num_grow_ch) for _ in range(num_block)])
        self.conv_body, self.conv_up1, self.conv_up2, self.conv_hr = (nn.Conv2d(num_feat, num_feat, 3, 1, 1) for _ in range(4))
        self.conv_last = nn.Conv2d(num_feat, num_out_ch, 3, 1, 1)
        self.lrelu = nn.LeakyReLU(0.2, inplace=True)

    def forward(self, x):
        feat = F.pixel_unshuffle(x, {4: 1, 2: 2, 1: 4}[self.scale]) if self.scale != 4 else x
        feat = self.conv_first(feat)
        feat = feat + self.conv_body(self.body(feat))
        feat = self.lrelu(self.conv_up1(F.interpolate(feat, scale_factor=2, mode="nearest")))
        feat = self.lrelu(self.conv_up2(F.interpolate(feat, scale_factor=2, mode="nearest")))
        return self.conv_last(self.lrelu(self.conv_hr(feat)))


def build_net_from_state_dict(sd: dict) -> nn.Module:
    if "conv_first.weight" in sd:
        blocks = sum(1 for k in sd if k.startswith("body.") and k.endswith(".rdb1.conv1.weight"))
        return RRDBNet(num_feat=sd["conv_first.weight"].shape[0], num_block=blocks, num_grow_ch=sd["body.0.rdb1.conv1.weight"].shape[0])
    convs = sorted((k for k in sd if k.startswith("body.") and k.endswith(".weight") and sd[k].dim() == 4),
                   key=lambda k: int(k.split(".")[1]))  # fmt: skip
    upscale = int(math.sqrt(sd[convs[-1]].shape[0] / 3))
    return SRVGGNetCompact(num_feat=sd["body.0.weight"].shape[0], num_conv=len(convs) - 2, upscale=upscale)


class RealESRGAN(BaseModel):
    def __init__(self, model_path: str | None = None, scale: int = 4, net: nn.Module | None = None) -> None:
        super().__init__()
        if net is None and (model_path is None or not os.path.isfile(model_path)):
            raise FileNotFoundError(f"Real-ESRGAN weights not found at {model_path!r}")
        self.model_path, self.target_scale = model_path, scale
        self._net = net
        self._native_scale = getattr(net, "upscale", getattr(net, "scale", 4)) if net is not None else 4

    @property
    def net(self) -> nn.Module:
        if self._net is None:
            sd = torch.load(self.model_path, map_location="cpu", weights_only=True)
            sd = sd.get("params_ema", sd.get("params", sd))
            self._net = build_net_from_state_dict(sd)
            self._net.load_state_dict(sd, strict=True)
            self._net.eval()
            self._native_scale = getattr(self._net, "upscale", getattr(self._net, "scale", 4))
        return self._net

    @property
    def native_scale(self) -> int:
        return self._native_scale

    def forward(self, x):
        return self.net(x)

    @torch.no_grad()
    def upscale_frame(self, frame: torch.Tensor, outscale: float | None = None) -> torch.Tensor:
        h, w = frame.shape[2:4]
        out = self.net(frame)
        if outscale is not None and outscale != self._native_scale:
            out = F.interpolate(out.float(), size=(int(h * outscale), int(w * outscale)), mode="bicubic", align_corners=False)
        return out.clamp(0.0, 1.0)

    @torch.no_grad()
    def upscale_frames(self, images: torch.Tensor, device="cuda", batch: int = 4) -> torch.Tensor:
        """images: [N, H, W, 3] in [0, 1] -> [N, H*s, W*s, 3] on the host."""
        net = self.net.to(device)
        p = next(net.parameters())
        outscale = self.target_scale if self.target_scale != self._native_scale else None
        outs = []
        for s in range(0, images.shape[0], batch):
            x = images[s : s + batch].permute(0, 3, 1, 2).to(device=device, dtype=p.dtype)
            outs.append(self.upscale_frame(x, outscale).permute(0, 2, 3, 1).to(images.dtype).cpu())
        return torch.cat(outs)

    @staticmethod
    def state_dict_converter():
        return RealESRGANStateDictConverter()


class RealESRGANStateDictConverter:
    def from_official(self, sd: dict):
        return sd, {}
