"""Full-reference quality measures between two videos / images in [-1, 1] (or any common peak): PSNR and mean SSIM.
Used by the example regression runner and the feature-cache benchmark; plain torch, no external metric package."""

from __future__ import annotations

import torch
import torch.nn.functional as F


def psnr(a: torch.Tensor, b: torch.Tensor, peak: float = 2.0) -> float:
    """10 log10(peak^2 / MSE); `inf` for identical inputs. `peak` is the value range (2 for data in [-1, 1])."""
    mse = torch.mean((a.double() - b.double()) ** 2).item()
    return float("inf") if mse == 0 else 10.0 * float(torch.log10(torch.tensor(peak * peak / mse)))


def ssim(a: torch.Tensor, b: torch.Tensor, peak: float = 2.0, window: int = 7) -> float:
    """Mean structural similarity over frames and channels with a uniform window; inputs [C, T, H, W] (or [C, H, W])."""
    if a.dim() == 3:
        a, b = a.unsqueeze(1), b.unsqueeze(1)
    x = a.double().permute(1, 0, 2, 3).reshape(-1, 1, *a.shape[-2:])
    y = b.double().permute(1, 0, 2, 3).reshape(-1, 1, *b.shape[-2:])
    k = torch.ones(1, 1, window, window, dtype=torch.float64) / (window * window)
    mu_x, mu_y = F.conv2d(x, k), F.conv2d(y, k)
    sxx = F.conv2d(x * x, k) - mu_x**2
    syy = F.conv2d(y * y, k) - mu_y**2
    sxy = F.conv2d(x * y, k) - mu_x * mu_y
    c1, c2 = (0.01 * peak) ** 2, (0.03 * peak) ** 2
    s = ((2 * mu_x * mu_y + c1) * (2 * sxy + c2)) / ((mu_x**2 + mu_y**2 + c1) * (sxx + syy + c2))
    return float(s.mean())
