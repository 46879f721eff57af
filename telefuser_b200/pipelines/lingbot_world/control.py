"""Camera / action control for LingBot-World streaming: poses -> Pluecker ray maps -> control tensor.

For every latent frame the control is a per-pixel 6-vector (ray origin, unit ray direction) in the
first camera's frame; the pixel grid is folded 8x8 into channels so the tensor matches the
latent grid: ``[1, 6*c1*c2, f, h, w]`` (384 channels at stride 8). The action variant carries the
3 direction channels plus a 4-vector action broadcast over pixels.
Maths parity: telefuser/pipelines/lingbot_world_fast/control.py:10-330. Also here: the seeded
smooth random-walk trajectory used for synthetic sessions and the key-state -> pose integrator
used by the interactive service.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch


def se3_inverse(poses: torch.Tensor) -> torch.Tensor:
    rot_t = poses[:, :3, :3].transpose(-1, -2)
    out = torch.eye(4, device=poses.device, dtype=poses.dtype).repeat(poses.shape[0], 1, 1)
    out[:, :3, :3] = rot_t
    out[:, :3, 3:] = -torch.bmm(rot_t, poses[:, :3, 3:])
    return out


def compute_relative_poses(c2ws: torch.Tensor, framewise: bool = False, normalize_trans: bool = True) -> torch.Tensor:
    """Poses relative to the first camera (optionally frame-to-frame), translations scaled to unit max norm."""
    rel = torch.matmul(se3_inverse(c2ws[0:1]), c2ws)
    rel[0] = torch.eye(4, device=c2ws.device, dtype=c2ws.dtype)
    if framewise and rel.shape[0] > 1:
        rel[1:] = torch.bmm(se3_inverse(rel[:-1]), rel[1:])
    if normalize_trans:
        m = torch.norm(rel[:, :3, 3], dim=-1).max()
        if float(m) > 0:
            rel[:, :3, 3] = rel[:, :3, 3] / m
    return rel


def scale_relative_translation(poses: torch.Tensor, scale) -> torch.Tensor:
    if scale is None:
        return poses
    if isinstance(scale, bool):
        raise ValueError("Translation scale must be a positive number")
    try:
        v = float(scale)
    except (TypeError, ValueError) as e:
        raise ValueError("Translation scale must be a positive number") from e
    if not math.isfinite(v) or v <= 0:
        raise ValueError("Translation scale must be a positive number")
    poses[:, :3, 3] *= v
    return poses


def transform_intrinsics(ks, h_org, w_org, h_resize, w_resize, h_final, w_final) -> torch.Tensor:
    """(fx, fy, cx, cy) after a resize to (h_resize, w_resize) and a centre crop to (h_final, w_final)."""
    fx, fy, cx, cy = ks.chunk(4, dim=-1)
    sx, sy = w_resize / w_org, h_resize / h_org
    return torch.cat([fx * sx, fy * sy, cx * sx - (w_resize - w_final) / 2, cy * sy - (h_resize - h_final) / 2], dim=-1)


def plucker_embeddings(c2ws: torch.Tensor, ks: torch.Tensor, height: int, width: int, only_rays_d: bool = False):
    """[F, H, W, 6] (origin, direction) or [F, H, W, 3] ray maps; pixel centres at +0.5."""
    F_ = c2ws.shape[0]
    dev, dt = c2ws.device, c2ws.dtype
    ys, xs = torch.meshgrid(torch.arange(height, device=dev, dtype=dt) + 0.5,
                            torch.arange(width, device=dev, dtype=dt) + 0.5, indexing="ij")  # fmt: skip
    i = xs.reshape(1, -1).expand(F_, -1)
    j = ys.reshape(1, -1).expand(F_, -1)
    fx, fy, cx, cy = ks.chunk(4, dim=-1)
    dirs = torch.stack([(i - cx) / fx, (j - cy) / fy, torch.ones_like(i)], dim=-1)
    dirs = dirs / dirs.norm(dim=-1, keepdim=True)
    rays_d = dirs @ c2ws[:, :3, :3].transpose(-1, -2)
    if only_rays_d:
        return rays_d.view(F_, height, width, 3)
    rays_o = c2ws[:, :3, 3][:, None, :].expand_as(rays_d)
    return torch.cat([rays_o, rays_d], dim=-1).view(F_, height, width, 6)


def fold_to_latent_grid(maps: torch.Tensor, latent_h: int, latent_w: int) -> torch.Tensor:
    """[F, H, W, C] -> [1, C*c1*c2, F, h, w] with (c, c1, c2) channel order."""
    F_, H, W, C = maps.shape
    c1, c2 = max(1, H // latent_h), max(1, W // latent_w)
    x = maps.reshape(F_, latent_h, c1, latent_w, c2, C).permute(5, 2, 4, 0, 1, 3)
    return x.reshape(1, C * c1 * c2, F_, latent_h, latent_w).contiguous()


def _fused_ok(poses, latent_h, latent_w, height, width) -> bool:
    return poses.is_cuda and height % latent_h == 0 and width % latent_w == 0


def build_camera_control_chunk(poses, intrinsics, latent_h, latent_w, height, width) -> torch.Tensor:
    if _fused_ok(poses, latent_h, latent_w, height, width):  # rays + fold in one kernel, no [F,H,W,6] intermediate
        from telefuser_b200.ops import functional as TF

        return TF.plucker_fold(poses, intrinsics, latent_h, latent_w, height, width).to(poses.dtype)
    return fold_to_latent_grid(plucker_embeddings(poses, intrinsics, height, width), latent_h, latent_w)


def build_action_control_chunk(poses, intrinsics, action, latent_h, latent_w, height, width) -> torch.Tensor:
    if _fused_ok(poses, latent_h, latent_w, height, width):
        from telefuser_b200.ops import functional as TF

        return TF.plucker_fold(poses, intrinsics, latent_h, latent_w, height, width, only_rays_d=True,
                               extra=action).to(poses.dtype)  # fmt: skip
    d = plucker_embeddings(poses, intrinsics, height, width, only_rays_d=True)
    a = action[:, None, None, :].expand(-1, height, width, -1)
    return fold_to_latent_grid(torch.cat([d, a], dim=-1), latent_h, latent_w)


def pinhole_intrinsics(height: int, width: int, fov_deg: float = 60.0) -> torch.Tensor:
    f = 0.5 * width / math.tan(math.radians(fov_deg) / 2)
    return torch.tensor([f, f, width / 2, height / 2], dtype=torch.float32)


def _rot(axis: int, angle: float) -> np.ndarray:
    """Right-handed rotation about x (0), y (1) or z (2)."""
    c, s = math.cos(angle), math.sin(angle)
    if axis == 0:
        return np.array([[1, 0, 0], [0, c, -s], [0, s, c]], dtype=np.float64)
    if axis == 1:
        return np.array([[c, 0, s], [0, 1, 0], [-s, 0, c]], dtype=np.float64)
    return np.array([[c, -s, 0], [s, c, 0], [0, 0, 1]], dtype=np.float64)


def random_walk_trajectory(num_frames: int, seed: int = 0, sigma_trans: float = 0.05, sigma_rot_deg: float = 1.0,
                           smooth: float = 0.9) -> torch.Tensor:  # fmt: skip
    """Seeded smooth random-walk camera path: [num_frames, 4, 4] camera-to-world matrices.

    Per-frame translation / rotation steps follow an AR(1) process (coefficient `smooth`) with
    stationary standard deviation `sigma_trans` / `sigma_rot_deg`; frame 0 is the identity.
    """
    rng = np.random.default_rng(seed)
    poses = np.tile(np.eye(4, dtype=np.float64), (num_frames, 1, 1))
    vel_t, vel_r = np.zeros(3), np.zeros(3)
    for i in range(1, num_frames):
        gain = math.sqrt(1 - smooth * smooth)  # keeps the per-step standard deviation at sigma
        vel_t = smooth * vel_t + gain * rng.normal(0, sigma_trans, 3)
        vel_r = smooth * vel_r + gain * rng.normal(0, math.radians(sigma_rot_deg), 3)
        step = np.eye(4)
        step[:3, :3] = _rot(0, vel_r[0]) @ _rot(1, vel_r[1]) @ _rot(2, vel_r[2])
        step[:3, 3] = vel_t
        poses[i] = poses[i - 1] @ step
    return torch.from_numpy(poses.astype(np.float32))


KEY_MOVES = {"w": (2, +1.0), "s": (2, -1.0), "a": (0, -1.0), "d": (0, +1.0), "q": (1, -1.0), "e": (1, +1.0)}
KEY_TURNS = {"j": (1, -1.0), "l": (1, +1.0), "i": (0, -1.0), "k": (0, +1.0)}


def integrate_keys(pose: torch.Tensor, keys, frames: int, move_step: float = 0.05, turn_step_deg: float = 1.5):
    """Advances `pose` ([4,4] c2w) by `frames` steps under the held `keys`; returns [frames, 4, 4]."""
    keys = {k.lower() for k in keys}
    t = np.zeros(3)
    r = np.zeros(3)
    for k in keys:
        if k in KEY_MOVES:
            ax, sg = KEY_MOVES[k]
            t[ax] += sg * move_step
        if k in KEY_TURNS:
            ax, sg = KEY_TURNS[k]
            r[ax] += sg * math.radians(turn_step_deg)
    step = np.eye(4)
    step[:3, :3] = _rot(0, r[0]) @ _rot(1, r[1]) @ _rot(2, r[2])
    step[:3, 3] = t
    out, cur = [], pose.double().numpy()
    for _ in range(frames):
        cur = cur @ step
        out.append(cur.copy())
    return torch.from_numpy(np.stack(out).astype(np.float32))


@dataclass(frozen=True)
class LingBotWorldFastControlContext:
    control_type: str
    device: object
    control_dtype: torch.dtype
    orig_height: int
    orig_width: int
    height: int
    width: int
    latent_h: int
    latent_w: int
    latent_frames: int
    chunk_size: int
    intrinsics: torch.Tensor


class LingBotWorldFastControlBuilder:
    """Turns external per-chunk actions ({poses, intrinsics, action} or a ready control tensor) into model input."""

    def __init__(self, context: LingBotWorldFastControlContext) -> None:
        self.context = context

    def defer(self, action: dict):
        return lambda: self.build(action)

    @staticmethod
    def _intrinsics_rows(intr: torch.Tensor, frames: int) -> torch.Tensor:
        if intr.ndim == 1:
            if intr.shape[0] != 4:
                raise ValueError(f"Static intrinsics must have shape (4,), got {tuple(intr.shape)}")
            return intr.unsqueeze(0).repeat(frames, 1)
        if intr.ndim != 2 or intr.shape[1] != 4 or intr.shape[0] < 1:
            raise ValueError(f"Intrinsics must have shape (4,) or (frames, 4), got {tuple(intr.shape)}")
        return intr[0:1].repeat(frames, 1)

    @staticmethod
    def _align_action(action: torch.Tensor, frames: int) -> torch.Tensor:
        if action.ndim == 1:
            action = action.unsqueeze(0)
        if action.shape[0] == frames:
            return action
        if action.shape[0] == (frames - 1) * 4 + 1:
            return action[::4]
        raise ValueError(f"Action length must be {frames} latent frames or {(frames - 1) * 4 + 1} video-rate frames, "
                         f"got {action.shape[0]}")  # fmt: skip

    def build(self, action: dict) -> torch.Tensor:
        c = self.context
        if "control_tensor" in action:
            return torch.as_tensor(action["control_tensor"], device=c.device, dtype=c.control_dtype)
        poses = action.get("poses")
        if poses is None:
            raise ValueError("External action requires poses")
        poses = torch.as_tensor(poses, dtype=torch.float32, device=c.device)
        frames = poses.shape[0]
        if poses.shape != (frames, 4, 4):
            raise ValueError(f"Poses must have shape (frames, 4, 4), got {tuple(poses.shape)}")
        intr = torch.as_tensor(action.get("intrinsics", c.intrinsics), dtype=torch.float32, device=c.device)
        ks = transform_intrinsics(self._intrinsics_rows(intr, frames), c.orig_height, c.orig_width, c.height, c.width,
                                  c.height, c.width)  # fmt: skip
        if not action.get("relative", False):
            poses = compute_relative_poses(poses, framewise=False, normalize_trans=action.get("normalize", True))
        poses = scale_relative_translation(poses, action.get("translation_scale"))
        if c.control_type == "cam":
            out = build_camera_control_chunk(poses, ks, c.latent_h, c.latent_w, c.height, c.width)
        else:
            act = self._align_action(torch.as_tensor(action["action"], dtype=torch.float32, device=c.device), frames)
            out = build_action_control_chunk(poses, ks, act, c.latent_h, c.latent_w, c.height, c.width)
        return out.to(c.control_dtype)

    def build_sequence(self, poses, intrinsics, action=None) -> list[torch.Tensor]:
        """Whole-trajectory version: relative poses once, then one control tensor per chunk of latent frames."""
        c = self.context
        poses = torch.as_tensor(np.asarray(poses), dtype=torch.float32, device=c.device)
        if poses.shape[0] == (c.latent_frames - 1) * 4 + 1:
            poses = poses[::4]
        rel = compute_relative_poses(poses[: c.latent_frames])
        intr = torch.as_tensor(np.asarray(intrinsics), dtype=torch.float32, device=c.device)
        out = []
        for s in range(0, rel.shape[0], c.chunk_size):
            item = {"poses": rel[s : s + c.chunk_size], "intrinsics": intr, "relative": True}
            if action is not None:
                a = torch.as_tensor(np.asarray(action), dtype=torch.float32)
                item["action"] = self._align_action(a, c.latent_frames)[s : s + c.chunk_size]
            out.append(self.build(item))
        return out
