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


# ---- offline control inputs: files, resampling, windows, deferred materialisation ----

def _quaternions(rot: np.ndarray) -> np.ndarray:
    """Rotation matrices [N, 3, 3] -> unit quaternions [N, 4] as (w, x, y, z), each on the hemisphere of its
    predecessor so that interpolation takes the short way round."""
    m = rot.astype(np.float64)
    q = np.empty((m.shape[0], 4))
    tr = np.trace(m, axis1=1, axis2=2)
    for i in range(m.shape[0]):
        r = m[i]
        if tr[i] > 0:
            s = 2.0 * math.sqrt(tr[i] + 1.0)
            q[i] = (0.25 * s, (r[2, 1] - r[1, 2]) / s, (r[0, 2] - r[2, 0]) / s, (r[1, 0] - r[0, 1]) / s)
        else:
            a = int(np.argmax(np.diag(r)))
            b, c = (a + 1) % 3, (a + 2) % 3
            s = 2.0 * math.sqrt(max(1.0 + r[a, a] - r[b, b] - r[c, c], 1e-30))
            v = np.empty(4)
            v[0], v[1 + a], v[1 + b], v[1 + c] = (r[c, b] - r[b, c]) / s, 0.25 * s, (r[b, a] + r[a, b]) / s, (r[c, a] + r[a, c]) / s
            q[i] = v
        q[i] /= np.linalg.norm(q[i])
        if i and np.dot(q[i], q[i - 1]) < 0:
            q[i] = -q[i]
    return q


def _rotation_matrices(q: np.ndarray) -> np.ndarray:
    w, x, y, z = q[:, 0], q[:, 1], q[:, 2], q[:, 3]
    return np.stack([np.stack([1 - 2 * (y * y + z * z), 2 * (x * y - z * w), 2 * (x * z + y * w)], -1),
                     np.stack([2 * (x * y + z * w), 1 - 2 * (x * x + z * z), 2 * (y * z - x * w)], -1),
                     np.stack([2 * (x * z - y * w), 2 * (y * z + x * w), 1 - 2 * (x * x + y * y)], -1)], 1)  # fmt: skip


def interpolate_camera_poses(src_indices, src_rot_mat, src_trans_vec, tgt_indices) -> torch.Tensor:
    """Camera path given at `src_indices` (ascending frame numbers) resampled at `tgt_indices`: translations linearly
    (extrapolated beyond the ends), rotations by spherical linear interpolation between the two neighbouring key
    frames (held at the ends). Returns [len(tgt), 4, 4] fp32 camera-to-world matrices.
    Role parity: telefuser/pipelines/lingbot_world_fast/control.py:57-89."""
    src = np.asarray(src_indices, dtype=np.float64)
    tgt = np.asarray(tgt_indices, dtype=np.float64)
    trans = np.asarray(src_trans_vec, dtype=np.float64)
    if src.ndim != 1 or src.size < 2 or np.any(np.diff(src) <= 0):
        raise ValueError("key-frame indices must be at least two strictly ascending numbers")
    hi = np.clip(np.searchsorted(src, tgt, side="right"), 1, src.size - 1)
    lo = hi - 1
    t = (tgt - src[lo]) / (src[hi] - src[lo])
    out_t = trans[lo] + (trans[hi] - trans[lo]) * t[:, None]
    q = _quaternions(np.asarray(src_rot_mat))
    tc = np.clip(t, 0.0, 1.0)
    dot = np.clip(np.sum(q[lo] * q[hi], axis=1), -1.0, 1.0)
    theta = np.arccos(dot)
    small = theta < 1e-6
    sin = np.where(small, 1.0, np.sin(theta))
    wa = np.where(small, 1.0 - tc, np.sin((1.0 - tc) * theta) / sin)
    wb = np.where(small, tc, np.sin(tc * theta) / sin)
    qi = wa[:, None] * q[lo] + wb[:, None] * q[hi]
    qi /= np.linalg.norm(qi, axis=1, keepdims=True)
    poses = np.zeros((tgt.size, 4, 4), dtype=np.float32)
    poses[:, :3, :3] = _rotation_matrices(qi)
    poses[:, :3, 3] = out_t
    poses[:, 3, 3] = 1.0
    return torch.from_numpy(poses)


def truncate_control_sequence(poses, intrinsics, action, frame_num: int):
    """The first `frame_num` video-rate poses (and actions) of a recorded trajectory, with the FIRST intrinsics row as
    the session's fixed calibration. Recordings shorter than the session are refused."""
    if frame_num < 1 or (frame_num - 1) % 4:
        raise ValueError(f"frame_num must have the form 4n+1, got {frame_num}")
    if len(poses) < frame_num:
        raise ValueError(f"the pose recording has {len(poses)} frames, the session needs {frame_num}")
    ks = np.asarray(intrinsics)
    if ks.ndim not in (1, 2) or ks.shape[-1] != 4 or ks.shape[0] < 1:
        raise ValueError(f"intrinsics are (fx, fy, cx, cy) or one such row per frame, got shape {ks.shape}")
    if action is not None and len(action) < frame_num:
        raise ValueError(f"the action recording has {len(action)} frames, the session needs {frame_num}")
    return poses[:frame_num], (ks[0] if ks.ndim == 2 else ks), (None if action is None else action[:frame_num])


class LingBotWorldFastOfflineControlSource:
    """A recorded trajectory kept outside the generation session: `control_at(i)` hands out a provider for chunk
    i, and the whole trajectory is converted to control tensors once, when the first provider is called (i.e. when
    the first chunk is admitted to the denoiser, not when the session is set up)."""

    def __init__(self, builder: LingBotWorldFastControlBuilder, poses, intrinsics, action=None) -> None:
        self._builder, self._inputs = builder, (poses, intrinsics, action)
        self._controls: list[torch.Tensor] | None = None
        self.materialize_count = 0

    def control_at(self, chunk_index: int):
        if chunk_index < 0:
            raise ValueError(f"chunk indices start at 0, got {chunk_index}")

        def provider() -> torch.Tensor:
            return self._materialized()[chunk_index]

        provider.source = self
        return provider

    def _materialized(self) -> list[torch.Tensor]:
        if self._controls is None:
            self._controls = self._builder.build_sequence(*self._inputs)
            self.materialize_count += 1
        return self._controls


def load_camera_control_inputs(action_path, intrinsics_path):
    """(`poses.npy` [frames, 4, 4] under `action_path`, the intrinsics file given explicitly)."""
    from pathlib import Path

    return np.load(Path(action_path) / "poses.npy"), np.load(Path(intrinsics_path))


def load_action_control_inputs(action_path, intrinsics_path):
    """As `load_camera_control_inputs`, plus `action.npy` [frames, 4] from the same folder."""
    from pathlib import Path

    poses, ks = load_camera_control_inputs(action_path, intrinsics_path)
    return poses, ks, np.load(Path(action_path) / "action.npy")
