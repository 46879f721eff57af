"""Per-(timestep, layer) key/value cache with optional fp8 storage and host offload (LiveAct-style
streaming models re-use the K,V of earlier chunks at every denoising step).

fp8 storage: one scale per (token, head) = amax over the head dimension / 448, values stored as
e4m3; de-quantised to the compute dtype on load. Host offload keeps the stored tensors in pinned
memory and brings them back on `load`.
Role parity: telefuser/cache/kv_cache.py:12-438 (KVCacheConfig, KVCache, KVCacheManager).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

FP8_MAX = 448.0


@dataclass
class KVCacheConfig:
    fp8_kv_cache: bool = False
    offload_cache: bool = False
    num_timesteps: int = 1
    num_layers: int = 1


def fp8_kv_quant_reference(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """x: [..., D] -> (e4m3 [..., D], fp32 scale [..., 1]) with scale = amax/448 (floor 1e-12)."""
    scale = (x.detach().abs().amax(dim=-1, keepdim=True).float() / FP8_MAX).clamp_min(1e-12)
    return (x / scale.to(x.dtype)).to(torch.float8_e4m3fn).contiguous(), scale.contiguous()


def fp8_kv_quant(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    from telefuser_b200.ops import functional as TF

    fn = getattr(TF, "fp8_kv_quant", None)
    return fn(x) if fn is not None else fp8_kv_quant_reference(x)


def fp8_kv_dequant(q: torch.Tensor, scale: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    return q.to(dtype) * scale.to(device=q.device, dtype=dtype)


class KVCache:
    def __init__(self, fp8_kv_cache: bool = False, offload_cache: bool = False) -> None:
        self.fp8_kv_cache, self.offload_cache = fp8_kv_cache, offload_cache
        self.k = self.v = self.k_scale = self.v_scale = None

    def allocate(self, shape, dtype, device) -> None:
        dev = "cpu" if self.offload_cache else device
        pin = self.offload_cache and torch.cuda.is_available()
        store = torch.float8_e4m3fn if self.fp8_kv_cache else dtype
        self.k = torch.zeros(shape, dtype=store, device=dev, pin_memory=pin)
        self.v = torch.zeros(shape, dtype=store, device=dev, pin_memory=pin)
        if self.fp8_kv_cache:
            sshape = (*shape[:-1], 1)
            self.k_scale = torch.ones(sshape, dtype=torch.float32, device=dev, pin_memory=pin)
            self.v_scale = torch.ones(sshape, dtype=torch.float32, device=dev, pin_memory=pin)

    def clear(self) -> None:
        self.k = self.v = self.k_scale = self.v_scale = None

    @property
    def is_allocated(self) -> bool:
        return self.k is not None

    def store(self, k: torch.Tensor, v: torch.Tensor) -> None:
        if self.fp8_kv_cache:
            k, ks = fp8_kv_quant(k)
            v, vs = fp8_kv_quant(v)
        else:
            ks = vs = None
        if self.offload_cache:
            k, v = self._to_host(k, self.k), self._to_host(v, self.v)
            if ks is not None:
                ks, vs = self._to_host(ks, self.k_scale), self._to_host(vs, self.v_scale)
        self.k, self.v, self.k_scale, self.v_scale = k, v, ks, vs

    @staticmethod
    def _to_host(t: torch.Tensor, old: torch.Tensor | None) -> torch.Tensor:
        if old is not None and old.device.type == "cpu" and old.shape == t.shape and old.dtype == t.dtype:
            old.copy_(t, non_blocking=True)  # reuse the pinned buffer
            return old
        host = torch.empty(t.shape, dtype=t.dtype, pin_memory=torch.cuda.is_available())
        host.copy_(t, non_blocking=True)
        return host

    def load(self, device, dtype) -> tuple[torch.Tensor, torch.Tensor]:
        if self.k is None:
            raise RuntimeError("KV cache is empty")
        k, v = self.k.to(device, non_blocking=True), self.v.to(device, non_blocking=True)
        if self.fp8_kv_cache:
            k = fp8_kv_dequant(k, self.k_scale.to(device, non_blocking=True), dtype)
            v = fp8_kv_dequant(v, self.v_scale.to(device, non_blocking=True), dtype)
        return k.to(dtype), v.to(dtype)

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.k, self.v, self.k_scale, self.v_scale) if t is not None)

    def to_dict(self) -> dict:
        return {"k": self.k, "v": self.v, "k_scale": self.k_scale, "v_scale": self.v_scale,
                "fp8_kv_cache": self.fp8_kv_cache, "offload_cache": self.offload_cache}  # fmt: skip

    @classmethod
    def from_dict(cls, d: dict) -> "KVCache":
        c = cls(d.get("fp8_kv_cache", False), d.get("offload_cache", False))
        c.k, c.v, c.k_scale, c.v_scale = d.get("k"), d.get("v"), d.get("k_scale"), d.get("v_scale")
        return c


class KVCacheManager:
    """`manager.get_cache(t_idx, layer_idx)`; one KVCache per denoising step and layer."""

    def __init__(self, num_timesteps: int, num_layers: int, fp8_kv_cache: bool = False, offload_cache: bool = False) -> None:
        self.num_timesteps, self.num_layers = num_timesteps, num_layers
        self.fp8_kv_cache, self.offload_cache = fp8_kv_cache, offload_cache
        self.caches = [[KVCache(fp8_kv_cache, offload_cache) for _ in range(num_layers)] for _ in range(num_timesteps)]
        self._shape = None

    @classmethod
    def from_config(cls, cfg: KVCacheConfig) -> "KVCacheManager":
        return cls(cfg.num_timesteps, cfg.num_layers, cfg.fp8_kv_cache, cfg.offload_cache)

    @classmethod
    def from_dit_model(cls, dit, num_timesteps: int, fp8_kv_cache: bool = False, offload_cache: bool = False):
        layers = getattr(dit, "num_layers", None) or len(getattr(dit, dit.layer_name_list[0]))
        return cls(num_timesteps, layers, fp8_kv_cache, offload_cache)

    def allocate(self, shape, dtype, device) -> None:
        self._shape = tuple(shape)
        for row in self.caches:
            for c in row:
                c.allocate(shape, dtype, device)

    def clear(self) -> None:
        for row in self.caches:
            for c in row:
                c.clear()
        self._shape = None

    def get_cache(self, t_idx: int, layer_idx: int) -> KVCache:
        if not (0 <= t_idx < self.num_timesteps and 0 <= layer_idx < self.num_layers):
            raise IndexError(f"cache index ({t_idx}, {layer_idx}) outside ({self.num_timesteps}, {self.num_layers})")
        return self.caches[t_idx][layer_idx]

    def get_timestep_caches(self, t_idx: int) -> list[KVCache]:
        return self.caches[t_idx]

    @property
    def shape(self):
        return self._shape

    @property
    def is_allocated(self) -> bool:
        return self._shape is not None

    def nbytes(self) -> int:
        return sum(c.nbytes() for row in self.caches for c in row)

    def to_dict(self) -> dict:
        return {t: {l: c.to_dict() for l, c in enumerate(row)} for t, row in enumerate(self.caches)}

    @classmethod
    def from_dict(cls, d: dict) -> "KVCacheManager":
        nt = len(d)
        nl = len(next(iter(d.values()))) if nt else 0
        first = d[0][0] if nt and nl else {}
        m = cls(nt, nl, first.get("fp8_kv_cache", False), first.get("offload_cache", False))
        for t, row in d.items():
            for l, cd in row.items():
                m.caches[int(t)][int(l)] = KVCache.from_dict(cd)
        return m
