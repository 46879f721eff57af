"""Rolling per-layer KV cache for chunk-autoregressive (streaming) DiTs.

One cache holds K and V of past chunks as ``[B, kv_size, H_local, D]``. New tokens are
appended after the current end; when the buffer is full and a *new* chunk arrives, the
oldest non-sink tokens are evicted by shifting the window left while the first
``sink_tokens`` stay pinned. Re-running the same chunk position (the 4 denoising steps
and the clean-latent commit of one chunk all write the same slot) overwrites in place.
Index semantics follow the reference's cache dict (`global_end_index`, `local_end_index`;
telefuser/models/lingbot_world_fast_dit.py:150-175).
"""

from __future__ import annotations

import torch


class RollingKVCache:
    def __init__(self, batch: int, kv_size: int, num_heads: int, head_dim: int, device, dtype,
                 sink_tokens: int = 0, rolling: bool = True) -> None:  # fmt: skip
        self.k = torch.zeros(batch, kv_size, num_heads, head_dim, device=device, dtype=dtype)
        self.v = torch.zeros_like(self.k)
        self.kv_size = kv_size
        self.sink_tokens = sink_tokens
        self.rolling = rolling
        self.global_end = 0  # absolute token index one past the newest token ever written
        self.local_end = 0  # buffer position one past the newest token

    def reset(self) -> None:
        self.global_end = 0
        self.local_end = 0

    def plan(self, current_start: int, num_new: int) -> tuple[int, int, int]:
        """Returns (evicted, local_start, local_end) for writing `num_new` tokens that start at `current_start`."""
        current_end = current_start + num_new
        advance = current_end - self.global_end
        evicted = 0
        if self.rolling and current_end > self.global_end and num_new + self.local_end > self.kv_size:
            evicted = num_new + self.local_end - self.kv_size
        local_end = self.local_end + advance - evicted
        if local_end > self.kv_size or local_end - num_new < 0:
            raise RuntimeError(f"KV cache overflow: local_end {local_end}, size {self.kv_size} (rolling={self.rolling})")
        return evicted, local_end - num_new, local_end

    def append(self, k: torch.Tensor, v: torch.Tensor, current_start: int) -> int:
        """Writes k/v ([B, n, H, D]) for absolute positions [current_start, current_start+n); returns local_end."""
        n = k.shape[1]
        evicted, lo, hi = self.plan(current_start, n)
        from telefuser_b200.ops import functional as TF

        keep = max(0, self.local_end - evicted - self.sink_tokens) if evicted > 0 else 0
        TF.kv_cache_roll_append(self.k, self.v, k, v, self.sink_tokens, evicted, keep, lo)  # shift + append, one call
        self.global_end = max(self.global_end, current_start + n)
        self.local_end = hi
        return hi

    def window(self, max_attention_size: int) -> tuple[torch.Tensor, torch.Tensor]:
        start = max(0, self.local_end - max_attention_size)
        return self.k[:, start : self.local_end], self.v[:, start : self.local_end]

    def nbytes(self) -> int:
        return 2 * self.k.numel() * self.k.element_size()
