"""World cache for chunk-autoregressive sessions: re-enter a world that was generated before without denoising it again.

A streaming world model generates a session chunk by chunk; chunk i depends on the reference image, the prompt, the
seed and on the controls of chunks 0..i. Two sessions that agree on all of that up to chunk k produce the same first k
chunks. The store keeps, per world (image + prompt + seed + geometry), the clean latent of every chunk together with a
digest of the control that produced it. A later session of the same world is checked chunk by chunk while it runs:
as long as its controls match the recorded ones, the recorded latent is used and the denoiser only replays the commit
pass (the one forward at timestep 0 that writes the chunk's K / V into the rolling cache) and advances its random
generators, i.e. one DiT forward instead of `steps + 1`. At the first control that differs the session simply continues
with normal denoising: the rolling cache holds exactly what a cold run would hold, because the commit passes were
replayed, so no K / V snapshots have to be stored and a divergence may happen at any chunk of an interactive session.

Role parity: the `world_kv_binding` hooks of telefuser/pipelines/lingbot_world_fast/{session.py:53-54,99-101,
pipeline.py:533-541, streaming.py:368-390}, which hand this job to an external cache package; here it is in-tree.
"""

from __future__ import annotations

import hashlib
import threading
from collections import OrderedDict
from dataclasses import dataclass, field

import torch


def tensor_digest(t) -> str:
    """Content hash of a tensor (shape, dtype and bytes), of a plain value, or of a sequence of either."""
    h = hashlib.sha256()

    def feed(x) -> None:
        if isinstance(x, torch.Tensor):
            c = x.detach().to("cpu").contiguous()
            h.update(f"{tuple(c.shape)}|{c.dtype}|".encode())
            h.update(c.view(torch.uint8).reshape(-1).numpy().tobytes() if c.numel() else b"")
        elif isinstance(x, (list, tuple)):
            h.update(f"[{len(x)}".encode())
            for item in x:
                feed(item)
        else:
            h.update(repr(x).encode())
        h.update(b";")

    feed(t)
    return h.hexdigest()


def world_key(condition_image, prompt_emb, seed: int, **geometry) -> str:
    """Identity of a world: everything that fixes chunk 0 apart from its control."""
    return tensor_digest([condition_image, prompt_emb, int(seed), sorted(geometry.items())])


@dataclass
class WorldRecord:
    """What is known about one world: per chunk, the digest of its control and its clean latent (on the host)."""

    key: str
    control_digests: list = field(default_factory=list)
    latents: list = field(default_factory=list)

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.latents)

    def __len__(self) -> int:
        return len(self.latents)


class WorldKVStore:
    """Least-recently-used store of world records, bounded by the bytes of the latents it holds."""

    def __init__(self, max_bytes: int = 1 << 30) -> None:
        self.max_bytes = int(max_bytes)
        self._records: "OrderedDict[str, WorldRecord]" = OrderedDict()
        self._lock = threading.Lock()
        self.hits = self.misses = self.evictions = 0

    def get(self, key: str) -> WorldRecord | None:
        with self._lock:
            rec = self._records.get(key)
            if rec is not None:
                self._records.move_to_end(key)
            return rec

    def record_chunk(self, key: str, index: int, control_digest: str, latent: torch.Tensor) -> None:
        """Chunk `index` of world `key` was produced under `control_digest`. A record only ever describes ONE
        control sequence: writing chunk i under another control than the recorded one drops the old chunks from i on."""
        lat = latent.detach().to("cpu").clone()
        with self._lock:
            rec = self._records.get(key)
            if rec is None:
                rec = self._records[key] = WorldRecord(key)
            self._records.move_to_end(key)
            if index > len(rec):
                return  # a gap (an earlier chunk was never recorded): nothing sound can be stored
            if index < len(rec):
                if rec.control_digests[index] == control_digest:
                    return
                del rec.control_digests[index:], rec.latents[index:]
            rec.control_digests.append(control_digest)
            rec.latents.append(lat)
            self._evict(keep=key)

    def _evict(self, keep: str) -> None:
        total = sum(r.nbytes() for r in self._records.values())
        while total > self.max_bytes and len(self._records) > 1:
            victim = next(k for k in self._records if k != keep)
            total -= self._records.pop(victim).nbytes()
            self.evictions += 1
        rec = self._records.get(keep)
        while rec is not None and total > self.max_bytes and len(rec):  # one world larger than the budget: keep its head
            total -= rec.latents[-1].numel() * rec.latents[-1].element_size()
            rec.latents.pop()
            rec.control_digests.pop()

    def drop(self, key: str) -> bool:
        with self._lock:
            return self._records.pop(key, None) is not None

    def clear(self) -> None:
        with self._lock:
            self._records.clear()

    def stats(self) -> dict:
        with self._lock:
            return {"worlds": len(self._records), "chunks": sum(len(r) for r in self._records.values()),
                    "bytes": sum(r.nbytes() for r in self._records.values()), "max_bytes": self.max_bytes,
                    "hits": self.hits, "misses": self.misses, "evictions": self.evictions}  # fmt: skip


class WorldKVBinding:
    """One session's view of the store. `lookup(i, digest)` answers, in chunk order, whether chunk i can be taken
    from the record (all earlier chunks matched and this control matches too); `finalize(i, digest, latent)` records
    what the session produced."""

    def __init__(self, store: WorldKVStore, key: str, read: bool = True, write: bool = True) -> None:
        self.store, self.key, self.read, self.write = store, key, read, write
        self._matching = read
        self.hits = 0
        self.misses = 0

    def lookup(self, index: int, control_digest: str) -> torch.Tensor | None:
        if not self._matching:
            self.misses += 1
            return None
        rec = self.store.get(self.key)
        if rec is not None and index < len(rec) and rec.control_digests[index] == control_digest:
            self.hits += 1
            self.store.hits += 1
            return rec.latents[index]
        self._matching = False  # the worlds part ways here; later chunks depend on this one
        self.misses += 1
        self.store.misses += 1
        return None

    def finalize(self, index: int, control_digest: str, latent: torch.Tensor) -> None:
        if self.write:
            self.store.record_chunk(self.key, index, control_digest, latent)


__all__ = ["tensor_digest", "world_key", "WorldRecord", "WorldKVStore", "WorldKVBinding"]
