"""Pipeline parallelism: contiguous block ranges per stage and point-to-point activation transfer.

Stage i owns blocks `stage_block_range(L, P, i)` (remainder blocks go to the first stages). Every
stage patchifies and embeds for itself (cheap, avoids shipping side inputs); only the token stream
`[B, S, C]` crosses stage boundaries through NCCL / gloo `isend` / `irecv`. Activation transfers stay
on the library's P2P path: NCCL moves them over NVLink with the copy engines while the next
micro-step (the other CFG branch) computes; `queue_*` + `commit` batches several transfers in one
`batch_isend_irecv` group.
Role parity: telefuser/distributed/pp_comm.py:30-310.
"""

from __future__ import annotations

import torch
import torch.distributed as dist


def stage_block_range(num_layers: int, pp_degree: int, stage: int) -> tuple[int, int]:
    if not 0 <= stage < pp_degree:
        raise ValueError(f"stage {stage} outside pp degree {pp_degree}")
    if pp_degree > num_layers:
        raise ValueError(f"pp degree {pp_degree} exceeds the number of layers {num_layers}")
    base, rem = divmod(num_layers, pp_degree)
    start = stage * base + min(stage, rem)
    return start, start + base + (1 if stage < rem else 0)


class PipelineP2PComm:
    def __init__(self, process_group=None, ranks: list[int] | None = None) -> None:
        self.group = process_group
        if process_group is None or not dist.is_initialized():
            self.world_size, self.rank, self.ranks = 1, 0, [0]
        else:
            self.world_size = dist.get_world_size(process_group)
            self.rank = dist.get_rank(process_group)
            self.ranks = ranks or dist.get_process_group_ranks(process_group)
        self._ops: list = []
        self._works: list = []

    @property
    def is_first(self) -> bool:
        return self.rank == 0

    @property
    def is_last(self) -> bool:
        return self.rank == self.world_size - 1

    @property
    def next_rank(self) -> int:
        return self.ranks[(self.rank + 1) % self.world_size]

    @property
    def prev_rank(self) -> int:
        return self.ranks[(self.rank - 1) % self.world_size]

    def get_stage_indices(self, num_layers: int) -> tuple[int, int]:
        return stage_block_range(num_layers, self.world_size, self.rank)

    # ---- immediate -----------------------------------------------------------
    def send(self, tensor: torch.Tensor, async_op: bool = True, dst: int | None = None):
        if self.world_size == 1:
            return None
        w = dist.isend(tensor.contiguous(), self.next_rank if dst is None else dst, group=self.group)
        if async_op:
            self._works.append(w)
            return w
        w.wait()
        return None

    def recv(self, shape=None, dtype=torch.bfloat16, device=None, buffer: torch.Tensor | None = None,
             async_op: bool = False, src: int | None = None):  # fmt: skip
        if self.world_size == 1:
            raise RuntimeError("recv on a single-stage pipeline")
        buf = buffer if buffer is not None else torch.empty(shape, dtype=dtype, device=device)
        w = dist.irecv(buf, self.prev_rank if src is None else src, group=self.group)
        if async_op:
            return buf, w
        w.wait()
        return buf

    # ---- batched ---------------------------------------------------------------
    def queue_send(self, tensor: torch.Tensor, dst: int | None = None) -> None:
        self._ops.append(dist.P2POp(dist.isend, tensor.contiguous(), self.next_rank if dst is None else dst, self.group))

    def queue_recv(self, buffer: torch.Tensor, src: int | None = None) -> None:
        self._ops.append(dist.P2POp(dist.irecv, buffer, self.prev_rank if src is None else src, self.group))

    def commit(self) -> None:
        if self._ops:
            self._works.extend(dist.batch_isend_irecv(self._ops))
            self._ops = []

    def wait(self) -> None:
        for w in self._works:
            w.wait()
        self._works = []

    # ---- latent helpers (names used by model code) ----------------------------------
    def send_latent(self, tensor: torch.Tensor) -> None:
        self.send(tensor, async_op=False)

    def recv_latent(self, shape, dtype=torch.bfloat16, device=None) -> torch.Tensor:
        return self.recv(shape, dtype, device)

    def send_latent_async(self, tensor: torch.Tensor):
        return self.send(tensor, async_op=True)

    def recv_latent_async(self, shape, dtype=torch.bfloat16, device=None):
        return self.recv(shape, dtype, device, async_op=True)
