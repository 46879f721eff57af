"""Process mesh: ranks laid out as DP x CFG x ring x Ulysses x PP x TP.

Dimension order and accessor names follow the reference's
``telefuser/distributed/device_mesh.py:19-347``. The mesh is a plain rank grid
with one ``torch.distributed`` group per (dimension, slice); it works the same
on NCCL (one process per B200) and on gloo (CPU tests). An ``ep`` view aliases
the CFG x SP ranks for expert-parallel MoE layers.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import os

import torch
import torch.distributed as dist

from telefuser_b200.core.config import ParallelConfig

DIM_NAMES = ("dp", "cfg", "ring", "ulysses", "pp", "tp")


@dataclass
class ParallelMesh:
    dims: tuple[int, ...]
    rank: int
    world_size: int
    coords: dict[str, int] = field(default_factory=dict)
    groups: dict[str, object] = field(default_factory=dict)
    group_ranks: dict[str, list[int]] = field(default_factory=dict)
    fused: bool = True  # peer-memory kernels instead of collective-library calls where both exist

    def size(self, name: str) -> int:
        if name == "sp":
            return self.size("ring") * self.size("ulysses")
        if name == "ep":
            return len(self.group_ranks.get("ep", [self.rank]))
        return self.dims[DIM_NAMES.index(name)]

    def coord(self, name: str) -> int:
        if name in ("sp", "ep"):
            return self.group_ranks[name].index(self.rank) if name in self.group_ranks else 0
        return self.coords.get(name, 0)

    def group(self, name: str):
        return self.groups.get(name)

    def ranks(self, name: str) -> list[int]:
        return self.group_ranks.get(name, [self.rank])


_MESH: ParallelMesh | None = None


def _make_groups(grid: torch.Tensor, dim_idx: list[int], rank: int):
    """Creates one group per slice along `dim_idx` (all ranks call new_group for every slice)."""
    nd = grid.dim()
    other = [d for d in range(nd) if d not in dim_idx]
    perm = grid.permute(*other, *dim_idx)
    n_in = 1
    for d in dim_idx:
        n_in *= grid.shape[d]
    flat = perm.reshape(-1, n_in)
    mine, mine_ranks = None, None
    for row in flat.tolist():
        g = dist.new_group(ranks=row) if (dist.is_initialized() and len(row) > 1) else None
        if rank in row:
            mine, mine_ranks = g, row
    return mine, mine_ranks


def create_mesh(config: ParallelConfig | None = None, rank: int | None = None, world_size: int | None = None,
                ) -> ParallelMesh:  # fmt: skip
    """Builds the mesh for this process and installs it as the current mesh."""
    global _MESH
    config = config or ParallelConfig()
    if rank is None:
        rank = dist.get_rank() if dist.is_initialized() else 0
    if world_size is None:
        world_size = dist.get_world_size() if dist.is_initialized() else 1
    dims = (config.dp_degree, config.cfg_degree, config.sp_ring_degree, config.sp_ulysses_degree,
            config.pp_degree, config.tp_degree)  # fmt: skip
    prod = 1
    for d in dims:
        prod *= d
    if prod != world_size:
        raise RuntimeError(f"mesh dims {dims} (product {prod}) do not match world size {world_size}")
    if config.sp_degree > 1 and config.tp_degree > 1:
        raise ValueError("sequence parallelism and tensor parallelism cannot be combined")
    grid = torch.arange(world_size).reshape(dims)
    pos = (grid == rank).nonzero()[0].tolist()
    mesh = ParallelMesh(dims=dims, rank=rank, world_size=world_size)
    mesh.fused = bool(config.fused_collectives) and os.environ.get("TFB_FUSED_COLLECTIVES", "1") != "0"
    for i, name in enumerate(DIM_NAMES):
        mesh.coords[name] = pos[i]
        g, ranks = _make_groups(grid, [i], rank)
        mesh.groups[name], mesh.group_ranks[name] = g, ranks
    g, ranks = _make_groups(grid, [2, 3], rank)  # ring x ulysses = whole SP group
    mesh.groups["sp"], mesh.group_ranks["sp"] = g, ranks
    if config.ep_degree > 1:
        # EP aliases the CFG x SP ranks, split into contiguous groups of ep_degree.
        g_all, ranks_all = _make_groups(grid, [1, 2, 3], rank)
        if config.ep_degree == len(ranks_all):
            mesh.groups["ep"], mesh.group_ranks["ep"] = g_all, ranks_all
        else:
            n = config.ep_degree
            chunks = [ranks_all[i:i + n] for i in range(0, len(ranks_all), n)]
            # every rank must create every group in the same order
            all_rows = torch.arange(world_size).reshape(dims).permute(0, 4, 5, 1, 2, 3).reshape(-1, len(ranks_all))
            for row in all_rows.tolist():
                for i in range(0, len(row), n):
                    sub = row[i:i + n]
                    gg = dist.new_group(ranks=sub) if dist.is_initialized() else None
                    if rank in sub:
                        mesh.groups["ep"], mesh.group_ranks["ep"] = gg, sub
            del chunks
    _MESH = mesh
    return mesh


def create_device_mesh_from_config(config: ParallelConfig) -> ParallelMesh:
    return create_mesh(config)


def get_mesh() -> ParallelMesh:
    global _MESH
    if _MESH is None:
        _MESH = ParallelMesh(dims=(1,) * 6, rank=0, world_size=1, coords={n: 0 for n in DIM_NAMES},
                             group_ranks={n: [0] for n in (*DIM_NAMES, "sp")})  # fmt: skip
    return _MESH


def set_mesh(mesh: ParallelMesh | None) -> None:
    global _MESH
    _MESH = mesh


def _acc(name):
    def group(mesh: ParallelMesh | None = None):
        return (mesh or get_mesh()).group(name)

    def rank(mesh: ParallelMesh | None = None) -> int:
        return (mesh or get_mesh()).coord(name)

    def world_size(mesh: ParallelMesh | None = None) -> int:
        return (mesh or get_mesh()).size(name)

    return group, rank, world_size


get_dp_group, get_dp_rank, get_dp_world_size = _acc("dp")
get_cfg_group, get_cfg_rank, get_cfg_world_size = _acc("cfg")
get_ring_group, get_ring_rank, get_ring_world_size = _acc("ring")
get_ulysses_group, get_ulysses_rank, get_ulysses_world_size = _acc("ulysses")
get_pp_group, get_pp_rank, get_pp_world_size = _acc("pp")
get_tp_group, get_tp_rank, get_tp_world_size = _acc("tp")
get_sp_group, get_sp_rank, get_sp_world_size = _acc("sp")
get_ep_group, get_ep_rank, get_ep_world_size = _acc("ep")


def is_pipeline_first_stage(mesh: ParallelMesh | None = None) -> bool:
    return get_pp_rank(mesh) == 0


def is_pipeline_last_stage(mesh: ParallelMesh | None = None) -> bool:
    return get_pp_rank(mesh) == get_pp_world_size(mesh) - 1


def get_attention_strategy(mesh: ParallelMesh | None = None) -> str:
    """'local', 'ulysses', 'ring' or 'usp' (ring x Ulysses)."""
    mesh = mesh or get_mesh()
    u, r = mesh.size("ulysses"), mesh.size("ring")
    if u > 1 and r > 1:
        return "usp"
    if u > 1:
        return "ulysses"
    if r > 1:
        return "ring"
    return "local"
