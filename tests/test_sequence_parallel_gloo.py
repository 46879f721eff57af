"""CPU plumbing checks: the tiny Wan-style DiT denoised on gloo ranks under each parallel strategy
(Ulysses, ring, ring x Ulysses, CFG, pipeline, tensor, sharded weights) must reproduce the
single-process run; plus unit checks of the stage split and of the TP text encoder."""
import os
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from telefuser_b200.parallel.pp import stage_block_range
from telefuser_b200.testing.distributed_checks import spawn_tiny_wan_denoise, tiny_wan_denoise


@pytest.fixture(scope="module")
def ref():
    out = tiny_wan_denoise()
    assert out.shape == (1, 16, 3, 8, 8) and torch.isfinite(out).all()
    return out


def test_ulysses2_matches_single_process(ref):
    assert (ref - spawn_tiny_wan_denoise(2, sp_ulysses_degree=2)).abs().max().item() <= 1e-5


def test_cfg_parallel2_matches_single_process(ref):
    assert (ref - spawn_tiny_wan_denoise(2, cfg_degree=2)).abs().max().item() <= 1e-5


def test_ring2_matches_single_process(ref):
    assert (ref - spawn_tiny_wan_denoise(2, sp_ring_degree=2)).abs().max().item() <= 1e-5


def test_usp_ring2_ulysses2_matches_single_process(ref):
    assert (ref - spawn_tiny_wan_denoise(4, sp_ring_degree=2, sp_ulysses_degree=2)).abs().max().item() <= 1e-5


def test_pipeline2_matches_single_process(ref):
    assert (ref - spawn_tiny_wan_denoise(2, pp_degree=2)).abs().max().item() <= 1e-5


def test_tensor_parallel2_matches_single_process(ref):
    assert (ref - spawn_tiny_wan_denoise(2, tp_degree=2)).abs().max().item() <= 1e-5


def test_sharded_weights2_match_single_process(ref):
    assert (ref - spawn_tiny_wan_denoise(2, sp_ulysses_degree=2, enable_fsdp=True)).abs().max().item() <= 1e-5


def test_stage_block_range():
    assert [stage_block_range(40, 4, i) for i in range(4)] == [(0, 10), (10, 20), (20, 30), (30, 40)]
    assert [stage_block_range(30, 4, i) for i in range(4)] == [(0, 8), (8, 16), (16, 23), (23, 30)]
    with pytest.raises(ValueError):
        stage_block_range(2, 4, 0)


def _tp_encoder_rank(rank, world, port, path):
    from telefuser_b200.models.umt5 import WanTextEncoder
    from telefuser_b200.parallel.tp import parallelize_module

    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        enc = WanTextEncoder(vocab=64, dim=32, dim_attn=32, dim_ffn=64, num_heads=4, num_layers=2, num_buckets=8).eval()
        ids = torch.arange(12).view(1, 12) % 64
        mask = torch.ones(1, 12, dtype=torch.long)
        mask[:, 9:] = 0
        full = enc(ids, mask)
        parallelize_module(enc, dist.group.WORLD, enc.get_tp_plan())
        assert enc.blocks[0].attn.q.weight.shape == (16, 32) and enc.blocks[0].attn.num_heads == 2
        assert enc.blocks[0].ffn.fc2.weight.shape == (32, 32)
        sharded = enc(ids, mask)
        if rank == 0:
            torch.save((full, sharded), path)
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_tensor_parallel_text_encoder():
    from telefuser_b200.utils.system import find_free_port

    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "o.pt")
        mp.spawn(_tp_encoder_rank, nprocs=2, join=True, args=(2, find_free_port(), path))
        full, sharded = torch.load(path)
    assert (full - sharded).abs().max().item() <= 1e-5


def _tp_fused_rank(rank, world, port, path):
    from telefuser_b200.testing.peer_checks import tp_fused_errors

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        errs = tp_fused_errors(dist.group.WORLD, torch.device("cpu"), None, M=64, K=32, N=24, rounds=1)
        if rank == 0:
            torch.save(errs, path)
    finally:
        dist.destroy_process_group()


def test_tensor_parallel_linears_compose_collectives_without_a_peer_workspace():
    from telefuser_b200.utils.system import find_free_port

    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "errs.pt")
        mp.spawn(_tp_fused_rank, nprocs=2, join=True, args=(2, find_free_port(), path))
        errs = torch.load(path)
    assert max(errs.values()) <= 1e-5, errs


def _remote_runs_case(device, dtype, D, tol):
    import torch

    from telefuser_b200.ops import functional as TF
    from telefuser_b200.parallel.symm import attend_remote_runs

    torch.manual_seed(0)
    P, Sk, H = 4, 64, 2
    k_full, v_full = (torch.randn(P * Sk, H * D, device=device, dtype=dtype) for _ in range(2))
    for rank in range(P):
        q = torch.randn(1, 48, H, D, device=device, dtype=dtype)
        own = slice(rank * Sk, (rank + 1) * Sk)
        o, lse = TF.attention(q, k_full[own].view(1, Sk, H, D), v_full[own].view(1, Sk, H, D), return_lse=True)
        o, lse = attend_remote_runs(q, o, lse, k_full, v_full, rank, P, Sk)
        want = TF.attention(q, k_full.view(1, P * Sk, H, D), v_full.view(1, P * Sk, H, D))
        assert (o.float() - want.float()).abs().max() < tol, rank


def test_context_parallel_remote_runs_cover_every_rank_position():
    import torch

    _remote_runs_case("cpu", torch.float32, 16, 1e-5)


@pytest.mark.gpu
def test_context_parallel_remote_runs_gpu():
    import torch

    _remote_runs_case("cuda", torch.bfloat16, 128, 2e-2)


@pytest.mark.parametrize("world", [2, 4])
def test_vae_spatial_parallelism_matches_the_single_process_result(world):
    """Tile round-robin + all-reduce (`_tiled`) and the 2-D domain split + all-gather (`decode_dist_2d`) under a
    process group: every rank ends with the full tensor, equal to what one process computes."""
    from telefuser_b200.testing.distributed_checks import spawn_vae_parallel, vae_parallel_outputs

    want = vae_parallel_outputs(1)
    # a halo as large as the latent makes every rank's tile see the whole input: the split decode is then exact
    assert (want["dist_2d"] - want["plain"]).abs().max() <= 1e-5
    outs = spawn_vae_parallel(world)
    assert len(outs) == world
    for rank, got in enumerate(outs):
        for key in ("tiled_decode", "tiled_encode", "dist_2d"):
            assert got[key].shape == want[key].shape, (rank, key)
            assert (got[key] - want[key]).abs().max() <= 2e-5, (rank, key, world)


def test_multi_gpu_suite_host_logic_on_two_cpu_ranks(tmp_path):
    """The layout sweep and the VAE split of the multi-GPU verification program, on gloo ranks."""
    import json
    import subprocess
    import sys

    from telefuser_b200.utils.system import find_free_port

    out = tmp_path / "suite.json"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(find_free_port()), "-m", "telefuser_b200.testing.multi_gpu_suite", "--backend", "gloo",
           "--out", str(out)]  # fmt: skip
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    rep = json.loads(out.read_text())
    assert rep["passed"] and {"cfg2/collectives", "u2/collectives", "r2/collectives", "tp2/collectives"} <= set(rep["rank0"]["layouts"])


def test_mesh_groups_partition_the_world_for_every_layout():
    """Without a process group (rank and world size given): every dimension's groups partition the ranks, members of a
    group differ in that coordinate only, the SP group is ring x Ulysses, and EP groups are contiguous slices of the
    CFG x SP ranks."""
    import itertools

    from telefuser_b200.core.config import ParallelConfig
    from telefuser_b200.parallel.mesh import DIM_NAMES, create_mesh, set_mesh

    layouts = [dict(cfg_degree=2, sp_ulysses_degree=4), dict(sp_ring_degree=2, sp_ulysses_degree=4), dict(dp_degree=2, cfg_degree=2, sp_ulysses_degree=2),
               dict(pp_degree=2, sp_ulysses_degree=2, cfg_degree=2), dict(tp_degree=8), dict(dp_degree=2, pp_degree=2, tp_degree=2),
               dict(cfg_degree=2, sp_ring_degree=2, sp_ulysses_degree=2, ep_degree=4), dict(sp_ulysses_degree=8, ep_degree=8)]  # fmt: skip
    try:
        for kw in layouts:
            cfg = ParallelConfig(device_ids=list(range(8)), **kw)
            meshes = [create_mesh(cfg, rank=r, world_size=8) for r in range(8)]
            for i, name in enumerate(DIM_NAMES):
                groups = {tuple(m.ranks(name)) for m in meshes}
                assert sorted(itertools.chain.from_iterable(groups)) == list(range(8)), (kw, name)  # a partition
                for m in meshes:
                    assert m.rank in m.ranks(name) and len(m.ranks(name)) == m.size(name) == m.dims[i]
                    assert m.ranks(name).index(m.rank) == m.coord(name)
                    for other in m.ranks(name):  # same group: all other coordinates agree
                        o = meshes[other]
                        assert all(o.coord(n) == m.coord(n) for n in DIM_NAMES if n != name), (kw, name)
            for m in meshes:
                assert len(m.ranks("sp")) == m.size("ring") * m.size("ulysses") == m.size("sp")
                assert set(m.ranks("ring")) | set(m.ranks("ulysses")) <= set(m.ranks("sp"))
                if kw.get("ep_degree", 1) > 1:
                    ep = m.ranks("ep")
                    assert len(ep) == kw["ep_degree"] == m.size("ep") and m.rank in ep and ep == list(range(ep[0], ep[0] + len(ep)))
                    assert m.coord("ep") == ep.index(m.rank)
        import pytest

        with pytest.raises(RuntimeError, match="do not match world size"):
            create_mesh(ParallelConfig(device_ids=list(range(8)), sp_ulysses_degree=4), rank=0, world_size=8)
        with pytest.raises(ValueError, match="cannot be combined"):
            create_mesh(ParallelConfig(device_ids=list(range(8)), sp_ulysses_degree=4, tp_degree=2), rank=0, world_size=8)
    finally:
        set_mesh(None)
