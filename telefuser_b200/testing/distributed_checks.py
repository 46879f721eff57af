"""Self-checks that run the same tiny workload single-process and as SPMD ranks.

`tiny_wan_denoise` is the plumbing check: a 2-block Wan-style DiT (dim 128, 4 heads
x 32, FFN 512, patch (1,2,2), 16 latent channels) denoises a [1,16,3,8,8] latent
(48 tokens) for 4 flow-matching Euler steps (shift 5, CFG 5, zero-context
unconditional branch). `spawn_tiny_wan_denoise` runs it on `world_size` ranks
(gloo on CPU, nccl on GPUs) with the requested parallel degrees and returns rank
0's result so callers can compare it with the single-process run.
"""

from __future__ import annotations

import os
import tempfile

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from telefuser_b200.core.config import ModelRuntimeConfig, ParallelConfig
from telefuser_b200.models.wan_dit import WanModel, WanModelConfig
from telefuser_b200.parallel import mesh as pmesh
from telefuser_b200.pipelines.wan.denoising import WanDenoisingStage
from telefuser_b200.schedulers.flow_match import FlowMatchScheduler


def make_tiny_inputs(seed: int = 0):
    g = torch.Generator().manual_seed(seed)
    latents = torch.randn(1, 16, 3, 8, 8, generator=g)
    context = torch.randn(1, 16, 256, generator=g)
    return latents, context, torch.zeros_like(context)


def make_tiny_model(seed: int = 0, dtype=torch.float32, preset: str = "tiny") -> WanModel:
    torch.manual_seed(seed)
    if preset == "native-small":  # head_dim 128 so the native attention kernel runs on GPUs
        model = WanModel(dim=512, ffn_dim=1024, num_heads=4, num_layers=2, text_dim=256).to(dtype)
    else:
        model = WanModel.from_config(WanModelConfig.preset(preset)).to(dtype)
    model.dtype = dtype
    return model.eval()


def tiny_wan_denoise(parallel: ParallelConfig | None = None, device: str = "cpu", dtype=torch.float32,
                     steps: int = 4, preset: str = "tiny") -> torch.Tensor:  # fmt: skip
    parallel = parallel or ParallelConfig()
    cfg = ModelRuntimeConfig(torch_dtype=dtype, parallel_config=parallel, device_type=device.split(":")[0],
                             device_id=int(device.split(":")[1]) if ":" in device else 0)  # fmt: skip
    model = make_tiny_model(dtype=dtype, preset=preset).to(device)
    stage = WanDenoisingStage("denoise", None, cfg, FlowMatchScheduler("Wan"), dit=model)
    if parallel.device_ids is not None and len(parallel.device_ids) > 1:
        stage.parallel_models()
    else:
        pmesh.set_mesh(None)
        stage.mesh = pmesh.get_mesh()
    stage.onload_models_flag = True
    latents, ctx, neg = make_tiny_inputs()
    out = stage.process(latents.to(device), steps, None, ctx.to(device=device, dtype=dtype),
                        neg.to(device=device, dtype=dtype), None, 5.0, 5.0)  # fmt: skip
    return out.float().cpu()


def _rank_main(rank: int, world_size: int, port: int, backend: str, parallel_kwargs: dict, out_path: str,
               dtype_name: str, preset: str = "tiny") -> None:  # fmt: skip
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world_size), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.set_num_threads(1)
    device = "cpu"
    if backend == "nccl":
        torch.cuda.set_device(rank)
        device = f"cuda:{rank}"
    dist.init_process_group(backend=backend, rank=rank, world_size=world_size)
    try:
        parallel = ParallelConfig(device_ids=list(range(world_size)), **parallel_kwargs)
        out = tiny_wan_denoise(parallel, device=device, dtype=getattr(torch, dtype_name), preset=preset)
        if rank == 0:
            torch.save(out, out_path)
        dist.barrier()
    finally:
        dist.destroy_process_group()


def spawn_tiny_wan_denoise(world_size: int, backend: str = "gloo", dtype=torch.float32, preset: str = "tiny",
                           **parallel_kwargs):  # fmt: skip
    from telefuser_b200.utils.system import find_free_port

    with tempfile.TemporaryDirectory() as d:
        out_path = os.path.join(d, "out.pt")
        mp.spawn(_rank_main, nprocs=world_size, join=True,
                 args=(world_size, find_free_port(), backend, parallel_kwargs, out_path, str(dtype).split(".")[-1],
                       preset))  # fmt: skip
        return torch.load(out_path)


if __name__ == "__main__":
    ref = tiny_wan_denoise()
    got = spawn_tiny_wan_denoise(2, sp_ulysses_degree=2)
    print("single vs ulysses-2 max abs diff:", (ref - got).abs().max().item())


# ---------------------------------------------------------------------------------------------------
# VAE spatial parallelism (tile round-robin with all-reduce, 2-D domain decomposition with all-gather)
# ---------------------------------------------------------------------------------------------------
def _tiny_vae(seed: int = 0):
    from telefuser_b200.models.wan_vae import WanVideoVAE
    from telefuser_b200.testing.synthetic import random_init_

    torch.manual_seed(seed)
    return random_init_(WanVideoVAE(dim=8).float(), seed, std=0.05).eval()


def vae_parallel_outputs(parallelism: int = 1) -> dict:
    """Tiled decode / encode and the 2-D split decode of a tiny VAE on fixed inputs; under a process group every rank
    computes its share and the collectives assemble the full result on every rank."""
    vae = _tiny_vae()
    vae.parallelism = parallelism
    g = torch.Generator().manual_seed(1)
    latents = torch.randn(1, 16, 2, 12, 10, generator=g)
    video = torch.rand(1, 3, 5, 64, 48, generator=g) * 2 - 1
    with torch.no_grad():
        return {"tiled_decode": vae.tiled_decode(latents, tile_size=(8, 6), tile_stride=(4, 4)),
                "tiled_encode": vae.tiled_encode(video, tile_size=(6, 4), tile_stride=(2, 2)),
                "dist_2d": vae.decode_dist_2d(latents, halo=12),
                "plain": vae.model.decode(latents, vae.scale).clamp(-1, 1)}  # fmt: skip


def _vae_rank_main(rank: int, world_size: int, port: int, out_dir: str) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world_size))
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world_size)
    try:
        torch.save(vae_parallel_outputs(world_size), os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


def spawn_vae_parallel(world_size: int) -> list[dict]:
    from telefuser_b200.utils.system import find_free_port

    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_vae_rank_main, nprocs=world_size, join=True, args=(world_size, find_free_port(), d))
        return [torch.load(os.path.join(d, f"rank{r}.pt")) for r in range(world_size)]
