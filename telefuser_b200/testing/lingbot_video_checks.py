"""SPMD checks of the LingBot-Video transformer: Ulysses sequence parallelism and expert parallelism
must reproduce the single-process forward (gloo ranks on CPU, NCCL ranks on GPUs)."""

from __future__ import annotations

import os
import tempfile

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from telefuser_b200.models.lingbot_video import LingBotVideoConfig, LingBotVideoTransformer3DModel


def make_model(preset: str, dtype=torch.float32, device="cpu", seed: int = 0, **overrides):
    torch.manual_seed(seed)
    cfg = LingBotVideoConfig.preset(preset)
    for k, v in overrides.items():
        setattr(cfg, k, v)
    m = LingBotVideoTransformer3DModel(cfg)
    for p in m.parameters():
        torch.nn.init.normal_(p, std=0.05)
    for n, b in m.named_buffers():
        if "correction" in n:
            b.normal_(std=0.1)
    m = m.to(dtype).to(device).eval()
    m.promote_stability_layers_to_fp32()
    m.dtype = dtype
    return m


def make_inputs(seed: int = 1, text_dim: int = 32, frames: int = 2, size: int = 8, text_len: int = 7):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(1, 16, frames, size, size, generator=g), torch.tensor([400.0]),
            torch.randn(1, text_len, text_dim, generator=g))  # fmt: skip


def _rank(rank, world, port, backend, preset, mode, dtype_name, out_path, overrides, input_kw):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                      NCCL_NVLS_ENABLE="0")  # fmt: skip
    torch.set_num_threads(1)
    device = "cpu"
    if backend == "nccl":
        torch.cuda.set_device(rank)
        device = f"cuda:{rank}"
    dist.init_process_group(backend, rank=rank, world_size=world)
    try:
        dtype = getattr(torch, dtype_name)
        model = make_model(preset, dtype, device, **overrides)
        if mode in ("ulysses", "both"):
            model.set_ulysses_group(dist.group.WORLD)
        if mode in ("ep", "both"):
            model.enable_expert_parallel(dist.group.WORLD)
        x, t, txt = make_inputs(text_dim=model.config.text_dim, **input_kw)
        out = model(x.to(device, dtype), t.to(device), txt.to(device, dtype))
        if rank == 0:
            torch.save(out.float().cpu(), out_path)
        dist.barrier()
        if backend == "nccl":
            from telefuser_b200.parallel import expert

            expert.release()
    finally:
        dist.destroy_process_group()


def spawn(world: int, preset: str, mode: str, backend: str = "gloo", dtype=torch.float32, overrides=None, **input_kw):
    from telefuser_b200.utils.system import find_free_port

    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "o.pt")
        mp.spawn(_rank, nprocs=world, join=True,
                 args=(world, find_free_port(), backend, preset, mode, str(dtype).split(".")[-1], path, overrides or {},
                       input_kw))  # fmt: skip
        return torch.load(path)
