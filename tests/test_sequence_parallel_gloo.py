"""CPU plumbing check: the tiny Wan-style DiT denoised on 2 gloo ranks with Ulysses
sequence parallelism (and with CFG parallelism) must reproduce the single-process run."""
import torch

from telefuser_b200.testing.distributed_checks import spawn_tiny_wan_denoise, tiny_wan_denoise


def test_ulysses2_matches_single_process():
    ref = tiny_wan_denoise()
    got = spawn_tiny_wan_denoise(2, sp_ulysses_degree=2)
    assert ref.shape == (1, 16, 3, 8, 8)
    assert torch.isfinite(ref).all()
    assert (ref - got).abs().max().item() <= 1e-5


def test_cfg_parallel2_matches_single_process():
    ref = tiny_wan_denoise()
    got = spawn_tiny_wan_denoise(2, cfg_degree=2)
    assert (ref - got).abs().max().item() <= 1e-5
