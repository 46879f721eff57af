"""Multi-GPU plumbing on real devices (NCCL): Ulysses and CFG-parallel denoising equal the single-GPU run."""
import pytest
import torch

from telefuser_b200.testing.distributed_checks import spawn_tiny_wan_denoise, tiny_wan_denoise

pytestmark = [pytest.mark.gpu, pytest.mark.multi_gpu]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("kw", [dict(sp_ulysses_degree=2), dict(cfg_degree=2)])
def test_two_gpu_denoise_matches_single(kw):
    ref = tiny_wan_denoise(device="cuda:0", dtype=torch.bfloat16, preset="native-small")
    got = spawn_tiny_wan_denoise(2, backend="nccl", dtype=torch.bfloat16, preset="native-small", **kw)
    err = ((ref - got).norm() / ref.norm()).item()
    assert err < 2e-2, err
