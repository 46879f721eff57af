"""Multi-GPU plumbing on real devices: Ulysses and CFG-parallel denoising equal the single-GPU run
(peer-memory kernels by default, the NCCL path with TFB_FUSED_COLLECTIVES=0), the peer-memory
paths equal the collective-library paths op by op, and a peer wait that nobody answers runs out
with a status instead of hanging. The file sorts after the single-GPU files on purpose: with `pytest -x` a failure that
needs several GPUs to show must not hide the single-GPU results."""
import ctypes

import pytest
import torch

from telefuser_b200.testing.distributed_checks import spawn_tiny_wan_denoise, tiny_wan_denoise

pytestmark = [pytest.mark.gpu]
two_gpus = pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")


@two_gpus
@pytest.mark.multi_gpu
@pytest.mark.parametrize("fused", ["1", "0"])
@pytest.mark.parametrize("kw", [dict(sp_ulysses_degree=2), dict(cfg_degree=2)])
def test_two_gpu_denoise_matches_single(kw, fused, monkeypatch):
    monkeypatch.setenv("TFB_FUSED_COLLECTIVES", fused)
    monkeypatch.setenv("NCCL_NVLS_ENABLE", "0")
    ref = tiny_wan_denoise(device="cuda:0", dtype=torch.bfloat16, preset="native-small")
    got = spawn_tiny_wan_denoise(2, backend="nccl", dtype=torch.bfloat16, preset="native-small", **kw)
    err = ((ref - got).norm() / ref.norm()).item()
    assert err < 2e-2, err


@two_gpus
@pytest.mark.multi_gpu
def test_peer_memory_paths_match_collectives():
    from telefuser_b200.testing.peer_checks import spawn

    n = 4 if torch.cuda.device_count() >= 4 else 2
    for errs in spawn(n):
        assert errs["status"] == 0, errs
        assert errs["ulysses"] <= 2e-2, errs  # bf16 outputs of two runs of the same kernel on the same data
        assert errs["gather"] == 0.0, errs
        assert errs["ring"] <= 2e-2, errs  # peer-store K / V exchange vs the NCCL ring and vs full-sequence attention
        if "cfg" in errs:
            assert errs["cfg"] <= 1e-6, errs
        for key in ("tp_rs", "tp_ar", "tp_ag"):  # fused GEMM + collective against the unsharded fp32 product
            assert errs[key] <= 1e-2, errs


def test_peer_wait_runs_out_with_a_status():
    """One GPU: the barrier waits for a second rank that does not exist. The wait is bounded (4 s), the
    kernel returns, the context stays usable and the status word names the barrier's wait site."""
    from telefuser_b200.ops import native

    lib = native.load()
    native.last_status()  # clear
    flags = [torch.zeros(64, dtype=torch.int32, device="cuda") for _ in range(2)]
    table = (ctypes.c_void_p * 2)(flags[0].data_ptr(), flags[1].data_ptr())
    assert lib.tfb_peer_barrier(table, 0, 2, 0, 1, torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    status = native.last_status()
    assert status & 0xFF == 1 and status >> 8 == 60, status  # TFB_ERR_TIMEOUT at site 60
    assert flags[1][0].item() == 1  # the signal to the absent rank was still written
    x = torch.ones(4, device="cuda") * 2  # context still answers
    assert x.sum().item() == 8.0


def _run_suite(n: int, backend: str, tmp_path, timeout: int = 1500):
    import json
    import subprocess
    import sys

    from telefuser_b200.utils.system import find_free_port

    out = tmp_path / f"suite_{n}.json"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", str(find_free_port()), "-m", "telefuser_b200.testing.multi_gpu_suite", "--backend", backend,
           "--out", str(out)]  # fmt: skip
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout)
    assert out.is_file(), res.stdout[-3000:] + res.stderr[-3000:]
    return res.returncode, json.loads(out.read_text())


@two_gpus
@pytest.mark.multi_gpu
def test_every_multi_gpu_path_on_all_visible_gpus(tmp_path):
    """All layouts (CFG x Ulysses, Ulysses, ring, Ulysses x ring, TP, PP x Ulysses, sharded weights), the peer-memory
    kernels against collectives and oracles, expert parallelism and the VAE split, on 2, 4 or 8 ranks in one launch."""
    n = max(k for k in (2, 4, 8) if k <= torch.cuda.device_count())
    code, rep = _run_suite(n, "nccl", tmp_path)
    assert code == 0 and rep["passed"], rep["failures"]
