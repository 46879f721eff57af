"""GEMM kernels with fused collectives, emulated on ONE GPU: the "peers" are local buffers and the ranks'
launches run one after another (no launch waits for another; the all-gather mode's waits are between CTAs
of one launch). Checked against the fp32 product of the unsharded operands."""

import ctypes

import pytest
import torch

from telefuser_b200.ops import native

pytestmark = [pytest.mark.gpu]


def _table(tensors):
    return (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


@pytest.mark.parametrize("P,seg,N,K", [(2, 700, 768, 1024), (3, 128, 256, 512), (4, 1920, 2048, 512)])
def test_gemm_reduce_scatter_epilogue_and_slab_reduce(P, seg, N, K):
    torch.manual_seed(0)
    lib = native.load()
    native.last_status()
    M = P * seg
    x = (torch.randn(M, K * P, device="cuda") / 4).bfloat16()
    w = (torch.randn(N, K * P, device="cuda") / (K * P) ** 0.5).bfloat16()
    bias = torch.randn(N, device="cuda").bfloat16()
    res = torch.randn(M, N, device="cuda").bfloat16()
    gate = torch.randn(1, N, device="cuda")
    slabs = [torch.zeros(P, seg, N, device="cuda", dtype=torch.bfloat16) for _ in range(P)]  # one buffer per owner
    st = torch.cuda.current_stream().cuda_stream
    for r in range(P):
        xs, wsh = x[:, r * K : (r + 1) * K], w[:, r * K : (r + 1) * K]  # strided K shards
        code = lib.tfb_gemm_bf16_rs(xs.data_ptr(), xs.stride(0), wsh.data_ptr(), wsh.stride(0), _table(slabs), N, P, r, seg,
                                    N, K, bias.data_ptr() if r == 0 else None, st)  # fmt: skip
        assert code == 0
    full = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16)
    for r in range(P):
        rows = res[r * seg : (r + 1) * seg]
        code = lib.tfb_slab_reduce(slabs[r].data_ptr(), P, seg, N, N, None, rows.data_ptr(), rows.stride(0), gate.data_ptr(),
                                   N, M, r * seg, _table([full]), 1, N, r * seg, st)  # fmt: skip
        assert code == 0
    torch.cuda.synchronize()
    assert native.last_status() == 0
    want = res.float() + gate * (x.float() @ w.float().t() + bias.float())
    err = ((full.float() - want).norm() / want.norm()).item()
    assert err < 6e-3, err


@pytest.mark.parametrize("P,seg,N,K,copiers", [(2, 700, 384, 1024, 4), (4, 350, 192, 256, 8), (3, 1024, 1024, 2048, 8),
                                               (2, 40, 128, 64, 8)])  # fmt: skip
def test_all_gather_gemm_with_copier_ctas(P, seg, N, K, copiers):
    torch.manual_seed(1)
    lib = native.load()
    native.last_status()
    shards = [(torch.randn(seg, K, device="cuda") / 4).bfloat16() for _ in range(P)]
    w = (torch.randn(N, K, device="cuda") / K**0.5).bfloat16()
    bias = torch.randn(N, device="cuda").bfloat16()
    want = torch.nn.functional.gelu(torch.cat(shards).float() @ w.float().t() + bias.float(), approximate="tanh")
    st = torch.cuda.current_stream().cuda_stream
    for r in range(P):
        gathered = torch.zeros(P * seg, K, device="cuda", dtype=torch.bfloat16)
        sync = torch.empty(16, device="cuda", dtype=torch.int32)
        out = torch.zeros(P * seg, N, device="cuda", dtype=torch.bfloat16)
        code = lib.tfb_gemm_bf16_ag(_table(shards), gathered.data_ptr(), sync.data_ptr(), copiers, w.data_ptr(), w.stride(0),
                                    out.data_ptr(), N, P, r, seg, N, K, bias.data_ptr(), 1, st)  # fmt: skip
        assert code == 0
        torch.cuda.synchronize()
        assert native.last_status() == 0
        assert torch.equal(gathered, torch.cat(shards))
        err = ((out.float() - want).norm() / want.norm()).item()
        assert err < 6e-3, (r, err)
        assert sync[1 : 1 + P].tolist() == [copiers] * P
