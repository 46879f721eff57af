"""Out-of-bounds writes: the native kernels run at edge shapes (ragged tiles, partial rows, odd counts) with every
output carved between guard zones; no guard byte may change. The checker itself is tested on CPU logic and with a
deliberate host-side overwrite (no kernel is ever asked to write out of range)."""

import pytest
import torch

from telefuser_b200.testing.guards import PATTERN, GuardedAllocations, GuardViolation


def test_guard_bookkeeping_on_cpu_allocations_is_transparent():
    with GuardedAllocations() as g:
        a = torch.empty(3, 5)
        b = torch.zeros(4, dtype=torch.int64)
        c = torch.empty_like(a)
    assert a.shape == (3, 5) and b.sum() == 0 and c.shape == a.shape and g.check() == 0
    assert torch.empty.__module__ == "torch" or torch.empty(1).shape == (1,)  # originals restored


@pytest.mark.gpu
def test_a_damaged_guard_is_reported_with_its_position():
    with pytest.raises(GuardViolation, match="above the tensor"):
        with GuardedAllocations() as g:
            t = torch.empty(100, dtype=torch.bfloat16, device="cuda")
            base, nbytes, _, _ = g.records[0]
            assert t.data_ptr() % 256 == 0 and (base[: g.guard] == PATTERN).all()
            base[g.guard + nbytes + 3] = 0  # host-side write into the upper guard
    with GuardedAllocations() as g:
        z = torch.zeros(7, 9, device="cuda")
        e = torch.empty_like(z)
        e.copy_(z + 1)
    assert g.check() == 2 and z.sum() == 0 and e.sum() == 63


@pytest.mark.gpu
def test_kernels_at_edge_shapes_leave_the_guards_alone():
    from telefuser_b200.ops import functional as TF
    from telefuser_b200.ops.quant import quantize_weight_fp8

    torch.manual_seed(0)
    dev = "cuda"
    with GuardedAllocations() as g:
        # GEMM: ragged M and N tiles, every epilogue
        x = torch.randn(3, 77, 144, device=dev).bfloat16()
        w = (torch.randn(72, 144, device=dev) * 0.1).bfloat16()
        bias, res = torch.randn(72, device=dev).bfloat16(), torch.randn(3, 77, 72, device=dev).bfloat16()
        gate = torch.randn(3, 1, 72, device=dev)
        TF.linear(x, w, bias, act="gelu_tanh")
        TF.linear(x, w, bias, residual=res, gate=gate)
        q8, s8 = quantize_weight_fp8(w)
        TF.linear_fp8(x, q8, s8, bias)
        wq, wsf = TF.quantize_weight_mxfp8(torch.randn(72, 256, device=dev).bfloat16())
        TF.linear_mxfp8(torch.randn(77, 256, device=dev).bfloat16(), wq, wsf, bias)
        # attention: partial query tiles, partial key tiles, both head dims, causal, LSE
        for D in (64, 128):
            q = torch.randn(2, 300, 3, D, device=dev).bfloat16()
            k = torch.randn(2, 515, 3, D, device=dev).bfloat16()
            v = torch.randn(2, 515, 3, D, device=dev).bfloat16()
            TF.attention(q, k, v, return_lse=True)
            TF.attention(q, k[:, :300], v[:, :300], causal=True)
        TF.attention(q, k, v, variant=21)
        # row kernels: odd row counts
        y = torch.randn(2, 333, 256, device=dev).bfloat16()
        sh, sc = torch.randn(2, 1, 256, device=dev), torch.randn(2, 1, 256, device=dev)
        TF.layernorm_modulate(y, sh, sc)
        TF.gated_residual(y, y, sh)
        TF.act_mul(torch.randn(333, 512, device=dev).bfloat16(), "silu")
        TF.quant_fp8_rowwise(y)
        TF.quant_mxfp8(y)
        TF.quant_mxfp8(y, tiled=True)
        lat = torch.randn(1, 16, 3, 10, 14, device=dev)
        TF.cfg_euler_step(lat, lat.bfloat16(), lat.bfloat16(), 5.0, -0.1)
    assert g.check() > 20


def test_peer_region_table_recarves_in_place_on_cpu_memory():
    """The region table of the peer workspace, exercised on a plain CPU buffer (no IPC): a name that comes back smaller
    keeps its offset, a name that outgrows its reservation resets the whole table, canary strips sit right behind every
    region and are checked, and a request beyond the buffer is refused."""
    import torch

    from telefuser_b200.parallel import symm

    ws = object.__new__(symm.PeerWorkspace)
    ws.nbytes = 1 << 20
    ws.local = torch.zeros(ws.nbytes, dtype=torch.uint8)
    ws.flag_off = ws.nbytes - symm.FLAG_BYTES
    ws._regions, ws._cursor, ws.canaries, ws._canaries = {}, 0, True, {}
    ws.ptrs, ws.rank, ws.world = [1000, 5000], 0, 2
    a = ws.region("q", (4, 64, 2, 128))  # 131072 bytes
    b = ws.region("o", (4, 64, 2, 128))
    assert a.shape == (4, 64, 2, 128) and a.dtype == torch.bfloat16
    off_a, off_b = ws._regions["q"][0], ws._regions["o"][0]
    assert off_a == 0 and off_b == 131072 + symm.CANARY_BYTES and off_b % 256 == 0
    assert ws.peer_ptr(1, "o") == 5000 + off_b
    ws.check_canaries()
    small = ws.region("q", (2, 64, 2, 128))  # fits the reservation: same place, other shape
    assert ws._regions["q"][0] == 0 and small.shape == (2, 64, 2, 128) and ws._regions["o"][0] == off_b
    a.view(torch.uint8).reshape(-1)[-1] = 7  # the last byte of the region itself: allowed
    ws.check_canaries()
    ws.local[ws._canaries["q"][0] + 3] = 0  # one byte behind the end of "q"
    with pytest.raises(AssertionError, match="'q'.*first at \\+3"):
        ws.check_canaries()
    big = ws.region("q", (8, 64, 2, 128))  # outgrows its reservation: everything is carved anew from offset 0
    assert big.shape == (8, 64, 2, 128) and list(ws._regions) == ["q"] and ws._regions["q"][0] == 0
    ws.check_canaries()  # the strips were rewritten with the new table
    assert ws.region("o", (4, 64, 2, 128)).data_ptr() == ws.local.data_ptr() + ws._regions["o"][0]
    with pytest.raises(MemoryError):
        ws.region("huge", (1 << 20,))
