"""The allocation-free token-permute entry point, called through its exported C symbol, against the
entry point that takes a caller-supplied scratch buffer: two calls in a row, then the size limit."""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

from telefuser_b200.ops import native  # noqa: E402

c_void_p, c_int, c_long = ctypes.c_void_p, ctypes.c_int, ctypes.c_long


def _symbols():
    lib = ctypes.CDLL(str(native.lib_path()))
    static = lib.tfb_moe_permute_static
    static.restype = c_int
    static.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_int, c_long, c_int, c_void_p, c_void_p, c_void_p]
    plain = lib.tfb_moe_permute
    plain.restype = c_int
    plain.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_long, c_int, c_void_p, c_void_p, c_void_p]
    plan = lib.tfb_moe_plan
    plan.restype = c_int
    plan.argtypes = [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p]
    return static, plain, plan


def _case(seed, T, K, E, hidden, dev):
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn(T, hidden, generator=g).bfloat16().to(dev)
    ids = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).to(torch.int32).to(dev)
    counts = torch.bincount(ids.reshape(-1).long(), minlength=E).to(torch.int32)
    return x, ids, counts


def test_static_permute_matches_buffer_version_twice_in_a_row():
    dev = torch.device("cuda:0")
    static, plain, plan = _symbols()
    stream = torch.cuda.current_stream().cuda_stream
    E, K, hidden = 96, 4, 256
    for call, (seed, T) in enumerate(((0, 700), (1, 431))):  # second call: different routing, stale cursors left behind
        x, ids, counts = _case(seed, T, K, E, hidden, dev)
        rows = -(-(T * K + E * 127) // 128) * 128
        offsets = torch.empty(E + 1, dtype=torch.int32, device=dev)
        tiles = torch.empty(rows // 128, dtype=torch.int32, device=dev)
        assert plan(counts.data_ptr(), E, 128, offsets.data_ptr(), tiles.data_ptr(), rows // 128, stream) == 0
        xp_a, xp_b = (torch.zeros(rows, hidden, dtype=torch.bfloat16, device=dev) for _ in range(2))
        map_a, map_b = (torch.empty(T * K, dtype=torch.int32, device=dev) for _ in range(2))
        cursor = torch.full((E,), 12345, dtype=torch.int32, device=dev)  # the entry point clears it itself
        assert plain(x.data_ptr(), hidden, ids.data_ptr(), offsets.data_ptr(), cursor.data_ptr(), E, T, K,
                     xp_a.data_ptr(), map_a.data_ptr(), stream) == 0  # fmt: skip
        assert static(x.data_ptr(), hidden, ids.data_ptr(), offsets.data_ptr(), E, T, K, xp_b.data_ptr(),
                      map_b.data_ptr(), stream) == 0  # fmt: skip
        torch.cuda.synchronize()
        # slot order inside an expert's segment depends on atomics, so compare what is order-free:
        # every (token, k) finds its token's row, inside its expert's segment, and the occupied rows coincide
        want = x.repeat_interleave(K, dim=0)
        assert torch.equal(xp_a[map_a.long()], want), call
        assert torch.equal(xp_b[map_b.long()], want), call
        assert torch.equal(map_a.sort().values, map_b.sort().values), call
        flat = ids.reshape(-1).long()
        lo, hi = offsets[flat], offsets[flat] + counts[flat]
        assert ((map_b >= lo) & (map_b < hi)).all(), call
        assert map_b.unique().numel() == T * K, call


def test_static_permute_rejects_more_experts_than_its_scratch_holds(capfd):
    dev = torch.device("cuda:0")
    static, _, _ = _symbols()
    x = torch.zeros(8, 64, dtype=torch.bfloat16, device=dev)
    ids = torch.zeros(8, 1, dtype=torch.int32, device=dev)
    offsets = torch.zeros(1026, dtype=torch.int32, device=dev)
    out = torch.zeros(8 + 1025 * 128, 64, dtype=torch.bfloat16, device=dev)
    row_map = torch.zeros(8, dtype=torch.int32, device=dev)
    code = static(x.data_ptr(), 64, ids.data_ptr(), offsets.data_ptr(), 1025, 8, 1, out.data_ptr(), row_map.data_ptr(),
                  torch.cuda.current_stream().cuda_stream)  # fmt: skip
    assert code == 5  # TFB_ERR_TOO_LARGE: nothing was launched
    assert "static scratch limit of 1024" in capfd.readouterr().err
    torch.cuda.synchronize()


def test_static_permute_at_its_limit_and_with_stale_cursors_beyond_e():
    """E = 1024 exactly (the whole scratch array), then E = 96 right after a call with E = 512: the cursors of
    experts 96..511 keep the counts of the earlier call, which no in-range id of the later call can touch."""
    dev = torch.device("cuda:0")
    static, _, plan = _symbols()
    stream = torch.cuda.current_stream().cuda_stream
    hidden, K = 64, 2
    for seed, (E, T) in enumerate(((1024, 1500), (512, 900), (96, 333))):
        x, ids, counts = _case(10 + seed, T, K, E, hidden, dev)
        rows = -(-(T * K + E * 127) // 128) * 128
        offsets = torch.empty(E + 1, dtype=torch.int32, device=dev)
        tiles = torch.empty(rows // 128, dtype=torch.int32, device=dev)
        assert plan(counts.data_ptr(), E, 128, offsets.data_ptr(), tiles.data_ptr(), rows // 128, stream) == 0
        xp = torch.zeros(rows, hidden, dtype=torch.bfloat16, device=dev)
        row_map = torch.empty(T * K, dtype=torch.int32, device=dev)
        assert static(x.data_ptr(), hidden, ids.data_ptr(), offsets.data_ptr(), E, T, K, xp.data_ptr(),
                      row_map.data_ptr(), stream) == 0  # fmt: skip
        torch.cuda.synchronize()
        assert torch.equal(xp[row_map.long()], x.repeat_interleave(K, dim=0)), E
        flat = ids.reshape(-1).long()
        assert ((row_map >= offsets[flat]) & (row_map < offsets[flat] + counts[flat])).all(), E
        assert row_map.unique().numel() == T * K, E


def test_an_expert_id_outside_the_range_is_skipped_and_reported():
    dev = torch.device("cuda:0")
    static, _, plan = _symbols()
    stream = torch.cuda.current_stream().cuda_stream
    E, T, K, hidden = 8, 16, 1, 64
    x, ids, _ = _case(3, T, K, E, hidden, dev)
    ids[5, 0] = 300  # inside the static array but not an expert of this call
    ids[9, 0] = -2
    valid = (ids.reshape(-1) >= 0) & (ids.reshape(-1) < E)
    counts = torch.bincount(ids.reshape(-1)[valid].long(), minlength=E).to(torch.int32)
    offsets = torch.empty(E + 1, dtype=torch.int32, device=dev)
    tiles = torch.empty(16, dtype=torch.int32, device=dev)
    assert plan(counts.data_ptr(), E, 128, offsets.data_ptr(), tiles.data_ptr(), 16, stream) == 0
    xp = torch.zeros(16 * 128, hidden, dtype=torch.bfloat16, device=dev)
    row_map = torch.empty(T, dtype=torch.int32, device=dev)
    native.last_status()
    assert static(x.data_ptr(), hidden, ids.data_ptr(), offsets.data_ptr(), E, T, K, xp.data_ptr(), row_map.data_ptr(),
                  stream) == 0  # fmt: skip
    torch.cuda.synchronize()
    status = native.last_status()
    assert status & 0xFF == 2 and status >> 8 == 70, status  # TFB_ERR_BAD_SHAPE at the permute's check
    assert row_map[5].item() == -1 and row_map[9].item() == -1
    keep = valid.nonzero().reshape(-1)
    assert torch.equal(xp[row_map[keep].long()], x[keep])
