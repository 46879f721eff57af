"""Peer-mapped workspaces and the fused compute + exchange paths built on them (one node, NVLink).

`PeerWorkspace(group, nbytes)`: every rank of `group` allocates `nbytes` of device memory, the CUDA
IPC handles are exchanged through the process group, and each rank maps all the others. Regions of
the workspace are carved by name (`region(name, shape, dtype)`): the same call sequence on every rank
gives the same offsets, so `peer_ptr(rank, name)` is the address of rank `rank`'s copy.

Exchanges are done by the kernels that produce or consume the data:
* `ulysses_attention_fused`: q/k/v go from the sequence-sharded projection output straight into the
  head-sharded slabs of every peer (one pass, no pack/unpack, no all-to-all), attention's epilogue
  stores each output row into the buffer of the rank that owns the token (no second all-to-all).
  Two flag barriers per layer order the slab reuse.
* `cfg_combine_step_fused`: each guidance rank publishes its prediction; the combine + Euler-step
  kernel reads the partner's prediction with peer loads (no all-gather).
* `all_gather_rows_fused`: a rank's token rows are pushed into every peer's full buffer.
The NCCL paths in `ulysses.py` / `shard.py` remain the oracle and the fallback.
"""

from __future__ import annotations

import ctypes
import math
import os

import torch
import torch.distributed as dist

from telefuser_b200.ops import native

FLAG_BYTES = 4096
CANARY_BYTES = 256
CANARY_PATTERN = 0x5A


class _DevMem:
    """Exposes a raw device pointer to torch through the CUDA array interface."""

    def __init__(self, ptr: int, nbytes: int) -> None:
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class PeerWorkspace:
    def __init__(self, group, nbytes: int, device=None) -> None:
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        if self.world > 8:
            raise ValueError("peer workspaces span at most 8 ranks (one node)")
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.nbytes = int(-(-nbytes // 256) * 256) + FLAG_BYTES
        lib = native.load()
        lib.tfb_ipc_alloc.argtypes = [ctypes.c_long, ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p]
        lib.tfb_ipc_open.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p)]
        lib.tfb_ipc_close.argtypes = [ctypes.c_void_p]
        lib.tfb_ipc_free.argtypes = [ctypes.c_void_p]
        ptr = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(64)
        with torch.cuda.device(self.device):
            native.check(lib.tfb_ipc_alloc(self.nbytes, ctypes.byref(ptr), handle), "tfb_ipc_alloc")
            handles: list = [None] * self.world
            dist.all_gather_object(handles, bytes(handle.raw), group=group)
            self.ptrs: list[int] = []
            for r, h in enumerate(handles):
                if r == self.rank:
                    self.ptrs.append(ptr.value)
                    continue
                p = ctypes.c_void_p()
                native.check(lib.tfb_ipc_open(ctypes.create_string_buffer(h, 64), ctypes.byref(p)), "tfb_ipc_open")
                self.ptrs.append(p.value)
        self._lib = lib
        self.local = torch.as_tensor(_DevMem(ptr.value, self.nbytes), device=self.device)
        self.flag_off = self.nbytes - FLAG_BYTES
        self._flag_table = (ctypes.c_void_p * self.world)(*[p + self.flag_off for p in self.ptrs])
        self._epoch = 0
        self._regions: dict[str, tuple[int, tuple, torch.dtype, int]] = {}  # offset, shape, dtype, reserved bytes
        self._cursor = 0
        self.canaries = os.environ.get("TFB_PEER_CANARY") == "1"
        self._canaries: dict[str, tuple[int, int]] = {}
        dist.barrier(group=group)  # every mapping exists before anyone stores

    # ---- regions ------------------------------------------------------------------
    def region(self, name: str, shape, dtype=torch.bfloat16) -> torch.Tensor:
        """This rank's view of a named region (carved on first use; same call order on every rank).

        A name that recurs with another shape or dtype (a request at another resolution, frame count or batch)
        keeps its place when the new extent fits the bytes reserved for it. Otherwise the whole table is carved
        anew from offset 0: every earlier view of this workspace is then invalid, which is safe because the
        callers' barriers order each reuse and a shape only changes between requests."""
        shape = tuple(int(s) for s in shape)
        n = math.prod(shape) * torch.empty((), dtype=dtype).element_size()
        hit = self._regions.get(name)
        if hit is not None and (hit[1] != shape or hit[2] != dtype):
            if n <= hit[3]:
                hit = self._regions[name] = (hit[0], shape, dtype, hit[3])
            else:
                self._regions.clear()
                self._canaries.clear()
                self._cursor = 0
                hit = None
        if hit is None:
            off = self._cursor
            gap = CANARY_BYTES if self.canaries else 0
            if off + n + gap > self.flag_off:
                raise MemoryError(f"peer workspace of {self.flag_off} bytes cannot hold region {name!r} ({n} bytes)")
            end = -(-(off + n) // 256) * 256
            if gap:  # a strip of a known pattern behind the region: peers that store past their slab land here
                self.local[end : end + gap].fill_(CANARY_PATTERN)
                self._canaries[name] = (end, gap)
            self._cursor = end + gap
            hit = self._regions[name] = (off, shape, dtype, end - off)
        off = hit[0]
        return self.local[off : off + n].view(dtype).view(shape)

    def check_canaries(self) -> None:
        """With `TFB_PEER_CANARY=1` every region is followed by a strip of a fixed byte pattern; raises when a
        peer (or this rank) stored past the end of a region. Synchronises the device: for tests and debugging."""
        for name, (off, n) in getattr(self, "_canaries", {}).items():
            strip = self.local[off : off + n]
            bad = (strip != CANARY_PATTERN).nonzero()
            if bad.numel():
                raise AssertionError(f"peer region {name!r}: {bad.numel()} bytes behind its end were overwritten "
                                     f"(first at +{int(bad[0])})")  # fmt: skip

    def peer_ptr(self, rank: int, name: str) -> int:
        return self.ptrs[rank] + self._regions[name][0]

    def peer_table(self, name: str):
        return (ctypes.c_void_p * self.world)(*[self.peer_ptr(r, name) for r in range(self.world)])

    # ---- synchronisation --------------------------------------------------------------
    def barrier(self, slot: int = 0) -> None:
        """Stream-ordered all-rank barrier (a one-warp kernel; bounded wait)."""
        self._epoch += 1
        code = self._lib.tfb_peer_barrier(self._flag_table, self.rank, self.world, slot, self._epoch, native.stream_ptr())
        native.check(code, "tfb_peer_barrier")

    def close(self) -> None:
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        for r, p in enumerate(self.ptrs):
            if r != self.rank:
                self._lib.tfb_ipc_close(ctypes.c_void_p(p))
        self._lib.tfb_ipc_free(ctypes.c_void_p(self.ptrs[self.rank]))
        self.ptrs = []


_WORKSPACES: dict = {}


_RESERVED: dict = {}


def reserve_workspace(group, nbytes: int, tag: str = "") -> None:
    """Declares the largest request a session will make (e.g. the full rolling window of a streaming session), so
    that the workspace is created once at that size instead of being re-created as requests grow."""
    key = (id(group), tag)
    _RESERVED[key] = max(int(nbytes), _RESERVED.get(key, 0))


def get_workspace(group, nbytes: int, tag: str = "") -> PeerWorkspace:
    """One workspace per (process group, tag). It is created at the larger of the request, the reserved size and
    `TFB_PEER_WORKSPACE_MB`; a later, larger request re-creates it with a quarter of headroom (a collective
    operation: free, allocate, exchange handles), smaller or differently shaped requests re-carve it in place.
    Callers whose regions must not compete for space (attention slabs, tensor-parallel slabs, the output gather)
    use own tags."""
    import os

    key = (id(group), tag)
    ws = _WORKSPACES.get(key)
    if ws is None or ws.flag_off < nbytes:
        want = max(int(nbytes), _RESERVED.get(key, 0), int(os.environ.get("TFB_PEER_WORKSPACE_MB", "0")) << 20)
        if ws is not None:
            ws.close()
            want = max(want, int(nbytes * 1.25))
        ws = _WORKSPACES[key] = PeerWorkspace(group, want)
    return ws


def release_workspaces() -> None:
    for ws in list(_WORKSPACES.values()):
        ws.close()
    _WORKSPACES.clear()


# ---------------------------------------------------------------------------
# fused paths
# ---------------------------------------------------------------------------
def ulysses_attention_fused(q, k, v, ws: PeerWorkspace, scale: float | None = None) -> torch.Tensor:
    """q, k, v: [B, S_loc, H, 128] bf16 (may be column slices of one fused buffer) -> [B, S_loc, H, 128].

    Equivalent to scatter_heads x3 -> attention -> gather_heads over `ws.group`."""
    B, S, H, D = q.shape
    P, r = ws.world, ws.rank
    if D != 128 or q.dtype != torch.bfloat16 or H % P:
        raise ValueError("fused Ulysses attention needs bf16, head_dim 128 and heads divisible by the group size")
    Hp, St = H // P, S * P
    slabs = [ws.region(f"ulysses_{n}", (B, St, Hp, D)) for n in ("q", "k", "v")]
    out = ws.region("ulysses_o", (B, S, H, D))
    lib = native.load()
    st = native.stream_ptr()

    def strides(t):
        if t.stride(-1) != 1 or t.stride(2) != D:
            t = t.contiguous()
        return t, t.stride(1), (t.stride(0) if B > 1 else S * t.stride(1))

    (q, ldq, bsq), (k, ldk, bsk), (v, ldv, bsv) = strides(q), strides(k), strides(v)
    srcs = (ctypes.c_void_p * 3)(q.data_ptr(), k.data_ptr(), v.data_ptr())
    lds = (ctypes.c_long * 3)(ldq, ldk, ldv)
    bss = (ctypes.c_long * 3)(bsq, bsk, bsv)
    dsts = (ctypes.c_void_p * (3 * P))(*[ws.peer_ptr(rr, f"ulysses_{n}") for n in ("q", "k", "v") for rr in range(P)])
    native.check(lib.tfb_ulysses_scatter(srcs, lds, bss, dsts, 3, B, S, H, D, P, r, st), "tfb_ulysses_scatter")
    ws.barrier()  # every peer's slice of q/k/v has landed in my slabs
    sq, sk, sv = slabs
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    code = lib.tfb_attn_fwd_peer(sq.data_ptr(), Hp * D, St * Hp * D, sk.data_ptr(), Hp * D, St * Hp * D, sv.data_ptr(),
                                 Hp * D, St * Hp * D, ws.peer_table("ulysses_o"), P, S, r * Hp, H * D, S * H * D, B, Hp,
                                 St, St, scale, 0, st)  # fmt: skip
    native.check(code, "tfb_attn_fwd_peer")
    ws.barrier()  # every peer has stored its heads of my tokens; slabs may be overwritten again
    return out


def cfg_combine_step_fused(latents, pred, ws: PeerWorkspace, cfg_scale: float, dsigma: float) -> torch.Tensor:
    """CFG-parallel pair: rank 0 holds the conditional prediction, rank 1 the unconditional one.
    Returns the updated latents (identical on both ranks)."""
    if ws.world != 2:
        raise ValueError("CFG combine runs on a group of two")
    buf = ws.region("cfg_pred", pred.shape, pred.dtype)
    buf.copy_(pred)
    ws.barrier()
    x = latents.float().contiguous()
    out = torch.empty_like(x)
    code = native.load().tfb_cfg_euler_step(x.data_ptr(), ws.peer_ptr(0, "cfg_pred"), ws.peer_ptr(1, "cfg_pred"),
                                            int(pred.dtype == torch.bfloat16), float(cfg_scale), float(dsigma),
                                            out.data_ptr(), None, x.numel(), native.stream_ptr())  # fmt: skip
    native.check(code, "tfb_cfg_euler_step")
    ws.barrier()  # the partner has read my prediction; the region may be reused
    return out


def all_gather_rows_fused(x_local: torch.Tensor, ws: PeerWorkspace, name: str = "gather") -> torch.Tensor:
    """x_local: [rows, C] (same shape on every rank) -> [rows * P, C], rank-major, by peer stores."""
    rows, C = x_local.shape
    full = ws.region(name, (rows * ws.world, C), x_local.dtype)
    xc = x_local.contiguous()
    rb = C * xc.element_size()
    ws.barrier()  # nobody still reads the previous contents of this region
    code = native.load().tfb_peer_push_rows(xc.data_ptr(), rb, ws.peer_table(name), ws.world, ws.rank * rows, rows, rb,
                                            rb, native.stream_ptr())  # fmt: skip
    native.check(code, "tfb_peer_push_rows")
    ws.barrier()
    return full


_SIDE_STREAMS: dict = {}


def _side_stream(device) -> "torch.cuda.Stream":
    key = str(device)
    if key not in _SIDE_STREAMS:
        _SIDE_STREAMS[key] = torch.cuda.Stream(device=device)
    return _SIDE_STREAMS[key]


def ring_workspace_bytes(S_local: int, H: int, D: int, world: int, itemsize: int = 2) -> int:
    return 2 * (world * S_local * H * D * itemsize + 256) + 4096


def ring_attention_fused(q, k, v, ws: PeerWorkspace, scale: float | None = None, return_lse: bool = False):
    """Context-parallel attention over `ws.group` with the K / V exchange done by peer stores.

    q, k, v: [1, S_local, H, 128] bf16 shards of one sequence. On a side stream one kernel pushes this rank's K and
    V rows into every peer's gather buffer (each shard crosses NVLink once and is then read from local memory),
    bracketed by flag barriers; meanwhile the main stream attends to the local shard. The remote shards form at
    most two contiguous runs in rank order; each is attended with one kernel launch and merged by log-sum-exp.
    All ranks hold all keys afterwards, so there are no ring steps: on an NVSwitch fabric every peer is one hop.
    """
    from telefuser_b200.ops import functional as TF

    B, S, H, D = q.shape
    if B != 1 or k.shape != v.shape or k.shape[0] != 1:
        raise ValueError("ring_attention_fused takes one sequence per call (batch 1)")
    P, rank, C = ws.world, ws.rank, H * D
    Sk = k.shape[1]
    kbuf = ws.region("ring_k", (P * Sk, C), k.dtype)
    vbuf = ws.region("ring_v", (P * Sk, C), v.dtype)
    lib, rb = native.load(), C * k.element_size()

    def rows(t):
        t2 = t.reshape(Sk, C) if t.is_contiguous() else t[0].reshape(Sk, C)
        if t2.stride(1) != 1 or (t2.stride(0) * t2.element_size()) % 16:
            t2 = t2.contiguous()
        return t2, t2.stride(0) * t2.element_size()

    (k2, ldk), (v2, ldv) = rows(k), rows(v)
    main, side = torch.cuda.current_stream(q.device), _side_stream(q.device)
    side.wait_stream(main)  # K / V are produced on the main stream; its earlier reads of the buffers are done too
    with torch.cuda.stream(side):
        ws.barrier(1)  # every rank is past its reads of the previous contents
        for src, ld, name in ((k2, ldk, "ring_k"), (v2, ldv, "ring_v")):
            code = lib.tfb_peer_push_rows(src.data_ptr(), ld, ws.peer_table(name), P, rank * Sk, Sk, rb, rb, native.stream_ptr())
            native.check(code, "tfb_peer_push_rows")
        ws.barrier(1)  # every shard has landed everywhere
    k2.record_stream(side)
    v2.record_stream(side)
    o, lse = TF.attention(q, k, v, scale, return_lse=True)  # local shard, overlaps the exchange
    main.wait_stream(side)
    o, lse = attend_remote_runs(q, o, lse, kbuf, vbuf, rank, P, Sk, scale)
    return (o, lse) if return_lse else o


def attend_remote_runs(q, o, lse, kbuf, vbuf, rank: int, P: int, Sk: int, scale=None):
    """Merges into (o, lse) the attention of `q` over the other ranks' shards held rank-major in kbuf / vbuf [P * Sk, H * D]:
    the rows before and after this rank's own shard are two contiguous runs, one kernel launch each."""
    from telefuser_b200.ops import functional as TF

    H, D = q.shape[2], q.shape[3]
    for lo, hi in ((0, rank), (rank + 1, P)):
        if hi > lo:
            kk = kbuf[lo * Sk : hi * Sk].view(1, (hi - lo) * Sk, H, D)
            vv = vbuf[lo * Sk : hi * Sk].view(1, (hi - lo) * Sk, H, D)
            o2, lse2 = TF.attention(q, kk, vv, scale, return_lse=True)
            o, lse = TF.merge_attn_states(o, lse, o2, lse2)
    return o, lse
