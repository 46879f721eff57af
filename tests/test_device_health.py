"""Peer workspace bookkeeping and the surfacing of expired device waits (host-side logic on CPU; the one
GPU case lets a flag barrier run out of time against a rank that does not exist, which leaves the context usable)."""

import ctypes

import pytest
import torch

from telefuser_b200.core.base_stage import BaseStage
from telefuser_b200.core.config import ModelRuntimeConfig
from telefuser_b200.ops import native
from telefuser_b200.parallel import symm


def _fake_workspace(nbytes: int) -> symm.PeerWorkspace:
    ws = symm.PeerWorkspace.__new__(symm.PeerWorkspace)
    ws.rank, ws.world = 0, 2
    ws.nbytes = nbytes + symm.FLAG_BYTES
    ws.flag_off = nbytes
    ws.local = torch.zeros(ws.nbytes, dtype=torch.uint8)
    ws.ptrs = [1 << 20, 2 << 20]
    ws._regions, ws._cursor = {}, 0
    ws.canaries, ws._canaries = False, {}
    return ws


def test_regions_are_recarved_when_a_name_recurs_with_another_shape():
    ws = _fake_workspace(64 * 1024)
    q = ws.region("ulysses_q", (1, 64, 2, 32))  # 8 KB
    k = ws.region("ulysses_k", (1, 64, 2, 32))
    assert ws.peer_ptr(1, "ulysses_k") - ws.peer_ptr(1, "ulysses_q") == 8192 and k.shape == (1, 64, 2, 32)
    # a smaller request keeps every offset
    q2 = ws.region("ulysses_q", (1, 32, 2, 32))
    assert q2.shape == (1, 32, 2, 32) and q2.data_ptr() == q.data_ptr()
    assert ws.peer_ptr(1, "ulysses_k") - ws.peer_ptr(1, "ulysses_q") == 8192
    # growing back into the bytes reserved at first use is also in place
    assert ws.region("ulysses_q", (1, 64, 2, 32)).data_ptr() == q.data_ptr()
    # a larger request starts the table over; the following names are carved behind it
    q3 = ws.region("ulysses_q", (1, 128, 2, 32))
    k3 = ws.region("ulysses_k", (1, 128, 2, 32))
    assert q3.data_ptr() == q.data_ptr() and ws.peer_ptr(0, "ulysses_k") - ws.peer_ptr(0, "ulysses_q") == 16384
    assert k3.shape == (1, 128, 2, 32)
    with pytest.raises(MemoryError):
        ws.region("too_big", (1 << 20,))


class _FakeLib:
    def __init__(self) -> None:
        self.word, self.host, self.cleared = 0, 0, 0

    def tfb_status_post(self, stream):
        self.host = self.word
        return 0

    def tfb_status_peek(self):
        return self.host

    def tfb_last_status(self):
        v, self.word, self.host = self.word, 0, 0
        self.cleared += 1
        return v


def test_poll_raises_once_the_posted_word_is_non_zero(monkeypatch):
    fake = _FakeLib()
    monkeypatch.setattr(native, "load", lambda: fake)
    monkeypatch.setattr(native, "stream_ptr", lambda: 0)
    native.poll_status()
    native.post_status()
    native.poll_status()  # still clean
    fake.word = 1 | (60 << 8)  # a barrier wait expired on the device
    native.poll_status()  # not posted yet: nothing to see, nothing blocks
    native.post_status()
    with pytest.raises(native.DeviceWaitTimeout, match="site 60"):
        native.poll_status("stage 'dit'")
    native.poll_status()  # cleared by the raise
    fake.word = 1 | (5 << 8)
    with pytest.raises(native.DeviceWaitTimeout, match="site 5"):
        native.finish_status()


class _BarrierStage(BaseStage):
    """A stage whose step waits for a second rank that does not exist."""

    def process(self, steps: int):
        lib = native.load()
        flags = [torch.zeros(64, dtype=torch.int32, device=self.device) for _ in range(2)]
        table = (ctypes.c_void_p * 2)(flags[0].data_ptr(), flags[1].data_ptr())
        for i in range(steps):
            native.check(lib.tfb_peer_barrier(table, 0, 2, 0, i + 1, native.stream_ptr()), "tfb_peer_barrier")
            self.check_device_waits()
        self.check_device_waits(final=True)
        return flags[1][0].item()


@pytest.mark.gpu
def test_a_stage_fails_loudly_when_a_peer_wait_runs_out():
    cfg = ModelRuntimeConfig()
    cfg.parallel_config.device_wait_timeout = 0.2
    stage = _BarrierStage("barrier", cfg)
    stage.configure_device_waits()
    native.last_status()
    try:
        with pytest.raises(native.DeviceWaitTimeout, match="site 60"):
            stage.process(2)
        assert native.last_status() == 0  # the record was consumed by the raise
        assert (torch.ones(4, device="cuda") * 2).sum().item() == 8.0  # the context still answers
    finally:
        native.set_peer_wait_ms(4000)


def test_canary_strips_behind_peer_regions():
    ws = _fake_workspace(64 * 1024)
    ws.canaries = True
    a = ws.region("slab_a", (100,), torch.uint8)  # 100 bytes -> strip starts at the next 256-byte boundary
    b = ws.region("slab_b", (1, 64, 2, 32))
    assert ws.peer_ptr(0, "slab_b") - ws.peer_ptr(0, "slab_a") == 256 + symm.CANARY_BYTES
    a.fill_(1)
    b.fill_(1.0)
    ws.check_canaries()  # writes inside the regions leave the strips alone
    ws.local[256 + 5] = 0  # what a store past the end of slab_a would do
    with pytest.raises(AssertionError, match="slab_a.*first at \\+5"):
        ws.check_canaries()
