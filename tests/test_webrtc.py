"""WebRTC transport against stand-ins of `aiortc` / `av` (neither is installed here): pacing and drop policy of
the video track, codec preference and bitrate settings, the offer/answer path with the data channel, and the
mapping of connection states onto the streaming session manager."""

import asyncio
import json
import sys
import types

import numpy as np
import pytest
import torch

from telefuser_b200.service.webrtc import FramePacer, WebRTCSessionManager, frame_to_rgb
from telefuser_b200.service.webrtc.track import make_track


# ---------------------------------------------------------------------------------------------------
# stand-ins
# ---------------------------------------------------------------------------------------------------
class _Emitter:
    def __init__(self):
        self.handlers = {}

    def on(self, event):
        def deco(fn):
            self.handlers[event] = fn
            return fn

        return deco


class FakeChannel(_Emitter):
    def __init__(self):
        super().__init__()
        self.readyState, self.sent = "open", []

    def send(self, data):
        self.sent.append(json.loads(data))


class FakePC(_Emitter):
    def __init__(self):
        super().__init__()
        self.tracks, self.connectionState, self.closed = [], "new", False
        self.transceivers = [types.SimpleNamespace(kind="video", prefs=None), types.SimpleNamespace(kind="audio", prefs=None)]
        for t in self.transceivers:
            t.setCodecPreferences = lambda codecs, t=t: setattr(t, "prefs", codecs)
        self.localDescription = None

    def addTrack(self, track):
        self.tracks.append(track)

    def getTransceivers(self):
        return self.transceivers

    async def setRemoteDescription(self, desc):
        self.remote = desc

    async def createAnswer(self):
        return types.SimpleNamespace(sdp="v=0 answer", type="answer")

    async def setLocalDescription(self, desc):
        self.localDescription = desc

    async def close(self):
        self.closed = True


class FakeVideoFrame:
    def __init__(self, arr):
        self.arr, self.pts, self.time_base = arr, None, None

    @classmethod
    def from_ndarray(cls, arr, format="rgb24"):  # noqa: A002
        assert format == "rgb24" and arr.dtype == np.uint8 and arr.ndim == 3
        return cls(arr)


def fake_modules():
    codec = lambda mime: types.SimpleNamespace(mimeType=mime)  # noqa: E731
    aiortc = types.ModuleType("aiortc")
    aiortc.MediaStreamTrack = type("MediaStreamTrack", (), {"__init__": lambda self: None})
    aiortc.RTCPeerConnection = FakePC
    aiortc.RTCSessionDescription = lambda sdp, type: types.SimpleNamespace(sdp=sdp, type=type)  # noqa: A002
    aiortc.RTCRtpSender = types.SimpleNamespace(getCapabilities=lambda kind: types.SimpleNamespace(
        codecs=[codec("video/VP8"), codec("video/rtx"), codec("video/H264"), codec("video/H264")]))
    av = types.ModuleType("av")
    av.VideoFrame = FakeVideoFrame
    return aiortc, av


class FakeSessions:
    """The part of StreamSessionManager the transport uses."""

    def __init__(self):
        self.events, self.session = [], None

    async def open(self, config):
        self.session = types.SimpleNamespace(session_id=config["session_id"], outbound=asyncio.Queue(), closed=False,
                                             chunks_sent=0, frames_dropped=0)
        return self.session

    def push(self, sid, msg):
        self.events.append(("push", sid, msg))

    def mark_disconnected(self, sid):
        self.events.append(("disconnected", sid))

    def mark_reconnected(self, sid):
        self.events.append(("reconnected", sid))

    async def close(self, sid, reason=""):
        self.events.append(("close", sid, reason))
        self.session.closed = True


# ---------------------------------------------------------------------------------------------------
# pacing
# ---------------------------------------------------------------------------------------------------
def test_pacer_drops_the_oldest_frame_when_the_client_falls_behind():
    p = FramePacer(fps=2, max_buffer_seconds=1.0)  # room for two frames
    p.push_frames([10, 20])
    p.push_frame(30)
    assert list(p.queue) == [20, 30] and p.dropped_frames == 1


def test_pacer_keeps_the_grid_and_holds_the_last_frame_after_the_stream_ends():
    async def run():
        now = [0.0]
        p = FramePacer(fps=100, clock=lambda: now[0])
        p.push_frames(["a", "b"])
        out = [await p.next_frame() for _ in range(2)]
        p.finish()
        now[0] = 1.0  # far behind schedule: no sleeping, frames keep coming
        out += [await p.next_frame() for _ in range(2)]
        return p, out

    p, out = asyncio.run(run())
    assert [o[0] for o in out] == ["a", "b", "b", "b"] and [o[1] for o in out] == [0, 1, 2, 3]
    assert out[0][2].denominator == 100 and p.repeated_frames == 2 and p.stats()["finished"]


def test_pacer_waits_for_the_first_frame():
    async def run():
        p = FramePacer(fps=1000)
        task = asyncio.ensure_future(p.next_frame())
        await asyncio.sleep(0.01)
        assert not task.done()
        p.push_frame("first")
        return (await asyncio.wait_for(task, 1.0))[0]

    assert asyncio.run(run()) == "first"


def test_frames_of_every_kind_become_rgb_arrays():
    chw = torch.full((3, 4, 6), -1.0)
    assert frame_to_rgb(chw).shape == (4, 6, 3) and frame_to_rgb(chw).max() == 0
    assert frame_to_rgb(torch.ones(4, 6, 3)).min() == 255
    u8 = torch.full((4, 6, 3), 7, dtype=torch.uint8)
    assert frame_to_rgb(u8).dtype == np.uint8 and frame_to_rgb(u8)[0, 0, 0] == 7
    assert frame_to_rgb(np.zeros((4, 6), dtype=np.uint8)).shape == (4, 6, 3)
    aiortc, av = fake_modules()
    p = FramePacer(fps=1000)
    track = make_track(p, aiortc, av)
    p.push_frame(chw)
    vf = asyncio.run(track.recv())
    assert isinstance(vf, FakeVideoFrame) and vf.pts == 0 and vf.arr.shape == (4, 6, 3)


# ---------------------------------------------------------------------------------------------------
# manager
# ---------------------------------------------------------------------------------------------------
def test_codec_preference_and_bitrate(monkeypatch):
    h264 = types.ModuleType("aiortc.codecs.h264")
    h264.DEFAULT_BITRATE, h264.MAX_BITRATE = 1_000_000, 3_000_000
    vpx = types.ModuleType("aiortc.codecs.vpx")
    vpx.DEFAULT_BITRATE, vpx.MAX_BITRATE = 500_000, 1_500_000
    monkeypatch.setitem(sys.modules, "aiortc.codecs.h264", h264)
    monkeypatch.setitem(sys.modules, "aiortc.codecs.vpx", vpx)
    mgr = WebRTCSessionManager(FakeSessions(), video_codec="h264", video_bitrate=8_000_000, modules=fake_modules())
    mgr.apply_video_bitrate()
    assert h264.DEFAULT_BITRATE == h264.MAX_BITRATE == vpx.DEFAULT_BITRATE == vpx.MAX_BITRATE == 8_000_000
    pc = FakePC()
    mgr.set_video_codec_preferences(pc)
    video, audio = pc.transceivers
    assert [c.mimeType for c in video.prefs] == ["video/H264", "video/H264", "video/VP8", "video/rtx"]
    assert audio.prefs is None


def test_offer_answer_pump_and_connection_states():
    async def run():
        sessions = FakeSessions()
        service = types.SimpleNamespace(stream_mode="bidirectional")
        mgr = WebRTCSessionManager(sessions, service, fps=500, modules=fake_modules())
        answer = await mgr.answer({"sdp": "v=0 offer", "type": "offer", "session_id": "s1", "config": {"height": 64}})
        assert answer == {"session_id": "s1", "sdp": "v=0 answer", "type": "answer"}
        conn = mgr.connections["s1"]
        pc = conn.pc
        assert len(pc.tracks) == 1 and pc.remote.sdp == "v=0 offer"
        # the browser opens the control channel and sends a key snapshot, rubbish, then asks to close
        ch = FakeChannel()
        pc.handlers["datachannel"](ch)
        ch.handlers["message"](json.dumps({"keys": ["w"]}))
        ch.handlers["message"]("not json")
        # the pipeline produces one chunk of three frames and finishes
        frames = [torch.zeros(3, 8, 8) for _ in range(3)]
        await sessions.session.outbound.put((frames, {"type": "chunk", "index": 0}))
        await sessions.session.outbound.put(([], {"type": "done"}))
        await asyncio.wait_for(conn.pump_task, 2.0)
        got = [await pc.tracks[0].recv() for _ in range(4)]
        await mgr.handle_state(conn, "disconnected")
        await mgr.handle_state(conn, "connected")
        ch.handlers["message"](json.dumps({"type": "close"}))
        await asyncio.sleep(0)
        await mgr.handle_state(conn, "failed")
        return sessions, mgr, ch, got, conn

    sessions, mgr, ch, got, conn = asyncio.run(run())
    assert [m["type"] for m in ch.sent] == ["chunk", "done"] and conn.messages_received == 2
    assert [f.pts for f in got] == [0, 1, 2, 3] and conn.pacer.repeated_frames == 1  # 4th: last frame held
    kinds = [e[0] for e in sessions.events]
    assert kinds == ["push", "disconnected", "reconnected", "close", "close"]
    assert sessions.events[0][2] == {"keys": ["w"]} and sessions.events[-1][2] == "webrtc failed"
    assert "s1" not in mgr.connections and sessions.session.chunks_sent == 2


# ---------------------------------------------------------------------------------------------------
# audio and encoded frames
# ---------------------------------------------------------------------------------------------------
class FakeAudioFrame:
    def __init__(self, arr, fmt, layout):
        self.arr, self.format, self.layout = arr, fmt, layout
        self.sample_rate = self.pts = self.time_base = None

    @classmethod
    def from_ndarray(cls, arr, format="s16", layout="mono"):  # noqa: A002
        assert arr.dtype == np.int16 and arr.ndim == 2 and arr.shape[0] == 1
        return cls(arr, format, layout)


def test_chunk_router_takes_encoded_frames_and_audio_in_every_form():
    import base64
    import io

    from PIL import Image

    from telefuser_b200.service.stream_service import AudioChunk, ChunkRouter, audio_from_chunk

    def jpeg(value):
        buf = io.BytesIO()
        Image.fromarray(np.full((8, 8, 3), value, dtype=np.uint8)).save(buf, format="JPEG")
        return buf.getvalue()

    pics = [jpeg(10), jpeg(200)]
    pcm = (np.arange(960, dtype=np.int16) - 480)
    chunk = {"type": "chunk", "index": 7, "fps": 24, "frames_b64": [base64.b64encode(p).decode() for p in pics],
             "audio_b64": base64.b64encode(pcm.tobytes()).decode(), "audio_sample_rate": 24000, "prompt": "waves"}
    media, msg = ChunkRouter().route(chunk, "s", 7)
    assert media[:2] == pics and isinstance(media[2], AudioChunk) and media[2].pcm16 == pcm.tobytes()
    assert msg["num_frames"] == 2 and msg["audio"] == {"sample_rate": 24000, "channels": 1, "num_samples": 960, "format": "pcm_s16le"}
    assert msg["data"] == {"type": "chunk", "index": 7, "fps": 24, "audio_sample_rate": 24000, "prompt": "waves"}  # no payload twice
    assert frame_to_rgb(pics[1]).shape == (8, 8, 3) and abs(int(frame_to_rgb(pics[1])[0, 0, 0]) - 200) <= 2
    stereo = audio_from_chunk({"audio": torch.tensor([[0.0, 1.0], [-1.0, 0.5]])})
    assert (stereo.channels, stereo.sample_rate, stereo.num_samples) == (2, 48000, 2)
    assert np.frombuffer(stereo.pcm16, dtype=np.int16).tolist() == [0, 32767, -32767, 16384]
    assert audio_from_chunk({"audio": pcm}).pcm16 == pcm.tobytes() and audio_from_chunk({"frames": []}) is None
    _, plain = ChunkRouter().route({"frames": [np.zeros((4, 4, 3), dtype=np.uint8)], "audio": False}, "s", 0)
    assert "audio" not in plain and plain["num_frames"] == 1 and plain["data"] == {"audio": False}  # a flag is not sound


def test_audio_pacer_packets_silence_and_drops():
    from telefuser_b200.service.webrtc import AudioPacer
    from telefuser_b200.service.webrtc.track import make_audio_track

    async def run():
        now = [0.0]
        p = AudioPacer(48000, 1, max_buffer_seconds=0.05, clock=lambda: now[0])
        p.push((np.arange(1500, dtype=np.int16)).tobytes())
        now[0] = 10.0  # behind schedule: no sleeping
        return p, [await p.next_packet() for _ in range(3)]

    p, out = asyncio.run(run())
    first, second, third = (np.frombuffer(o[0], dtype=np.int16) for o in out)
    assert first.tolist() == list(range(960)) and second[:540].tolist() == list(range(960, 1500)) and not second[540:].any()
    assert not third.any() and [o[1] for o in out] == [0, 960, 1920] and out[0][2].denominator == 48000
    assert p.stats()["silent_packets"] == 2 and p.packet_samples == 960
    p.push(bytes(2 * 5000))  # capacity is 0.05 s = 2400 samples
    assert p.stats()["queued_samples"] == 2400 and p.dropped_samples == 2600
    with pytest.raises(ValueError, match="negotiated"):
        p.push(b"\0\0", sample_rate=16000)
    with pytest.raises(ValueError, match="mono or stereo"):
        AudioPacer(48000, 6)
    aiortc, av = fake_modules()
    av.AudioFrame = FakeAudioFrame
    st = AudioPacer(48000, 2, clock=lambda: 10.0)
    st.push(np.arange(2 * 960, dtype=np.int16).tobytes())
    frame = asyncio.run(make_audio_track(st, aiortc, av).recv())
    assert frame.layout == "stereo" and frame.arr.shape == (1, 1920) and frame.sample_rate == 48000 and frame.pts == 0


def test_offer_with_audio_adds_a_second_track_and_feeds_it():
    from telefuser_b200.service.stream_service import AudioChunk

    async def run(want_audio):
        sessions = FakeSessions()
        aiortc, av = fake_modules()
        av.AudioFrame = FakeAudioFrame
        mgr = WebRTCSessionManager(sessions, types.SimpleNamespace(stream_mode="server_push"), fps=500, modules=(aiortc, av))
        body = {"sdp": "v=0 offer", "session_id": "a1", "config": {"audio": {"sample_rate": 24000} if want_audio else False}}
        await mgr.answer(body)
        conn = mgr.connections["a1"]
        pcm = np.ones(480, dtype=np.int16).tobytes()
        media = [torch.zeros(3, 8, 8), AudioChunk(pcm, 24000, 1)]
        await sessions.session.outbound.put((media, {"type": "chunk", "index": 0}))
        await sessions.session.outbound.put(([AudioChunk(pcm, 48000, 1)], {"type": "chunk", "index": 1}))  # not what was negotiated
        await sessions.session.outbound.put(([], {"type": "done"}))
        await asyncio.wait_for(conn.pump_task, 2.0)
        return mgr, conn

    mgr, conn = asyncio.run(run(True))
    assert [t.kind for t in conn.pc.tracks] == ["video", "audio"] and conn.audio_pacer.sample_rate == 24000
    assert conn.audio_pacer.stats()["queued_samples"] == 480 and conn.audio_unsent_chunks == 1 and list(conn.pacer.queue)[0].shape == (3, 8, 8)
    assert mgr.stats()["a1"]["audio"]["queued_samples"] == 480
    mgr, conn = asyncio.run(run(False))
    assert [t.kind for t in conn.pc.tracks] == ["video"] and conn.audio_unsent_chunks == 2 and len(conn.pacer.queue) == 1
