"""WebRTC transport of streaming sessions: paced media track, per-connection session manager, signalling.

`aiortc` and `av` are optional; they are looked up through `backend()` when a connection is made, so the package
imports (and its pacing / routing / bookkeeping logic is testable) without them.
Role parity: telefuser/service/webrtc/{track,session_manager,chunk_router}.py and api/routers/webrtc.py.
"""

from .session_manager import WebRTCSessionManager, answer_offer, backend
from .track import AudioPacer, FramePacer, frame_to_rgb

__all__ = ["AudioPacer", "FramePacer", "WebRTCSessionManager", "answer_offer", "backend", "frame_to_rgb"]
