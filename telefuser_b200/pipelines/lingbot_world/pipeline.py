"""LingBot-World-Fast pipeline and its streaming runtime.

`LingBotWorldFastPipeline` owns three stages (condition encode, chunk denoise, chunk decode)
and one `LingBotWorldFastStreamingRuntime`: a `StreamingPipelineOrchestrator` graph

    encode_request -> [encode] -> condition -+
                                   control  -+-> [denoise] -> latent -> [decode] -> frames

with edge capacity 2, so encode(k+1), denoise(k) and decode(k-1) overlap. Stages that are plain
objects run behind `LocalStageActor`s (tensors stay on the device), stages wrapped in a
`ParallelWorker` behind `ParallelWorkerStageActor`s. Role parity:
telefuser/pipelines/lingbot_world_fast/pipeline.py:66-620, streaming.py:52-419, session.py.
"""

from __future__ import annotations

import itertools
import threading
import time
from dataclasses import dataclass, field
from typing import Callable

import torch

from telefuser_b200.core.base_pipeline import BasePipeline
from telefuser_b200.core.config import ModelRuntimeConfig
from telefuser_b200.orchestrator import (LocalStageActor, StreamingEdgeSpec, StreamingPipelineOrchestrator,
                                         StreamingPipelineSpec, StreamingSessionStatus, StreamingStageSpec)  # fmt: skip
from telefuser_b200.orchestrator.worker_actor import ParallelWorkerStageActor
from telefuser_b200.utils.logging import logger
from telefuser_b200.worker.parallel_worker import ParallelWorker

from .control import (LingBotWorldFastControlBuilder, LingBotWorldFastControlContext, LingBotWorldFastOfflineControlSource,
                      load_action_control_inputs, load_camera_control_inputs, pinhole_intrinsics, random_walk_trajectory,
                      truncate_control_sequence)  # fmt: skip
from .session import LingBotWorldFastSessionConfig, resolve_lingbot_frame_count
from .stages import LingBotWorldFastDenoisingStage, LingBotWorldFastVAEDecodeStage, LingBotWorldFastVAEEncodeStage


@dataclass
class LingBotWorldFastPipelineConfig:
    dit_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    vae_encode_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    vae_decode_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    text_encoding_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    chunk_size: int = 4  # latent frames per chunk
    local_attn_size: int = 18  # latent frames attended to (-1: unbounded)
    sink_size: int = 6
    timestep_indices: tuple = (0, 250, 500, 750)
    sample_shift: float = 10.0
    max_sequence_length: int = 512
    fps: int = 16
    control_type: str = "cam"
    enable_denoising_parallel: bool = False
    edge_capacity: int = 2
    # the output resolution of a session keeps the reference image's aspect ratio at (about) this many pixels;
    # orig_height / orig_width: the image size that recorded intrinsics files refer to unless the caller says otherwise
    max_area: int = 480 * 832
    orig_height: int = 480
    orig_width: int = 832
    # > 0: keep the chunk latents of generated worlds (on the host, least recently used first out) so that a session
    # of the same image / prompt / seed replays matching chunks with one forward pass each instead of denoising them
    world_cache_bytes: int = 0


@dataclass
class LingBotWorldFastGenerationSession:
    cache_handle: int
    prompt_emb: torch.Tensor
    chunk_count: int
    chunk_size: int
    height: int
    width: int
    latent_h: int
    latent_w: int
    frame_tokens: int
    kv_size: int
    max_attention_size: int
    control_builder: LingBotWorldFastControlBuilder
    created_at: float = field(default_factory=time.monotonic)
    world: object | None = None  # WorldKVBinding when the session reads / feeds the world cache
    control_digests: dict = field(default_factory=dict)


@dataclass(frozen=True)
class LingBotWorldFastStreamingSession:
    session_id: str
    session_epoch: int
    cache_handle: int


def _call(stage, name: str, *args):
    """Calls a stage method, in process or through a ParallelWorker."""
    if isinstance(stage, ParallelWorker):
        return stage.call(name, *args)
    return getattr(stage, name)(*args)


class LingBotWorldFastStreamingRuntime:
    def __init__(self, pipeline: "LingBotWorldFastPipeline") -> None:
        self.pipeline = pipeline
        self._lock = threading.RLock()
        self._sessions: dict[str, tuple[LingBotWorldFastGenerationSession, int]] = {}
        self._closed = False
        cap = pipeline.config.edge_capacity
        actors = {
            "encode": self._actor("encode", pipeline.vae_encode_stage, "encode_condition_chunk", self._encode_inputs,
                                  lambda r, inv: {"condition": r}, self._release("vae_encode_stage")),  # fmt: skip
            "denoise": self._actor("denoise", pipeline.denoise_stage, "denoise_and_update_cache", self._denoise_inputs,
                                   self._denoise_outputs, self._release("denoise_stage")),  # fmt: skip
            "decode": self._actor("decode", pipeline.vae_decode_stage, "decode_chunk", self._decode_inputs,
                                  lambda r, inv: {"frames": r}, self._release("vae_decode_stage")),  # fmt: skip
        }
        spec = StreamingPipelineSpec(
            stages=(StreamingStageSpec("encode", {"encode_request"}, {"condition"}),
                    StreamingStageSpec("denoise", {"condition", "control"}, {"latent"}),
                    StreamingStageSpec("decode", {"latent"}, {"frames"})),
            edges=(StreamingEdgeSpec("encode_request", "encode", None, cap),
                   StreamingEdgeSpec("condition", "denoise", "encode", cap),
                   StreamingEdgeSpec("control", "denoise", None, cap),
                   StreamingEdgeSpec("latent", "decode", "denoise", cap)),
            output_artifacts=frozenset({"frames"}), output_capacity_per_session=cap)  # fmt: skip
        self.orchestrator = StreamingPipelineOrchestrator(spec, actors)

    # ---- actor construction ---------------------------------------------------------
    def _actor(self, stage_id, stage, method, input_builder, output_builder, session_closer):
        if isinstance(stage, ParallelWorker):
            return ParallelWorkerStageActor(stage, method, input_builder, output_builder, close_worker=False,
                                            session_closer=session_closer)  # fmt: skip

        def handler(inv):
            args, kwargs = input_builder(inv)
            return output_builder(getattr(stage, method)(*args, **kwargs), inv)

        return LocalStageActor(stage_id, handler, 1, session_closer)

    def _release(self, stage_attr: str):
        def closer(ctx, reason):
            entry = self._sessions.get(ctx.session_id)
            if entry is not None and entry[1] == ctx.session_epoch:
                _call(getattr(self.pipeline, stage_attr), "release_cache", entry[0].cache_handle)

        return closer

    def _entry(self, session_id: str) -> LingBotWorldFastGenerationSession:
        return self._sessions[session_id][0]

    def _encode_inputs(self, inv):
        rt = self._entry(inv.key.session_id)
        return (rt.cache_handle, inv.key.sequence_id, rt.chunk_count, rt.chunk_size, rt.height, rt.width), {}

    def _denoise_inputs(self, inv):
        rt = self._entry(inv.key.session_id)
        control = inv.inputs["control"]
        if callable(control):
            control = control()
        start = inv.key.sequence_id * rt.chunk_size * rt.frame_tokens
        kwargs = {}
        if rt.world is not None:
            from telefuser_b200.cache.world_kv import tensor_digest

            digest = rt.control_digests[inv.key.sequence_id] = tensor_digest(control)
            cached = rt.world.lookup(inv.key.sequence_id, digest)
            if cached is not None:
                kwargs["cached_latent"] = cached
        return (rt.cache_handle, inv.inputs["condition"], rt.prompt_emb, control, start, rt.max_attention_size), kwargs

    def _denoise_outputs(self, latent, inv):
        rt = self._entry(inv.key.session_id)
        if rt.world is not None:
            try:
                rt.world.finalize(inv.key.sequence_id, rt.control_digests.pop(inv.key.sequence_id), latent)
            except Exception as exc:  # noqa: BLE001 - the cache is best effort; the session goes on
                logger.warning(f"world cache: chunk {inv.key.sequence_id} was not recorded: {exc}")
        return {"latent": latent}

    def _decode_inputs(self, inv):
        rt = self._entry(inv.key.session_id)
        return (rt.cache_handle, inv.inputs["latent"]), {}

    # ---- session API ---------------------------------------------------------------------
    def create_session(self, runtime: LingBotWorldFastGenerationSession) -> LingBotWorldFastStreamingSession:
        sid = f"lingbot-{runtime.cache_handle}"
        with self._lock:
            if self._closed:
                raise RuntimeError("LingBot streaming runtime is closed")
            if sid in self._sessions:
                raise ValueError(f"LingBot streaming session {sid!r} already exists")
            epoch = self.orchestrator.create_session(sid, final_sequence_id=runtime.chunk_count - 1)
            self._sessions[sid] = (runtime, epoch)
        return LingBotWorldFastStreamingSession(sid, epoch, runtime.cache_handle)

    def can_submit_chunk(self, session) -> bool:
        try:
            if self.orchestrator.status(session.session_id) != StreamingSessionStatus.RUNNING:
                return False
            return self.orchestrator.can_push_inputs(session.session_id, ("encode_request", "control"))
        except RuntimeError:
            return False

    def try_submit_chunk(self, session, chunk_index: int, control) -> bool:
        return self.orchestrator.try_push_inputs(session.session_id, chunk_index,
                                                 {"encode_request": chunk_index, "control": control})  # fmt: skip

    def poll_frames(self, session) -> list:
        """[(chunk_index, frames)] in order."""
        return [(seq, v) for seq, _, v in self.orchestrator.poll_outputs(session.session_id)]

    def status(self, session) -> StreamingSessionStatus:
        return self.orchestrator.status(session.session_id)

    def error(self, session):
        return self.orchestrator.error(session.session_id)

    def metrics(self, session) -> dict:
        m = self.orchestrator.session_metrics(session.session_id)
        idle = {s: [i.idle_seconds for i in self.orchestrator.stage_idle_intervals(session.session_id, s)]
                for s in ("encode", "denoise", "decode")}  # fmt: skip
        busy = {}
        for s in ("encode", "denoise", "decode"):
            t = self.orchestrator.stage_timings(session.session_id, s)
            busy[s] = [x.completed_at - x.admitted_at for x in t if x.completed_at and x.admitted_at]
        return {"first_output_latency_s": m.first_output_latency_seconds,
                "chunk_period_p50_s": m.chunk_period.p50_seconds, "chunk_period_p95_s": m.chunk_period.p95_seconds,
                "control_to_output_p50_s": m.control_to_output_latency.p50_seconds, "chunks": len(m.output_emitted_at),
                "stage_busy_s": busy, "stage_idle_s": idle, **self._world_metrics(session)}  # fmt: skip

    def _world_metrics(self, session) -> dict:
        entry = self._sessions.get(session.session_id)
        world = entry[0].world if entry is not None else None
        return {} if world is None else {"world_cache_hits": world.hits, "world_cache_misses": world.misses}

    def close_session(self, session, cancel: bool = False) -> None:
        try:
            (self.orchestrator.cancel_session if cancel else self.orchestrator.close_session)(session.session_id, 30.0)
        finally:
            with self._lock:
                self._sessions.pop(session.session_id, None)

    def close(self) -> None:
        with self._lock:
            if self._closed:
                return
            self._closed = True
        self.orchestrator.close()


class LingBotWorldFastPipeline(BasePipeline):
    def __init__(self, device="cuda", torch_dtype=torch.bfloat16) -> None:
        super().__init__(device=device, torch_dtype=torch_dtype)
        self._handles = itertools.count(1)
        self.runtime: LingBotWorldFastStreamingRuntime | None = None

    def _get_stages(self) -> list:
        return [self.vae_encode_stage, self.denoise_stage, self.vae_decode_stage]

    def init(self, module_manager, config: LingBotWorldFastPipelineConfig, text_stage=None):
        self.config = config
        self._model_info = module_manager.get_model_info()
        self.vae_encode_stage = LingBotWorldFastVAEEncodeStage("vae_encode", module_manager, config.vae_encode_config)
        self.vae_decode_stage = LingBotWorldFastVAEDecodeStage("vae_decode", module_manager, config.vae_decode_config)
        self.denoise_stage = LingBotWorldFastDenoisingStage("denoise", module_manager, config.dit_config)
        self.dit_meta = dict(patch=self.denoise_stage.dit.patch_size, control_type=self.denoise_stage.dit.control_type)
        enc, dec = self.vae_encode_stage, self.vae_decode_stage
        if enc.device.type == "cuda" and dec.vae is enc.vae and dec.device != enc.device:
            # The two VAE actors may sit on different GPUs (decode next to the last denoiser rank): the module they
            # fetched is one object, so the decoder gets its own copy on its own device (a few hundred MB).
            import copy

            dec.vae = copy.deepcopy(enc.vae).to(dec.device)
        if enc.device.type == "cuda" and next(enc.vae.parameters()).device != enc.device:
            enc.vae.to(enc.device)
        for st in (self.vae_encode_stage, self.vae_decode_stage, self.denoise_stage):
            st.onload_models_flag = True
        if config.enable_denoising_parallel:
            self.denoise_stage = ParallelWorker(self.denoise_stage)
        self.text_encoding_stage = text_stage
        if text_stage is None and module_manager.fetch_module("wan_video_text_encoder") is not None:
            from telefuser_b200.pipelines.wan.stages import TextEncodingStage

            self.text_encoding_stage = TextEncodingStage("text_encoding", module_manager, config.text_encoding_config,
                                                         config.max_sequence_length)  # fmt: skip
        self.world_store = None
        if config.world_cache_bytes > 0:
            from telefuser_b200.cache.world_kv import WorldKVStore

            self.world_store = WorldKVStore(config.world_cache_bytes)
        self.runtime = LingBotWorldFastStreamingRuntime(self)

    # ---- sessions -------------------------------------------------------------------------
    def _create_initialized_session(self, prompt, image, num_frames: int, height: int, width: int, seed: int = 0,
                                    prompt_emb: torch.Tensor | None = None, world_cache: bool | str = True) -> LingBotWorldFastGenerationSession:  # fmt: skip
        """`world_cache`: True reads and feeds the pipeline's world store (when it has one), "read" / "write" only one
        side, False neither."""
        cfg = self.config
        if (num_frames - 1) % 4:
            raise ValueError(f"num_frames must be 4n+1, got {num_frames}")
        latent_frames = (num_frames - 1) // 4 + 1
        if latent_frames % cfg.chunk_size:
            raise ValueError(f"{latent_frames} latent frames are not a multiple of chunk size {cfg.chunk_size}")
        latent_h, latent_w = height // 8, width // 8
        patch = self.dit_meta["patch"]
        frame_tokens = (latent_h // patch[1]) * (latent_w // patch[2])
        window = cfg.local_attn_size if cfg.local_attn_size != -1 else latent_frames
        kv_size = frame_tokens * window
        if prompt_emb is None:
            prompt_emb = self.text_encoding_stage.process([prompt])[0]
        if isinstance(image, torch.Tensor):
            cond = image
            if tuple(cond.shape[-2:]) != (height, width):  # a tensor image of another size: resample as a PIL image would be
                cond = torch.nn.functional.interpolate(cond.reshape(1, *cond.shape[-3:]).float(), size=(height, width),
                                                       mode="bilinear", antialias=True, align_corners=False)[0].to(image.dtype)  # fmt: skip
        else:
            cond = self.preprocess_image(image, height, width)[0]
        handle = next(self._handles)
        noise_shape = (1, 16, cfg.chunk_size, latent_h, latent_w)
        _call(self.vae_encode_stage, "initialize_cache", handle, cond)
        _call(self.vae_decode_stage, "initialize_cache", handle)
        _call(self.denoise_stage, "initialize_cache", handle, 1, kv_size, cfg.max_sequence_length, cfg.sample_shift,
              seed, seed + 1, noise_shape, tuple(cfg.timestep_indices), frame_tokens)  # fmt: skip
        ctx = LingBotWorldFastControlContext(
            control_type=self.dit_meta["control_type"], device=self.device, control_dtype=self.torch_dtype,
            orig_height=height, orig_width=width, height=height, width=width, latent_h=latent_h, latent_w=latent_w,
            latent_frames=latent_frames, chunk_size=cfg.chunk_size, intrinsics=pinhole_intrinsics(height, width))  # fmt: skip
        world = None
        if self.world_store is not None and world_cache:
            from telefuser_b200.cache.world_kv import WorldKVBinding, world_key

            key = world_key(cond, prompt_emb, seed, height=height, width=width, chunk=cfg.chunk_size, window=cfg.local_attn_size,
                            sink=cfg.sink_size, steps=tuple(cfg.timestep_indices), shift=cfg.sample_shift, dtype=str(self.torch_dtype))  # fmt: skip
            world = WorldKVBinding(self.world_store, key, read=world_cache in (True, "read"), write=world_cache in (True, "write"))
        return LingBotWorldFastGenerationSession(
            cache_handle=handle, prompt_emb=prompt_emb, chunk_count=latent_frames // cfg.chunk_size,
            chunk_size=cfg.chunk_size, height=height, width=width, latent_h=latent_h, latent_w=latent_w,
            frame_tokens=frame_tokens, kv_size=kv_size, max_attention_size=kv_size,
            control_builder=LingBotWorldFastControlBuilder(ctx), world=world)  # fmt: skip

    def release_session(self, session: LingBotWorldFastStreamingSession, cancel: bool = False) -> None:
        self.runtime.close_session(session, cancel)

    # ---- session records, output geometry, recorded trajectories ----------------------------------
    @staticmethod
    def best_output_size(width: int, height: int, expected_area: int, dw: int = 16, dh: int = 16) -> tuple[int, int]:
        """(width, height) of about `expected_area` pixels with the aspect ratio of a width x height image, each side
        rounded DOWN to its own multiple (16 by default: stride-8 VAE x patch 2)."""
        import math

        aspect = height / width
        return int(math.sqrt(expected_area / aspect) // dw * dw), int(math.sqrt(expected_area * aspect) // dh * dh)

    @staticmethod
    def _image_size(image) -> tuple[int, int]:
        if isinstance(image, torch.Tensor):
            return int(image.shape[-1]), int(image.shape[-2])
        return int(image.width), int(image.height)

    def control_context(self, session_config: LingBotWorldFastSessionConfig) -> LingBotWorldFastControlContext:
        """Geometry of a session's control tensors, worked out from the record alone (no caches are allocated, no
        model runs): output size from the reference image and `max_area`, latent frame count from the frame policy,
        intrinsics either given (first row, with their calibration size) or a pinhole of focal length = image width.
        Role parity: telefuser/pipelines/lingbot_world_fast/pipeline.py:192-242."""
        cfg = self.config
        session_config.validate(self.dit_meta["control_type"])
        img_w, img_h = self._image_size(session_config.image)
        width, height = self.best_output_size(img_w, img_h, cfg.max_area)
        height, width = self.check_resize_height_width(height, width)
        _, latent_frames = resolve_lingbot_frame_count(session_config.frame_num, session_config.chunk_size,
                                                       session_config.frame_policy)  # fmt: skip
        if session_config.intrinsics is None:
            cal_w, cal_h = img_w, img_h
            ks = torch.tensor([float(img_w), float(img_w), img_w * 0.5, img_h * 0.5], dtype=torch.float32, device=self.device)
        else:
            cal_w = session_config.intrinsics_width or cfg.orig_width
            cal_h = session_config.intrinsics_height or cfg.orig_height
            ks = torch.as_tensor(session_config.intrinsics, dtype=torch.float32, device=self.device)
            if ks.ndim == 2 and ks.shape[0] >= 1 and ks.shape[1] == 4:
                ks = ks[0]
            if ks.shape != (4,):
                raise ValueError(f"session intrinsics are (fx, fy, cx, cy) or one such row per frame, got {tuple(ks.shape)}")
        return LingBotWorldFastControlContext(
            control_type=self.dit_meta["control_type"], device=self.device, control_dtype=self.torch_dtype,
            orig_height=cal_h, orig_width=cal_w, height=height, width=width, latent_h=height // 8, latent_w=width // 8,
            latent_frames=latent_frames, chunk_size=session_config.chunk_size, intrinsics=ks)  # fmt: skip

    def prepare_offline_controls(self, session_config: LingBotWorldFastSessionConfig, action_path, intrinsics_path,
                                 intrinsics_width: int | None = None, intrinsics_height: int | None = None) -> list:  # fmt: skip
        """One deferred control per chunk from a recorded trajectory (`poses.npy`, for the action mode also
        `action.npy`, under `action_path`; the intrinsics file is named explicitly). The recording is cut to the
        session's length, its first intrinsics row is the calibration (measured on `intrinsics_width` x
        `intrinsics_height` pixels; default: the configured original size), and the conversion to control tensors runs
        once, when the first chunk asks for its control."""
        if (intrinsics_width is None) != (intrinsics_height is None):
            raise ValueError("intrinsics_width and intrinsics_height name one calibration image: give both or neither")
        for name, v in (("intrinsics_width", intrinsics_width), ("intrinsics_height", intrinsics_height)):
            if v is not None and (isinstance(v, bool) or not isinstance(v, int) or v < 1):
                raise ValueError(f"{name} must be a positive integer, got {v!r}")
        from dataclasses import replace

        ctx = replace(self.control_context(session_config), orig_width=intrinsics_width or self.config.orig_width,
                      orig_height=intrinsics_height or self.config.orig_height)  # fmt: skip
        if ctx.control_type == "act":
            poses, ks, action = load_action_control_inputs(action_path, intrinsics_path)
        else:
            (poses, ks), action = load_camera_control_inputs(action_path, intrinsics_path), None
        poses, ks, action = truncate_control_sequence(poses, ks, action, session_config.frame_num)
        source = LingBotWorldFastOfflineControlSource(LingBotWorldFastControlBuilder(ctx), poses, ks, action)
        return [source.control_at(i) for i in range(ctx.latent_frames // ctx.chunk_size)]

    def validate_control(self, rt: LingBotWorldFastGenerationSession, control: torch.Tensor) -> None:
        """A control tensor must be [1, c * (H / h) * (W / w), chunk, h, w] with c = 6 (camera) or 7 (action)."""
        per_pixel = 7 if self.dit_meta["control_type"] == "act" else 6
        fold = max(1, rt.height // rt.latent_h) * max(1, rt.width // rt.latent_w)
        want = (1, per_pixel * fold, rt.chunk_size, rt.latent_h, rt.latent_w)
        if tuple(control.shape) != want:
            raise ValueError(f"control tensor has shape {tuple(control.shape)}, this session takes {want}")

    def create_session(self, session_config: LingBotWorldFastSessionConfig, prompt_emb: torch.Tensor | None = None):
        """Generation session for a session record: the frame policy is applied, the output size follows the reference
        image, and the session's calibration is taken from the record. Returns (generation session, control context)."""
        ctx = self.control_context(session_config)
        if session_config.chunk_size != self.config.chunk_size:
            raise ValueError(f"the session asks for chunks of {session_config.chunk_size} latent frames, the pipeline was "
                             f"initialised with {self.config.chunk_size}")  # fmt: skip
        rt = self._create_initialized_session(session_config.prompt, session_config.image, session_config.frame_num,
                                              ctx.height, ctx.width, session_config.seed, prompt_emb)  # fmt: skip
        rt.control_builder = LingBotWorldFastControlBuilder(ctx)
        return rt, ctx

    # ---- offline generation through the streaming graph ---------------------------------------
    @torch.no_grad()
    def generate_video(self, prompt, image, num_frames: int = 61, height: int = 480, width: int = 832, seed: int = 0,
                       poses: torch.Tensor | None = None, prompt_emb=None, on_chunk: Callable | None = None,
                       timeout_s: float = 3600.0, bind_controls_late: bool = False, controls: list | None = None,
                       frame_policy: str = "strict", session_config: LingBotWorldFastSessionConfig | None = None,
                       world_cache: bool | str = True):  # fmt: skip
        """Returns (frames [1, 3, T, H, W], metrics). `poses`: [latent_frames, 4, 4] camera path (default: seeded walk).
        `controls`: one ready control tensor or provider per chunk instead of `poses` (what `prepare_offline_controls`
        returns). `frame_policy="truncate"` rounds `num_frames` down to a whole number of chunks. `session_config`: a
        session record in place of the individual arguments (its image fixes the output size). `world_cache`: whether the
        session reads / feeds the pipeline's world store (`LingBotWorldFastPipelineConfig.world_cache_bytes`): chunks whose
        controls match an earlier session of the same image, prompt and seed are replayed with one forward pass each;
        `metrics["world_cache_hits"]` counts them.
        `bind_controls_late`: hand each chunk's control to the denoiser as a provider that is read when the chunk is
        admitted (what the interactive service does); `metrics["control_bound_to_output_p50_s"]` is then the time
        from that moment to the chunk's frames."""
        if session_config is not None:
            rt, _ = self.create_session(session_config, prompt_emb)
            seed = session_config.seed
        else:
            num_frames, _ = resolve_lingbot_frame_count(num_frames, self.config.chunk_size, frame_policy)
            rt = self._create_initialized_session(prompt, image, num_frames, height, width, seed, prompt_emb, world_cache)
        latent_frames = rt.chunk_count * rt.chunk_size
        if controls is None:
            if poses is None:
                poses = random_walk_trajectory(latent_frames, seed=seed)
            controls = rt.control_builder.build_sequence(poses, rt.control_builder.context.intrinsics)
        elif len(controls) < rt.chunk_count:
            raise ValueError(f"{len(controls)} controls were given for {rt.chunk_count} chunks")
        session = self.runtime.create_session(rt)
        frames, nxt, t0 = {}, 0, time.monotonic()
        bound_at, latencies = {}, []

        def provider(i):
            def bind():
                bound_at[i] = time.monotonic()
                return controls[i]() if callable(controls[i]) else controls[i]

            return bind

        try:
            while len(frames) < rt.chunk_count:
                if time.monotonic() - t0 > timeout_s:
                    raise TimeoutError("LingBot generation timed out")
                if self.runtime.status(session) == StreamingSessionStatus.FAILED:
                    raise RuntimeError("LingBot streaming session failed") from self.runtime.error(session)
                progressed = False
                if nxt < rt.chunk_count and self.runtime.try_submit_chunk(
                        session, nxt, provider(nxt) if bind_controls_late else controls[nxt]):  # fmt: skip
                    nxt += 1
                    progressed = True
                for idx, f in self.runtime.poll_frames(session):
                    frames[idx] = f
                    progressed = True
                    if idx in bound_at:
                        latencies.append(time.monotonic() - bound_at[idx])
                    if on_chunk is not None:
                        on_chunk(idx, f)
                if not progressed:
                    time.sleep(0.001)
            metrics = self.runtime.metrics(session)
            if latencies:
                metrics["control_bound_to_output_p50_s"] = sorted(latencies)[len(latencies) // 2]
        finally:
            self.release_session(session, cancel=len(frames) < rt.chunk_count)
        video = torch.cat([frames[i] for i in range(rt.chunk_count)], dim=2)
        return video, metrics

    def warmup(self, height: int = 480, width: int = 832, chunks: int = 2) -> None:
        cs = self.config.chunk_size
        n = (cs * chunks - 1) * 4 + 1
        emb = torch.zeros(1, self.config.max_sequence_length, self.denoise_stage_text_dim(), device=self.device,
                          dtype=self.torch_dtype)  # fmt: skip
        self.generate_video("", torch.zeros(3, height, width), n, height, width, prompt_emb=emb)

    def denoise_stage_text_dim(self) -> int:
        st = self.denoise_stage.stage if isinstance(self.denoise_stage, ParallelWorker) else self.denoise_stage
        return st.dit.text_dim

    def close(self) -> None:
        if self.runtime is not None:
            self.runtime.close()
        if isinstance(self.denoise_stage, ParallelWorker):
            self.denoise_stage.close()
        logger.info("LingBot pipeline closed")
