"""ctypes binding of libtfb200.so, the hand-written sm_100a kernel library.

The library is built in-tree by ``telefuser_b200/csrc/build.py`` and loaded
lazily. On a machine with a CUDA device the ops in this package *require* it
and fail loudly when it is missing; on CPU-only machines nothing here is
touched and the pure-PyTorch reference implementations are used instead.
"""

from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path

import torch

_LIB = None
_LOCK = threading.Lock()
_LAUNCHES = 0  # number of native kernel launches issued through this module

c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_long = ctypes.c_long
c_float = ctypes.c_float


class NativeLibraryError(RuntimeError):
    pass


def lib_path() -> Path:
    return Path(__file__).resolve().parent.parent / "_native" / "libtfb200.so"


def _declare(lib) -> None:
    lib.tfb_abi_version.restype = c_int
    lib.tfb_sm_count.restype = c_int
    lib.tfb_last_status.restype = c_int
    lib.tfb_gemm_bf16.restype = c_int
    lib.tfb_gemm_bf16.argtypes = [
        c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
        c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p,
    ]  # fmt: skip
    lib.tfb_attn_fwd.restype = c_int
    lib.tfb_attn_fwd.argtypes = [
        c_void_p, c_long, c_long, c_void_p, c_long, c_long, c_void_p, c_long, c_long,
        c_void_p, c_long, c_long, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p,
    ]  # fmt: skip
    lib.tfb_status_post.restype = c_int
    lib.tfb_status_post.argtypes = [c_void_p]
    lib.tfb_status_peek.restype = c_int
    lib.tfb_set_peer_wait_ms.restype = c_int
    lib.tfb_set_peer_wait_ms.argtypes = [c_int]
    lib.tfb_layernorm_modulate.restype = c_int
    lib.tfb_layernorm_modulate.argtypes = [
        c_void_p, c_long, c_void_p, c_long, c_int, c_int, c_float, c_void_p, c_void_p,
        c_void_p, c_void_p, c_long, c_int, c_void_p,
    ]  # fmt: skip
    lib.tfb_rmsnorm_rope.restype = c_int
    lib.tfb_rmsnorm_rope.argtypes = [
        c_void_p, c_long, c_long, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p,
        c_void_p, c_void_p, c_void_p,
    ]  # fmt: skip
    lib.tfb_gated_residual.restype = c_int
    lib.tfb_gated_residual.argtypes = [
        c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_long, c_int, c_void_p,
    ]
    lib.tfb_act_mul.restype = c_int
    lib.tfb_act_mul.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
    lib.tfb_cfg_euler_step.restype = c_int
    lib.tfb_cfg_euler_step.argtypes = [
        c_void_p, c_void_p, c_void_p, c_int, c_float, c_float, c_void_p, c_void_p, c_long, c_void_p,
    ]
    lib.tfb_quant_mxfp8.restype = c_int
    lib.tfb_quant_mxfp8.argtypes = [c_void_p, c_long, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
    table = {
        "tfb_gemm_bf16_grouped": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                  c_void_p, c_int, c_void_p],
        "tfb_moe_route": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p,
                          c_void_p, c_void_p],
        "tfb_moe_plan": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p],
        "tfb_moe_permute": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_long, c_int, c_void_p, c_void_p,
                            c_void_p],
        "tfb_moe_combine": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p],
        "tfb_kv_cache_roll_append": [c_void_p, c_void_p, c_long, c_void_p, c_void_p, c_long, c_long, c_int, c_int,
                                     c_int, c_int, c_int, c_int, c_int, c_void_p],
        "tfb_fp8_kv_quant": [c_void_p, c_void_p, c_void_p, c_long, c_int, c_void_p],
        "tfb_merge_attn_states": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                  c_int, c_void_p],
        "tfb_taylor_update": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float,
                              c_long, c_void_p],
        "tfb_taylor_apply": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_float, c_float, c_float,
                             c_int, c_void_p, c_long, c_void_p],
        "tfb_plucker_fold": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                             c_void_p],
        "tfb_frames_to_u8": [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p],
        "tfb_attn_fwd_sparse": [c_void_p, c_long, c_long, c_void_p, c_long, c_long, c_void_p, c_long, c_long, c_void_p,
                                c_long, c_long, c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_int,
                                c_int, c_void_p],
        "tfb_gemm_fp8": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                         c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p],
        "tfb_gemm_mxfp8": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                           c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p],
        "tfb_attn_fwd_qk8": [c_void_p, c_long, c_long, c_void_p, c_long, c_long, c_void_p, c_long, c_long, c_void_p, c_void_p,
                             c_void_p, c_long, c_long, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p],
        "tfb_attn_k_stats": [c_void_p, c_long, c_long, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p],
        "tfb_attn_quant_int8": [c_void_p, c_long, c_long, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                c_void_p, c_void_p],
        "tfb_conv3d_causal": [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                              c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
        "tfb_pixel_norm_act": [c_void_p, c_void_p, c_long, c_int, c_void_p, c_int, c_void_p],
        "tfb_upsample2x_nearest": [c_void_p, c_void_p, c_long, c_int, c_int, c_int, c_void_p],
        "tfb_quant_fp8_rowwise": [c_void_p, c_long, c_void_p, c_long, c_void_p, c_int, c_int, c_void_p],
        "tfb_softmax_rows": [c_void_p, c_long, c_int, c_int, c_float, c_void_p],
        "tfb_quant_int8_rowwise": [c_void_p, c_long, c_void_p, c_long, c_void_p, c_int, c_int, c_void_p],
        "tfb_quant_fp8_per_tensor": [c_void_p, c_void_p, c_void_p, c_void_p, c_long, c_int, c_void_p],
        "tfb_gemm_int8": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                          c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p],
        "tfb_nf4_dequant": [c_void_p, c_void_p, c_void_p, c_long, c_int, c_void_p],
        "tfb_rmsnorm_modulate": [c_void_p, c_long, c_void_p, c_long, c_int, c_int, c_float, c_void_p, c_void_p,
                                 c_void_p, c_long, c_int, c_void_p],
        "tfb_rmsnorm_gate_residual": [c_void_p, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_int, c_float,
                                      c_void_p, c_void_p, c_long, c_int, c_int, c_void_p],
        "tfb_headnorm_rope": [c_void_p, c_long, c_long, c_int, c_long, c_int, c_int, c_float, c_void_p, c_void_p,
                              c_void_p, c_void_p, c_void_p],
        "tfb_moe_ep_plan": [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p],
        "tfb_moe_ep_dispatch": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_long, c_int, c_void_p,
                                c_void_p, c_void_p],
        "tfb_moe_ep_combine": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p],
        "tfb_peer_barrier": [c_void_p, c_int, c_int, c_int, c_int, c_void_p],
        "tfb_ulysses_scatter": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                c_int, c_void_p],
        "tfb_peer_push_rows": [c_void_p, c_long, c_void_p, c_int, c_long, c_long, c_int, c_long, c_void_p],
        "tfb_gemm_bf16_rs": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                             c_void_p, c_void_p],
        "tfb_gemm_bf16_ag": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                             c_int, c_int, c_void_p, c_int, c_void_p],
        "tfb_slab_reduce": [c_void_p, c_int, c_long, c_int, c_long, c_void_p, c_void_p, c_long, c_void_p, c_long, c_int,
                            c_long, c_void_p, c_int, c_long, c_long, c_void_p],
        "tfb_attn_fwd_peer": [c_void_p, c_long, c_long, c_void_p, c_long, c_long, c_void_p, c_long, c_long, c_void_p,
                              c_int, c_int, c_int, c_long, c_long, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p],
    }  # fmt: skip
    for name, args in table.items():
        fn = getattr(lib, name)
        fn.restype = c_int
        fn.argtypes = args


def available() -> bool:
    """True when the native library file exists (it may still fail to load)."""
    return lib_path().exists()


def load():
    """Loads (once) and returns the ctypes handle. Raises NativeLibraryError if absent."""
    global _LIB
    if _LIB is not None:
        return _LIB
    with _LOCK:
        if _LIB is not None:
            return _LIB
        path = lib_path()
        if not path.exists():
            raise NativeLibraryError(
                f"{path} is missing: run `python -m telefuser_b200.csrc.build` (or __graft_entry__.build()) first"
            )
        try:
            lib = ctypes.CDLL(os.fspath(path))
        except OSError as e:  # pragma: no cover - depends on the machine
            raise NativeLibraryError(f"cannot load {path}: {e}") from e
        _declare(lib)
        _LIB = lib
    return _LIB


def use_native(t: torch.Tensor) -> bool:
    """Native kernels run for CUDA tensors; CPU tensors take the PyTorch reference path."""
    return t.is_cuda


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def check(code: int, what: str) -> None:
    global _LAUNCHES
    if code != 0:
        raise NativeLibraryError(f"{what} failed with status {code} (site {code >> 8}, kind {code & 0xff})")
    _LAUNCHES += 1


def launch_count() -> int:
    return _LAUNCHES


def reset_launch_count() -> None:
    global _LAUNCHES
    _LAUNCHES = 0


def last_status() -> int:
    """Synchronising read-and-clear of the device status word (bounded-wait expiry etc.)."""
    return int(load().tfb_last_status())


class DeviceWaitTimeout(NativeLibraryError):
    """A bounded wait inside a kernel (on a peer's flag, an mbarrier, a gathered segment) ran out: the data the
    following kernels consumed may be stale, so the result of the current call must be discarded."""


def post_status() -> None:
    """Enqueues, on the current stream, a copy of the status word to pinned host memory (no synchronisation)."""
    check(load().tfb_status_post(stream_ptr()), "tfb_status_post")


def poll_status(what: str = "device kernels") -> None:
    """Raises `DeviceWaitTimeout` when the last posted status word that has reached the host is non-zero.
    Never blocks: a word posted after work still in flight is seen by a later poll."""
    code = int(load().tfb_status_peek())
    if code:
        last_status()  # clear, so that a restarted worker does not trip over the same record
        raise DeviceWaitTimeout(f"{what}: a bounded device wait expired (site {code >> 8}, kind {code & 0xff})")


def finish_status(what: str = "device kernels") -> None:
    """Synchronising check for the end of a call whose result is about to be read anyway."""
    code = last_status()
    if code:
        raise DeviceWaitTimeout(f"{what}: a bounded device wait expired (site {code >> 8}, kind {code & 0xff})")


def set_peer_wait_ms(ms: int) -> None:
    check(load().tfb_set_peer_wait_ms(int(ms)), "tfb_set_peer_wait_ms")


def ptr(t: torch.Tensor | None) -> int | None:
    """Device address of an optional operand. A host tensor is refused: a kernel given a host address faults."""
    if t is None:
        return None
    if not t.is_cuda:
        raise NativeLibraryError(f"a native kernel was handed a {t.device} tensor of shape {tuple(t.shape)}")
    return t.data_ptr()


def same_device(ref: torch.Tensor, *others: torch.Tensor | None) -> None:
    """Raises when an operand lives on another device than `ref` (a module moved after its tensors were tagged)."""
    for t in others:
        if t is not None and t.device != ref.device:
            raise NativeLibraryError(f"operand on {t.device}, expected {ref.device} (shape {tuple(t.shape)})")
