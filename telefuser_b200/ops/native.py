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
        c_void_p, c_long, c_long, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p,
    ]  # fmt: skip
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
    lib.tfb_quant_mxfp8.argtypes = [c_void_p, c_long, c_void_p, c_void_p, c_int, c_int, c_void_p]
    lib.tfb_umma_probe.restype = c_int
    lib.tfb_umma_probe.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
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
                                c_void_p],
        "tfb_gemm_fp8": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                         c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p],
        "tfb_quant_fp8_rowwise": [c_void_p, c_long, c_void_p, c_long, c_void_p, c_int, c_int, c_void_p],
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
                              c_int, c_int, c_int, c_long, c_long, c_int, c_int, c_int, c_int, c_float, c_void_p],
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


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()
