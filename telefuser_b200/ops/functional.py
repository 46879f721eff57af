"""Functional ops: each has an fp32 PyTorch reference (`*_reference`, used on CPU and as
the numerics oracle) and dispatches CUDA tensors to the sm_100a kernels of libtfb200.

There is one native implementation per op and no backend selection: a CUDA tensor
either runs the native kernel or raises (missing library / unsupported shape).
Set ``TFB_FORCE_REFERENCE=1`` to run the reference path on CUDA for debugging.
"""

from __future__ import annotations

import math
import os

import torch
import torch.nn.functional as F

from . import native

_FORCE_REF = os.environ.get("TFB_FORCE_REFERENCE", "0") == "1"


def _native(t: torch.Tensor) -> bool:
    return t.is_cuda and not _FORCE_REF


def set_force_reference(flag: bool) -> None:
    """Route CUDA tensors through the PyTorch reference implementations (debug / A-B checks)."""
    global _FORCE_REF
    _FORCE_REF = bool(flag)


# ---------------------------------------------------------------------------
# Linear (GEMM + fused epilogue)
# ---------------------------------------------------------------------------
def linear_reference(x, weight, bias=None, act=None, residual=None, gate=None):
    y = x.float() @ weight.float().t()
    if bias is not None:
        y = y + bias.float()
    if act == "gelu_tanh":
        y = F.gelu(y, approximate="tanh")
    elif act is not None:
        raise ValueError(f"unknown activation {act}")
    if gate is not None:
        y = y * gate.float()
    if residual is not None:
        y = y + residual.float()
    return y.to(x.dtype)


def linear(x, weight, bias=None, act=None, residual=None, gate=None, out=None):
    """``residual + gate * act(x @ weight.T + bias)`` in one kernel.

    x: [..., K] bf16; weight: [N, K]; gate: fp32 broadcastable over rows as
    [..., 1, N] (one gate row per leading batch entry) or per row [..., N].
    """
    if weight.dtype == torch.float8_e4m3fn:
        mx_sf = getattr(weight, "tfb_mx_sf", None)
        if mx_sf is not None:
            if mx_sf.device != weight.device:  # the module was moved after quantisation
                mx_sf = weight.tfb_mx_sf = mx_sf.to(weight.device)
            r = linear_mxfp8(x, weight, mx_sf, bias, act, residual, gate)
        else:
            r = linear_fp8(x, weight, fp8_weight_scale(weight), bias, act, residual, gate)
        if out is not None:
            out.copy_(r)
            return out
        return r
    if weight.dtype == torch.int8:
        r = linear_int8(x, weight, fp8_weight_scale(weight), bias, act, residual, gate)
        if out is not None:
            out.copy_(r)
            return out
        return r
    if weight.dtype == torch.uint8 and hasattr(weight, "tfb_nf4_absmax"):
        from telefuser_b200.ops.nf4 import expand_nf4_weight

        weight = expand_nf4_weight(weight, x.dtype)  # packed 4-bit codes -> [N, K] in a shared scratch buffer
    elif weight.dtype == torch.uint8 and hasattr(weight, "tfb_nvfp4_sf"):
        from telefuser_b200.ops.nvfp4 import expand_nvfp4_weight

        weight = expand_nvfp4_weight(weight, x.dtype)  # e2m1 codes + e4m3 block scales -> [N, K]
    K = x.shape[-1]
    N = weight.shape[0]
    # The tensor-core kernel moves 16-byte rows: widths that are not multiples of 8 elements (toy configurations)
    # take the fp32 evaluation.
    if not _native(x) or x.dtype != torch.bfloat16 or K % 8 or N % 8:
        r = linear_reference(x, weight, bias, act, residual, gate)
        if out is not None:
            out.copy_(r)
            return out
        return r
    lib = native.load()
    x2 = x.reshape(-1, K)
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    M = x2.shape[0]
    if weight.stride(-1) != 1:
        weight = weight.contiguous()
    if out is None:
        out = torch.empty(*x.shape[:-1], N, device=x.device, dtype=torch.bfloat16)
    out2 = out.view(-1, N)
    res2 = None
    if residual is not None:
        res2 = residual.reshape(-1, N)
        if res2.stride(-1) != 1:
            res2 = res2.contiguous()
    gate_ptr, ldg, rpg = None, 0, 1
    if gate is not None:
        g = gate
        if g.dtype != torch.float32:
            g = g.float()
        g2 = g.reshape(-1, N)
        if g2.stride(-1) != 1:
            g2 = g2.contiguous()
        if M % g2.shape[0]:
            raise ValueError("gate rows must divide the number of rows")
        gate_ptr, ldg, rpg = g2.data_ptr(), g2.stride(0) if g2.shape[0] > 1 else N, M // g2.shape[0]
        gate = g2  # keep alive
    if bias is not None and bias.dtype != torch.bfloat16:
        bias = bias.to(torch.bfloat16)
    native.same_device(x2, weight, bias, res2)
    code = lib.tfb_gemm_bf16(
        x2.data_ptr(), x2.stride(0), weight.data_ptr(), weight.stride(0), out2.data_ptr(), out2.stride(0),
        M, N, K, native.ptr(bias), 1 if act == "gelu_tanh" else 0,
        native.ptr(res2), res2.stride(0) if res2 is not None else 0, gate_ptr, ldg, rpg, 0, native.stream_ptr(),
    )  # fmt: skip
    if act not in (None, "gelu_tanh"):
        raise ValueError(f"unknown activation {act}")
    native.check(code, "tfb_gemm_bf16")
    return out


def quant_fp8_rowwise(x):
    """x [..., C] -> (e4m3 [..., C], fp32 scale [..., 1]) with scale = row amax / 448 (floor 1e-12)."""
    C = x.shape[-1]
    if not _native(x) or x.dtype != torch.bfloat16 or C % 8:
        s = (x.float().abs().amax(-1, keepdim=True) / 448.0).clamp_min(1e-12)
        return (x.float() / s).clamp(-448, 448).to(torch.float8_e4m3fn), s
    x2 = x.reshape(-1, C)
    if x2.stride(-1) != 1 or x2.stride(0) % 8:
        x2 = x2.contiguous()
    q = torch.empty(x2.shape, device=x.device, dtype=torch.float8_e4m3fn)
    s = torch.empty(x2.shape[0], device=x.device, dtype=torch.float32)
    code = native.load().tfb_quant_fp8_rowwise(x2.data_ptr(), x2.stride(0), q.data_ptr(), C, s.data_ptr(), x2.shape[0],
                                               C, native.stream_ptr())  # fmt: skip
    native.check(code, "tfb_quant_fp8_rowwise")
    return q.view(x.shape), s.view(*x.shape[:-1], 1)


def use_native_kernels(t) -> bool:
    """True when ops on `t` run on the native kernels (a CUDA tensor and the fp32 oracle is not forced)."""
    return _native(t)


def is_quantized_weight(weight) -> bool:
    """True for every stored format whose rows cannot be sliced along K like a dense matrix: e4m3 and int8 (one scale
    per output row), MXFP8 / NVFP4 (scale per K block, tiled layout) and packed NF4."""
    return weight.dtype in (torch.float8_e4m3fn, torch.int8, torch.uint8)


def fp8_weight_scale(weight):
    """Per-output-channel scale tagged on an e4m3 weight (`tfb_scale`), on the weight's own device.

    The tag is set when a layer is quantised. `Module.to()` moves the parameter's storage but keeps the Python
    object, so after a move the tag still points at the old device; it is re-homed here (and cached back) so that
    the GEMM never receives an address of another device."""
    s = getattr(weight, "tfb_scale", None)
    if s is not None and s.device != weight.device:
        s = s.to(device=weight.device, dtype=torch.float32)
        weight.tfb_scale = s
    return s


def quant_int8_rowwise(x):
    """x [..., C] -> (int8 [..., C] in [-127, 127], fp32 scale [..., 1]) with scale = row amax / 127 (floor 1e-12)."""
    C = x.shape[-1]
    if not _native(x) or x.dtype != torch.bfloat16 or C % 8:
        s = (x.float().abs().amax(-1, keepdim=True) / 127.0).clamp_min(1e-12)
        return torch.round(x.float() / s).clamp(-127, 127).to(torch.int8), s
    x2 = x.reshape(-1, C)
    if x2.stride(-1) != 1 or x2.stride(0) % 8:
        x2 = x2.contiguous()
    q = torch.empty(x2.shape, device=x.device, dtype=torch.int8)
    s = torch.empty(x2.shape[0], device=x.device, dtype=torch.float32)
    code = native.load().tfb_quant_int8_rowwise(x2.data_ptr(), x2.stride(0), q.data_ptr(), C, s.data_ptr(), x2.shape[0],
                                                C, native.stream_ptr())  # fmt: skip
    native.check(code, "tfb_quant_int8_rowwise")
    return q.view(x.shape), s.view(*x.shape[:-1], 1)


def quantize_weight_int8(weight):
    """[N, K] weight -> (int8 [N, K], fp32 per-output-channel scale [N]); symmetric, range [-127, 127]."""
    w = weight.float()
    s = (w.abs().amax(-1, keepdim=True) / 127.0).clamp_min(1e-12)
    return torch.round(w / s).clamp(-127, 127).to(torch.int8), s.reshape(-1)


def quant_fp8_per_tensor(x, scale=None):
    """Whole-tensor FP8 quantisation: (e4m3 tensor of x's shape, fp32 scale [1]). With `scale` given (a calibrated,
    static scale) it is used as is; otherwise scale = amax / 448 (floor 1e-12). Role of the reference's
    tf_per_tensor_quant_fp8 (tf-kernel/tf_kernel/gemm.py:123)."""
    if not _native(x) or x.dtype != torch.bfloat16 or not x.is_contiguous():
        s = (x.float().abs().amax() / 448.0).clamp_min(1e-12).reshape(1) if scale is None else scale.float().reshape(1)
        return (x.float() / s).clamp(-448, 448).to(torch.float8_e4m3fn), s
    q = torch.empty(x.shape, device=x.device, dtype=torch.float8_e4m3fn)
    static = scale is not None
    s = scale.to(device=x.device, dtype=torch.float32).reshape(1).clone() if static else torch.empty(1, device=x.device)
    scratch = torch.empty(1, device=x.device, dtype=torch.int32)
    code = native.load().tfb_quant_fp8_per_tensor(x.data_ptr(), q.data_ptr(), s.data_ptr(), scratch.data_ptr(), x.numel(),
                                                  1 if static else 0, native.stream_ptr())  # fmt: skip
    native.check(code, "tfb_quant_fp8_per_tensor")
    return q, s


def _linear_w8a8(x, weight, weight_scale, bias, act, residual, gate, int8):
    """Shared body of the two W8A8 linears (e4m3 or int8 operands): quantise the activations per token, multiply on
    the 8-bit tensor-core path, apply both scale vectors and the epilogue in fp32."""
    name = "int8" if int8 else "fp8"
    if weight_scale is None:
        raise ValueError(f"an {name} weight needs its per-channel scale (attribute `tfb_scale` or argument)")
    ws = weight_scale.to(device=x.device, dtype=torch.float32).reshape(-1)
    quant = quant_int8_rowwise if int8 else quant_fp8_rowwise
    K, N = x.shape[-1], weight.shape[0]
    if not _native(x) or x.dtype != torch.bfloat16 or K % 16 or N % 8:
        q, s = quant(x)
        y = (q.float() @ weight.float().t()) * s.float() * ws
        if bias is not None:
            y = y + bias.float()
        if act == "gelu_tanh":
            y = F.gelu(y, approximate="tanh")
        elif act is not None:
            raise ValueError(f"unknown activation {act}")
        if gate is not None:
            y = y * gate.float()
        if residual is not None:
            y = y + residual.float()
        return y.to(x.dtype)
    q, s = quant(x.reshape(-1, K))
    M = q.shape[0]
    ws = ws.contiguous()
    out = torch.empty(*x.shape[:-1], N, device=x.device, dtype=torch.bfloat16)
    res2 = None if residual is None else residual.reshape(-1, N).contiguous()
    gate_ptr, ldg, rpg, g2 = None, 0, 1, None
    if gate is not None:
        g2 = gate.float().reshape(-1, N).contiguous()
        gate_ptr, ldg, rpg = g2.data_ptr(), N, M // g2.shape[0]
    if bias is not None and bias.dtype != torch.bfloat16:
        bias = bias.to(torch.bfloat16)
    if act not in (None, "gelu_tanh"):
        raise ValueError(f"unknown activation {act}")
    w = weight if weight.stride(-1) == 1 else weight.contiguous()
    native.same_device(x, w, ws, bias, res2, g2)
    fn = native.load().tfb_gemm_int8 if int8 else native.load().tfb_gemm_fp8
    code = fn(q.data_ptr(), K, w.data_ptr(), w.stride(0), out.data_ptr(), N, M, N, K, s.data_ptr(), ws.data_ptr(),
              native.ptr(bias), 1 if act == "gelu_tanh" else 0, native.ptr(res2), N if res2 is not None else 0, gate_ptr,
              ldg, rpg, native.stream_ptr())  # fmt: skip
    native.check(code, f"tfb_gemm_{name}")
    return out


def bmm_fp8(a, b, a_scale, b_scale, out_dtype=torch.bfloat16, out=None):
    """Batched FP8 product with one scale per operand: out[i] = (a[i] @ b[i]) * a_scale * b_scale.

    a: e4m3 [B, M, K]; b: e4m3 [B, K, N] whose K axis is the contiguous one (a transposed view of a [B, N, K] tensor,
    the column-major operand a batched FP8 library GEMM takes); a_scale / b_scale: one fp32 value each. On CUDA
    every batch entry runs on the W8A8 tensor-core GEMM with the two scalars broadcast as its per-row / per-column scale
    vectors; elsewhere the product is evaluated in fp32. Role of the reference's `bmm_fp8`
    (tf-kernel/tf_kernel/gemm.py:60, tf-kernel/csrc/gemm/bmm_fp8.cu)."""
    if a.dim() != 3 or b.dim() != 3 or a.shape[0] != b.shape[0] or a.shape[2] != b.shape[1]:
        raise ValueError(f"bmm_fp8: shapes {tuple(a.shape)} x {tuple(b.shape)} do not multiply")
    B, M, K = a.shape
    N = b.shape[2]
    sa = a_scale.to(device=a.device, dtype=torch.float32).reshape(-1)[:1]
    sb = b_scale.to(device=a.device, dtype=torch.float32).reshape(-1)[:1]
    if out is None:
        out = torch.empty(B, M, N, device=a.device, dtype=out_dtype)
    bt = b.transpose(1, 2)  # [B, N, K]
    native_ok = (_native(a) and a.dtype == torch.float8_e4m3fn and b.dtype == torch.float8_e4m3fn and K % 16 == 0
                 and N % 8 == 0 and a.stride(2) == 1 and bt.stride(2) == 1 and a.stride(1) % 16 == 0 and bt.stride(1) % 16 == 0)  # fmt: skip
    if not native_ok:
        out.copy_((torch.bmm(a.float(), b.float()) * (sa * sb)).to(out.dtype))
        return out
    row_scale, col_scale = sa.expand(M).contiguous(), sb.expand(N).contiguous()
    lib = native.load()
    tmp = out if out.dtype == torch.bfloat16 and out.is_contiguous() else torch.empty(B, M, N, device=a.device, dtype=torch.bfloat16)
    for i in range(B):
        ai, bi = a[i], bt[i]
        if ai.data_ptr() % 16 or bi.data_ptr() % 16:
            ai, bi = ai.contiguous(), bi.contiguous()
        code = lib.tfb_gemm_fp8(ai.data_ptr(), ai.stride(0), bi.data_ptr(), bi.stride(0), tmp[i].data_ptr(), N, M, N, K,
                                row_scale.data_ptr(), col_scale.data_ptr(), None, 0, None, 0, None, 0, 1,
                                native.stream_ptr())  # fmt: skip
        native.check(code, "tfb_gemm_fp8")
    if tmp is not out:
        out.copy_(tmp)
    return out


def linear_fp8(x, weight, weight_scale, bias=None, act=None, residual=None, gate=None):
    """W8A8: weight e4m3 [N, K] with per-output-channel scale [N] or [N, 1]; activations are quantised
    per token on the fly; fp32 accumulate; epilogue as `linear`."""
    return _linear_w8a8(x, weight, weight_scale, bias, act, residual, gate, False)


def linear_int8(x, weight, weight_scale, bias=None, act=None, residual=None, gate=None):
    """W8A8 on integers: weight int8 [N, K] with per-output-channel scale, activations quantised per token to
    [-127, 127]; exact int32 accumulation on the tensor cores; epilogue as `linear`. Role of the reference's
    int8_scaled_mm (tf-kernel/tf_kernel/gemm.py:8)."""
    return _linear_w8a8(x, weight, weight_scale, bias, act, residual, gate, True)


# ---------------------------------------------------------------------------
# LayerNorm + modulation
# ---------------------------------------------------------------------------
def layernorm_modulate_reference(x, shift=None, scale=None, weight=None, bias=None, eps=1e-6):
    y = F.layer_norm(x.float(), (x.shape[-1],), None if weight is None else weight.float(),
                     None if bias is None else bias.float(), eps)  # fmt: skip
    if scale is not None:
        y = y * (1 + scale.float())
    if shift is not None:
        y = y + shift.float()
    return y.to(x.dtype)


def layernorm_modulate(x, shift=None, scale=None, weight=None, bias=None, eps=1e-6):
    """LN over the last dim (optional affine) then ``y*(1+scale)+shift``.

    x: [B, S, C]; shift/scale: fp32 [B, 1, C] (per batch) or [B, S, C] (per token).
    """
    if not _native(x) or x.dtype != torch.bfloat16:
        return layernorm_modulate_reference(x, shift, scale, weight, bias, eps)
    lib = native.load()
    C = x.shape[-1]
    x2 = x.reshape(-1, C)
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    rows = x2.shape[0]
    out = torch.empty_like(x2)
    sh_ptr = sc_ptr = None
    ldmod, rpm = 0, 1
    keep = []
    if (shift is None) != (scale is None):
        z = torch.zeros_like(shift if shift is not None else scale)
        shift = z if shift is None else shift
        scale = z if scale is None else scale
    if scale is not None:
        sh = shift.float() if shift.dtype != torch.float32 else shift
        sc = scale.float() if scale.dtype != torch.float32 else scale
        sh2, sc2 = sh.reshape(-1, C), sc.reshape(-1, C)
        if sh2.stride(-1) != 1 or sc2.stride(-1) != 1 or sh2.stride(0) != sc2.stride(0):
            sh2, sc2 = sh2.contiguous(), sc2.contiguous()
        if rows % sh2.shape[0]:
            raise ValueError("modulation rows must divide the number of rows")
        ldmod = sh2.stride(0) if sh2.shape[0] > 1 else C
        rpm = rows // sh2.shape[0]
        sh_ptr, sc_ptr = sh2.data_ptr(), sc2.data_ptr()
        keep = [sh2, sc2]
    code = lib.tfb_layernorm_modulate(
        x2.data_ptr(), x2.stride(0), out.data_ptr(), out.stride(0), rows, C, eps,
        native.ptr(weight), native.ptr(bias), sh_ptr, sc_ptr, ldmod, rpm, native.stream_ptr())  # fmt: skip
    native.check(code, "tfb_layernorm_modulate")
    del keep
    return out.view(x.shape)


# ---------------------------------------------------------------------------
# RMSNorm (+ RoPE)
# ---------------------------------------------------------------------------
def rope_reference(x, cos, sin):
    """Interleaved-pair RoPE. x: [B, S, H, D]; cos/sin: [S, D/2] (fp32)."""
    B, S, H, D = x.shape
    xf = x.float().reshape(B, S, H, D // 2, 2)
    a, b = xf[..., 0], xf[..., 1]
    c = cos.float().reshape(1, S, 1, D // 2)
    s = sin.float().reshape(1, S, 1, D // 2)
    return torch.stack([a * c - b * s, a * s + b * c], dim=-1).reshape(B, S, H, D).to(x.dtype)


def rmsnorm_reference(x, weight=None, eps=1e-6):
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    if weight is not None:
        y = y * weight.float()
    return y.to(x.dtype)


def rmsnorm_rope_(x, weight, num_heads, cos=None, sin=None, eps=1e-6, x2=None, weight2=None):
    """In-place RMSNorm over the full channel dim followed by optional RoPE.

    x: [B, S, C] view (may be a column slice of a fused qkv buffer). When ``x2``
    is given (same shape/strides, e.g. the k slice) both are processed in one launch.
    cos/sin: fp32 [B*S, D/2] or [S, D/2] with B == 1.
    """
    B, S, C = x.shape
    D = C // num_heads
    if not _native(x) or x.dtype != torch.bfloat16:
        for t, w in ((x, weight), (x2, weight2)):
            if t is None:
                continue
            y = rmsnorm_reference(t, w, eps)
            if cos is not None:
                c2, s2 = cos.reshape(-1, D // 2), sin.reshape(-1, D // 2)
                if c2.shape[0] == B * S and B > 1:
                    y = torch.cat([rope_reference(y[i : i + 1].reshape(1, S, num_heads, D), c2[i * S : (i + 1) * S],
                                                  s2[i * S : (i + 1) * S]) for i in range(B)]).reshape(B, S, C)  # fmt: skip
                else:
                    y = rope_reference(y.reshape(B, S, num_heads, D), c2, s2).reshape(B, S, C)
            t.copy_(y)
        return x
    lib = native.load()
    if x.stride(-1) != 1 or (B > 1 and x.stride(0) != S * x.stride(1)):
        raise ValueError("rmsnorm_rope_ needs row-strided input")
    nmat, mat_stride = 1, 0
    if x2 is not None:
        if x2.stride() != x.stride() or x2.shape != x.shape:
            raise ValueError("x2 must match x")
        mat_stride = (x2.data_ptr() - x.data_ptr()) // x.element_size()
        nmat = 2
    if cos is not None:
        if cos.dtype != torch.float32 or not cos.is_contiguous():
            cos, sin = cos.float().contiguous(), sin.float().contiguous()
        if cos.numel() != B * S * (D // 2):
            if B == 1:
                raise ValueError("cos/sin must have one row per token")
            cos = cos.reshape(1, S, D // 2).expand(B, S, D // 2).contiguous()
            sin = sin.reshape(1, S, D // 2).expand(B, S, D // 2).contiguous()
    code = lib.tfb_rmsnorm_rope(
        x.data_ptr(), x.stride(1), mat_stride, nmat, B * S, num_heads, D, eps, native.ptr(weight),
        native.ptr(weight2), native.ptr(cos), native.ptr(sin), native.stream_ptr())  # fmt: skip
    native.check(code, "tfb_rmsnorm_rope")
    return x


# ---------------------------------------------------------------------------
# Attention
# ---------------------------------------------------------------------------
def attention_reference(q, k, v, scale=None, return_lse=False, causal=False, mask=None, q_block: int | None = None,
                        bias=None):
    """q: [B, Sq, H, D], k/v: [B, Skv, H, D] -> [B, Sq, H, D] (fp32 softmax).

    `causal`: key j is visible to query i when j <= i + (Skv - Sq). `mask`: boolean, broadcastable to
    [B, H, Sq, Skv], True = visible. `bias`: added to the scaled scores, broadcastable to [B, H, Sq, Skv].
    `q_block` bounds the score matrix held at once to [B, H, q_block, Skv]."""
    D = q.shape[-1]
    Sq, Skv = q.shape[1], k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    kf, vf = (t.float().permute(0, 2, 1, 3) for t in (k, v))
    outs, lses = [], []
    step = q_block or Sq
    for s0 in range(0, Sq, step):
        s1 = min(Sq, s0 + step)
        qf = q[:, s0:s1].float().permute(0, 2, 1, 3)
        s = (qf @ kf.transpose(-1, -2)) * scale
        if causal:
            rows = torch.arange(s0, s1, device=q.device).unsqueeze(1) + (Skv - Sq)
            s = s.masked_fill(torch.arange(Skv, device=q.device).unsqueeze(0) > rows, float("-inf"))
        if bias is not None:
            s = s + (bias if bias.dim() < 2 or bias.shape[-2] == 1 else bias[..., s0:s1, :]).float()
        if mask is not None:
            m = mask if mask.dim() < 2 or mask.shape[-2] == 1 else mask[..., s0:s1, :]
            s = s.masked_fill(~m, float("-inf"))
        outs.append((torch.softmax(s, dim=-1) @ vf).permute(0, 2, 1, 3).to(q.dtype))
        if return_lse:
            lses.append(torch.logsumexp(s, dim=-1))
    o = outs[0] if len(outs) == 1 else torch.cat(outs, dim=1)
    if return_lse:
        return o, (lses[0] if len(lses) == 1 else torch.cat(lses, dim=-1))
    return o


def _pad_head_dim(t, D_to):
    return F.pad(t, (0, D_to - t.shape[-1]))


def softmax_rows_(x, scale: float = 1.0):
    """In place: x[r, :] = softmax(scale * x[r, :]) for a 2-D bf16 CUDA tensor (fp32 maths); other inputs go through
    torch.softmax in fp32."""
    C = x.shape[-1]
    if not _native(x) or x.dtype != torch.bfloat16 or x.dim() != 2 or C % 8 or x.stride(1) != 1 or x.stride(0) % 8 \
            or scale <= 0:  # fmt: skip
        x.copy_(torch.softmax(x.float() * scale, dim=-1))
        return x
    code = native.load().tfb_softmax_rows(x.data_ptr(), x.stride(0), x.shape[0], C, float(scale), native.stream_ptr())
    native.check(code, "tfb_softmax_rows")
    return x


def _attention_wide_heads(q, k, v, scale):
    """Heads wider than 128 (the single-head attention of the VAEs: D = 384 / 512) on the native kernels, unfused:
    per (batch, head) a scores GEMM [Sq, Skv], the row softmax in place, and the P.V GEMM. The score matrix of ONE
    head is held at a time (bf16)."""
    B, Sq, H, D = q.shape
    out = torch.empty(B, Sq, H, D, device=q.device, dtype=q.dtype)
    for b in range(B):
        for h in range(H):
            p = linear(q[b, :, h].contiguous(), k[b, :, h].contiguous())  # [Sq, Skv]
            softmax_rows_(p, scale)
            out[b, :, h] = linear(p, v[b, :, h].t().contiguous())  # weight [D, Skv]
    return out


def attention(q, k, v, scale=None, return_lse=False, variant=0, causal=False, mask=None, quant=None, bias=None):
    """Attention, layout BSHD: q [B, Sq, H, D], k / v [B, Skv, H, D] -> [B, Sq, H, D].
    `quant="int8"` computes the scores on int8 operands (`attention_int8`; no LSE output).

    CUDA bf16 / fp16 inputs with D <= 128 run on the tcgen05 kernel (head dims other than 64 / 128 are zero-padded
    to the next of the two, fp16 is computed in bf16); `causal` is handled inside the kernel. Heads wider than 128
    without mask / bias and with at least 1024 keys run as two tensor-core GEMMs around a row-softmax kernel (the
    scores pass through bf16 there; shorter sequences, where speed does not matter, keep fp32 scores). A general boolean `mask`
    (True = visible) or an additive `bias` take the fp32 evaluation in query blocks, so that no [Sq, Skv] score
    matrix is ever held for the whole sequence. CPU tensors always take the fp32 evaluation."""
    D = q.shape[-1]
    if (_native(q) and q.dtype == torch.bfloat16 and D > 128 and D % 8 == 0 and mask is None and bias is None
            and not causal and not return_lse and quant is None and k.shape[1] % 8 == 0 and k.shape[1] >= 1024):
        return _attention_wide_heads(q, k, v, scale if scale is not None else 1.0 / math.sqrt(D))
    if quant is not None:
        if quant != "int8" or return_lse or mask is not None or bias is not None:
            raise ValueError("quantised attention: quant='int8', without LSE output or a mask")
        if D == 128:
            return attention_int8(q, k, v, scale, causal)
    if not _native(q) or q.dtype not in (torch.bfloat16, torch.float16) or D > 128 or mask is not None or D % 8 \
            or bias is not None or (causal and k.shape[1] < q.shape[1]):  # fmt: skip
        blk = None
        if q.is_cuda and q.shape[1] * k.shape[1] > (1 << 24):
            blk = max(128, (1 << 24) // k.shape[1])
        return attention_reference(q, k, v, scale, return_lse, causal, mask, blk, bias)
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    in_dtype = q.dtype
    if in_dtype != torch.bfloat16:
        q, k, v = q.bfloat16(), k.bfloat16(), v.bfloat16()
    Dk = 64 if D <= 64 else 128
    if Dk != D:
        q, k, v = _pad_head_dim(q, Dk), _pad_head_dim(k, Dk), _pad_head_dim(v, Dk)
    lib = native.load()
    B, Sq, H, _ = q.shape
    Skv = k.shape[1]

    def prep(t):
        S = t.shape[1]
        if t.stride(-1) != 1 or t.stride(2) != Dk or (B > 1 and t.stride(0) % 8) or t.stride(1) % 8:
            t = t.contiguous()
        return t, t.stride(1), (t.stride(0) if B > 1 else S * t.stride(1))

    q, ldq, bsq = prep(q)
    k, ldk, bsk = prep(k)
    v, ldv, bsv = prep(v)
    out = torch.empty(B, Sq, H, Dk, device=q.device, dtype=torch.bfloat16)
    lse = torch.empty(B, H, Sq, device=q.device, dtype=torch.float32) if return_lse else None
    code = lib.tfb_attn_fwd(
        q.data_ptr(), ldq, bsq, k.data_ptr(), ldk, bsk, v.data_ptr(), ldv, bsv, out.data_ptr(), H * Dk, Sq * H * Dk,
        native.ptr(lse), B, H, Sq, Skv, Dk, int(bool(causal)), scale, variant, native.stream_ptr())  # fmt: skip
    native.check(code, "tfb_attn_fwd")
    if Dk != D:
        out = out[..., :D]
    if in_dtype != torch.bfloat16:
        out = out.to(in_dtype)
    return (out, lse) if return_lse else out


def quantize_qk_int8_reference(q, k):
    """q, k [B, S, H, D] -> (q8 int8, q_scale fp32 [B, H, Sq], k8 int8, k_scale fp32 [B, H], k_mean fp32 [B, H, D]).

    Q: one scale per token and head (max |q| / 127). K: the per-channel mean over the tokens is removed (softmax is
    invariant to it), then one scale per head, taken from the bound max |k| + max |mean| so that it needs no
    second pass over K."""
    qf, kf = q.float(), k.float()
    qs = (qf.abs().amax(-1) / 127.0).clamp_min(1e-12)  # [B, S, H]
    q8 = torch.round(qf / qs.unsqueeze(-1)).clamp(-127, 127).to(torch.int8)
    mean = kf.mean(dim=1)  # [B, H, D]
    ks = ((kf.abs().amax(dim=(1, 3)) + mean.abs().amax(-1)) / 127.0).clamp_min(1e-12)  # [B, H]
    k8 = torch.round((kf - mean.unsqueeze(1)) / ks[:, None, :, None]).clamp(-127, 127).to(torch.int8)
    return q8, qs.permute(0, 2, 1).contiguous(), k8, ks, mean


def quantize_qk_int8(q, k):
    """As `quantize_qk_int8_reference`, by the native kernels on CUDA bf16 inputs with head_dim 128."""
    B, Sq, H, D = q.shape
    if not _native(q) or q.dtype != torch.bfloat16 or D != 128:
        return quantize_qk_int8_reference(q, k)
    lib, st = native.load(), native.stream_ptr()
    Skv = k.shape[1]

    def prep(t):
        S = t.shape[1]
        if t.stride(-1) != 1 or t.stride(2) != D or (B > 1 and t.stride(0) % 8) or t.stride(1) % 8:
            t = t.contiguous()
        return t, t.stride(1), (t.stride(0) if B > 1 else S * t.stride(1))

    (q, ldq, bsq), (k, ldk, bsk) = prep(q), prep(k)
    dev = q.device
    sums = torch.empty(B, H * D, device=dev, dtype=torch.float32)
    amax = torch.empty(B, H, device=dev, dtype=torch.float32)
    native.check(lib.tfb_attn_k_stats(k.data_ptr(), ldk, bsk, B, Skv, H, sums.data_ptr(), amax.data_ptr(), st), "tfb_attn_k_stats")
    mean = (sums / Skv).view(B, H, D)
    ks = ((amax + mean.abs().amax(-1)) / 127.0).clamp_min(1e-12).contiguous()
    q8 = torch.empty(B, Sq, H, D, device=dev, dtype=torch.int8)
    k8 = torch.empty(B, Skv, H, D, device=dev, dtype=torch.int8)
    qs = torch.empty(B, H, Sq, device=dev, dtype=torch.float32)
    native.check(lib.tfb_attn_quant_int8(q.data_ptr(), ldq, bsq, q8.data_ptr(), B, Sq, H, 0, None, None, qs.data_ptr(), st),
                 "tfb_attn_quant_int8")  # fmt: skip
    native.check(lib.tfb_attn_quant_int8(k.data_ptr(), ldk, bsk, k8.data_ptr(), B, Skv, H, 1, mean.data_ptr(), ks.data_ptr(),
                                         None, st), "tfb_attn_quant_int8")  # fmt: skip
    return q8, qs, k8, ks, mean


def attention_int8(q, k, v, scale=None, causal=False):
    """Attention with int8 scores: Q and K are quantised on the fly (per token / per head, K mean-centred), the score
    matrix is accumulated in int32 on the tensor core (`tcgen05.mma.kind::i8`), softmax and P.V run as in the bf16
    kernel. The place of the reference's SageAttention int8-QK modes (telefuser/ops/attention/attention_impl.py:245-300).
    CPU tensors and shapes the kernel does not cover evaluate the same quantised maths in fp32."""
    B, Sq, H, D = q.shape
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if not _native(q) or q.dtype != torch.bfloat16 or D != 128 or (causal and k.shape[1] < Sq):
        q8, qs, k8, ks, _ = quantize_qk_int8_reference(q, k)
        s = torch.einsum("bqhd,bkhd->bhqk", q8.float(), k8.float()) * qs.unsqueeze(-1) * ks[:, :, None, None] * scale
        if causal:
            Skv = k.shape[1]
            rows = torch.arange(Sq, device=q.device).unsqueeze(1) + (Skv - Sq)
            s = s.masked_fill(torch.arange(Skv, device=q.device).unsqueeze(0) > rows, float("-inf"))
        return torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, dim=-1), v.float()).to(q.dtype)
    q8, qs, k8, ks, _ = quantize_qk_int8(q, k)
    Skv = k.shape[1]
    if v.stride(-1) != 1 or v.stride(2) != D or (B > 1 and v.stride(0) % 8) or v.stride(1) % 8:
        v = v.contiguous()
    ldv, bsv = v.stride(1), (v.stride(0) if B > 1 else Skv * v.stride(1))
    out = torch.empty(B, Sq, H, D, device=q.device, dtype=torch.bfloat16)
    code = native.load().tfb_attn_fwd_qk8(q8.data_ptr(), H * D, Sq * H * D, k8.data_ptr(), H * D, Skv * H * D, v.data_ptr(), ldv,
                                          bsv, qs.data_ptr(), ks.data_ptr(), out.data_ptr(), H * D, Sq * H * D, B, H, Sq, Skv,
                                          int(bool(causal)), scale, native.stream_ptr())  # fmt: skip
    native.check(code, "tfb_attn_fwd_qk8")
    return out


def merge_attn_states_reference(o1, lse1, o2, lse2):
    l1 = lse1.float().transpose(1, 2).unsqueeze(-1)
    l2 = lse2.float().transpose(1, 2).unsqueeze(-1)
    m = torch.maximum(l1, l2)
    w1, w2 = torch.exp(l1 - m), torch.exp(l2 - m)
    o = (o1.float() * w1 + o2.float() * w2) / (w1 + w2)
    lse = (m + torch.log(w1 + w2)).squeeze(-1).transpose(1, 2)
    return o.to(o1.dtype), lse


def merge_attn_states(o1, lse1, o2, lse2):
    """Combine two partial attention results by their log-sum-exp (ring attention step).

    o*: [B, S, H, D]; lse*: [B, H, S]. Same maths as the reference's
    ``merge_attn_states`` (telefuser/distributed/ring.py:159-214).
    """
    if _native(o1) and o1.dtype == torch.bfloat16 and o1.shape[-1] % 8 == 0:
        B, S, H, D = o1.shape
        o1c, o2c = o1.contiguous(), o2.contiguous()
        l1c, l2c = lse1.float().contiguous(), lse2.float().contiguous()
        out, lse = torch.empty_like(o1c), torch.empty_like(l1c)
        code = native.load().tfb_merge_attn_states(o1c.data_ptr(), l1c.data_ptr(), o2c.data_ptr(), l2c.data_ptr(),
                                                   out.data_ptr(), lse.data_ptr(), B, S, H, D, native.stream_ptr())  # fmt: skip
        native.check(code, "tfb_merge_attn_states")
        return out, lse
    l1 = lse1.float().transpose(1, 2).unsqueeze(-1)
    l2 = lse2.float().transpose(1, 2).unsqueeze(-1)
    m = torch.maximum(l1, l2)
    w1, w2 = torch.exp(l1 - m), torch.exp(l2 - m)
    o = (o1.float() * w1 + o2.float() * w2) / (w1 + w2)
    lse = (m + torch.log(w1 + w2)).squeeze(-1).transpose(1, 2)
    return o.to(o1.dtype), lse


# ---------------------------------------------------------------------------
# Elementwise
# ---------------------------------------------------------------------------
def gated_residual(x, y, gate=None):
    """``x + gate * y``; gate fp32 [B, 1, C] or [B, S, C] or None."""
    if not _native(x) or x.dtype != torch.bfloat16:
        r = x.float() + (y.float() if gate is None else gate.float() * y.float())
        return r.to(x.dtype)
    lib = native.load()
    C = x.shape[-1]
    x2, y2 = x.reshape(-1, C).contiguous(), y.reshape(-1, C).contiguous()
    rows = x2.shape[0]
    out = torch.empty_like(x2)
    gp, ldg, rpg = None, 0, 1
    if gate is not None:
        g2 = gate.float().reshape(-1, C).contiguous()
        gp, ldg, rpg = g2.data_ptr(), C, rows // g2.shape[0]
    code = lib.tfb_gated_residual(x2.data_ptr(), y2.data_ptr(), out.data_ptr(), rows, C, gp, ldg, rpg,
                                  native.stream_ptr())  # fmt: skip
    native.check(code, "tfb_gated_residual")
    return out.view(x.shape)


_ACTS = {"silu": 0, "gelu_tanh": 1, "gelu": 2}


def act_mul_reference(x, act="silu"):
    d = x.shape[-1] // 2
    a, g = x[..., :d].float(), x[..., d:].float()
    if act == "silu":
        a = F.silu(a)
    elif act == "gelu_tanh":
        a = F.gelu(a, approximate="tanh")
    else:
        a = F.gelu(a)
    return (a * g).to(x.dtype)


def act_mul(x, act="silu"):
    """``act(x[..., :d]) * x[..., d:]`` (silu_and_mul / gelu_and_mul of the reference)."""
    if not _native(x) or x.dtype != torch.bfloat16 or (x.shape[-1] // 2) % 8:
        return act_mul_reference(x, act)
    lib = native.load()
    d = x.shape[-1] // 2
    x2 = x.reshape(-1, 2 * d).contiguous()
    out = torch.empty(x2.shape[0], d, device=x.device, dtype=x.dtype)
    code = lib.tfb_act_mul(x2.data_ptr(), out.data_ptr(), x2.shape[0], d, _ACTS[act], native.stream_ptr())
    native.check(code, "tfb_act_mul")
    return out.view(*x.shape[:-1], d)


def silu_and_mul(x):
    return act_mul(x, "silu")


def gelu_and_mul(x, approximate="none"):
    return act_mul(x, "gelu_tanh" if approximate == "tanh" else "gelu")


def cfg_euler_step_reference(x, cond, uncond, cfg_scale, dsigma):
    c = cond.float()
    v = c if uncond is None else uncond.float() + cfg_scale * (c - uncond.float())
    return x.float() + v * dsigma, v


def cfg_euler_step(x, cond, uncond, cfg_scale, dsigma, return_v=False):
    """Guidance ``u + s(c-u)`` and Euler update ``x + v*dsigma`` in one pass over fp32 latents."""
    if not _native(x) or x.dtype != torch.float32:
        xo, v = cfg_euler_step_reference(x, cond, uncond, cfg_scale, dsigma)
        xo = xo.to(x.dtype)
        return (xo, v) if return_v else xo
    lib = native.load()
    cond = cond.contiguous()
    if uncond is not None:
        uncond = uncond.contiguous()
        if uncond.dtype != cond.dtype:
            uncond = uncond.to(cond.dtype)
    if cond.dtype not in (torch.bfloat16, torch.float32):
        cond = cond.float()
        uncond = None if uncond is None else uncond.float()
    x = x.contiguous()
    xo = torch.empty_like(x)
    v = torch.empty_like(x) if return_v else None
    code = lib.tfb_cfg_euler_step(
        x.data_ptr(), cond.data_ptr(), native.ptr(uncond), 1 if cond.dtype == torch.bfloat16 else 0,
        float(cfg_scale), float(dsigma), xo.data_ptr(), native.ptr(v), x.numel(), native.stream_ptr())  # fmt: skip
    native.check(code, "tfb_cfg_euler_step")
    return (xo, v) if return_v else xo


# ---------------------------------------------------------------------------
# Causal 3-D convolution (VAE)
# ---------------------------------------------------------------------------
def conv3d_causal_reference(x, weight, bias=None, prev=None, residual=None, pad_t=None):
    """x [B, Cin, T, H, W], weight [Cout, Cin, kt, kh, kw], stride 1: zero padding (kh-1)/2, (kw-1)/2 in space and
    `pad_t` (default kt - 1) frames in front in time, of which the last `prev.shape[2]` are the frames of `prev`."""
    kt, kh, kw = weight.shape[2:]
    pad_t = kt - 1 if pad_t is None else pad_t
    xf = x.float()
    if prev is not None and pad_t > 0:
        prev = prev[:, :, -pad_t:]
        xf = torch.cat([prev.float().to(x.device), xf], dim=2)
        pad_t -= prev.shape[2]
    xf = F.pad(xf, ((kw - 1) // 2, (kw - 1) // 2, (kh - 1) // 2, (kh - 1) // 2, pad_t, 0))
    y = F.conv3d(xf, weight.float(), None if bias is None else bias.float())
    if residual is not None:
        y = y + residual.float()
    return y.to(x.dtype)


def conv_weight_taps(weight: torch.Tensor) -> torch.Tensor:
    """[Cout, Cin, kt, kh, kw] -> [Cout, kt*kh*kw, Cin] bf16 contiguous, the operand layout of the native kernel."""
    co, ci = weight.shape[:2]
    return weight.detach().reshape(co, ci, -1).permute(0, 2, 1).to(torch.bfloat16).contiguous()


def conv3d_causal(x, weight, bias=None, prev=None, residual=None, pad_t=None, weight_taps=None):
    """Causal stride-1 3-D convolution on the tensor cores. Tensors are logically [B, C, T, H, W]; CUDA bf16 inputs are
    used in channels-last-3d memory (converted when they are not) and the result comes back in that format, so a chain
    of convolutions, norms and activations never changes layout. Spatial and causal padding are produced by the
    loads' out-of-range fill (no padded copy); `prev` (the last frames of the previous chunk) is read in place.
    Other inputs take the fp32 evaluation. `weight_taps`: cached `conv_weight_taps(weight)`."""
    co, ci, kt, kh, kw = weight.shape
    pad_t = kt - 1 if pad_t is None else pad_t
    ok = (_native(x) and x.dtype == torch.bfloat16 and ci % 8 == 0 and ci >= 8 and (co % 8 == 0 or co <= 32)
          and kh % 2 == 1 and kw % 2 == 1)  # fmt: skip
    if not ok:
        return conv3d_causal_reference(x, weight, bias, prev, residual, pad_t)
    B, _, T, H, W = x.shape
    cl = torch.channels_last_3d
    x = x.contiguous(memory_format=cl)
    prev_T = 0
    if prev is not None and pad_t > 0:
        prev = prev[:, :, -pad_t:].to(device=x.device, dtype=x.dtype).contiguous(memory_format=cl)
        if prev.shape[2] > 1 and not prev.permute(0, 2, 3, 4, 1).is_contiguous():
            prev = prev.permute(0, 2, 3, 4, 1).contiguous().permute(0, 4, 1, 2, 3)
        prev_T = prev.shape[2]
    if residual is not None:
        residual = residual.to(x.dtype).contiguous(memory_format=cl)
    wt = weight_taps if weight_taps is not None else conv_weight_taps(weight)
    if bias is not None and bias.dtype != torch.bfloat16:
        bias = bias.to(torch.bfloat16)
    out = torch.empty((B, co, T, H, W), device=x.device, dtype=torch.bfloat16, memory_format=cl)
    native.same_device(x, wt, bias, prev, residual)
    code = native.load().tfb_conv3d_causal(x.data_ptr(), native.ptr(prev) if prev_T else None, prev_T, wt.data_ptr(),
                                           native.ptr(bias), native.ptr(residual), out.data_ptr(), B, T, H, W, ci, co, kt, kh,
                                           kw, pad_t, (kh - 1) // 2, (kw - 1) // 2, native.stream_ptr())  # fmt: skip
    native.check(code, "tfb_conv3d_causal")
    return out


def pixel_norm_act(x, gamma, silu: bool = True):
    """x [B, C, ...] (channel dim 1): per-position L2 normalisation over the channels times sqrt(C) * gamma, then SiLU
    when asked: the norm + activation pair in front of every convolution of the video VAE, one pass instead of five.
    CUDA bf16 tensors are used in channels-last memory (2-D or 3-D) and stay in it."""
    C = x.shape[1]
    g = gamma.reshape(-1)
    if not _native(x) or x.dtype != torch.bfloat16 or x.dim() not in (4, 5) or C % 8:
        y = F.normalize(x.float(), dim=1) * (C**0.5) * g.float().view(1, C, *([1] * (x.dim() - 2)))
        return (F.silu(y) if silu else y).to(x.dtype)
    fmt = torch.channels_last_3d if x.dim() == 5 else torch.channels_last
    x = x.contiguous(memory_format=fmt)
    out = torch.empty_like(x, memory_format=fmt)
    gf = g.to(device=x.device, dtype=torch.float32).contiguous()
    code = native.load().tfb_pixel_norm_act(x.data_ptr(), out.data_ptr(), x.numel() // C, C, gf.data_ptr(), int(silu),
                                            native.stream_ptr())  # fmt: skip
    if code == 2:  # a channel count the row kernel has no instance for
        y = F.normalize(x.float(), dim=1) * (C**0.5) * g.float().view(1, C, *([1] * (x.dim() - 2)))
        return (F.silu(y) if silu else y).to(x.dtype)
    native.check(code, "tfb_pixel_norm_act")
    return out


def upsample2x_nearest(x):
    """[N, C, H, W] -> [N, C, 2H, 2W], out(h, w) = in(h // 2, w // 2) (what `nearest-exact` gives at scale 2)."""
    N, C, H, W = x.shape
    if not _native(x) or x.dtype != torch.bfloat16 or C % 8:
        return x.repeat_interleave(2, dim=-2).repeat_interleave(2, dim=-1)
    x = x.contiguous(memory_format=torch.channels_last)
    out = torch.empty((N, C, 2 * H, 2 * W), device=x.device, dtype=x.dtype, memory_format=torch.channels_last)
    native.check(native.load().tfb_upsample2x_nearest(x.data_ptr(), out.data_ptr(), N, H, W, C, native.stream_ptr()),
                 "tfb_upsample2x_nearest")  # fmt: skip
    return out


# ---------------------------------------------------------------------------
# MXFP8 quantisation
# ---------------------------------------------------------------------------
def quant_mxfp8_reference(x):
    """Returns (e4m3 payload as uint8 [rows, C], UE8M0 scales uint8 [rows, C/32])."""
    C = x.shape[-1]
    xf = x.float().reshape(-1, C // 32, 32)
    amax = xf.abs().amax(-1)
    e = torch.where(amax > 0, torch.ceil(torch.log2(amax / 448.0)), torch.zeros_like(amax)).clamp(-126, 126)
    q = (xf * torch.exp2(-e)[..., None]).clamp(-448, 448).to(torch.float8_e4m3fn)
    return q.view(torch.uint8).reshape(-1, C), (e + 127).to(torch.uint8)


def dequant_mxfp8(q, sf):
    C = q.shape[-1]
    v = q.view(torch.float8_e4m3fn).float().reshape(-1, C // 32, 32)
    return (v * torch.exp2(sf.float() - 127)[..., None]).reshape(-1, C)


def mx_tile_scales(sf: torch.Tensor) -> torch.Tensor:
    """Row-major UE8M0 scales [rows, C/32] (C a multiple of 128) -> the tiled order of the block-scaled GEMM:
    uint8 [ceil(rows/128), C/128, 512], row r / block b of a tile at (r%32)*16 + (r/32)*4 + b. Rows of padding
    get the exponent 0 (scale 2^-127)."""
    rows, nb = sf.shape
    if nb % 4:
        raise ValueError("the tiled scale layout needs a multiple of 128 columns")
    mt = -(-rows // 128)
    full = torch.zeros(mt * 128, nb, dtype=torch.uint8, device=sf.device)
    full[:rows] = sf
    # [mt, r/32 (4), r%32 (32), kb, b (4)] -> [mt, kb, r%32, r/32, b]
    return full.view(mt, 4, 32, nb // 4, 4).permute(0, 3, 2, 1, 4).contiguous().view(mt, nb // 4, 512)


def mx_untile_scales(tiled: torch.Tensor, rows: int) -> torch.Tensor:
    mt, kb, _ = tiled.shape
    return tiled.view(mt, kb, 32, 4, 4).permute(0, 3, 2, 1, 4).reshape(mt * 128, kb * 4)[:rows].contiguous()


def quant_mxfp8(x, tiled: bool = False):
    """x [..., C] -> (e4m3 payload uint8 [rows, C], UE8M0 scales). `tiled=False`: scales [rows, C/32];
    `tiled=True`: the order read by the block-scaled GEMM (`mx_tile_scales`), written directly by the kernel."""
    C = x.shape[-1]
    if not _native(x) or x.dtype != torch.bfloat16:
        q, sf = quant_mxfp8_reference(x)
        return (q, mx_tile_scales(sf)) if tiled else (q, sf)
    lib = native.load()
    x2 = x.reshape(-1, C)
    if x2.stride(-1) != 1 or x2.stride(0) % 8:
        x2 = x2.contiguous()
    rows = x2.shape[0]
    q = torch.empty(rows, C, device=x.device, dtype=torch.uint8)
    if tiled:
        sf = torch.zeros(-(-rows // 128), C // 128, 512, device=x.device, dtype=torch.uint8)
    else:
        sf = torch.empty(rows, C // 32, device=x.device, dtype=torch.uint8)
    code = lib.tfb_quant_mxfp8(x2.data_ptr(), x2.stride(0), q.data_ptr(), sf.data_ptr(), rows, C, int(tiled),
                               native.stream_ptr())  # fmt: skip
    native.check(code, "tfb_quant_mxfp8")
    return q, sf


def quantize_weight_mxfp8(w: torch.Tensor):
    """[N, K] (K a multiple of 128) -> (e4m3 [N, K], tiled UE8M0 scales uint8 [ceil(N/128), K/128, 512])."""
    q, sf = quant_mxfp8_reference(w) if not (w.is_cuda and w.dtype == torch.bfloat16) else quant_mxfp8(w)
    return q.view(torch.float8_e4m3fn).reshape(w.shape), mx_tile_scales(sf.reshape(w.shape[0], -1))


def linear_mxfp8(x, weight, weight_sf, bias=None, act=None, residual=None, gate=None):
    """Block-scaled W8A8: weight e4m3 [N, K] with tiled UE8M0 scales per 32 K-elements (`quantize_weight_mxfp8`);
    activations are quantised to the same format on the fly (one scale per token and 32 channels) and both scalings
    happen inside the tensor core. Epilogue as `linear`."""
    K, N = x.shape[-1], weight.shape[0]
    if act not in (None, "gelu_tanh"):
        raise ValueError(f"unknown activation {act}")
    if not _native(x) or x.dtype != torch.bfloat16 or K % 128 or N % 8:
        xq, xsf = quant_mxfp8_reference(x)
        wsf = mx_untile_scales(weight_sf, N)
        y = dequant_mxfp8(xq, xsf) @ dequant_mxfp8(weight.view(torch.uint8).reshape(N, K), wsf).t()
        y = y.reshape(*x.shape[:-1], N)
        if bias is not None:
            y = y + bias.float()
        if act == "gelu_tanh":
            y = F.gelu(y, approximate="tanh")
        if gate is not None:
            y = y * gate.float()
        if residual is not None:
            y = y + residual.float()
        return y.to(x.dtype)
    q, sf = quant_mxfp8(x.reshape(-1, K), tiled=True)
    M = q.shape[0]
    out = torch.empty(*x.shape[:-1], N, device=x.device, dtype=torch.bfloat16)
    res2 = None if residual is None else residual.reshape(-1, N).contiguous()
    gate_ptr, ldg, rpg, g2 = None, 0, 1, None
    if gate is not None:
        g2 = gate.float().reshape(-1, N).contiguous()
        gate_ptr, ldg, rpg = g2.data_ptr(), N, M // g2.shape[0]
    if bias is not None and bias.dtype != torch.bfloat16:
        bias = bias.to(torch.bfloat16)
    w = weight if weight.stride(-1) == 1 else weight.contiguous()
    native.same_device(x, w, weight_sf, bias, res2, g2)
    code = native.load().tfb_gemm_mxfp8(q.data_ptr(), K, sf.data_ptr(), w.data_ptr(), w.stride(0), weight_sf.data_ptr(),
                                        out.data_ptr(), N, M, N, K, native.ptr(bias), 1 if act == "gelu_tanh" else 0,
                                        native.ptr(res2), N if res2 is not None else 0, gate_ptr, ldg, rpg,
                                        native.stream_ptr())  # fmt: skip
    native.check(code, "tfb_gemm_mxfp8")
    return out


# ---------------------------------------------------------------------------
# Streaming / caching ops
# ---------------------------------------------------------------------------
def fp8_kv_quant(x):
    """x: [..., D] -> (e4m3 [..., D], fp32 scale [..., 1]); scale = amax over D / 448 (floor 1e-12)."""
    D = x.shape[-1]
    if not _native(x) or x.dtype != torch.bfloat16 or D % 32 or D > 256:
        scale = (x.detach().abs().amax(dim=-1, keepdim=True).float() / 448.0).clamp_min(1e-12)
        return (x / scale.to(x.dtype)).to(torch.float8_e4m3fn).contiguous(), scale.contiguous()
    xc = x.contiguous()
    q = torch.empty(xc.shape, device=x.device, dtype=torch.float8_e4m3fn)
    scale = torch.empty(*xc.shape[:-1], 1, device=x.device, dtype=torch.float32)
    code = native.load().tfb_fp8_kv_quant(xc.data_ptr(), q.data_ptr(), scale.data_ptr(), xc.numel() // D, D,
                                          native.stream_ptr())  # fmt: skip
    native.check(code, "tfb_fp8_kv_quant")
    return q, scale


def kv_cache_roll_append(k_cache, v_cache, new_k, new_v, sink: int, evicted: int, keep: int, local_start: int):
    """In-place: shift `keep` tokens left by `evicted` (starting after `sink`), then write new_k/new_v
    ([B, n, H, D]) at token `local_start`. k_cache / v_cache: [B, kv_size, H, D]."""
    n = new_k.shape[1]
    native_ok = (_native(k_cache) and k_cache.dtype == torch.bfloat16 and new_k.dtype == torch.bfloat16
                 and new_v.dtype == torch.bfloat16 and n > 0 and k_cache.is_contiguous()
                 and v_cache.is_contiguous() and new_k.stride() == new_v.stride() and new_k.stride(-1) == 1
                 and new_k.stride(2) == new_k.shape[3] and (k_cache.shape[2] * k_cache.shape[3]) % 8 == 0
                 and new_k.stride(1) % 8 == 0 and new_k.stride(0) % 8 == 0 and new_k.data_ptr() % 16 == 0
                 and new_v.data_ptr() % 16 == 0)  # fmt: skip
    if not native_ok:
        if evicted > 0 and keep > 0:
            for done in range(0, keep, evicted):  # pieces whose source and destination do not overlap
                ln = min(evicted, keep - done)
                d, s = sink + done, sink + done + evicted
                k_cache[:, d : d + ln] = k_cache[:, s : s + ln]
                v_cache[:, d : d + ln] = v_cache[:, s : s + ln]
        k_cache[:, local_start : local_start + n] = new_k
        v_cache[:, local_start : local_start + n] = new_v
        return
    B, _, H, D = k_cache.shape
    code = native.load().tfb_kv_cache_roll_append(
        k_cache.data_ptr(), v_cache.data_ptr(), k_cache.stride(0), new_k.data_ptr(), new_v.data_ptr(), new_k.stride(1),
        new_k.stride(0) if B > 1 else n * new_k.stride(1), B, H * D, sink, evicted, keep, local_start, n,
        native.stream_ptr())  # fmt: skip
    native.check(code, "tfb_kv_cache_roll_append")


def taylor_update_(out, ori, terms: list, n_old: int, n_new: int, window: float) -> None:
    """In place on the bf16 term buffers: terms[0] = out - ori; terms[i+1] = (new[i] - old[i]) / window."""
    if _native(out) and out.dtype == torch.bfloat16 and out.numel() % 8 == 0 and out.is_contiguous() \
            and ori.is_contiguous():  # fmt: skip
        p = [t.data_ptr() if t is not None else None for t in (terms + [None] * 4)[:4]]
        code = native.load().tfb_taylor_update(out.data_ptr(), ori.data_ptr(), p[0], p[1], p[2], p[3], n_old, n_new,
                                               float(window), out.numel(), native.stream_ptr())  # fmt: skip
        native.check(code, "tfb_taylor_update")
        return
    cur = out - ori
    for i in range(n_new):
        old = terms[i].clone() if (i < n_old and i + 1 < n_new) else None
        terms[i].copy_(cur)
        if old is None:
            break
        cur = (cur - old) / window


def taylor_apply(x, terms: list, coefs: list):
    """x + sum_i terms[i] * coefs[i]."""
    if _native(x) and x.dtype == torch.bfloat16 and x.numel() % 8 == 0 and x.is_contiguous():
        p = [t.data_ptr() for t in terms] + [None] * (4 - len(terms))
        c = [float(v) for v in coefs] + [0.0] * (4 - len(coefs))
        y = torch.empty_like(x)
        code = native.load().tfb_taylor_apply(x.data_ptr(), p[0], p[1], p[2], p[3], c[0], c[1], c[2], c[3], len(terms),
                                              y.data_ptr(), x.numel(), native.stream_ptr())  # fmt: skip
        native.check(code, "tfb_taylor_apply")
        return y
    r = None
    for t, c in zip(terms, coefs):
        r = t * c if r is None else r + t * c
    return x + r


def plucker_fold(c2ws, ks, latent_h: int, latent_w: int, height: int, width: int, only_rays_d=False, extra=None):
    """Camera poses [F,4,4] + intrinsics [F,4] -> ray maps folded to [1, C*c1*c2, F, h, w] (fp32), with
    optional per-frame extra channels [F, n] appended after the ray channels. CUDA tensors only."""
    F_ = c2ws.shape[0]
    c1, c2 = max(1, height // latent_h), max(1, width // latent_w)
    n_extra = 0 if extra is None else extra.shape[-1]
    C = (3 if only_rays_d else 6) + n_extra
    out = torch.empty(1, C * c1 * c2, F_, latent_h, latent_w, device=c2ws.device, dtype=torch.float32)
    e = None if extra is None else extra.float().contiguous()
    code = native.load().tfb_plucker_fold(c2ws.float().contiguous().data_ptr(), ks.float().contiguous().data_ptr(),
                                          native.ptr(e), n_extra, out.data_ptr(), F_, latent_h, latent_w, c1, c2,
                                          int(only_rays_d), native.stream_ptr())  # fmt: skip
    native.check(code, "tfb_plucker_fold")
    return out


def frames_to_uint8(frames):
    """[3, T, H, W] in [-1, 1] -> uint8 [T, H, W, 3]."""
    if not _native(frames) or frames.dtype not in (torch.bfloat16, torch.float32) or frames.shape[-1] % 4:
        return ((frames.float() + 1) * 127.5).round().clamp(0, 255).to(torch.uint8).permute(1, 2, 3, 0).contiguous()
    f = frames.contiguous()
    _, T, H, W = f.shape
    out = torch.empty(T, H, W, 3, device=f.device, dtype=torch.uint8)
    code = native.load().tfb_frames_to_u8(f.data_ptr(), int(f.dtype == torch.bfloat16), out.data_ptr(), T, H, W,
                                          native.stream_ptr())  # fmt: skip
    native.check(code, "tfb_frames_to_u8")
    return out


# ---------------------------------------------------------------------------
# RMSNorm block glue (sandwich-norm DiTs)
# ---------------------------------------------------------------------------
def _rms(x, w, eps):
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w.float()


def _table(t, rows):
    """fp32 [B, S|1, C] (or [rows|1, C]) table -> (contiguous 2-D view, row stride, rows per table row)."""
    t2 = t.float().reshape(-1, t.shape[-1]).contiguous()
    return t2, t2.shape[-1], max(1, rows // t2.shape[0])


def rmsnorm_modulate(x, weight=None, shift=None, scale=None, eps=1e-6):
    """(w * rmsnorm(x)) * (1 + scale) + shift; x [..., C] bf16 on CUDA, fp32 weight / tables."""
    if not _native(x) or x.dtype != torch.bfloat16 or x.shape[-1] % 8 or x.shape[-1] > 8192:
        y = _rms(x, weight, eps)
        if scale is not None:
            y = y * (1.0 + scale.float())
        if shift is not None:
            y = y + shift.float()
        return y.to(x.dtype)
    C = x.shape[-1]
    x2 = x.reshape(-1, C).contiguous()
    rows = x2.shape[0]
    out = torch.empty_like(x2)
    w = None if weight is None else weight.float().contiguous()
    sh = sc = None
    ld, rpm = C, 1
    if shift is not None:
        sh, ld, rpm = _table(shift, rows)
    if scale is not None:
        sc, ld, rpm = _table(scale, rows)
    code = native.load().tfb_rmsnorm_modulate(x2.data_ptr(), C, out.data_ptr(), C, rows, C, float(eps), native.ptr(w),
                                              native.ptr(sh), native.ptr(sc), ld, rpm, native.stream_ptr())  # fmt: skip
    native.check(code, "tfb_rmsnorm_modulate")
    return out.view(x.shape)


def rmsnorm_gate_residual(res, y, weight=None, gate=None, eps=1e-6, tanh_gate=True):
    """res + tanh(gate) * (w * rmsnorm(y))."""
    if not _native(y) or y.dtype != torch.bfloat16 or res.dtype != torch.bfloat16 or y.shape[-1] % 8 or y.shape[-1] > 8192:
        n = _rms(y, weight, eps)
        if gate is not None:
            n = (gate.float().tanh() if tanh_gate else gate.float()) * n
        return (res.float() + n).to(res.dtype)
    C = y.shape[-1]
    y2, r2 = y.reshape(-1, C).contiguous(), res.reshape(-1, C).contiguous()
    rows = y2.shape[0]
    out = torch.empty_like(r2)
    w = None if weight is None else weight.float().contiguous()
    g, ld, rpg = None, C, 1
    if gate is not None:
        g, ld, rpg = _table(gate, rows)
    code = native.load().tfb_rmsnorm_gate_residual(y2.data_ptr(), C, r2.data_ptr(), C, out.data_ptr(), C, rows, C,
                                                   float(eps), native.ptr(w), native.ptr(g), ld, rpg, int(tanh_gate),
                                                   native.stream_ptr())  # fmt: skip
    native.check(code, "tfb_rmsnorm_gate_residual")
    return out.view(res.shape)


def headnorm_rope_(q, weight_q, cos=None, sin=None, eps=1e-6, k=None, weight_k=None):
    """In place on q (and k): per-head RMSNorm over the last dim, then interleaved-pair RoPE.
    q / k: [B, S, H, D] views (possibly slices of one fused buffer); cos / sin: fp32 [B*S, D/2]."""
    B, S, H, D = q.shape

    def ref(t, w):
        y = _rms(t, w, eps)
        if cos is not None:
            y = rope_reference(y.reshape(1, B * S, H, D), cos, sin).reshape(B, S, H, D)
        t.copy_(y.to(t.dtype))

    ok = (_native(q) and q.dtype == torch.bfloat16 and D % 64 == 0 and D <= 256 and q.stride(-1) == 1
          and q.stride(2) == D and (B == 1 or q.stride(0) == S * q.stride(1)))  # fmt: skip
    if k is not None:
        ok = ok and k.stride() == q.stride() and k.dtype == q.dtype
    if not ok:
        ref(q, weight_q)
        if k is not None:
            ref(k, weight_k)
        return
    nmat, stride = 1, 0
    if k is not None:
        delta = (k.data_ptr() - q.data_ptr()) // 2
        if 0 < delta < q.stride(1):
            nmat, stride = 2, delta
    lib = native.load()
    c = None if cos is None else cos.float().contiguous()
    s = None if sin is None else sin.float().contiguous()
    wq = None if weight_q is None else weight_q.float().contiguous()
    wk = None if weight_k is None else weight_k.float().contiguous()
    code = lib.tfb_headnorm_rope(q.data_ptr(), q.stride(1), stride, nmat, B * S, H, D, float(eps), native.ptr(wq),
                                 native.ptr(wk), native.ptr(c), native.ptr(s), native.stream_ptr())  # fmt: skip
    native.check(code, "tfb_headnorm_rope")
    if k is not None and nmat == 1:
        code = lib.tfb_headnorm_rope(k.data_ptr(), k.stride(1), 0, 1, B * S, H, D, float(eps), native.ptr(wk), None,
                                     native.ptr(c), native.ptr(s), native.stream_ptr())  # fmt: skip
        native.check(code, "tfb_headnorm_rope")
