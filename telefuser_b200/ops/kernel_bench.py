"""Micro-benchmarks of the native kernels against the measured roofline of the machine.

    python -m telefuser_b200.ops.kernel_bench attn  --seq 8192 --heads 12
    python -m telefuser_b200.ops.kernel_bench gemm  --m 8192 --n 5120 --k 5120
    python -m telefuser_b200.ops.kernel_bench elementwise --rows 75600 --dim 5120
    python -m telefuser_b200.ops.kernel_bench moe   --tokens 16384
    python -m telefuser_b200.ops.kernel_bench vae   --frames 17 --height 480 --width 832
    python -m telefuser_b200.ops.kernel_bench all

Timing: CUDA events on the launching stream, `--warmup` untimed launches, then `--iters` timed ones;
between timed launches a 256 MB buffer is rewritten so that the 126 MB L2 does not hold the inputs.
Fractions are of the measured peaks in MEASURED_PEAKS.json at the repository root (copy bandwidth and
cuBLAS bf16 throughput); without that file the stated fallback figures are used and labelled.
Each case prints one JSON line. `--once` runs a single launch per case (for profiler captures).
"""

from __future__ import annotations

import argparse
import json
import os
from pathlib import Path

import torch

from telefuser_b200.ops import functional as TF
from telefuser_b200.ops import moe as MOE


def peaks() -> dict:
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if p.is_file():
        d = json.loads(p.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "label": "of measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "label": "of fallback"}


class Timer:
    def __init__(self, warmup: int, iters: int, once: bool) -> None:
        self.warmup, self.iters = (0, 1) if once else (warmup, iters)
        self.flush = None if once else torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def __call__(self, fn) -> float:
        for _ in range(self.warmup):
            fn()
        torch.cuda.synchronize()
        times = []
        for _ in range(self.iters):
            if self.flush is not None:
                self.flush.fill_(1)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
        times.sort()
        return times[len(times) // 2]  # median, ms


def report(name: str, ms: float, flops: float = 0.0, bytes_: float = 0.0, **cfg) -> None:
    pk = peaks()
    out = {"kernel": name, "ms": round(ms, 4), **cfg}
    if flops:
        tf = flops / ms / 1e9
        out.update(tflops=round(tf, 1), frac_tensor=round(tf / pk["bf16_tflops"], 3))
    if bytes_:
        gbs = bytes_ / ms / 1e6
        out.update(gbs=round(gbs, 1), frac_hbm=round(gbs / pk["hbm_gbs"], 3))
    out["peaks"] = pk["label"]
    print(json.dumps(out), flush=True)


def bench_attn(t: Timer, seq: int, heads: int, compare: bool, variant: int = 0, head_dim: int = 128,
               causal: bool = False) -> None:  # fmt: skip
    q, k, v = (torch.randn(1, seq, heads, head_dim, device="cuda").bfloat16() for _ in range(3))
    flops = 4.0 * seq * seq * heads * head_dim * (0.5 if causal else 1.0)
    variants = [variant] if variant >= 0 else [30, 31, 32, 20, 21, 22]  # -1: every kernel form and exp2 share
    for vr in variants:
        report("attn_fwd_tcgen05", t(lambda: TF.attention(q, k, v, variant=vr, causal=causal)), flops, seq=seq,
               heads=heads, head_dim=head_dim, causal=causal, variant=vr)  # fmt: skip
    if head_dim != 128 or causal:
        return
    if variant == 0 and seq >= 8192:
        from telefuser_b200.ops import sparse_attention as SA

        frames = 16
        mm = SA.RadialMaskMap(seq // frames * frames, frames)
        mask = mm.query_block_mask(seq, 0.5, "cuda")
        lists = SA.lists_from_mask(SA._broadcast_mask(mask, 1, heads))
        dens = mask.float().mean().item()
        report("attn_fwd_tcgen05 block-sparse (radial mask; FLOPs counted for visited blocks only)",
               t(lambda: SA.block_sparse_attention(q, k, v, mask, lists)), flops * dens, seq=seq, heads=heads,
               frames=frames, block_density=round(dens, 3))  # fmt: skip
    if compare:
        qt, kt, vt = (x.transpose(1, 2) for x in (q, k, v))
        fn = lambda: torch.nn.functional.scaled_dot_product_attention(qt, kt, vt)  # noqa: E731
        report("torch_sdpa (library)", t(fn), flops, seq=seq, heads=heads)


def bench_gemm(t: Timer, m: int, n: int, k: int, compare: bool) -> None:
    a = torch.randn(m, k, device="cuda").bfloat16()
    w = (torch.randn(n, k, device="cuda") / k**0.5).bfloat16()
    bias = torch.randn(n, device="cuda").bfloat16()
    flops = 2.0 * m * n * k
    report("gemm_bf16_tcgen05 (+bias, gelu)", t(lambda: TF.linear(a, w, bias, act="gelu_tanh")), flops, m=m, n=n, k=k)
    report("gemm_bf16_tcgen05 (+bias)", t(lambda: TF.linear(a, w, bias)), flops, m=m, n=n, k=k)
    from telefuser_b200.ops.quant import quantize_weight_fp8

    w8, ws = quantize_weight_fp8(w)
    a8, as_ = TF.quant_fp8_rowwise(a)
    report("quant_fp8_rowwise", t(lambda: TF.quant_fp8_rowwise(a)), bytes_=m * k * 3, m=m, k=k)
    report("gemm_fp8_tcgen05 W8A8 (+bias, incl. activation quant)", t(lambda: TF.linear_fp8(a, w8, ws, bias)), flops,
           m=m, n=n, k=k)  # fmt: skip
    lib = TF.native.load()
    out = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
    wsf, asf = ws.reshape(-1).contiguous(), as_.reshape(-1).contiguous()

    def gemm_only():
        lib.tfb_gemm_fp8(a8.data_ptr(), k, w8.data_ptr(), k, out.data_ptr(), n, m, n, k, asf.data_ptr(), wsf.data_ptr(),
                         bias.data_ptr(), 0, None, 0, None, 0, 1, TF.native.stream_ptr())

    report("gemm_fp8_tcgen05 (GEMM only; fraction is of the bf16 peak)", t(gemm_only), flops, m=m, n=n, k=k)
    if k % 128 == 0:
        wq, wsf = TF.quantize_weight_mxfp8(w)
        aq, asf = TF.quant_mxfp8(a, tiled=True)
        report("quant_mxfp8 (tiled scales)", t(lambda: TF.quant_mxfp8(a, tiled=True)), bytes_=m * k * 3 + m * k // 32, m=m, k=k)
        report("gemm_mxfp8_tcgen05 block-scaled (+bias, incl. activation quant)", t(lambda: TF.linear_mxfp8(a, wq, wsf, bias)),
               flops, m=m, n=n, k=k)  # fmt: skip

        def mx_only():
            lib.tfb_gemm_mxfp8(aq.data_ptr(), k, asf.data_ptr(), wq.data_ptr(), k, wsf.data_ptr(), out.data_ptr(), n, m, n, k,
                               bias.data_ptr(), 0, None, 0, None, 0, 1, TF.native.stream_ptr())

        report("gemm_mxfp8_tcgen05 (GEMM only; fraction is of the bf16 peak)", t(mx_only), flops, m=m, n=n, k=k)
    if compare:
        try:  # the library's row-wise FP8 GEMM (cuBLASLt through torch._scaled_mm), same operands and scales
            fn = lambda: torch._scaled_mm(a8, w8.t(), scale_a=as_.reshape(m, 1), scale_b=ws.reshape(1, n), bias=bias,
                                          out_dtype=torch.bfloat16)  # noqa: E731
            report("torch._scaled_mm row-wise FP8 (cuBLASLt, library; fraction is of the bf16 peak)", t(fn), flops, m=m, n=n, k=k)
        except Exception as e:  # noqa: BLE001 - depends on the library build
            print(json.dumps({"kernel": "torch._scaled_mm row-wise FP8", "unavailable": f"{type(e).__name__}: {e}"[:200]}), flush=True)
        report("torch F.linear (cuBLAS)", t(lambda: torch.nn.functional.linear(a, w, bias)), flops, m=m, n=n, k=k)


def bench_elementwise(t: Timer, rows: int, dim: int) -> None:
    x = torch.randn(1, rows, dim, device="cuda").bfloat16()
    y = torch.randn_like(x)
    shift, scale, gate = (torch.randn(1, 1, dim, device="cuda") for _ in range(3))
    nb = rows * dim * 2
    report("layernorm_modulate", t(lambda: TF.layernorm_modulate(x, shift, scale)), bytes_=2 * nb, rows=rows, dim=dim)
    report("gated_residual", t(lambda: TF.gated_residual(x, y, gate)), bytes_=3 * nb, rows=rows, dim=dim)
    h = torch.randn(rows, 2 * dim, device="cuda").bfloat16()
    report("act_mul (silu)", t(lambda: TF.act_mul(h, "silu")), bytes_=3 * nb, rows=rows, dim=dim)
    heads = dim // 128
    qk = torch.randn(1, rows, 2 * dim, device="cuda").bfloat16()
    w = torch.ones(dim, device="cuda").bfloat16()
    cos, sin = torch.randn(rows, 64, device="cuda"), torch.randn(rows, 64, device="cuda")
    q, k = qk[..., :dim], qk[..., dim:]
    report("rmsnorm_rope (q and k)", t(lambda: TF.rmsnorm_rope_(q, w, heads, cos, sin, 1e-6, x2=k, weight2=w)),
           bytes_=4 * nb + 2 * rows * 64 * 4, rows=rows, dim=dim)  # fmt: skip
    report("quant_mxfp8", t(lambda: TF.quant_mxfp8(x)), bytes_=nb + nb // 2 + nb // 64, rows=rows, dim=dim)
    from telefuser_b200.ops import nf4

    wq = torch.randint(0, 256, (4 * dim * dim // 2,), device="cuda", dtype=torch.uint8)  # a [4 dim, dim] MLP weight, packed
    am = torch.rand(4 * dim * dim // 64, device="cuda")
    wout = torch.empty(4 * dim, dim, device="cuda", dtype=torch.bfloat16)
    report("nf4_dequant", t(lambda: nf4.dequantize_nf4(wq, am, wout.shape, out=wout)), bytes_=wq.numel() + am.numel() * 4 + wout.numel() * 2,
           n=4 * dim, k=dim)  # fmt: skip
    lat = torch.randn(1, 16, 21, 90, 160, device="cuda")
    c, u = torch.randn_like(lat).bfloat16(), torch.randn_like(lat).bfloat16()
    report("cfg_euler_step", t(lambda: TF.cfg_euler_step(lat, c, u, 5.0, -0.02)), bytes_=lat.numel() * (4 + 2 + 2 + 4))
    fr = torch.randn(3, 12, 480, 832, device="cuda").bfloat16()
    report("frames_to_uint8", t(lambda: TF.frames_to_uint8(fr)), bytes_=fr.numel() * 3)
    kc, vc = (torch.zeros(1, 32768, heads, 128, device="cuda").bfloat16() for _ in range(2))
    nk, nv = (torch.randn(1, 4680, heads, 128, device="cuda").bfloat16() for _ in range(2))
    keep = 32768 - 4680 - 1560
    report("kv_cache_roll_append", t(lambda: TF.kv_cache_roll_append(kc, vc, nk, nv, 1560, 4680, keep, 32768 - 4680)),
           bytes_=2 * 2 * (keep + 4680) * dim * 2, kv_tokens=32768, new_tokens=4680)  # fmt: skip


def bench_moe(t: Timer, tokens: int, compare: bool) -> None:
    E, K, C, I = 128, 8, 2048, 768
    x = torch.randn(tokens, C, device="cuda").bfloat16()
    w13 = (torch.randn(E, 2 * I, C, device="cuda") / C**0.5).bfloat16()
    w2 = (torch.randn(E, C, I, device="cuda") / I**0.5).bfloat16()
    logits = torch.randn(tokens, E, device="cuda")
    bias = torch.zeros(E, device="cuda")
    report("moe_route (128 experts, 4 groups, top-8)", t(lambda: MOE.route_topk(logits, 4, 2, K, bias, 2.5)),
           bytes_=tokens * E * 4, tokens=tokens)  # fmt: skip
    ids, w, counts = MOE.route_topk(logits, 4, 2, K, bias, 2.5, return_counts=True)
    flops = 2.0 * tokens * K * (2 * I * C + C * I)
    report("moe experts_forward (plan+permute+2 grouped GEMMs+silu+combine)",
           t(lambda: MOE.experts_forward(x, ids, w, w13, w2, counts=counts)), flops, tokens=tokens, experts=E, top_k=K)
    if compare and hasattr(torch, "_grouped_mm"):
        order = ids.reshape(-1).long().argsort(stable=True)
        xs = x[order // K]
        offs = counts.cumsum(0).to(torch.int32)

        def lib():
            g = torch._grouped_mm(xs, w13.transpose(-2, -1), offs=offs)
            h = torch.nn.functional.silu(g[:, :I]) * g[:, I:]
            return torch._grouped_mm(h, w2.transpose(-2, -1), offs=offs)

        try:
            report("torch._grouped_mm x2 + silu (library, no permute/combine)", t(lib), flops, tokens=tokens)
        except Exception as e:  # noqa: BLE001
            print(json.dumps({"kernel": "torch._grouped_mm", "unavailable": str(e)[:120]}))


def bench_vae(t: Timer, frames: int, height: int, width: int, compare: bool) -> None:
    """Wan VAE decode of `frames` video frames at height x width (random-init weights, bf16): the native path
    (implicit-GEMM convolutions, fused norm + SiLU, channels-last) against the same module on the library path
    (cuDNN convolutions, torch elementwise ops), plus the single convolution that dominates it."""
    from telefuser_b200.models.wan_vae import WanVideoVAE
    from telefuser_b200.testing.synthetic import random_init_

    vae = random_init_(WanVideoVAE().to("cuda").to(torch.bfloat16), 0, std=0.03).eval()
    z = torch.randn(1, 16, (frames - 1) // 4 + 1, height // 8, width // 8, device="cuda").bfloat16()
    out_bytes = 3 * frames * height * width * 2
    with torch.no_grad():
        ms = t(lambda: vae.model.decode(z, vae.scale))
        report("wan_vae_decode native", ms, bytes_=out_bytes, frames=frames, height=height, width=width,
               frames_per_s=round(frames / ms * 1e3, 1))  # fmt: skip
        if compare:
            TF.set_force_reference(True)
            try:
                ms = t(lambda: vae.model.decode(z, vae.scale))
            finally:
                TF.set_force_reference(False)
            report("wan_vae_decode library path (cuDNN + torch ops)", ms, bytes_=out_bytes, frames=frames, height=height,
                   width=width, frames_per_s=round(frames / ms * 1e3, 1))  # fmt: skip
    T = min(frames, 8)
    x = torch.randn(1, 96, T, height, width, device="cuda").bfloat16().contiguous(memory_format=torch.channels_last_3d)
    w = (torch.randn(96, 96, 3, 3, 3, device="cuda") / 50).bfloat16()
    b = torch.zeros(96, device="cuda").bfloat16()
    wt = TF.conv_weight_taps(w)
    flops = 2.0 * T * height * width * 96 * 96 * 27
    report("conv3d_tcgen05 96->96 3x3x3 (full resolution)", t(lambda: TF.conv3d_causal(x, w, b, weight_taps=wt)), flops,
           frames=T, height=height, width=width)  # fmt: skip
    if compare:
        xp = torch.nn.functional.pad(x, (1, 1, 1, 1, 2, 0)).contiguous(memory_format=torch.channels_last_3d)
        report("torch conv3d (cuDNN, library; input already padded)", t(lambda: torch.nn.functional.conv3d(xp, w, b)), flops,
               frames=T, height=height, width=width)  # fmt: skip


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["attn", "gemm", "elementwise", "moe", "vae", "all"])
    ap.add_argument("--frames", type=int, default=17)
    ap.add_argument("--height", type=int, default=480)
    ap.add_argument("--width", type=int, default=832)
    ap.add_argument("--seq", type=int, default=8192)
    ap.add_argument("--heads", type=int, default=12)
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=5120)
    ap.add_argument("--k", type=int, default=5120)
    ap.add_argument("--rows", type=int, default=75600)
    ap.add_argument("--dim", type=int, default=5120)
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--variant", type=int, default=0, help="attention kernel variant (0 = default, -1 = all forms)")
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--causal", action="store_true")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--once", action="store_true", help="one launch per case, no flush, no comparison")
    ap.add_argument("--no-compare", action="store_true", help="skip the library kernels")
    a = ap.parse_args()
    os.environ.setdefault("CUDA_MODULE_LOADING", "LAZY")
    torch.manual_seed(0)
    t = Timer(a.warmup, a.iters, a.once)
    cmp_ = not (a.once or a.no_compare)
    if a.what in ("attn", "all"):
        bench_attn(t, a.seq, a.heads, cmp_, a.variant, a.head_dim, a.causal)
    if a.what in ("gemm", "all"):
        bench_gemm(t, a.m, a.n, a.k, cmp_)
    if a.what in ("elementwise", "all"):
        bench_elementwise(t, a.rows, a.dim)
    if a.what in ("moe", "all"):
        bench_moe(t, a.tokens, cmp_)
    if a.what == "vae":
        bench_vae(t, a.frames, a.height, a.width, cmp_)


if __name__ == "__main__":
    main()
