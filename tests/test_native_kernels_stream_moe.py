"""GPU numerics of the streaming / caching kernels and the mixture-of-experts kernels against plain
PyTorch references of the same ops."""

import pytest
import torch

pytestmark = pytest.mark.gpu

from telefuser_b200.ops import functional as TF  # noqa: E402
from telefuser_b200.ops import moe as MOE  # noqa: E402

DEV = "cuda"


def test_merge_attn_states_matches_reference():
    torch.manual_seed(0)
    B, S, H, D = 2, 333, 3, 128
    o1, o2 = (torch.randn(B, S, H, D, device=DEV).bfloat16() for _ in range(2))
    l1, l2 = (torch.randn(B, H, S, device=DEV) * 3 for _ in range(2))
    o, lse = TF.merge_attn_states(o1, l1, o2, l2)
    ro, rl = TF.merge_attn_states_reference(o1, l1, o2, l2)
    assert (o.float() - ro.float()).abs().max() <= 2e-2
    assert (lse - rl).abs().max() <= 1e-4


def test_fp8_kv_quant_matches_reference():
    torch.manual_seed(0)
    x = (torch.randn(2, 257, 5, 128, device=DEV) * 4).bfloat16()
    x[0, 0, 0] = 0  # all-zero row: scale floor
    q, s = TF.fp8_kv_quant(x)
    scale = (x.abs().amax(dim=-1, keepdim=True).float() / 448.0).clamp_min(1e-12)
    rq = (x / scale.to(x.dtype)).to(torch.float8_e4m3fn)
    assert q.dtype == torch.float8_e4m3fn and s.shape == (2, 257, 5, 1)
    assert torch.allclose(s, scale, rtol=1e-6, atol=0)
    mism = (q.view(torch.uint8) != rq.view(torch.uint8)).float().mean().item()
    assert mism < 1e-3, mism
    back = q.float() * s
    assert (back - x.float()).abs().max() <= x.float().abs().max() * 0.07


def test_kv_cache_roll_append_matches_slicing():
    torch.manual_seed(0)
    B, size, H, D, sink = 1, 40, 2, 128, 4
    k = torch.randn(B, size, H, D, device=DEV).bfloat16()
    v = torch.randn(B, size, H, D, device=DEV).bfloat16()
    qkv = torch.randn(B, 6, 3 * H * D, device=DEV).bfloat16()  # new k/v as column slices of a fused buffer
    nk = qkv[..., H * D : 2 * H * D].unflatten(-1, (H, D))
    nv = qkv[..., 2 * H * D :].unflatten(-1, (H, D))
    for evicted, keep, lo in ((6, 30, 34), (5, 31, 34), (0, 0, 10), (3, 2, 9)):
        rk, rv = k.clone(), v.clone()
        if evicted and keep:
            rk[:, sink : sink + keep] = k[:, sink + evicted : sink + evicted + keep]
            rv[:, sink : sink + keep] = v[:, sink + evicted : sink + evicted + keep]
        rk[:, lo : lo + 6], rv[:, lo : lo + 6] = nk, nv
        gk, gv = k.clone(), v.clone()
        TF.kv_cache_roll_append(gk, gv, nk, nv, sink, evicted, keep, lo)
        assert torch.equal(gk, rk) and torch.equal(gv, rv), (evicted, keep, lo)


def test_rolling_cache_native_equals_cpu_semantics():
    from telefuser_b200.cache.rolling_kv import RollingKVCache

    torch.manual_seed(0)
    cg = RollingKVCache(1, 24, 2, 128, DEV, torch.bfloat16, sink_tokens=4)
    cc = RollingKVCache(1, 24, 2, 128, "cpu", torch.bfloat16, sink_tokens=4)
    pos = 0
    for _ in range(6):
        k, v = torch.randn(1, 6, 2, 128).bfloat16(), torch.randn(1, 6, 2, 128).bfloat16()
        for _rep in range(2):  # the same chunk position is written more than once
            cg.append(k.to(DEV), v.to(DEV), pos)
            cc.append(k, v, pos)
        pos += 6
        assert cg.local_end == cc.local_end
        assert torch.equal(cg.k.cpu(), cc.k) and torch.equal(cg.v.cpu(), cc.v)


def test_taylor_update_apply_match_reference():
    torch.manual_seed(0)
    n = 8 * 1001
    hist = [torch.randn(n, device=DEV).bfloat16() for _ in range(3)]
    out, ori, x = (torch.randn(n, device=DEV).bfloat16() for _ in range(3))
    for n_old, n_new, window in ((0, 1, 1), (1, 2, 3), (2, 3, 2), (3, 3, 5)):
        terms = [h.clone() for h in hist]
        ref = [h.clone() for h in hist]
        cur = out - ori
        for i in range(n_new):
            old = ref[i].clone() if (i < n_old and i + 1 < n_new) else None
            ref[i].copy_(cur)
            if old is None:
                break
            cur = (cur - old) / window
        TF.taylor_update_(out, ori, terms, n_old, n_new, float(window))
        for i in range(3):
            assert torch.equal(terms[i], ref[i]), (n_old, n_new, window, i)
    coefs = [1.0, 2.0, 2.0]
    y = TF.taylor_apply(x, hist, coefs)
    want = x.float() + sum(h.float() * c for h, c in zip(hist, coefs))
    assert (y.float() - want).abs().max() <= 6e-2


def test_ada_taylor_cache_fused_tracks_eager():
    from telefuser_b200.feature_cache.ada_taylor import TaylorBranchState

    torch.manual_seed(0)
    kw = dict(num_inference_steps=10, thresh=0.1, K=3, mag_ratios=[1.0] * 10, retention_ratio=0.2, n_derivatives=2)
    fused, eager = TaylorBranchState(**kw), TaylorBranchState(**kw)
    for step in range(8):
        fused.advance(), eager.advance()
        x = torch.randn(1, 64, 256, device=DEV).bfloat16()
        if step in (0, 1, 2, 5):
            out = x + torch.randn_like(x) * 0.1
            fused.update(out, x)
            eager.update(out.float().cpu().bfloat16(), x.float().cpu().bfloat16())
        else:
            a, b = fused.approximate(x), eager.approximate(x.cpu())
            assert (a.float().cpu() - b.float()).abs().max() <= 4e-2


def test_plucker_fold_matches_reference():
    from telefuser_b200.pipelines.lingbot_world import control as C

    torch.manual_seed(0)
    F_, H, W, h, w = 3, 48, 64, 6, 8
    poses = torch.eye(4).repeat(F_, 1, 1)
    poses[:, :3, :3] = torch.linalg.qr(torch.randn(F_, 3, 3)).Q
    poses[:, :3, 3] = torch.randn(F_, 3)
    ks = torch.tensor([[50.0, 55.0, 32.0, 24.0]]).repeat(F_, 1) + torch.rand(F_, 4)
    action = torch.randn(F_, 4)
    ref_cam = C.fold_to_latent_grid(C.plucker_embeddings(poses, ks, H, W), h, w)
    got_cam = C.build_camera_control_chunk(poses.to(DEV), ks.to(DEV), h, w, H, W)
    assert got_cam.shape == ref_cam.shape == (1, 6 * 64, F_, h, w)
    assert (got_cam.cpu() - ref_cam).abs().max() <= 1e-5
    d = C.plucker_embeddings(poses, ks, H, W, only_rays_d=True)
    ref_act = C.fold_to_latent_grid(torch.cat([d, action[:, None, None, :].expand(-1, H, W, -1)], -1), h, w)
    got_act = C.build_action_control_chunk(poses.to(DEV), ks.to(DEV), action.to(DEV), h, w, H, W)
    assert (got_act.cpu() - ref_act).abs().max() <= 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_frames_to_uint8(dtype):
    torch.manual_seed(0)
    f = (torch.rand(3, 5, 36, 64, device=DEV) * 2.4 - 1.2).to(dtype)
    got = TF.frames_to_uint8(f)
    want = ((f.float() + 1) * 127.5).round().clamp(0, 255).to(torch.uint8).permute(1, 2, 3, 0)
    assert got.shape == (5, 36, 64, 3) and got.dtype == torch.uint8
    assert (got.int() - want.int()).abs().max() <= 1
    assert (got != want).float().mean() < 1e-3


@pytest.mark.parametrize("E,G,TG,K,softmax", [(128, 4, 2, 8, False), (64, 1, 1, 6, False), (256, 8, 4, 8, True),
                                              (8, 1, 1, 2, False)])  # fmt: skip
def test_moe_route_matches_reference(E, G, TG, K, softmax):
    torch.manual_seed(0)
    T = 777
    logits = torch.randn(T, E, device=DEV) * 2
    bias = torch.randn(E, device=DEV) * 0.1
    ids, w, counts = MOE.route_topk(logits, G, TG, K, bias, 2.5, softmax, return_counts=True)
    rid, rw = MOE.route_topk_reference(logits, G, TG, K, bias, 2.5, softmax)
    sid, order = ids.long().sort(-1)
    rsid, rorder = rid.sort(-1)
    same = (sid == rsid).all(-1)
    assert same.float().mean() > 0.995  # ties / last-ulp score differences may flip a borderline expert
    assert (w.gather(-1, order)[same] - rw.gather(-1, rorder)[same]).abs().max() <= 1e-4
    assert torch.equal(counts.long(), torch.bincount(ids.reshape(-1).long(), minlength=E))
    assert torch.allclose(w.sum(-1), torch.full((T,), 2.5, device=DEV), atol=1e-4)


def test_grouped_gemm_and_experts_forward():
    torch.manual_seed(0)
    T, C, I, E, K = 1500, 256, 128, 16, 4
    x = torch.randn(T, C, device=DEV).bfloat16()
    w13 = (torch.randn(E, 2 * I, C, device=DEV) / C**0.5).bfloat16()
    w2 = (torch.randn(E, C, I, device=DEV) / I**0.5).bfloat16()
    logits = torch.randn(T, E, device=DEV)
    logits[:, 3] = -30.0  # an expert that receives no token
    ids, w, counts = MOE.route_topk(logits, 1, 1, K, None, 1.0, False, return_counts=True)
    assert counts[3].item() == 0
    res = torch.randn(T, C, device=DEV).bfloat16()
    got = MOE.experts_forward(x, ids, w, w13, w2, counts=counts, residual=res)
    ref = MOE.experts_forward_reference(x.float(), ids.long(), w, w13.float(), w2.float()) + res.float()
    err = (got.float() - ref).abs().max().item()
    assert err <= 6e-2, err
    again = MOE.experts_forward(x, ids, w, w13, w2, counts=counts, residual=res)  # workspace reuse
    assert torch.equal(got, again)
