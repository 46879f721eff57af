"""Block-sparse attention: mask builders (radial, top-k, local window), list conversion, the masked
reference, and on GPUs the sparse tcgen05 kernel against the masked fp32 evaluation."""

import pytest
import torch

from telefuser_b200.ops import functional as TF
from telefuser_b200.ops import sparse_attention as SA


def test_radial_mask_structure():
    frames, tpf, text = 8, 512, 256
    vt = frames * tpf
    s = vt + text
    m = SA.radial_block_mask_128(s, vt, frames, 0.5, "wan")
    nb, vb, fb = s // 128, vt // 128, tpf // 128
    assert m.shape == (nb, nb)
    assert m[vb:].all() and m[:, vb:].all()  # text rows / columns dense
    assert m[:, :fb].all()  # first frame is an attention sink for every row
    for i in range(frames):  # each frame attends to itself and to its neighbours
        for j in (i - 1, i, i + 1):
            if 0 <= j < frames:
                assert m[i * fb : (i + 1) * fb, j * fb : (j + 1) * fb].all(), (i, j)
    far = m[7 * fb : 8 * fb, 3 * fb : 4 * fb]  # distance 4: band of width 128 plus the marked first / last row blocks
    assert not far.all() and far.any()
    assert SA.radial_block_mask_128(s, vt, frames, 1.0, "wan").sum() >= m.sum()  # wider bands with a larger decay factor
    # kernel granularity (256 query rows): needs frames of many blocks to stay sparse, since every frame
    # pair marks its first and last row block
    frames, tpf = 8, 2048
    vt = frames * tpf
    s = vt + 256
    mm = SA.RadialMaskMap(vt, frames)
    k = mm.query_block_mask(s, 0.5)
    assert k.shape == ((s + 255) // 256, (s + 127) // 128) and 0.2 < mm.sparsity(s, 0.5) < 1.0
    assert mm.query_block_mask(s, 0.5) is not None and len(mm._cache) == 1


def test_lists_and_reference_semantics():
    torch.manual_seed(0)
    B, Sq, Skv, H, D = 1, 600, 500, 2, 16
    q, k, v = torch.randn(B, Sq, H, D), torch.randn(B, Skv, H, D), torch.randn(B, Skv, H, D)
    nQ, nK = 3, 4
    mask = torch.zeros(H, nQ, nK, dtype=torch.bool)
    mask[0, 0, [0, 2]] = True
    mask[0, 1, :] = True
    mask[1, :, 3] = True  # head 0 group 2 has no block: zero rows
    idx, cnt = SA.lists_from_mask(mask)
    assert cnt.tolist() == [[2, 4, 0], [1, 1, 1]] and idx[0, 0, :2].tolist() == [0, 2] and idx[1, 2, 0].item() == 3
    out = SA.block_sparse_attention(q, k, v, mask)
    assert out[0, 512:, 0].abs().max() == 0
    full = TF.attention_reference(q, k, v)
    assert torch.allclose(out[0, 256:512, 0], full[0, 256:512, 0], atol=1e-5)  # all blocks listed == dense
    only_last = TF.attention_reference(q[:, :, 1:], k[:, 384:, 1:], v[:, 384:, 1:])
    assert torch.allclose(out[:, :, 1:], only_last, atol=1e-5)


def test_topk_and_local_window_masks():
    torch.manual_seed(0)
    q, k = torch.randn(1, 1024, 2, 16), torch.randn(1, 1024, 2, 16)
    k[:, 640:768] += 3 * q[:, :256].mean(1, keepdim=True)  # key block 5 matches query group 0
    m = SA.topk_block_mask(q, k, sparsity=0.75)
    assert m.shape == (1, 2, 4, 8) and m[..., 0].all() and m[0, :, 0, 5].all()
    assert m[0, 0, 2, 4] and m[0, 0, 2, 5]  # diagonal blocks kept
    assert m.sum(-1).min() >= 2 and m.sum(-1).max() <= 2 + 1 + 2
    lw = SA.local_window_block_mask((4, 16, 16), (1, 16, 16))
    assert lw.shape == (4, 8) and lw[0, 0] and lw[0, 3] and not lw[0, 6] and lw[3, 7]
    pooled = SA.mean_pool_blocks(torch.ones(1, 300, 1, 4), 128)
    assert pooled.shape == (1, 3, 1, 4) and torch.allclose(pooled, torch.ones_like(pooled))


def test_wan_model_routes_to_radial_attention_outside_the_dense_steps():
    from telefuser_b200.testing.distributed_checks import make_tiny_model

    model = make_tiny_model()
    x = torch.randn(1, 16, 4, 32, 32)  # 4 frames x 256 tokens
    ctx, t = torch.randn(1, 8, 256), torch.tensor([500.0])
    dense = model(x, t, ctx)
    model.enable_radial_attention(dense_layers=1, dense_timesteps=2, decay_factor=0.5)
    late = model(x, t, ctx, numeral_timestep=0)  # inside the dense steps
    assert torch.equal(late, dense)
    assert [b.self_attn.sparse_ctx[2] for b in model.blocks] == [True, True]
    early = model(x, t, ctx, numeral_timestep=5)
    assert [b.self_attn.sparse_ctx[2] for b in model.blocks] == [True, False]  # layer 0 stays dense
    assert torch.isfinite(early).all() and early.shape == dense.shape


@pytest.mark.gpu
@pytest.mark.parametrize("Sq,Skv,H", [(1024, 1024, 2), (777, 1300, 3)])
def test_sparse_kernel_matches_masked_reference(Sq, Skv, H):
    torch.manual_seed(0)
    B, D = 2, 128
    q, k, v = (torch.randn(B, s, H, D, device="cuda").bfloat16() for s in (Sq, Skv, Skv))
    nQ, nK = (Sq + 255) // 256, (Skv + 127) // 128
    mask = torch.rand(B, H, nQ, nK, device="cuda") < 0.4
    mask[..., -1] = True  # the ragged last key block
    mask[0, 0, 1] = False  # a query group with nothing to attend to
    out = SA.block_sparse_attention(q, k, v, mask).float()
    ref = SA.block_sparse_attention_reference(q.float(), k.float(), v.float(), mask)
    assert out[0, 256:512, 0].abs().max() == 0
    assert (out - ref).abs().max() <= 3e-2
    dense = SA.block_sparse_attention(q, k, v, torch.ones(nQ, nK, dtype=torch.bool, device="cuda")).float()
    assert (dense - TF.attention(q, k, v).float()).abs().max() <= 1e-2


@pytest.mark.gpu
def test_radial_attention_on_gpu():
    torch.manual_seed(0)
    frames, tpf, text = 6, 640, 256
    s = frames * tpf + text
    q, k, v = (torch.randn(1, s, 2, 128, device="cuda").bfloat16() for _ in range(3))
    mm = SA.RadialMaskMap(frames * tpf, frames)
    out = SA.radial_attention(q, k, v, mm).float()
    ref = SA.block_sparse_attention_reference(q.float(), k.float(), v.float(), mm.query_block_mask(s, 0.5, "cuda"))
    assert (out - ref).abs().max() <= 3e-2
    assert (SA.radial_attention(q, k, v, mm, dense=True).float() - TF.attention(q, k, v).float()).abs().max() == 0


def test_reference_attention_bias_and_blocking_on_cpu():
    torch.manual_seed(0)
    q, k, v = (torch.randn(2, 19, 3, 16) for _ in range(3))
    bias = torch.randn(1, 3, 19, 19)
    want = torch.nn.functional.scaled_dot_product_attention(
        q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), attn_mask=bias, scale=1.0).transpose(1, 2)
    assert torch.allclose(TF.attention(q, k, v, scale=1.0, bias=bias), want, atol=1e-5)
    assert torch.allclose(TF.attention_reference(q, k, v, 1.0, bias=bias, q_block=5), want, atol=1e-5)
    x = torch.randn(4, 24)
    assert torch.allclose(TF.softmax_rows_(x.clone(), 0.3), torch.softmax(x * 0.3, -1), atol=1e-6)
