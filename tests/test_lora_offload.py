"""LoRA merging (key spellings, alpha, diff keys, fp8 weights, run-time network), layer offload
(async ring and sequential) and single-rank weight sharding: outputs must not change."""

import pytest
import torch
from torch import nn

from telefuser_b200.offload import AsyncOffloadManager, enable_sequential_cpu_offload
from telefuser_b200.parallel.fsdp import shard_model
from telefuser_b200.testing.distributed_checks import make_tiny_inputs, make_tiny_model
from telefuser_b200.utils.lora import LoRALoader, create_lora_network


def _tiny_forward(model):
    latents, ctx, _ = make_tiny_inputs()
    return model(latents, torch.tensor([500.0]), ctx)


def test_lora_merge_formats_and_alpha():
    torch.manual_seed(0)
    model = nn.ModuleDict({"blocks": nn.ModuleList([nn.ModuleDict({"q": nn.Linear(8, 8), "k": nn.Linear(8, 8)})])})
    w_q, w_k, b_q = (model["blocks"][0]["q"].weight.clone(), model["blocks"][0]["k"].weight.clone(),
                     model["blocks"][0]["q"].bias.clone())  # fmt: skip
    up, down = torch.randn(8, 2), torch.randn(2, 8)
    up2, down2 = torch.randn(8, 4), torch.randn(4, 8)
    sd = {
        "diffusion_model.blocks.0.q.lora_up.weight": up, "diffusion_model.blocks.0.q.lora_down.weight": down,
        "diffusion_model.blocks.0.q.alpha": torch.tensor(1.0),
        "transformer.blocks.0.k.lora_B.default.weight": up2, "transformer.blocks.0.k.lora_A.default.weight": down2,
        "blocks.0.q.diff_b": torch.ones(8),
        "blocks.9.q.lora_B.weight": up, "blocks.9.q.lora_A.weight": down,
    }  # fmt: skip
    res = LoRALoader().apply_lora(model, sd, strength=0.5)
    assert res["merged"] == 3 and res["missing"] == ["blocks.9.q.weight"]
    assert torch.allclose(model["blocks"][0]["q"].weight, w_q + up @ down * (1.0 / 2) * 0.5, atol=1e-6)
    assert torch.allclose(model["blocks"][0]["k"].weight, w_k + up2 @ down2 * 0.5, atol=1e-6)  # no alpha: scale 1
    assert torch.allclose(model["blocks"][0]["q"].bias, b_q + 0.5)
    # key mapping rules
    m2 = nn.ModuleDict({"layers": nn.ModuleList([nn.Linear(8, 8)])})
    w = m2["layers"][0].weight.clone()
    LoRALoader([(r"^blocks\.(\d+)\.q", r"layers.\1")]).apply_lora(
        m2, {"blocks.0.q.lora_B.weight": up, "blocks.0.q.lora_A.weight": down})  # fmt: skip
    assert torch.allclose(m2["layers"][0].weight, w + up @ down, atol=1e-6)


def test_lora_merge_into_fp8_weight():
    torch.manual_seed(0)
    w = torch.randn(16, 32)
    scale = w.abs().amax(dim=1, keepdim=True) / 448.0
    lin = nn.Module()
    lin.weight = nn.Parameter((w / scale).to(torch.float8_e4m3fn), requires_grad=False)
    lin.register_buffer("weight_scale", scale.clone())
    model = nn.ModuleDict({"proj": lin})
    up, down = torch.randn(16, 4) * 0.5, torch.randn(4, 32) * 0.5
    LoRALoader().apply_lora(model, {"proj.lora_B.weight": up, "proj.lora_A.weight": down})
    got = lin.weight.float() * lin.weight_scale
    want = w + up @ down
    assert (got - want).abs().max() / want.abs().max() < 0.08  # e4m3: 3 mantissa bits
    assert not torch.allclose(lin.weight_scale, scale)


@pytest.mark.parametrize("kind,limit", [("fp8", 0.08), ("int8", 0.03), ("mxfp8", 0.08), ("nvfp4", 0.3), ("nf4", 0.3)])
def test_lora_merge_into_every_stored_format_of_a_model(kind, limit):
    """The merge works on the matrix a quantised layer stands for and stores it back in the same format; fused QKV views
    (which hold copies of scales) are rebuilt, so the model's output follows the merged weights."""
    from telefuser_b200.ops.quant import dense_weight, stored_format, update_weight_

    torch.manual_seed(0)
    model = make_tiny_model()
    blk = model.blocks[0]
    dense_q = blk.self_attn.q.weight.detach().clone()
    rank = 4
    up, down = torch.randn(dense_q.shape[0], rank) * 0.15, torch.randn(rank, dense_q.shape[1]) * 0.15
    lora = {"blocks.0.self_attn.q.lora_B.weight": up, "blocks.0.self_attn.q.lora_A.weight": down,
            "blocks.0.ffn.0.lora_B.weight": torch.randn(blk.ffn[0].out_features, rank) * 0.15,
            "blocks.0.ffn.0.lora_A.weight": torch.randn(rank, blk.ffn[0].in_features) * 0.15}  # fmt: skip
    reference = make_tiny_model()
    LoRALoader().apply_lora(reference, lora)
    want = _tiny_forward(reference)

    model.enable_quant(kind)
    assert stored_format(blk.self_attn.q) == kind and stored_format(model.head.head) == "dense"
    before = _tiny_forward(model)  # also builds the fused QKV view of the un-merged weights
    res = LoRALoader().apply_lora(model, lora)
    assert res["merged"] == 2 and stored_format(blk.self_attn.q) == kind and stored_format(blk.ffn[0]) == kind
    merged = dense_weight(blk.self_attn.q)
    target = dense_q + up @ down
    assert ((merged - target).norm() / target.norm()).item() < limit
    unmerged = dense_weight(make_quantised_copy(dense_q, kind))
    assert (merged - target).norm() < 0.5 * (unmerged - target).norm()  # the delta went in: far closer than the old weights
    after = _tiny_forward(model)
    assert not torch.allclose(after, before) and ((after - want).norm() / want.norm()).item() < 1.5 * limit
    # the two helpers on their own: a round trip through the dense view keeps the format and (nearly) the values
    lin = blk.self_attn.o
    d0 = dense_weight(lin)
    update_weight_(lin, d0)
    assert stored_format(lin) == kind and ((dense_weight(lin) - d0).norm() / d0.norm()).item() < 0.02


def make_quantised_copy(weight, kind):
    from telefuser_b200.ops.quant import quantize_model_

    lin = nn.Sequential(nn.Linear(weight.shape[1], weight.shape[0], bias=False))
    lin[0].weight.data.copy_(weight)
    quantize_model_(lin, kind, ("*",))
    return lin[0]


def test_runtime_lora_network_switch():
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(8, 8), nn.ReLU(), nn.Linear(8, 4))
    x = torch.randn(3, 8)
    base = model(x)
    net = create_lora_network(model, [r"^0$"], rank=2, alpha=2.0)
    assert torch.allclose(model(x), base)  # up is zero-initialised
    lora = next(iter(net.loras.values()))
    lora.up.weight.data.normal_()
    changed = model(x)
    assert not torch.allclose(changed, base)
    assert torch.allclose(nn.functional.linear(x, lora.weight, lora.bias), lora(x), atol=1e-5)  # merged view == side path
    net.set_use_lora(False)
    assert torch.allclose(model(x), base)
    net.set_use_lora(True)
    net.set_multiplier(0.0)
    assert torch.allclose(model(x), base)


def test_async_offload_ring_keeps_outputs():
    model = make_tiny_model()
    ref = _tiny_forward(model)
    mgr = AsyncOffloadManager(model.blocks, enabled=True, offload_ratio=1.0, prefetch_size=1, device="cpu", min_numel=1)
    model.async_offload_manager, model.async_offload_flag = mgr, True
    assert mgr.first_offloaded == 0 and len(mgr.slots) == 2 and mgr.offloaded_bytes() > 0
    out1 = _tiny_forward(model)
    out2 = _tiny_forward(model)
    assert torch.equal(out1, ref) and torch.equal(out2, ref)
    assert mgr.copies >= 2
    # half of the blocks offloaded, one slot
    model2 = make_tiny_model()
    mgr2 = AsyncOffloadManager(model2.blocks, offload_ratio=0.5, prefetch_size=1, device="cpu", min_numel=1)
    model2.async_offload_manager, model2.async_offload_flag = mgr2, True
    assert mgr2.first_offloaded == 1 and len(mgr2.slots) == 1
    assert torch.equal(_tiny_forward(model2), ref)


def test_sequential_offload_states():
    model = make_tiny_model()
    ref = _tiny_forward(model)
    units = enable_sequential_cpu_offload(model, "cpu")
    assert len(units) == len(model.blocks)
    assert torch.equal(_tiny_forward(model), ref)
    assert all(u.state == 0 for u in units)  # offloaded again after the forward
    units[0].keep()
    assert torch.equal(_tiny_forward(model), ref) and units[0].state == 2


def test_single_rank_sharding_keeps_outputs_and_fused_views():
    model = make_tiny_model()
    ref = _tiny_forward(model)
    shard_model(model, None, ["blocks"], min_shard_numel=1)
    sb = model._sharded_blocks
    assert sb.bytes_per_rank() > 0 and len(sb.slots) == 2
    attn = model.blocks[0].self_attn
    W, _ = attn.fused_qkv()
    assert W.data_ptr() == attn.q.weight.data_ptr() and W.shape[0] == 3 * attn.q.weight.shape[0]  # zero-copy view
    assert torch.equal(_tiny_forward(model), ref)
    assert torch.equal(_tiny_forward(model), ref)


import pytest  # noqa: E402


@pytest.mark.gpu
def test_async_offload_ring_on_the_device_rotates_slots_and_keeps_outputs():
    """Four blocks behind two device slots: every forward streams each block from pinned host memory on the copy stream
    while the previous block computes; the result must equal the all-resident run bit for bit, forward after forward,
    and sequential offload must agree as well."""
    from telefuser_b200.models.wan_dit import WanModel

    def build():
        torch.manual_seed(0)
        m = WanModel(dim=512, ffn_dim=1024, num_heads=4, num_layers=4, text_dim=256).to(torch.bfloat16).cuda().eval()
        m.dtype = torch.bfloat16
        return m

    latents, ctx, _ = make_tiny_inputs()
    args = (latents.cuda(), torch.tensor([500.0], device="cuda"), ctx.cuda().bfloat16())
    with torch.no_grad():
        ref = build()(*args)
        model = build()
        mgr = AsyncOffloadManager(model.blocks, enabled=True, offload_ratio=1.0, prefetch_size=1, device="cuda", min_numel=1)
        model.async_offload_manager, model.async_offload_flag = mgr, True
        assert mgr.first_offloaded == 0 and len(mgr.slots) == 2 and mgr.offloaded_bytes() > 0
        outs = [model(*args) for _ in range(3)]
        torch.cuda.synchronize()
        assert all(torch.equal(o, ref) for o in outs)
        assert mgr.copies >= 3 * 4 - 2  # two slots for four blocks: (almost) every block is copied again on every forward
        half = build()
        mgr2 = AsyncOffloadManager(half.blocks, offload_ratio=0.5, prefetch_size=1, device="cuda", min_numel=1)
        half.async_offload_manager, half.async_offload_flag = mgr2, True
        assert mgr2.first_offloaded == 2
        assert torch.equal(half(*args), ref) and torch.equal(half(*args), ref)
        seq = build()
        units = enable_sequential_cpu_offload(seq, "cuda")
        assert len(units) == 4 and torch.equal(seq(*args), ref) and all(u.state == 0 for u in units)
