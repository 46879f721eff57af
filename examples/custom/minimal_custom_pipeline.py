"""Template: a model, a stage, a pipeline and the service entry points in one file, small enough to read in a minute and
complete enough to run (random weights, CPU or GPU).

    python examples/custom/minimal_custom_pipeline.py --prompt "anything" --output work_dirs/custom.png
    telefuser serve examples/custom/minimal_custom_pipeline.py -t t2i

What each part shows:
* `TinyDiT(BaseModel)`: blocks written with `telefuser_b200.ops.functional` calls (attention, fused LayerNorm + modulation,
  linear with fused activation / gated residual), so the same code runs the fp32 reference on CPU and the native kernels on a
  B200; the hooks a model gives the framework (`get_fsdp_module_names`, `enable_quant` through the default, a fingerprint
  registration so `ModuleManager.load_model` recognises its checkpoints).
* `TinyDenoisingStage(BaseStage)`: owns the model, `@with_model_offload` around the entry point, a flow-match Euler loop.
* `TinyPipeline(BasePipeline)`: `init(module_manager, config)` builds the stages, `__call__` runs them.
* module level: `PPL_CONFIG`, `PIPELINE_MANIFEST`, `get_pipeline(parallelism)`, `run_with_file(...)`.
"""

from __future__ import annotations

import math
import os
from dataclasses import dataclass, field

import torch
from torch import nn

from telefuser_b200.core.base_model import BaseModel
from telefuser_b200.core.base_pipeline import BasePipeline
from telefuser_b200.core.base_stage import BaseStage, with_model_offload
from telefuser_b200.core.config import ModelRuntimeConfig
from telefuser_b200.core.model_registry import register_architecture
from telefuser_b200.core.module_manager import ModuleManager
from telefuser_b200.ops import functional as TF
from telefuser_b200.schedulers.flow_match import FlowMatchScheduler

PPL_CONFIG = dict(name="tiny_custom_t2i", height=32, width=32, num_inference_steps=4, seed=0, dim=128, heads=1, depth=2)
PIPELINE_MANIFEST = {"tasks": ["t2i"], "media_type": "image", "required_inputs": {"t2i": ["prompt"]}}


# ---- the model ----------------------------------------------------------------------------------------------------
class TinyBlock(nn.Module):
    def __init__(self, dim: int, heads: int) -> None:
        super().__init__()
        self.heads = heads
        self.qkv, self.proj = nn.Linear(dim, 3 * dim), nn.Linear(dim, dim)
        self.ffn_in, self.ffn_out = nn.Linear(dim, 4 * dim), nn.Linear(4 * dim, dim)
        self.modulation = nn.Parameter(torch.zeros(6, dim))  # shift / scale / gate for the two halves of the block

    def forward(self, x, t_emb):
        B, S, C = x.shape
        sh1, sc1, g1, sh2, sc2, g2 = (self.modulation.float() + t_emb.float()).unsqueeze(1).unbind(2)  # each [B, 1, C] fp32
        h = TF.layernorm_modulate(x, sh1, sc1)  # LayerNorm (no affine) * (1 + scale) + shift, one pass
        q, k, v = TF.linear(h, self.qkv.weight, self.qkv.bias).view(B, S, 3, self.heads, C // self.heads).unbind(2)
        a = TF.attention(q, k, v).reshape(B, S, C)
        x = TF.linear(a, self.proj.weight, self.proj.bias, residual=x, gate=g1)  # x + gate * proj(a), fused epilogue
        h = TF.linear(TF.layernorm_modulate(x, sh2, sc2), self.ffn_in.weight, self.ffn_in.bias, act="gelu_tanh")
        return TF.linear(h, self.ffn_out.weight, self.ffn_out.bias, residual=x, gate=g2)


class TinyDiT(BaseModel):
    """Pixels in, velocity out: 4 x 4 patches -> tokens -> blocks -> patches."""

    def __init__(self, dim: int = 128, heads: int = 1, depth: int = 2, patch: int = 4, text_dim: int = 32) -> None:
        super().__init__()
        self.dim, self.patch = dim, patch
        self.patch_in, self.text_in = nn.Linear(3 * patch * patch, dim), nn.Linear(text_dim, dim)
        self.time_in = nn.Sequential(nn.Linear(dim, dim), nn.SiLU(), nn.Linear(dim, 6 * dim))
        self.blocks = nn.ModuleList(TinyBlock(dim, heads) for _ in range(depth))
        self.head = nn.Linear(dim, 3 * patch * patch)

    def get_fsdp_module_names(self) -> list[str]:  # block lists: what weight sharding wraps and `enable_quant` quantises
        return ["blocks"]

    def forward(self, image, timestep, text):
        B, _, H, W = image.shape
        p = self.patch
        tokens = image.unfold(2, p, p).unfold(3, p, p).permute(0, 2, 3, 1, 4, 5).reshape(B, (H // p) * (W // p), 3 * p * p)
        x = torch.cat([self.text_in(text.to(image.dtype)), self.patch_in(tokens)], dim=1)
        half = self.dim // 2
        freqs = torch.exp(-math.log(10000.0) * torch.arange(half, device=image.device) / half)
        ang = timestep.float()[:, None] * freqs
        t_emb = self.time_in(torch.cat([ang.cos(), ang.sin()], dim=-1).to(image.dtype)).view(B, 6, self.dim)
        for blk in self.blocks:
            x = blk(x, t_emb)
        out = self.head(x[:, text.shape[1] :]).view(B, H // p, W // p, 3, p, p)
        return out.permute(0, 3, 1, 4, 2, 5).reshape(B, 3, H, W)


# the checkpoint fingerprint follows from the definition: files saved from this class are recognised by `load_model`
register_architecture("tiny_custom_dit", TinyDiT, lambda: TinyDiT(PPL_CONFIG["dim"], PPL_CONFIG["heads"], PPL_CONFIG["depth"]))


# ---- the stage ----------------------------------------------------------------------------------------------------
class TinyDenoisingStage(BaseStage):
    def __init__(self, name: str, module_manager: ModuleManager, config: ModelRuntimeConfig) -> None:
        super().__init__(name, config)
        self.dit = module_manager.fetch_module("tiny_custom_dit")
        self.model_names = ["dit"]  # what on- / off-loading moves
        self.scheduler = FlowMatchScheduler("Wan")

    @with_model_offload(["dit"])
    @torch.no_grad()
    def process(self, noise: torch.Tensor, text: torch.Tensor, num_inference_steps: int) -> torch.Tensor:
        x = noise.to(self.device, self.torch_dtype)
        text = text.to(self.device, self.torch_dtype)
        self.scheduler.set_timesteps(num_inference_steps, shift=3.0)
        for i, t in enumerate(self.scheduler.timesteps):
            velocity = self.dit(x, t.expand(x.shape[0]).to(self.device), text)
            x = self.scheduler.step(velocity, t, x, to_final=i == num_inference_steps - 1)
        return x


# ---- the pipeline ------------------------------------------------------------------------------------------------
@dataclass
class TinyPipelineConfig:
    dit_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)


class TinyPipeline(BasePipeline):
    def _get_stages(self) -> list:
        return [self.denoise_stage]

    def init(self, module_manager: ModuleManager, config: TinyPipelineConfig) -> None:
        self.config = config
        self.denoise_stage = TinyDenoisingStage("denoise", module_manager, config.dit_config)

    def __call__(self, prompt: str, height: int = 32, width: int = 32, num_inference_steps: int = 4, seed: int = 0) -> torch.Tensor:
        height, width = self.check_resize_height_width(height, width)
        g = torch.Generator().manual_seed(sum(prompt.encode()) + 1)  # stands in for a text encoder
        text = torch.randn(1, 4, 32, generator=g)
        noise = self.generate_noise((1, 3, height, width), seed=seed)
        return self.denoise_stage.process(noise, text, num_inference_steps)  # [1, 3, H, W] in about [-1, 1]


# ---- what `telefuser serve` loads ------------------------------------------------------------------------------------
def get_pipeline(parallelism: int = 1) -> TinyPipeline:
    device = "cuda" if torch.cuda.is_available() else "cpu"
    dtype = torch.bfloat16 if device == "cuda" else torch.float32
    torch.manual_seed(0)
    model = TinyDiT(PPL_CONFIG["dim"], PPL_CONFIG["heads"], PPL_CONFIG["depth"]).to(dtype).eval()
    model.dtype = dtype
    mm = ModuleManager(torch_dtype=dtype, device=device)
    mm.add_module(model, "tiny_custom_dit")  # a real pipeline calls mm.load_model(path) here
    pipe = TinyPipeline(device=device, torch_dtype=dtype)
    pipe.init(mm, TinyPipelineConfig(ModelRuntimeConfig(device_type=device, torch_dtype=dtype)))
    return pipe


def run_with_file(pipeline, prompt: str, output_path: str, seed: int = PPL_CONFIG["seed"], height: int = PPL_CONFIG["height"],
                  width: int = PPL_CONFIG["width"], num_inference_steps: int = PPL_CONFIG["num_inference_steps"]):  # fmt: skip
    from PIL import Image

    image = pipeline(prompt, height=height, width=width, num_inference_steps=num_inference_steps, seed=seed)
    arr = ((image[0].float().clamp(-1, 1) + 1) * 127.5).round().to(torch.uint8).permute(1, 2, 0).cpu().numpy()
    os.makedirs(os.path.dirname(os.path.abspath(output_path)), exist_ok=True)
    Image.fromarray(arr).save(output_path)
    return {"output_path": output_path}


if __name__ == "__main__":
    import click

    @click.command()
    @click.option("--prompt", default="a template")
    @click.option("--output", default="work_dirs/custom.png")
    def main(prompt, output):
        print(run_with_file(get_pipeline(), prompt, output))

    main()
