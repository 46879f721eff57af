"""HunyuanVideo-1.5 VAE, latent upsamplers and the logic around the transformers-backed encoders (with fakes)."""

from types import SimpleNamespace

import numpy as np
import pytest
import torch
from torch import nn

from telefuser_b200.models import hunyuan_video_encoders as E
from telefuser_b200.models import hunyuan_video_vae as V


def _vae(**kw):
    torch.manual_seed(0)
    vae = V.HunyuanVideoVAE(latent_channels=4, block_out_channels=(16, 32, 64, 64), layers_per_block=1, ffactor_spatial=8, ffactor_temporal=4,
                            sample_size=32, **kw)  # fmt: skip
    for p in vae.parameters():
        torch.nn.init.normal_(p, std=0.1)
    return vae.float().eval()


def test_vae_shapes_causality_and_scaled_helpers():
    vae = _vae()
    x = torch.randn(1, 3, 9, 32, 48)
    post = vae.encode(x).latent_dist
    assert post.mode().shape == (1, 4, 3, 4, 6) and vae.decode(post.mode()).sample.shape == x.shape
    assert vae.get_latent_size((8, 32, 48)) == (2, 4, 6) and vae.get_video_size((2, 4, 6)) == (8, 32, 48)
    x2 = x.clone()
    x2[:, :, 5:] += 1.0  # frames 5.. belong to the third latent only
    assert torch.allclose(vae.encode(x2).latent_dist.mode()[:, :, :2], post.mode()[:, :, :2], atol=1e-4)
    assert torch.allclose(vae.encode_latents(x), post.mode() * vae.scaling_factor)
    z = torch.randn(1, 4, 2, 4, 6)
    assert torch.allclose(vae.decode_latents(z * vae.scaling_factor, memory_efficient=False), vae.decode(z).sample, atol=1e-5)
    g = torch.Generator().manual_seed(1)
    s = post.sample(g)
    assert s.shape == post.mean.shape and not torch.equal(s, post.mean) and post.kl().shape == (1,)
    assert torch.equal(V.frame_causal_mask(2, 2, "cpu"), torch.tensor([[1, 1, 0, 0], [1, 1, 0, 0], [1, 1, 1, 1], [1, 1, 1, 1]], dtype=torch.bool))
    out = vae(x, return_dict=False)
    assert out[0].shape == x.shape and out[1] is not None


def test_vae_tiling_and_slicing():
    vae = _vae()
    z = torch.randn(2, 4, 2, 7, 9)
    with vae.memory_efficient_context():
        assert vae.use_slicing and vae.use_spatial_tiling
        tiled = vae.decode(z).sample
    assert not vae.use_slicing and tiled.shape == (2, 3, 5, 56, 72)
    # tiles that fit the window are decoded directly
    small = torch.randn(1, 4, 2, 4, 4)
    vae.enable_tiling()
    assert torch.allclose(vae.decode(small).sample, vae.decoder(small))
    # the first tile's interior (before any blend region) equals a direct decode of that tile
    direct = vae.decoder(z[:1, :, :, :4, :4])
    assert torch.allclose(tiled[:1, :, :, :24, :24], direct[..., :24, :24], atol=1e-5)
    a, b = torch.zeros(1, 1, 1, 2, 4), torch.ones(1, 1, 1, 2, 4)
    assert torch.allclose(V._blend(a, b, 2, -1)[0, 0, 0, 0], torch.tensor([0.0, 0.5, 1.0, 1.0]))
    sd = {"vae." + k: v for k, v in vae.state_dict().items()}
    conv, cfg = vae.state_dict_converter().from_official(sd)
    assert set(conv) == set(vae.state_dict()) and cfg == {"latent_channels": 4, "block_out_channels": [16, 32, 64, 64]}


def test_latent_upsamplers():
    up = V.SRTo720pUpsampler(in_channels=4, out_channels=4, hidden_channels=8, num_blocks=2, global_residual=True).float().eval()
    z = torch.randn(1, 4, 3, 4, 6)
    assert up(z).shape == z.shape
    up2 = V.SRTo1080pUpsampler(z_channels=4, out_channels=4, block_out_channels=(8, 16), num_res_blocks=1).float().eval()
    assert up2(z, (6, 10)).shape == (1, 4, 3, 6, 10) and up2(z).shape == z.shape
    assert V.resize_latents(z, (8, 12)).shape == (1, 4, 3, 8, 12) and V.resize_latents(z, (4, 6)) is z


class _ByteTokenizer:
    """One token per byte (+3), id 0 pads; chat templates are rendered as <|im_start|>role\\ncontent<|im_end|>\\n."""

    def __init__(self):
        self.extra = []

    def __len__(self):
        return 259 + len(self.extra)

    def add_tokens(self, tokens, special_tokens=False):
        self.extra += list(tokens)

    def _ids(self, text):
        return [b + 3 for b in text.encode()]

    def __call__(self, text, padding=None, max_length=None, truncation=False, add_special_tokens=True, return_tensors=None, **kw):
        texts = [text] if isinstance(text, str) else list(text)
        rows = [self._ids(t) for t in texts]
        if return_tensors is None:
            return {"input_ids": rows[0] if isinstance(text, str) else rows}
        n = max_length or max(len(r) for r in rows)
        ids = torch.zeros(len(rows), n, dtype=torch.long)
        mask = torch.zeros(len(rows), n, dtype=torch.long)
        for i, r in enumerate(rows):
            r = r[:n]
            ids[i, : len(r)] = torch.tensor(r)
            mask[i, : len(r)] = 1
        return {"input_ids": ids, "attention_mask": mask}

    def apply_chat_template(self, chats, add_generation_prompt=True, tokenize=True, return_dict=True, **kw):
        chats = chats if isinstance(chats[0], list) else [chats]
        texts = ["".join(f"<|im_start|>{m['role']}\n{m['content']}<|im_end|>\n" for m in c) + "<|im_start|>assistant\n" for c in chats]
        return self(texts, **kw)


class _FakeLM(nn.Module):
    def __init__(self, dim=8, layers=3):
        super().__init__()
        self.emb = nn.Embedding(600, dim)
        self.norm = nn.LayerNorm(dim)
        self.layers = layers

    def forward(self, input_ids, attention_mask=None, output_hidden_states=False):
        h = self.emb(input_ids)
        hs = tuple(h * (i + 1) for i in range(self.layers + 1))
        return {"last_hidden_state": hs[-1], "hidden_states": hs} if not output_hidden_states else SimpleNamespace(last_hidden_state=hs[-1], hidden_states=hs)


def test_text_encoder_template_crop_and_skip_layer():
    tok, lm = _ByteTokenizer(), _FakeLM()
    image_t = {"template": [{"role": "system", "content": "Describe the image."}, {"role": "user", "content": "{}"}], "crop_start": -1}
    video_t = {"template": [{"role": "system", "content": "Describe the video in detail."}, {"role": "user", "content": "{}"}], "crop_start": -1}
    enc = E.HunyuanVideoTextEncoder(max_length=48, prompt_template=image_t, prompt_template_video=video_t, hidden_state_skip_layer=2,
                                    model=lm, tokenizer=tok)  # fmt: skip
    sys_len = len("<|im_start|>system\nDescribe the image.<|im_end|>\n" + E.USER_TURN_MARKER)
    assert enc.prompt_template["crop_start"] == sys_len and image_t["crop_start"] == -1  # the caller's dict is not modified
    assert set(E.PROMPT_TEMPLATE) == {"li-dit-encode-image-json", "li-dit-encode-video-json"}
    assert enc.prompt_template_video["crop_start"] > sys_len
    out = enc("a red fox")
    assert out.hidden_state.shape == (1, 48, 8) and out.attention_mask.shape == (1, 48)
    n = len("a red fox<|im_end|>\n<|im_start|>assistant\n")
    assert int(out.attention_mask.sum()) == n
    ids = tok("a red fox", return_tensors="pt", max_length=9)["input_ids"]
    assert torch.allclose(out.hidden_state[:, :9], lm.emb(ids) * 2)  # hidden_states[-3] of 4 -> scale 2
    both = enc(["a", ""], data_type="video", output_hidden_states=True)
    assert both.hidden_state.shape == (2, 48, 8) and len(both.hidden_states_list) == 4
    assert E.HunyuanVideoTextEncoder.apply_text_to_template("", [{"role": "user", "content": "{}"}])[0]["content"] == " "
    with pytest.raises(ValueError):
        E.HunyuanVideoTextEncoder(prompt_template={"template": "no placeholder"}, model=lm, tokenizer=tok)


class _FakeT5(nn.Module):
    def __init__(self):
        super().__init__()
        self.emb = nn.Embedding(300, 6)
        self.resized = None

    def resize_token_embeddings(self, n, mean_resizing=False):
        self.resized = n

    def forward(self, input_ids, attention_mask=None):
        return SimpleNamespace(last_hidden_state=self.emb(input_ids) * attention_mask[..., None])


def test_glyph_encoder(tmp_path):
    assert E.extract_glyph_texts('a sign saying "OPEN" and “24h” and "OPEN"') == ["OPEN", "24h"]
    assert E.extract_glyph_texts("nothing quoted") == [] and E.extract_glyph_texts('"x"') == ["x"]
    (tmp_path / "c.json").write_text('{"red": 0, "blue": 1}')
    (tmp_path / "f.json").write_text('{"en-Arial": 3}')
    fmt = E.MultilingualPromptFormat(str(tmp_path / "f.json"), str(tmp_path / "c.json"))
    assert fmt.format_prompt(["Hi", "Yo"], [{"color": 1, "font-family": "en-Arial"}, {"color": None, "font-family": "xx"}]) == "<color-1><en-font-3>Hi Yo"
    model, tok = _FakeT5(), _ByteTokenizer()
    enc = E.HunyuanVideoByT5Encoder(E.ByT5Config(max_length=16, hidden_dim=6, color_ann_path=str(tmp_path / "c.json"),
                                                  font_ann_path=str(tmp_path / "f.json")), torch.float32, model=model, tokenizer=tok)  # fmt: skip
    assert tok.extra == ["<color-0>", "<color-1>", "<en-font-3>"] and model.resized == 262
    out = enc(['say "hello"', "plain"])
    assert out["byt5_text_states"].shape == (2, 16, 6) and out["byt5_text_mask"].sum(dim=1).tolist() == [5, 0]
    assert bool((out["byt5_text_states"][1] == 0).all()) and bool((out["byt5_text_states"][0, 5:] == 0).all())


def test_image_encoder_and_crop():
    class _Proc:
        def preprocess(self, images, return_tensors="pt"):
            return {"pixel_values": torch.as_tensor(images).permute(0, 3, 1, 2).float() / 255.0}

    class _Vision(nn.Module):
        def __init__(self):
            super().__init__()
            self.proj = nn.Linear(3, 5)
            self.config = SimpleNamespace(hidden_size=5)

        def forward(self, pixel_values):
            return SimpleNamespace(last_hidden_state=self.proj(pixel_values.flatten(2).transpose(1, 2)), pooler_output=None)

    enc = E.HunyuanVideoImageEncoder(_Vision(), _Proc(), dtype=torch.float32)
    out = enc(np.zeros((1, 4, 6, 3), dtype=np.uint8))
    assert out.last_hidden_state.shape == (1, 24, 5) and enc.hidden_size == 5 and out.hidden_states is None
    img = (np.random.rand(40, 60, 3) * 255).astype(np.uint8)
    assert E.resize_and_center_crop(img, 32, 32).shape == (32, 32, 3) and E.resize_and_center_crop(img, 60, 40) is img
