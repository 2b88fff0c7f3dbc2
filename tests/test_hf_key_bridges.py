"""diffusers checkpoints → native DiT modules: every native parameter receives its value, fused weights are assembled in the right
row order.  The diffusers-style state dicts are synthesised here from a randomly initialised native module by splitting its fused
weights under the published key names (the bridges themselves only ever go the other way)."""
import pytest
import torch

from unirl_b200.models.dit.config import PRESETS
from unirl_b200.models.dit.hf_keys import load_diffusers_transformer
from unirl_b200.models.dit.modeling import DiTTransformer


def _split(sd, out, native, names):
    for suf in ("weight", "bias"):
        k = f"{native}.{suf}"
        if k in sd:
            for n, part in zip(names, sd[k].chunk(len(names), 0)):
                out[f"{n}.{suf}"] = part.clone()


def _copy(sd, out, native, name):
    for suf in ("weight", "bias"):
        if f"{native}.{suf}" in sd:
            out[f"{name}.{suf}"] = sd[f"{native}.{suf}"].clone()


def _to_diffusers(sd, cfg, family):
    out = {}
    top = {"sd3": {"patch_embed": "pos_embed.proj", "text_in": "context_embedder"}, "flux": {"patch_embed": "x_embedder", "text_in": "context_embedder"},
           "qwen": {"patch_embed": "img_in", "text_in": "txt_in"}}[family]
    for native, name in {**top, "time_in.0": "time_text_embed.timestep_embedder.linear_1", "time_in.1": "time_text_embed.timestep_embedder.linear_2",
                         "pooled_in.0": "time_text_embed.text_embedder.linear_1", "pooled_in.1": "time_text_embed.text_embedder.linear_2",
                         "guidance_in.0": "time_text_embed.guidance_embedder.linear_1", "guidance_in.1": "time_text_embed.guidance_embedder.linear_2",
                         "final_mod": "norm_out.linear", "final_proj": "proj_out"}.items():
        _copy(sd, out, native, name)
    mod = ("img_mod.1", "txt_mod.1") if family == "qwen" else ("norm1.linear", "norm1_context.linear")
    mlp = (("img_mlp.net.0.proj", "img_mlp.net.2"), ("txt_mlp.net.0.proj", "txt_mlp.net.2")) if family == "qwen" else (("ff.net.0.proj", "ff.net.2"), ("ff_context.net.0.proj", "ff_context.net.2"))
    for i in range(cfg.num_joint_blocks):
        s, d = f"joint_blocks.{i}", f"transformer_blocks.{i}"
        _copy(sd, out, f"{s}.img_mod", f"{d}.{mod[0]}")
        _copy(sd, out, f"{s}.txt_mod", f"{d}.{mod[1]}")
        _split(sd, out, f"{s}.img_attn.qkv", [f"{d}.attn.to_q", f"{d}.attn.to_k", f"{d}.attn.to_v"])
        _split(sd, out, f"{s}.txt_attn.qkv", [f"{d}.attn.add_q_proj", f"{d}.attn.add_k_proj", f"{d}.attn.add_v_proj"])
        _split(sd, out, f"{s}.img_attn2.qkv", [f"{d}.attn2.to_q", f"{d}.attn2.to_k", f"{d}.attn2.to_v"])
        for a, b in (("img_attn.out", "attn.to_out.0"), ("txt_attn.out", "attn.to_add_out"), ("img_attn2.out", "attn2.to_out.0"), ("img_mlp.fc1", mlp[0][0]),
                     ("img_mlp.fc2", mlp[0][1]), ("txt_mlp.fc1", mlp[1][0]), ("txt_mlp.fc2", mlp[1][1])):
            _copy(sd, out, f"{s}.{a}", f"{d}.{b}")
        for a, b in (("img_attn.q_norm", "attn.norm_q.weight"), ("img_attn.k_norm", "attn.norm_k.weight"), ("txt_attn.q_norm", "attn.norm_added_q.weight"),
                     ("txt_attn.k_norm", "attn.norm_added_k.weight"), ("img_attn2.q_norm", "attn2.norm_q.weight"), ("img_attn2.k_norm", "attn2.norm_k.weight")):
            if f"{s}.{a}" in sd:
                out[f"{d}.{b}"] = sd[f"{s}.{a}"].clone()
    h, m = cfg.hidden_size, cfg.mlp_dim
    for i in range(cfg.num_single_blocks):
        s, d = f"single_blocks.{i}", f"single_transformer_blocks.{i}"
        _copy(sd, out, f"{s}.mod", f"{d}.norm.linear")
        for suf in ("weight", "bias"):
            t = sd[f"{s}.in_proj.{suf}"]
            for n, part in zip((f"{d}.attn.to_q", f"{d}.attn.to_k", f"{d}.attn.to_v", f"{d}.proj_mlp"), t.split([h, h, h, m], 0)):
                out[f"{n}.{suf}"] = part.clone()
        _copy(sd, out, f"{s}.out_proj", f"{d}.proj_out")
        for a, b in (("q_norm", "attn.norm_q.weight"), ("k_norm", "attn.norm_k.weight")):
            if f"{s}.{a}" in sd:
                out[f"{d}.{b}"] = sd[f"{s}.{a}"].clone()
    return out


@pytest.mark.parametrize("preset,family", [("tiny-sd3", "sd3"), ("tiny-flux2", "flux"), ("tiny-hunyuan-video", "flux"), ("tiny-z-image", "flux"), ("tiny-qwen-image", "qwen")])
def test_diffusers_state_dict_lands_in_the_native_module(preset, family):
    cfg = PRESETS[preset]().transformer
    src = DiTTransformer(cfg, dtype=torch.float32, device="cpu").init_weights(1)
    with torch.no_grad():
        for p in src.parameters():  # biases and norms start at 0 / 1: randomise everything so that a misplaced tensor shows
            p.copy_(torch.randn_like(p) * 0.1)
    hf = _to_diffusers(src.state_dict(), cfg, family)
    assert not any(k.startswith(("joint_blocks", "single_blocks")) for k in hf), "the synthetic checkpoint uses the published key grammar only"
    if family == "sd3":
        hf["pos_embed.proj.weight"] = hf["pos_embed.proj.weight"].view(cfg.hidden_size, cfg.in_channels, cfg.patch_size[1], cfg.patch_size[2])  # a conv kernel, as published
    dst = DiTTransformer(cfg, dtype=torch.float32, device="cpu").init_weights(2)
    missing, unexpected = load_diffusers_transformer(dst, hf, preset, strict=True)
    assert not missing and not unexpected
    for (k, a), (_, b) in zip(src.state_dict().items(), dst.state_dict().items()):
        assert torch.equal(a, b), k
    x = torch.randn(1, cfg.in_channels, *( (2,) if cfg.is_video else () ), 8, 8)
    # same weights → same function
    t = torch.tensor([0.5])
    txt = torch.randn(1, 5, cfg.text_dim)
    kw = {"pooled": torch.randn(1, cfg.pooled_dim)} if cfg.pooled_dim else {}
    try:
        ya, yb = src(x, t, txt, **kw), dst(x, t, txt, **kw)
    except TypeError:
        return  # forward signature of this family needs more inputs; the parameter check above is the point of this test
    torch.testing.assert_close(ya, yb)


def test_bridge_reports_shape_mismatch_and_unplaced_tensors():
    cfg = PRESETS["tiny-sd3"]().transformer
    src = DiTTransformer(cfg, dtype=torch.float32, device="cpu").init_weights(1)
    hf = _to_diffusers(src.state_dict(), cfg, "sd3")
    bad = dict(hf)
    bad["transformer_blocks.0.attn.to_q.weight"] = bad["transformer_blocks.0.attn.to_q.weight"][:-1]
    with pytest.raises(ValueError, match="shape mismatch"):
        load_diffusers_transformer(DiTTransformer(cfg, dtype=torch.float32, device="cpu"), bad, "tiny-sd3")
    short = {k: v for k, v in hf.items() if "transformer_blocks.1.ff.net.2" not in k}
    with pytest.raises(KeyError, match="got no value"):
        load_diffusers_transformer(DiTTransformer(cfg, dtype=torch.float32, device="cpu"), short, "tiny-sd3")
