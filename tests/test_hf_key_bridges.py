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
        pe = cfg.patch_size[1] * cfg.patch_size[2]
        for suf in ("weight", "bias"):  # ... and the output projection keeps the channel last inside a patch
            t = hf[f"proj_out.{suf}"]
            hf[f"proj_out.{suf}"] = t.reshape(-1, pe, *t.shape[1:]).transpose(0, 1).reshape(t.shape)
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


# ---- WAN: an independent statement of the published forward (WanTransformer3DModel, text-to-video), written against the published key names
def _wan_reference(sd, cfg, latents, t, text, image=None):
    import math

    import torch.nn.functional as F

    h, nh, hd = cfg.hidden_size, cfg.num_heads, cfg.head_dim
    lin = lambda x, k: F.linear(x, sd[f"{k}.weight"], sd.get(f"{k}.bias"))  # noqa: E731
    rms = lambda x, w: x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.eps) * w  # noqa: E731
    ln = lambda x: F.layer_norm(x, (h,), eps=cfg.eps)  # noqa: E731
    b, c, f, hh, ww = latents.shape
    pf, ph, pw = cfg.patch_size
    x = F.conv3d(latents, sd["patch_embedding.weight"], sd["patch_embedding.bias"], stride=(pf, ph, pw))  # [b, h, F, H, W]
    grid = x.shape[2:]
    x = x.flatten(2).transpose(1, 2)
    # rotary tables: the head dimension is split over (frame, row, column); consecutive pairs rotate together
    pos = torch.stack(torch.meshgrid(*[torch.arange(n) for n in grid], indexing="ij"), -1).reshape(-1, 3).float()
    ang = torch.cat([pos[:, a : a + 1] / (cfg.rope_theta ** (torch.arange(0, d, 2).float() / d))[None] for a, d in enumerate(cfg.rope_axes)], -1)
    rot = torch.polar(torch.ones_like(ang), ang)  # [L, hd / 2] complex

    def rope(v):  # [b, L, nh, hd]
        vc = torch.view_as_complex(v.float().reshape(*v.shape[:-1], -1, 2))
        return torch.view_as_real(vc * rot[None, :, None, :]).flatten(-2)

    half = cfg.time_freq_dim // 2
    freqs = torch.exp(-math.log(10000.0) * torch.arange(half).float() / half)
    emb = t.float()[:, None] * freqs[None]
    temb = lin(F.silu(lin(torch.cat([emb.cos(), emb.sin()], -1), "condition_embedder.time_embedder.linear_1")), "condition_embedder.time_embedder.linear_2")
    tproj = lin(F.silu(temb), "condition_embedder.time_proj").unflatten(1, (6, -1))
    ctx = lin(F.gelu(lin(text, "condition_embedder.text_embedder.linear_1"), approximate="tanh"), "condition_embedder.text_embedder.linear_2")

    img_ctx = None
    if image is not None:  # image-to-video: the image encoder's tokens through the checkpoint's image embedder
        e = "condition_embedder.image_embedder"
        y = F.layer_norm(image, (image.shape[-1],), sd[f"{e}.norm1.weight"], sd[f"{e}.norm1.bias"])
        y = lin(F.gelu(lin(y, f"{e}.ff.net.0.proj")), f"{e}.ff.net.2")
        img_ctx = F.layer_norm(y, (h,), sd[f"{e}.norm2.weight"], sd[f"{e}.norm2.bias"])

    def attend(q, k, v):
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2))
        return o.transpose(1, 2).flatten(2)

    for i in range(cfg.num_cross_blocks):
        p = f"blocks.{i}"
        sh1, sc1, g1, sh2, sc2, g2 = (sd[f"{p}.scale_shift_table"] + tproj).unbind(1)
        y = ln(x) * (1 + sc1[:, None]) + sh1[:, None]
        q = rms(lin(y, f"{p}.attn1.to_q"), sd[f"{p}.attn1.norm_q.weight"]).unflatten(2, (nh, hd))
        k = rms(lin(y, f"{p}.attn1.to_k"), sd[f"{p}.attn1.norm_k.weight"]).unflatten(2, (nh, hd))
        v = lin(y, f"{p}.attn1.to_v").unflatten(2, (nh, hd))
        x = x + lin(attend(rope(q), rope(k), v), f"{p}.attn1.to_out.0") * g1[:, None]
        y = F.layer_norm(x, (h,), sd[f"{p}.norm2.weight"], sd[f"{p}.norm2.bias"], cfg.eps)
        q = rms(lin(y, f"{p}.attn2.to_q"), sd[f"{p}.attn2.norm_q.weight"]).unflatten(2, (nh, hd))
        k = rms(lin(ctx, f"{p}.attn2.to_k"), sd[f"{p}.attn2.norm_k.weight"]).unflatten(2, (nh, hd))
        v = lin(ctx, f"{p}.attn2.to_v").unflatten(2, (nh, hd))
        o = attend(q, k, v)
        if img_ctx is not None:  # a second attention of the same queries over the image tokens, added before the output projection
            ki = rms(lin(img_ctx, f"{p}.attn2.add_k_proj"), sd[f"{p}.attn2.norm_added_k.weight"]).unflatten(2, (nh, hd))
            o = o + attend(q, ki, lin(img_ctx, f"{p}.attn2.add_v_proj").unflatten(2, (nh, hd)))
        x = x + lin(o, f"{p}.attn2.to_out.0")
        y = ln(x) * (1 + sc2[:, None]) + sh2[:, None]
        x = x + lin(F.gelu(lin(y, f"{p}.ffn.net.0.proj"), approximate="tanh"), f"{p}.ffn.net.2") * g2[:, None]
    shift, scale = (sd["scale_shift_table"] + temb[:, None]).unbind(1)
    x = lin(ln(x) * (1 + scale[:, None]) + shift[:, None], "proj_out")
    x = x.reshape(b, *grid, pf, ph, pw, -1).permute(0, 7, 1, 4, 2, 5, 3, 6)
    return x.reshape(b, -1, grid[0] * pf, grid[1] * ph, grid[2] * pw)


@pytest.mark.parametrize("i2v", [False, True])
def test_wan_checkpoint_in_published_layout_matches_the_published_forward(i2v):
    """``i2v``: the WAN 2.1 image-to-video layout — an image embedder and, in every block, keys / values for the image encoder's tokens."""
    from unirl_b200.models.dit.hf_keys import wan_from_diffusers

    cfg = PRESETS["tiny-wan"]().transformer
    idim = 24
    if i2v:
        cfg.image_dim = idim
    h, m, g = cfg.hidden_size, cfg.mlp_dim, torch.Generator().manual_seed(0)
    rnd = lambda *s: torch.randn(*s, generator=g) * 0.2  # noqa: E731
    sd = {"patch_embedding.weight": rnd(h, cfg.in_channels, *cfg.patch_size), "patch_embedding.bias": rnd(h), "scale_shift_table": rnd(1, 2, h),
          "proj_out.weight": rnd(cfg.in_channels * 4, h), "proj_out.bias": rnd(cfg.in_channels * 4)}
    for name, (i, o) in {"condition_embedder.time_embedder.linear_1": (cfg.time_freq_dim, h), "condition_embedder.time_embedder.linear_2": (h, h),
                         "condition_embedder.time_proj": (h, 6 * h), "condition_embedder.text_embedder.linear_1": (cfg.text_dim, h),
                         "condition_embedder.text_embedder.linear_2": (h, h)}.items():
        sd[f"{name}.weight"], sd[f"{name}.bias"] = rnd(o, i), rnd(o)
    for b in range(cfg.num_cross_blocks):
        p = f"blocks.{b}"
        sd[f"{p}.scale_shift_table"] = rnd(1, 6, h)
        for a in ("attn1", "attn2"):
            for pr in ("to_q", "to_k", "to_v", "to_out.0"):
                sd[f"{p}.{a}.{pr}.weight"], sd[f"{p}.{a}.{pr}.bias"] = rnd(h, h), rnd(h)
            sd[f"{p}.{a}.norm_q.weight"], sd[f"{p}.{a}.norm_k.weight"] = 1 + rnd(h), 1 + rnd(h)
        if i2v:
            for pr in ("add_k_proj", "add_v_proj"):
                sd[f"{p}.attn2.{pr}.weight"], sd[f"{p}.attn2.{pr}.bias"] = rnd(h, h), rnd(h)
            sd[f"{p}.attn2.norm_added_k.weight"] = 1 + rnd(h)
        sd[f"{p}.norm2.weight"], sd[f"{p}.norm2.bias"] = 1 + rnd(h), rnd(h)
        sd[f"{p}.ffn.net.0.proj.weight"], sd[f"{p}.ffn.net.0.proj.bias"] = rnd(m, h), rnd(m)
        sd[f"{p}.ffn.net.2.weight"], sd[f"{p}.ffn.net.2.bias"] = rnd(h, m), rnd(h)
    if i2v:
        e = "condition_embedder.image_embedder"
        for name, (i, o) in {f"{e}.ff.net.0.proj": (idim, idim), f"{e}.ff.net.2": (idim, h)}.items():
            sd[f"{name}.weight"], sd[f"{name}.bias"] = rnd(o, i), rnd(o)
        sd[f"{e}.norm1.weight"], sd[f"{e}.norm1.bias"], sd[f"{e}.norm2.weight"], sd[f"{e}.norm2.bias"] = 1 + rnd(idim), rnd(idim), 1 + rnd(h), rnd(h)
    model = DiTTransformer(cfg, dtype=torch.float32, device="cpu").init_weights(3)
    missing, unexpected = load_diffusers_transformer(model, sd, "tiny-wan", strict=True)
    assert not missing and not unexpected
    assert set(wan_from_diffusers(sd, cfg.num_cross_blocks, strict=True)) == set(model.state_dict())
    lat, t, text = torch.randn(2, cfg.in_channels, 3, 8, 12, generator=g), torch.tensor([0.3, 0.9]) * 1000, torch.randn(2, 7, cfg.text_dim, generator=g)
    image = torch.randn(2, 5, idim, generator=g) if i2v else None
    with torch.no_grad():
        got, want = model(lat, t, text, image_embeds=image), _wan_reference(sd, cfg, lat, t, text, image)
    torch.testing.assert_close(got, want, rtol=2e-4, atol=2e-4)
    if i2v:
        with torch.no_grad():
            assert float((model(lat, t, text) - got).abs().max()) > 1e-3, "the image tokens reach the output"


def test_sd3_position_table_follows_the_published_formula_and_is_taken_from_the_checkpoint():
    """The table a random-init SD3 model computes equals the published construction (numpy restatement below); a checkpoint's stored table
    replaces it; the output projection's rows are reordered from channel-last to channel-first patches."""
    import numpy as np

    from unirl_b200.models.dit.modeling import sincos_2d_table

    dim, size, base = 32, 12, 4
    gh = np.arange(size, dtype=np.float32) / (size / base)
    gw = np.arange(size, dtype=np.float32) / (size / base)
    grid = np.stack(np.meshgrid(gw, gh), 0).reshape(2, 1, size, size)  # the column coordinate comes first

    def one_d(d, pos):
        omega = 1.0 / 10000 ** (np.arange(d // 2, dtype=np.float64) / (d / 2.0))
        out = np.einsum("m,d->md", pos.reshape(-1), omega)
        return np.concatenate([np.sin(out), np.cos(out)], 1)

    want = np.concatenate([one_d(dim // 2, grid[0]), one_d(dim // 2, grid[1])], 1)  # [size * size, dim]
    got = sincos_2d_table(dim, size, "cpu", base).reshape(size * size, dim)
    np.testing.assert_allclose(got.numpy(), want, rtol=1e-5, atol=1e-6)

    cfg = PRESETS["tiny-sd3"]().transformer
    src = DiTTransformer(cfg, dtype=torch.float32, device="cpu").init_weights(1)
    hf = _to_diffusers(src.state_dict(), cfg, "sd3")
    pe = cfg.patch_size[1] * cfg.patch_size[2]
    for suf in ("weight", "bias"):  # a published checkpoint keeps the channel last inside a patch
        t = hf[f"proj_out.{suf}"]
        hf[f"proj_out.{suf}"] = t.reshape(-1, pe, *t.shape[1:]).transpose(0, 1).reshape(t.shape)
    stored = torch.randn(1, cfg.pos_embed_max_size ** 2, cfg.hidden_size)
    hf["pos_embed.pos_embed"] = stored
    dst = DiTTransformer(cfg, dtype=torch.float32, device="cpu").init_weights(2)
    load_diffusers_transformer(dst, hf, "tiny-sd3", strict=True)
    assert torch.equal(dst.pos_table.reshape(-1), stored.reshape(-1))
    assert torch.equal(dst.final_proj.weight, src.final_proj.weight) and torch.equal(dst.final_proj.bias, src.final_proj.bias)
