"""The published KL auto-encoder as a native module: its parameter names are the checkpoint's key grammar, and its forward equals a plain
functional statement of the published computation written directly over those keys."""
import json

import torch
import torch.nn.functional as F

from unirl_b200.models.dit.vae_kl import AutoencoderKL, KLConfig

CFG = dict(in_channels=3, out_channels=3, latent_channels=4, block_out_channels=[8, 16, 16], layers_per_block=1, norm_num_groups=4, scaling_factor=1.5305,
           shift_factor=0.0609, use_quant_conv=False, use_post_quant_conv=False, _class_name="AutoencoderKL", sample_size=32)


def _gn(sd, k, x, groups=4):
    return F.group_norm(x, groups, sd[k + ".weight"], sd[k + ".bias"], eps=1e-6)


def _conv(sd, k, x, **kw):
    return F.conv2d(x, sd[k + ".weight"], sd[k + ".bias"], **kw)


def _resnet(sd, k, x):
    h = _conv(sd, k + ".conv1", F.silu(_gn(sd, k + ".norm1", x)), padding=1)
    h = _conv(sd, k + ".conv2", F.silu(_gn(sd, k + ".norm2", h)), padding=1)
    return h + (_conv(sd, k + ".conv_shortcut", x) if k + ".conv_shortcut.weight" in sd else x)


def _mid(sd, k, x):
    x = _resnet(sd, k + ".resnets.0", x)
    a = k + ".attentions.0"
    b, c, h, w = x.shape
    y = _gn(sd, a + ".group_norm", x).flatten(2).transpose(1, 2)
    q, kk, v = (F.linear(y, sd[a + f".to_{n}.weight"], sd[a + f".to_{n}.bias"]) for n in "qkv")
    att = torch.softmax(q @ kk.transpose(1, 2) / c ** 0.5, -1) @ v
    x = x + F.linear(att, sd[a + ".to_out.0.weight"], sd[a + ".to_out.0.bias"]).transpose(1, 2).reshape(b, c, h, w)
    return _resnet(sd, k + ".resnets.1", x)


def _encode(sd, x, levels=3, layers=1):
    x = _conv(sd, "encoder.conv_in", x, padding=1)
    for i in range(levels):
        for j in range(layers):
            x = _resnet(sd, f"encoder.down_blocks.{i}.resnets.{j}", x)
        if i < levels - 1:
            x = _conv(sd, f"encoder.down_blocks.{i}.downsamplers.0.conv", F.pad(x, (0, 1, 0, 1)), stride=2)
    x = _mid(sd, "encoder.mid_block", x)
    return _conv(sd, "encoder.conv_out", F.silu(_gn(sd, "encoder.conv_norm_out", x)), padding=1)


def _decode(sd, z, levels=3, layers=1):
    x = _mid(sd, "decoder.mid_block", _conv(sd, "decoder.conv_in", z, padding=1))
    for i in range(levels):
        for j in range(layers + 1):
            x = _resnet(sd, f"decoder.up_blocks.{i}.resnets.{j}", x)
        if i < levels - 1:
            x = _conv(sd, f"decoder.up_blocks.{i}.upsamplers.0.conv", F.interpolate(x, scale_factor=2.0, mode="nearest"), padding=1)
    return _conv(sd, "decoder.conv_out", F.silu(_gn(sd, "decoder.conv_norm_out", x)), padding=1)


def _published_keys(levels=3, layers=1, ch=(8, 16, 16)):
    """Key list of the published class for this configuration, written out by rule (no module of this repository involved)."""
    keys = []

    def wb(k):
        keys.extend([k + ".weight", k + ".bias"])

    def resnet(k, cin, cout):
        for n in ("norm1", "conv1", "norm2", "conv2"):
            wb(f"{k}.{n}")
        if cin != cout:
            wb(f"{k}.conv_shortcut")

    def mid(k, c):
        resnet(k + ".resnets.0", c, c)
        for n in ("group_norm", "to_q", "to_k", "to_v", "to_out.0"):
            wb(f"{k}.attentions.0.{n}")
        resnet(k + ".resnets.1", c, c)

    wb("encoder.conv_in")
    for i in range(levels):
        for j in range(layers):
            resnet(f"encoder.down_blocks.{i}.resnets.{j}", ch[max(i - 1, 0)] if j == 0 else ch[i], ch[i])
        if i < levels - 1:
            wb(f"encoder.down_blocks.{i}.downsamplers.0.conv")
    mid("encoder.mid_block", ch[-1])
    wb("encoder.conv_norm_out"), wb("encoder.conv_out")
    rch = tuple(reversed(ch))
    wb("decoder.conv_in")
    mid("decoder.mid_block", rch[0])
    for i in range(levels):
        for j in range(layers + 1):
            resnet(f"decoder.up_blocks.{i}.resnets.{j}", rch[max(i - 1, 0)] if j == 0 else rch[i], rch[i])
        if i < levels - 1:
            wb(f"decoder.up_blocks.{i}.upsamplers.0.conv")
    wb("decoder.conv_norm_out"), wb("decoder.conv_out")
    return sorted(keys)


def test_parameter_names_are_the_published_key_grammar_and_forward_matches_its_functional_statement(tmp_path):
    from safetensors.torch import save_file

    torch.manual_seed(0)
    model = AutoencoderKL(KLConfig.from_hf_dict(CFG)).init_weights(3)
    with torch.no_grad():
        for p in model.parameters():
            if p.dim() == 1:
                p.add_(torch.randn_like(p) * 0.1)  # norm scales and biases away from their constant initial values
    sd = {k: v.clone() for k, v in model.state_dict().items()}
    assert sorted(sd) == _published_keys()
    # round trip through a checkpoint folder in the published layout
    (tmp_path / "config.json").write_text(json.dumps(CFG))
    save_file(sd, str(tmp_path / "diffusion_pytorch_model.safetensors"))
    loaded = AutoencoderKL.from_hf(str(tmp_path))
    assert loaded.cfg.block_out_channels == (8, 16, 16) and loaded.cfg.spatial_factor == 4 and loaded.quant_conv is None
    img = torch.rand(2, 3, 32, 40)
    with torch.no_grad():
        moments = _encode(sd, img * 2 - 1)
        want_lat = (moments[:, :4] - 0.0609) * 1.5305
        got_lat = loaded.encode(img)
        torch.testing.assert_close(got_lat, want_lat, rtol=1e-4, atol=1e-5)
        assert got_lat.shape == (2, 4, 8, 10)
        z = torch.randn(2, 4, 8, 10)
        want_px = (_decode(sd, z / 1.5305 + 0.0609) / 2 + 0.5).clamp(0, 1)
        torch.testing.assert_close(loaded.decode(z), want_px, rtol=1e-4, atol=1e-5)


def test_older_files_with_quant_convs_and_conv_shaped_attention(tmp_path):
    """Checkpoints written by older library versions: 1x1 quant / post-quant convolutions present, attention projections stored under
    query / key / value / proj_attn as 1x1 convolutions."""
    from safetensors.torch import save_file

    cfg = dict(CFG, use_quant_conv=True, use_post_quant_conv=True)
    model = AutoencoderKL(KLConfig.from_hf_dict(cfg)).init_weights(5)
    sd = {}
    for k, v in model.state_dict().items():
        for new, old in ((".to_q.", ".query."), (".to_k.", ".key."), (".to_v.", ".value."), (".to_out.0.", ".proj_attn.")):
            if new in k:
                k = k.replace(new, old)
                v = v[:, :, None, None] if v.dim() == 2 else v
        sd[k] = v.clone().contiguous()
    (tmp_path / "config.json").write_text(json.dumps(CFG))  # the flags come from what the file holds
    save_file(sd, str(tmp_path / "diffusion_pytorch_model.safetensors"))
    loaded = AutoencoderKL.from_hf(str(tmp_path))
    assert loaded.quant_conv is not None and loaded.post_quant_conv is not None
    z = torch.randn(1, 4, 4, 4)
    torch.testing.assert_close(loaded.decode(z), model.decode(z))
    img = torch.rand(1, 3, 16, 16)
    torch.testing.assert_close(loaded.encode(img), model.encode(img))


def test_bundle_uses_the_checkpoints_codec(tmp_path):
    """A checkpoint folder with a ``vae`` sub-folder in the published layout: the pipeline decodes with that codec."""
    from safetensors.torch import save_file

    from unirl_b200.models.sd3.config import SD3PipelineConfig
    from unirl_b200.models.sd3.pipeline import SD3Pipeline

    rnd = SD3Pipeline.from_config(SD3PipelineConfig(pretrained_model_ckpt_path="random:tiny-sd3", model_precision="fp32", autocast_precision="fp32", device="cpu"))
    lat_ch = rnd.bundle.spec.transformer.in_channels
    save_file({k: v.contiguous() for k, v in rnd.bundle.transformer.state_dict().items()}, str(tmp_path / "transformer.safetensors"))
    (tmp_path / "config.json").write_text(json.dumps({"preset": "tiny-sd3"}))
    cfg = dict(CFG, latent_channels=lat_ch)
    codec = AutoencoderKL(KLConfig.from_hf_dict(cfg)).init_weights(11)
    (tmp_path / "vae").mkdir()
    (tmp_path / "vae" / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.contiguous() for k, v in codec.state_dict().items()}, str(tmp_path / "vae" / "diffusion_pytorch_model.safetensors"))
    pipe = SD3Pipeline.from_config(SD3PipelineConfig(pretrained_model_ckpt_path=str(tmp_path), model_precision="fp32", autocast_precision="fp32", device="cpu"))
    assert isinstance(pipe.bundle.vae, AutoencoderKL)
    z = torch.randn(2, lat_ch, 4, 4)
    torch.testing.assert_close(pipe.bundle.vae.decode(z), codec.decode(z))
