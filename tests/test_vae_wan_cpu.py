"""The causal 3-D codec of WAN / Qwen-Image: the one-pass evaluation of this package against a streamed evaluation written here as plain
functions over the checkpoint's key names (first frame alone, then one latent frame at a time, every causal convolution fed from a cache
of its last two input frames — the procedure of the published implementation), plus key grammar, size and normalisation."""
import json
import os

import pytest
import torch
import torch.nn.functional as F

from unirl_b200.models.dit.vae_wan import AutoencoderKLWan, WanVAEConfig, is_wan_vae


# ------------------------------------------------------------------------------------------------ streamed statement over the keys
def _conv(sd, key, x, cache, pad=(1, 1, 1), stride=1):
    """Causal convolution of one chunk: the cache holds the last two frames this convolution has seen."""
    w, b = sd[key + ".weight"], sd[key + ".bias"]
    front = 2 * pad[0]
    if front:
        prev = cache.get(key)
        keep = x[:, :, -2:]
        if keep.shape[2] < 2 and prev is not None:
            keep = torch.cat([prev[:, :, -1:], keep], 2)
        if prev is not None:
            x = torch.cat([prev, x], 2)
            front -= prev.shape[2]
        cache[key] = keep
    return F.conv3d(F.pad(x, (pad[2], pad[2], pad[1], pad[1], max(front, 0), 0)), w, b, stride=stride)


def _rms(sd, key, x):
    g = sd[key + ".gamma"]
    return F.normalize(x, dim=1) * (x.shape[1] ** 0.5) * g


def _res(sd, p, x, cache):
    h = _conv(sd, p + ".conv1", F.silu(_rms(sd, p + ".norm1", x)), cache)
    h = _conv(sd, p + ".conv2", F.silu(_rms(sd, p + ".norm2", h)), cache)
    return h + (_conv(sd, p + ".conv_shortcut", x, cache, pad=(0, 0, 0)) if p + ".conv_shortcut.weight" in sd else x)


def _attn(sd, p, x):
    b, c, t, h, w = x.shape
    y = x.permute(0, 2, 1, 3, 4).reshape(b * t, c, h, w)
    qkv = F.conv2d(_rms(sd, p + ".norm", y), sd[p + ".to_qkv.weight"], sd[p + ".to_qkv.bias"]).reshape(b * t, 3, c, h * w)
    q, k, v = (qkv[:, i].transpose(1, 2) for i in range(3))
    o = torch.softmax(q @ k.transpose(1, 2) / c ** 0.5, -1) @ v
    o = F.conv2d(o.transpose(1, 2).reshape(b * t, c, h, w), sd[p + ".proj.weight"], sd[p + ".proj.bias"])
    return x + o.view(b, t, c, h, w).permute(0, 2, 1, 3, 4)


def _frames(fn, x):
    b, c, t, h, w = x.shape
    y = fn(x.permute(0, 2, 1, 3, 4).reshape(b * t, c, h, w))
    return y.view(b, t, *y.shape[1:]).permute(0, 2, 1, 3, 4)


def _mid(sd, p, x, cache):
    return _res(sd, p + ".resnets.1", _attn(sd, p + ".attentions.0", _res(sd, p + ".resnets.0", x, cache)), cache)


def _down(sd, p, x, cache):
    x = _frames(lambda y: F.conv2d(F.pad(y, (0, 1, 0, 1)), sd[p + ".resample.1.weight"], sd[p + ".resample.1.bias"], stride=2), x)
    if p + ".time_conv.weight" in sd:
        if p not in cache:
            cache[p] = x.clone()  # first chunk: one frame, passes through
        else:
            last = x[:, :, -1:].clone()
            x = F.conv3d(torch.cat([cache[p][:, :, -1:], x], 2), sd[p + ".time_conv.weight"], sd[p + ".time_conv.bias"], stride=(2, 1, 1))
            cache[p] = last
    return x


def _up(sd, p, x, cache):
    if p + ".time_conv.weight" in sd:
        if p not in cache:
            cache[p] = "first"  # the first latent frame is not doubled
        else:
            keep = x[:, :, -2:]
            if isinstance(cache[p], str):
                if keep.shape[2] < 2:
                    keep = torch.cat([torch.zeros_like(keep), keep], 2)
                y = F.conv3d(F.pad(x, (0, 0, 0, 0, 2, 0)), sd[p + ".time_conv.weight"], sd[p + ".time_conv.bias"])
            else:
                if keep.shape[2] < 2:
                    keep = torch.cat([cache[p][:, :, -1:], keep], 2)
                y = F.conv3d(torch.cat([cache[p], x], 2), sd[p + ".time_conv.weight"], sd[p + ".time_conv.bias"])
            cache[p] = keep
            b, c2, t, h, w = y.shape
            y = y.reshape(b, 2, c2 // 2, t, h, w)
            x = torch.stack((y[:, 0], y[:, 1]), 3).reshape(b, c2 // 2, 2 * t, h, w)
    return _frames(lambda y: F.conv2d(F.interpolate(y, scale_factor=2.0, mode="nearest-exact"), sd[p + ".resample.1.weight"], sd[p + ".resample.1.bias"], padding=1), x)


def _encode_streamed(sd, video, z_dim):
    cache, outs = {}, []
    n_down = max(int(k.split(".")[2]) for k in sd if k.startswith("encoder.down_blocks.")) + 1
    chunks = [video[:, :, :1]] + [video[:, :, 1 + 4 * i : 5 + 4 * i] for i in range((video.shape[2] - 1) // 4)]
    for x in chunks:
        x = _conv(sd, "encoder.conv_in", x, cache)
        for i in range(n_down):
            p = f"encoder.down_blocks.{i}"
            x = _res(sd, p, x, cache) if p + ".conv1.weight" in sd else _down(sd, p, x, cache)
        x = _mid(sd, "encoder.mid_block", x, cache)
        outs.append(_conv(sd, "encoder.conv_out", F.silu(_rms(sd, "encoder.norm_out", x)), cache))
    enc = F.conv3d(torch.cat(outs, 2), sd["quant_conv.weight"], sd["quant_conv.bias"])
    return enc[:, :z_dim]


def _decode_streamed(sd, z):
    cache, outs = {}, []
    z = F.conv3d(z, sd["post_quant_conv.weight"], sd["post_quant_conv.bias"])
    n_up = max(int(k.split(".")[2]) for k in sd if k.startswith("decoder.up_blocks.")) + 1
    for f in range(z.shape[2]):
        x = _mid(sd, "decoder.mid_block", _conv(sd, "decoder.conv_in", z[:, :, f : f + 1], cache), cache)
        for i in range(n_up):
            p, j = f"decoder.up_blocks.{i}", 0
            while f"{p}.resnets.{j}.conv1.weight" in sd:
                x = _res(sd, f"{p}.resnets.{j}", x, cache)
                j += 1
            if f"{p}.upsamplers.0.resample.1.weight" in sd:
                x = _up(sd, f"{p}.upsamplers.0", x, cache)
        outs.append(_conv(sd, "decoder.conv_out", F.silu(_rms(sd, "decoder.norm_out", x)), cache))
    return torch.cat(outs, 2).clamp(-1, 1)


# ------------------------------------------------------------------------------------------------------------------------- tests
@pytest.fixture(scope="module")
def tiny():
    torch.manual_seed(0)
    vae = AutoencoderKLWan(WanVAEConfig.tiny()).init_weights(3)
    return vae, {k: v.clone() for k, v in vae.state_dict().items()}


def test_decode_in_one_pass_equals_the_streamed_decode(tiny):
    vae, sd = tiny
    c = vae.cfg
    z = torch.randn(2, c.z_dim, 4, 3, 5)
    mean = torch.tensor(c.latents_mean).view(1, -1, 1, 1, 1)
    std = torch.tensor(c.latents_std).view(1, -1, 1, 1, 1)
    want = _decode_streamed(sd, z * std + mean) / 2 + 0.5  # [B, 3, T, H, W]
    got = vae.decode(z)  # [B, T, 3, H, W]
    assert got.shape == (2, 13, 3, 24, 40)
    assert float(want.std()) > 1e-3
    torch.testing.assert_close(got, want.permute(0, 2, 1, 3, 4), atol=2e-5, rtol=1e-4)
    # one frame in, one frame out (Qwen-Image uses the codec this way)
    one = vae.decode(z[:, :, 0])
    torch.testing.assert_close(one, got[:, 0], atol=2e-5, rtol=1e-4)


def test_encode_in_one_pass_equals_the_streamed_encode(tiny):
    vae, sd = tiny
    c = vae.cfg
    video = torch.rand(1, 3, 9, 16, 24)
    mean = torch.tensor(c.latents_mean).view(1, -1, 1, 1, 1)
    std = torch.tensor(c.latents_std).view(1, -1, 1, 1, 1)
    want = (_encode_streamed(sd, video * 2 - 1, c.z_dim) - mean) / std
    got = vae.encode_video(video)
    assert got.shape == (1, c.z_dim, 3, 2, 3)
    torch.testing.assert_close(got, want, atol=2e-5, rtol=1e-4)
    torch.testing.assert_close(vae.encode(video[:, :, 0]), got[:, :, 0], atol=2e-5, rtol=1e-4)
    with pytest.raises(ValueError, match="4k \\+ 1"):
        vae.encode_video(video[:, :, :8])


def test_published_geometry_has_the_published_key_names_and_size():
    with torch.device("meta"):
        vae = AutoencoderKLWan(WanVAEConfig(), device="meta")
    sd = vae.state_dict()
    assert round(sum(v.numel() for v in sd.values()) / 1e6) == 127, "the WAN 2.1 codec has 127 M parameters"
    for key, shape in {
        "encoder.conv_in.weight": (96, 3, 3, 3, 3),
        "encoder.down_blocks.0.norm1.gamma": (96, 1, 1, 1),
        "encoder.down_blocks.2.resample.1.weight": (96, 96, 3, 3),
        "encoder.down_blocks.3.conv_shortcut.weight": (192, 96, 1, 1, 1),
        "encoder.down_blocks.5.time_conv.weight": (192, 192, 3, 1, 1),
        "encoder.mid_block.attentions.0.norm.gamma": (384, 1, 1),
        "encoder.mid_block.attentions.0.to_qkv.weight": (1152, 384, 1, 1),
        "encoder.conv_out.weight": (32, 384, 3, 3, 3),
        "quant_conv.weight": (32, 32, 1, 1, 1),
        "post_quant_conv.weight": (16, 16, 1, 1, 1),
        "decoder.conv_in.weight": (384, 16, 3, 3, 3),
        "decoder.up_blocks.0.resnets.2.conv2.weight": (384, 384, 3, 3, 3),
        "decoder.up_blocks.0.upsamplers.0.time_conv.weight": (768, 384, 3, 1, 1),
        "decoder.up_blocks.0.upsamplers.0.resample.1.weight": (192, 384, 3, 3),
        "decoder.up_blocks.1.resnets.0.conv_shortcut.weight": (384, 192, 1, 1, 1),
        "decoder.up_blocks.3.resnets.0.conv1.weight": (96, 96, 3, 3, 3),
        "decoder.norm_out.gamma": (96, 1, 1, 1),
        "decoder.conv_out.bias": (3,),
    }.items():
        assert key in sd and tuple(sd[key].shape) == shape, key
    assert "decoder.up_blocks.2.upsamplers.0.time_conv.weight" not in sd and "decoder.up_blocks.3.upsamplers.0.resample.1.weight" not in sd
    assert vae.cfg.spatial_factor == 8 and vae.cfg.temporal_factor == 4 and vae.cfg.latent_channels == 16


def test_a_vae_folder_round_trips_through_the_importer(tmp_path, tiny):
    from safetensors.torch import save_file

    vae, sd = tiny
    c = vae.cfg
    folder = tmp_path / "vae"
    os.makedirs(folder)
    with open(folder / "config.json", "w") as f:
        json.dump({"_class_name": "AutoencoderKLWan", "base_dim": c.base_dim, "z_dim": c.z_dim, "dim_mult": list(c.dim_mult), "num_res_blocks": c.num_res_blocks,
                   "attn_scales": [], "temperal_downsample": list(c.temporal_downsample), "latents_mean": list(c.latents_mean), "latents_std": list(c.latents_std)}, f)
    save_file({k: v.contiguous() for k, v in sd.items()}, str(folder / "diffusion_pytorch_model.safetensors"))
    assert is_wan_vae(str(folder))
    back = AutoencoderKLWan.from_hf(str(folder))
    z = torch.randn(1, c.z_dim, 2, 2, 2)
    torch.testing.assert_close(back.decode(z), vae.decode(z))


def test_wan_bundle_uses_the_checkpoints_codec_and_encodes_the_first_frame_as_a_clip(tmp_path):
    """A checkpoint folder with a ``vae`` sub-folder in the published layout: the image-to-video condition is the codec's encoding of
    "first frame, then grey", whose later latent frames are not zero (the codec is causal in time)."""
    from safetensors.torch import save_file

    from unirl_b200.models.wan21.pipeline import Wan21Pipeline, Wan21PipelineConfig

    rnd = Wan21Pipeline.from_config(Wan21PipelineConfig(pretrained_model_ckpt_path="random:tiny-wan", model_precision="fp32", autocast_precision="fp32", device="cpu", image_to_video=True))
    zc = rnd.bundle.spec.transformer.in_channels
    save_file({k: v.contiguous() for k, v in rnd.bundle.transformer.state_dict().items()}, str(tmp_path / "transformer.safetensors"))
    (tmp_path / "config.json").write_text(json.dumps({"preset": "tiny-wan"}))
    c = WanVAEConfig.tiny(zc)
    codec = AutoencoderKLWan(c).init_weights(5)
    (tmp_path / "vae").mkdir()
    (tmp_path / "vae" / "config.json").write_text(json.dumps({"_class_name": "AutoencoderKLWan", "base_dim": c.base_dim, "z_dim": c.z_dim, "dim_mult": list(c.dim_mult),
                                                              "num_res_blocks": c.num_res_blocks, "attn_scales": [], "temperal_downsample": list(c.temporal_downsample),
                                                              "latents_mean": list(c.latents_mean), "latents_std": list(c.latents_std)}))
    save_file({k: v.contiguous() for k, v in codec.state_dict().items()}, str(tmp_path / "vae" / "diffusion_pytorch_model.safetensors"))
    pipe = Wan21Pipeline.from_config(Wan21PipelineConfig(pretrained_model_ckpt_path=str(tmp_path), model_precision="fp32", autocast_precision="fp32", device="cpu", image_to_video=True))
    assert isinstance(pipe.bundle.vae, AutoencoderKLWan)
    image = torch.rand(2, 3, 16, 16)
    cond = pipe.bundle.first_frame_condition(image, num_latent_frames=3).latents
    assert cond.shape == (2, 4 + zc, 3, 2, 2)
    assert bool((cond[:, :4, 0] == 1).all()) and bool((cond[:, :4, 1:] == 0).all())
    clip = torch.full((2, 3, 9, 16, 16), 0.5)
    clip[:, :, 0] = image
    torch.testing.assert_close(cond[:, 4:], codec.encode_video(clip))
    assert float(cond[:, 4:, 1:].abs().max()) > 1e-3
    # and the sampler decodes 4 (F - 1) + 1 frames through it
    z = torch.randn(1, zc, 3, 2, 2)
    assert pipe.bundle.vae.decode(z).shape == (1, 9, 3, 16, 16)
