"""Key bridges from diffusers transformer checkpoints to the native fused-parameter DiT module.

diffusers keeps ``to_q / to_k / to_v`` (and ``add_*_proj``) as separate matrices and names modulation, patch and time embedders per
family; the native module fuses QKV per stream (and, in single-stream blocks, QKV with the MLP input projection) and uses one naming
scheme.  A bridge is a table of (native name ← diffusers name) plus the row-wise concatenations of the fused weights.

Families covered: the joint-block (MMDiT) layouts -- Stable Diffusion 3.x (``SD3Transformer2DModel``), FLUX-style double + single
stream models (``FluxTransformer2DModel`` naming: FLUX.2 klein, HunyuanVideo, Z-Image single-stream) and Qwen-Image
(``QwenImageTransformer2DModel``).  The reference loads these through diffusers itself (``unirl/models/sd3/bundle.py``,
``unirl/models/qwen_image/bundle.py``, ``unirl/models/flux2_klein/bundle.py``); here the published weights go straight into the native module.
WAN 2.1 / 2.2 text-to-video (``WanTransformer3DModel``: cross-attention blocks with full-width q/k norms, a two-layer text embedder and
table-based modulation; ``unirl/models/wan21/diffusion.py:62-158``) has a bridge of its own; the image-to-video checkpoints carry an
extra image embedder that the native module does not have and are refused.
"""

from __future__ import annotations

from typing import Callable, Dict, Iterable, List, Optional, Tuple

import torch

Tensor = torch.Tensor


def _cat(sd: Dict[str, Tensor], names: Iterable[str], suffix: str) -> Optional[Tensor]:
    parts = [sd.get(f"{n}.{suffix}") for n in names]
    if any(p is None for p in parts):
        return None
    return torch.cat(parts, 0)


class _Writer:
    def __init__(self, src: Dict[str, Tensor]):
        self.src, self.out, self.used = src, {}, set()

    def put(self, dst: str, src: str) -> None:
        """Copy ``<src>.weight/.bias`` (whichever exist) to ``<dst>.*``."""
        for s in ("weight", "bias"):
            k = f"{src}.{s}"
            if k in self.src:
                self.out[f"{dst}.{s}"] = self.src[k]
                self.used.add(k)

    def raw(self, dst: str, src: str) -> None:
        if src in self.src:
            self.out[dst] = self.src[src]
            self.used.add(src)

    def fuse(self, dst: str, names: List[str]) -> None:
        """Row-wise concatenation of several diffusers linears into one fused native linear."""
        for s in ("weight", "bias"):
            t = _cat(self.src, names, s)
            if t is not None:
                self.out[f"{dst}.{s}"] = t
                self.used.update(f"{n}.{s}" for n in names)


def _joint_block(w: _Writer, s: str, d: str, *, mod: Tuple[str, str], img_mlp: Tuple[str, str], txt_mlp: Tuple[str, str], dual: bool) -> None:
    w.put(f"{d}.img_mod", f"{s}.{mod[0]}")
    w.put(f"{d}.txt_mod", f"{s}.{mod[1]}")
    w.fuse(f"{d}.img_attn.qkv", [f"{s}.attn.to_q", f"{s}.attn.to_k", f"{s}.attn.to_v"])
    w.fuse(f"{d}.txt_attn.qkv", [f"{s}.attn.add_q_proj", f"{s}.attn.add_k_proj", f"{s}.attn.add_v_proj"])
    w.put(f"{d}.img_attn.out", f"{s}.attn.to_out.0")
    w.put(f"{d}.txt_attn.out", f"{s}.attn.to_add_out")
    for a, b in (("img_attn.q_norm", "attn.norm_q.weight"), ("img_attn.k_norm", "attn.norm_k.weight"), ("txt_attn.q_norm", "attn.norm_added_q.weight"),
                 ("txt_attn.k_norm", "attn.norm_added_k.weight")):
        w.raw(f"{d}.{a}", f"{s}.{b}")
    if dual:
        w.fuse(f"{d}.img_attn2.qkv", [f"{s}.attn2.to_q", f"{s}.attn2.to_k", f"{s}.attn2.to_v"])
        w.put(f"{d}.img_attn2.out", f"{s}.attn2.to_out.0")
        w.raw(f"{d}.img_attn2.q_norm", f"{s}.attn2.norm_q.weight")
        w.raw(f"{d}.img_attn2.k_norm", f"{s}.attn2.norm_k.weight")
    w.put(f"{d}.img_mlp.fc1", f"{s}.{img_mlp[0]}")
    w.put(f"{d}.img_mlp.fc2", f"{s}.{img_mlp[1]}")
    w.put(f"{d}.txt_mlp.fc1", f"{s}.{txt_mlp[0]}")
    w.put(f"{d}.txt_mlp.fc2", f"{s}.{txt_mlp[1]}")


def _single_block(w: _Writer, s: str, d: str) -> None:
    w.put(f"{d}.mod", f"{s}.norm.linear")
    w.fuse(f"{d}.in_proj", [f"{s}.attn.to_q", f"{s}.attn.to_k", f"{s}.attn.to_v", f"{s}.proj_mlp"])  # one GEMM: q | k | v | mlp-in
    w.raw(f"{d}.q_norm", f"{s}.attn.norm_q.weight")
    w.raw(f"{d}.k_norm", f"{s}.attn.norm_k.weight")
    w.put(f"{d}.out_proj", f"{s}.proj_out")  # diffusers applies it to cat(attention, mlp): the same column order as here


def _channel_major_out(w: _Writer, patch_elems: int) -> None:
    """SD3 and WAN un-patchify their output with the channel LAST inside a patch (row ``p * C + c`` of ``proj_out``); the native module
    keeps the channel first, as on the input side (row ``c * P + p``).  Reorder the rows of the output projection accordingly."""
    for suf in ("weight", "bias"):
        k = f"final_proj.{suf}"
        if k in w.out and patch_elems > 1:
            t = w.out[k]
            w.out[k] = t.reshape(patch_elems, -1, *t.shape[1:]).transpose(0, 1).reshape(t.shape)


def _finish(w: _Writer, strict: bool) -> Dict[str, Tensor]:
    if "patch_embed.weight" in w.out and w.out["patch_embed.weight"].dim() > 2:  # a conv patch embedder: [h, c, (t,) p, p] -> [h, c * t * p * p]
        w.out["patch_embed.weight"] = w.out["patch_embed.weight"].flatten(1)
    if strict:
        left = sorted(k for k in w.src if k not in w.used)
        if left:
            raise KeyError(f"diffusers checkpoint has {len(left)} tensors this bridge does not place, e.g. {left[:6]}")
    return w.out


def sd3_from_diffusers(sd: Dict[str, Tensor], num_joint_blocks: int, dual: Iterable[int] = (), strict: bool = False, patch_elems: int = 4) -> Dict[str, Tensor]:
    w = _Writer(sd)
    w.put("patch_embed", "pos_embed.proj")
    w.put("time_in.0", "time_text_embed.timestep_embedder.linear_1")
    w.put("time_in.1", "time_text_embed.timestep_embedder.linear_2")
    w.put("pooled_in.0", "time_text_embed.text_embedder.linear_1")
    w.put("pooled_in.1", "time_text_embed.text_embedder.linear_2")
    w.put("text_in", "context_embedder")
    w.put("final_mod", "norm_out.linear")
    w.put("final_proj", "proj_out")
    w.raw("pos_embed_table", "pos_embed.pos_embed")
    dual = set(dual)
    for i in range(num_joint_blocks):
        _joint_block(w, f"transformer_blocks.{i}", f"joint_blocks.{i}", mod=("norm1.linear", "norm1_context.linear"), img_mlp=("ff.net.0.proj", "ff.net.2"),
                     txt_mlp=("ff_context.net.0.proj", "ff_context.net.2"), dual=i in dual)
    _channel_major_out(w, patch_elems)
    return _finish(w, strict)


def flux_from_diffusers(sd: Dict[str, Tensor], num_joint_blocks: int, num_single_blocks: int, strict: bool = False) -> Dict[str, Tensor]:
    """``FluxTransformer2DModel`` naming (double blocks ``transformer_blocks.*``, single blocks ``single_transformer_blocks.*``)."""
    w = _Writer(sd)
    w.put("patch_embed", "x_embedder")
    w.put("text_in", "context_embedder")
    w.put("time_in.0", "time_text_embed.timestep_embedder.linear_1")
    w.put("time_in.1", "time_text_embed.timestep_embedder.linear_2")
    w.put("guidance_in.0", "time_text_embed.guidance_embedder.linear_1")
    w.put("guidance_in.1", "time_text_embed.guidance_embedder.linear_2")
    w.put("pooled_in.0", "time_text_embed.text_embedder.linear_1")
    w.put("pooled_in.1", "time_text_embed.text_embedder.linear_2")
    w.put("final_mod", "norm_out.linear")
    w.put("final_proj", "proj_out")
    for i in range(num_joint_blocks):
        _joint_block(w, f"transformer_blocks.{i}", f"joint_blocks.{i}", mod=("norm1.linear", "norm1_context.linear"), img_mlp=("ff.net.0.proj", "ff.net.2"),
                     txt_mlp=("ff_context.net.0.proj", "ff_context.net.2"), dual=False)
    for i in range(num_single_blocks):
        _single_block(w, f"single_transformer_blocks.{i}", f"single_blocks.{i}")
    return _finish(w, strict)


def qwen_image_from_diffusers(sd: Dict[str, Tensor], num_joint_blocks: int, strict: bool = False) -> Dict[str, Tensor]:
    """``QwenImageTransformer2DModel`` naming (``img_in`` / ``txt_in``, ``img_mod.1`` / ``txt_mod.1``, ``img_mlp`` / ``txt_mlp``)."""
    w = _Writer(sd)
    w.put("patch_embed", "img_in")
    w.put("text_in", "txt_in")
    w.raw("text_norm", "txt_norm.weight")
    w.put("time_in.0", "time_text_embed.timestep_embedder.linear_1")
    w.put("time_in.1", "time_text_embed.timestep_embedder.linear_2")
    w.put("final_mod", "norm_out.linear")
    w.put("final_proj", "proj_out")
    for i in range(num_joint_blocks):
        _joint_block(w, f"transformer_blocks.{i}", f"joint_blocks.{i}", mod=("img_mod.1", "txt_mod.1"), img_mlp=("img_mlp.net.0.proj", "img_mlp.net.2"),
                     txt_mlp=("txt_mlp.net.0.proj", "txt_mlp.net.2"), dual=False)
    return _finish(w, strict)


def wan_from_diffusers(sd: Dict[str, Tensor], num_cross_blocks: int, strict: bool = False, patch_elems: int = 4) -> Dict[str, Tensor]:
    """``WanTransformer3DModel`` naming (``condition_embedder.*``, ``blocks.<i>.attn1 / attn2 / ffn / norm2 / scale_shift_table``)."""
    w = _Writer(sd)
    i2v = any(k.startswith("condition_embedder.image_embedder.") for k in sd)  # WAN 2.1 image-to-video: image-encoder tokens as a second context
    if i2v:
        e = "condition_embedder.image_embedder"
        w.put("image_in.norm1", f"{e}.norm1")
        w.put("image_in.fc1", f"{e}.ff.net.0.proj")
        w.put("image_in.fc2", f"{e}.ff.net.2")
        w.put("image_in.norm2", f"{e}.norm2")
    w.put("patch_embed", "patch_embedding")  # a Conv3d kernel [h, c, 1, 2, 2]: flattened to the patchify order (c, t, rows, cols) below
    w.put("time_in.0", "condition_embedder.time_embedder.linear_1")
    w.put("time_in.1", "condition_embedder.time_embedder.linear_2")
    w.put("time_proj", "condition_embedder.time_proj")
    w.put("text_in", "condition_embedder.text_embedder.linear_1")
    w.put("text_in2", "condition_embedder.text_embedder.linear_2")
    w.put("final_proj", "proj_out")
    if "scale_shift_table" in sd:
        w.out["final_table"] = sd["scale_shift_table"].reshape(2, -1)
        w.used.add("scale_shift_table")
    for i in range(num_cross_blocks):
        s_, d = f"blocks.{i}", f"cross_blocks.{i}"
        if f"{s_}.scale_shift_table" in sd:
            w.out[f"{d}.modulation"] = sd[f"{s_}.scale_shift_table"].reshape(6, -1)
            w.used.add(f"{s_}.scale_shift_table")
        w.fuse(f"{d}.self_attn.qkv", [f"{s_}.attn1.to_q", f"{s_}.attn1.to_k", f"{s_}.attn1.to_v"])
        w.put(f"{d}.self_attn.out", f"{s_}.attn1.to_out.0")
        w.raw(f"{d}.self_attn.q_norm", f"{s_}.attn1.norm_q.weight")
        w.raw(f"{d}.self_attn.k_norm", f"{s_}.attn1.norm_k.weight")
        w.put(f"{d}.cross_q", f"{s_}.attn2.to_q")
        w.fuse(f"{d}.cross_kv", [f"{s_}.attn2.to_k", f"{s_}.attn2.to_v"])
        w.put(f"{d}.cross_out", f"{s_}.attn2.to_out.0")
        w.raw(f"{d}.cross_q_norm", f"{s_}.attn2.norm_q.weight")
        w.raw(f"{d}.cross_k_norm", f"{s_}.attn2.norm_k.weight")
        if i2v:
            w.fuse(f"{d}.cross_kv_img", [f"{s_}.attn2.add_k_proj", f"{s_}.attn2.add_v_proj"])
            w.raw(f"{d}.cross_k_img_norm", f"{s_}.attn2.norm_added_k.weight")
        w.put(f"{d}.cross_norm", f"{s_}.norm2")
        w.put(f"{d}.mlp.fc1", f"{s_}.ffn.net.0.proj")
        w.put(f"{d}.mlp.fc2", f"{s_}.ffn.net.2")
    _channel_major_out(w, patch_elems)
    return _finish(w, strict)


def bridge_for(preset: str) -> Optional[Callable[..., Dict[str, Tensor]]]:
    """The bridge of a preset family, or ``None`` when the family loads native checkpoints only."""
    p = preset.lower()
    if "sd3" in p:
        return lambda sd, cfg, strict=False: sd3_from_diffusers(sd, cfg.num_joint_blocks, cfg.dual_attention_blocks, strict,
                                                                 cfg.patch_size[0] * cfg.patch_size[1] * cfg.patch_size[2])
    if "qwen-image" in p or "qwen_image" in p:
        return lambda sd, cfg, strict=False: qwen_image_from_diffusers(sd, cfg.num_joint_blocks, strict)
    if "wan" in p:
        return lambda sd, cfg, strict=False: wan_from_diffusers(sd, cfg.num_cross_blocks, strict, cfg.patch_size[0] * cfg.patch_size[1] * cfg.patch_size[2])
    if any(k in p for k in ("flux", "hunyuan-video", "z-image")) and "15" not in p:
        return lambda sd, cfg, strict=False: flux_from_diffusers(sd, cfg.num_joint_blocks, cfg.num_single_blocks, strict)
    return None


def load_diffusers_transformer(model: torch.nn.Module, sd: Dict[str, Tensor], preset: str, strict: bool = True) -> Tuple[List[str], List[str]]:
    """Place a diffusers state dict into ``model`` (a ``DiTTransformer``).  Returns ``(missing, unexpected)`` native keys; with ``strict`` a
    tensor whose shape disagrees with the module, or a native parameter left without a value, raises."""
    fn = bridge_for(preset)
    if fn is None:
        raise KeyError(f"no diffusers key bridge for preset {preset!r}")
    native = fn(sd, model.cfg, False)
    own = model.state_dict()
    bad = [k for k, v in native.items() if k in own and tuple(v.shape) != tuple(own[k].shape)]
    if bad:
        k = bad[0]
        raise ValueError(f"shape mismatch for {k}: checkpoint {tuple(native[k].shape)} vs module {tuple(own[k].shape)} ({len(bad)} in total)")
    table = native.pop("pos_embed_table", None)  # SD3 stores its sin-cos table [1, S * S, h]: take it as published instead of recomputing it
    if table is not None and getattr(model, "pos_table", None) is not None:
        if table.numel() != model.pos_table.numel():
            raise ValueError(f"position table of {table.numel()} values does not fit the module's {tuple(model.pos_table.shape)}")
        model.pos_table.copy_(table.reshape(model.pos_table.shape).to(model.pos_table.dtype))
    missing, unexpected = model.load_state_dict({k: v for k, v in native.items() if k in own}, strict=False)
    unexpected = list(unexpected) + [k for k in native if k not in own]
    if strict and missing:
        raise KeyError(f"{len(missing)} native parameters got no value from the checkpoint, e.g. {list(missing)[:6]}")
    return list(missing), unexpected


__all__ = ["sd3_from_diffusers", "flux_from_diffusers", "qwen_image_from_diffusers", "wan_from_diffusers", "bridge_for", "load_diffusers_transformer"]
