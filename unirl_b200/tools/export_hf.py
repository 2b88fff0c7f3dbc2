"""Export a training checkpoint as a Hugging Face style model directory.

``python -m unirl_b200.tools.export_hf --checkpoint <dir with checkpoint.pt> --base <model spec or dir> --out <dir> [--family qwen3|sd3]
[--adapter-only]``

* full checkpoints: the policy weights are written in the family's HF key grammar (un-fused q/k/v, gate/up) as sharded
  ``model-0000x-of-0000y.safetensors`` + ``model.safetensors.index.json`` + ``config.json``;
* LoRA checkpoints (``save_mode="adapter"`` or a ``lora_config`` in the checkpoint): adapters are merged into the base
  weights first (``W += B·A·alpha/r``) unless ``--adapter-only``, which writes a PEFT-format ``adapter_model.safetensors`` +
  ``adapter_config.json`` instead.
Parity: ``unirl/tools/export_hf.py`` (merge LoRA / load distributed checkpoint → HF export).
"""

from __future__ import annotations

import argparse
import json
import os
from typing import Dict, Optional

import torch


def _build(family: str, base: str, device: str = "cpu"):
    if family == "qwen3":
        from unirl_b200.models.qwen3.bundle import Qwen3Bundle
        from unirl_b200.models.qwen3.config import Qwen3PipelineConfig

        return Qwen3Bundle.from_config(Qwen3PipelineConfig(pretrained_model_ckpt_path=base, device=device, model_precision="bf16"))
    if family == "sd3":
        from unirl_b200.models.sd3.bundle import SD3Bundle
        from unirl_b200.models.sd3.config import SD3PipelineConfig

        return SD3Bundle.from_config(SD3PipelineConfig(pretrained_model_ckpt_path=base, device=device, model_precision="bf16"))
    raise ValueError(f"unknown family {family!r} (qwen3 | sd3)")


def _hf_tensors(family: str, model: torch.nn.Module) -> Dict[str, torch.Tensor]:
    if family == "qwen3":
        return {k: v.detach().cpu().contiguous() for k, v in model.hf_state_dict().items()}
    from unirl_b200.models.sd3.hf_keys import to_diffusers

    sd = {k: v.detach().cpu() for k, v in model.state_dict().items()}
    out = to_diffusers(sd, model.cfg.num_joint_blocks, model.cfg.hidden_size)
    out.update({k: v for k, v in sd.items() if ".qkv." not in k})  # non-fused tensors keep their native names
    return {k: v.contiguous() for k, v in out.items()}


def write_sharded(tensors: Dict[str, torch.Tensor], out: str, max_shard_bytes: int = 5 << 30) -> None:
    from safetensors.torch import save_file

    shards, cur, size = [], {}, 0
    for k, v in tensors.items():
        n = v.numel() * v.element_size()
        if cur and size + n > max_shard_bytes:
            shards.append(cur)
            cur, size = {}, 0
        cur[k] = v
        size += n
    if cur:
        shards.append(cur)
    index = {"metadata": {"total_size": sum(v.numel() * v.element_size() for v in tensors.values())}, "weight_map": {}}
    for i, sh in enumerate(shards):
        name = "model.safetensors" if len(shards) == 1 else f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        save_file(sh, os.path.join(out, name))
        index["weight_map"].update({k: name for k in sh})
    if len(shards) > 1:
        with open(os.path.join(out, "model.safetensors.index.json"), "w") as f:
            json.dump(index, f, indent=1)


def export(checkpoint: str, base: str, out: str, family: str = "qwen3", adapter_only: bool = False) -> Dict[str, int]:
    ckpt = torch.load(os.path.join(checkpoint, "checkpoint.pt"), map_location="cpu", weights_only=False)
    sd, lora_cfg = ckpt["policy_state_dict"], ckpt.get("lora_config")
    bundle = _build(family, base)
    model = bundle.transformer
    os.makedirs(out, exist_ok=True)
    if lora_cfg:
        from unirl_b200.train import inject
        from unirl_b200.utils.peft_merge import merged_state_dict

        inject.inject_lora(model, rank=int(lora_cfg["rank"]), alpha=float(lora_cfg["alpha"]), target_modules=tuple(lora_cfg["target_modules"]))
    missing, unexpected = model.load_state_dict(sd, strict=False)
    if unexpected:
        raise RuntimeError(f"checkpoint holds tensors the model does not have: {unexpected[:5]}")
    if lora_cfg and adapter_only:
        from safetensors.torch import save_file

        tensors = {k: v.detach().cpu().contiguous() for k, v in inject.lora_named_tensors(model).items()}
        save_file(tensors, os.path.join(out, "adapter_model.safetensors"))
        with open(os.path.join(out, "adapter_config.json"), "w") as f:
            json.dump(inject.peft_config_dict(lora_cfg["rank"], lora_cfg["alpha"], lora_cfg["target_modules"]), f, indent=1)
        return {"tensors": len(tensors), "adapter": 1}
    if lora_cfg:
        merged = dict(merged_state_dict(model))
        for m in model.modules():  # drop the adapters, keep merged base weights
            if hasattr(m, "lora"):
                del m.lora
                m._lora_index = {}
        model.load_state_dict(merged, strict=False)
    tensors = _hf_tensors(family, model)
    write_sharded(tensors, out)
    cfg = getattr(model, "cfg", None)
    with open(os.path.join(out, "config.json"), "w") as f:
        json.dump({k: (list(v) if isinstance(v, tuple) else v) for k, v in vars(cfg).items() if isinstance(v, (int, float, str, bool, tuple, list, type(None)))}, f, indent=1)
    return {"tensors": len(tensors), "adapter": 0}


def main(argv: Optional[list] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--checkpoint", required=True)
    ap.add_argument("--base", required=True, help="model spec the checkpoint was trained from (random:<preset> or a checkpoint directory)")
    ap.add_argument("--out", required=True)
    ap.add_argument("--family", default="qwen3", choices=["qwen3", "sd3"])
    ap.add_argument("--adapter-only", action="store_true")
    a = ap.parse_args(argv)
    print(json.dumps(export(a.checkpoint, a.base, a.out, a.family, a.adapter_only)))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
