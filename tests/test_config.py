import os

import pytest

from unirl_b200.config import ConfigNode, compose, get_method, instantiate, parse_cfg, require
from unirl_b200.config.loader import apply_overrides, parse_cli


def test_interpolation_and_access(monkeypatch):
    monkeypatch.setenv("UB_X", "7")
    monkeypatch.delenv("UB_Y", raising=False)
    c = ConfigNode({"a": {"b": "${oc.env:UB_X}", "c": "${oc.env:UB_Y,${oc.env:UB_X}}", "d": "${oc.env:UB_Y,null}", "e": "${a.b}-x"}, "l": [1, {"k": "${a.b}"}]})
    assert c.a.b == "7" and c.a.c == "7" and c.a.d is None and c.a.e == "7-x" and c.l[1].k == "7"
    assert c.get("zzz", 3) == 3 and "a" in c and c.a.get("d", 5) == 5
    with pytest.raises(KeyError):
        ConfigNode({"x": "${oc.env:UB_Y}"}).x
    with pytest.raises(AttributeError):
        c.nope


def test_overrides_and_cli():
    d = apply_overrides({"a": {"b": 1}, "z": 2}, ["a.b=5", "+a.c=[1,2]", "~z", "+n.m=true"])
    assert d == {"a": {"b": 5, "c": [1, 2]}, "n": {"m": True}}
    with pytest.raises(KeyError):
        apply_overrides({"a": 1}, ["b=2"])
    name, cdir, ov, flags = parse_cli(["--config-name=ar/x", "--config-dir", "ex", "k=v", "--cfg", "job", "--resolve"])
    assert (name, cdir, ov) == ("ar/x", "ex", ["k=v"]) and flags == {"cfg": True, "resolve": True}


def test_instantiate_and_reference_target_names():
    obj = instantiate({"_target_": "unirl.types.sampling.ARSamplingParams", "samples_per_prompt": 4, "temperature": 1.0})
    assert type(obj).__module__ == "unirl_b200.types.sampling" and obj.samples_per_prompt == 4
    cls = instantiate({"_target_": "hydra.utils.get_class", "path": "unirl.models.qwen3.conditions.Qwen3ARConditions"})
    assert cls.__name__ == "Qwen3ARConditions"
    nested = parse_cfg(ConfigNode({"_target_": "unirl_b200.train.stack.TrainStack", "micro_batch_size": 2, "inner": {"_target_": "x.y"}}))
    assert nested["role_cls"].__name__ == "TrainStack" and nested["inner"] == {"_target_": "x.y"}
    assert get_method("unirl_b200.models.qwen3.bundle.Qwen3Bundle.from_config").__self__.__name__ == "Qwen3Bundle"
    part = instantiate({"_target_": "builtins.int", "_partial_": True, "base": 2})
    assert part("101") == 5
    with pytest.raises(ValueError):
        require(False, "nope")


def test_every_recipe_target_resolves():
    """Static recipe check (the reference ships this as a pre-commit hook, scripts/check_recipe_targets.py)."""
    from unirl_b200.tools.check_recipe_targets import check_tree

    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples")
    problems = check_tree(root)
    assert not problems, "\n".join(problems)


def test_compose_recipe():
    cfg = compose("ar/tiny_qwen3_grpo_cpu", overrides=["num_rollouts=3"])
    assert cfg.num_rollouts == 3 and cfg.bundle.config.pretrained_model_ckpt_path == "random:tiny"


def test_recipe_validators_flag_cross_component_mistakes():
    from unirl_b200.config.loader import compose
    from unirl_b200.config.validation import ConfigValidationError, validate_recipe

    validate_recipe(compose("ar/qwen3_4b_grpo_b200", overrides=[]))
    validate_recipe(compose("diffusion/tiny_sd3_flowgrpo_cpu", overrides=[]))
    for ov, needle in ((["rollout.config.tp_size=4"], "rollout_parallel"), (["sampling.max_new_tokens=8192"], "max_new_tokens"), (["batch_size=3", "num_devices=8", "sampling.samples_per_prompt=1"], "data-parallel")):
        with pytest.raises(ConfigValidationError, match=needle):
            validate_recipe(compose("ar/qwen3_4b_grpo_b200", overrides=ov))
    with pytest.raises(ConfigValidationError, match="guidance"):
        validate_recipe(compose("diffusion/tiny_sd3_flowgrpo_cpu", overrides=["sampling.guidance_scale=5.0"]))
    with pytest.raises(ConfigValidationError, match="sde_indices"):
        validate_recipe(compose("diffusion/tiny_sd3_flowgrpo_cpu", overrides=["sampling.sde_indices=[0, 9]"]))
    with pytest.raises(ConfigValidationError, match="not executed"):
        validate_recipe(compose("ar/qwen3_4b_grpo_b200", overrides=["+train_parallel={cp: 2}"]))
    with pytest.raises(ConfigValidationError, match="sp_size"):
        validate_recipe(compose("diffusion/wan21_14b_dancegrpo_sp8_b200", overrides=["backend.fsdp_cfg.sp_size=4"]))
    validate_recipe(compose("diffusion/wan21_14b_dancegrpo_sp8_b200", overrides=[]))


def test_export_hf_full_and_lora(tmp_path):
    import torch
    from safetensors.torch import load_file

    from unirl_b200.models.qwen3.bundle import Qwen3Bundle
    from unirl_b200.models.qwen3.config import Qwen3PipelineConfig
    from unirl_b200.tools.export_hf import export
    from unirl_b200.train import inject

    b = Qwen3Bundle.from_config(Qwen3PipelineConfig(pretrained_model_ckpt_path="random:tiny", device="cpu", model_precision="bf16"))
    m = b.transformer
    (tmp_path / "full").mkdir()
    torch.save({"policy_state_dict": {k: v.detach().clone() for k, v in m.state_dict().items()}, "lora_config": None}, tmp_path / "full" / "checkpoint.pt")
    assert export(str(tmp_path / "full"), "random:tiny", str(tmp_path / "out_full"))["tensors"] > 10
    hf = load_file(str(tmp_path / "out_full" / "model.safetensors"))
    nq = m.layers[0].n_q * m.cfg.head_dim
    assert torch.equal(hf["model.layers.0.self_attn.q_proj.weight"], m.layers[0].qkv_proj[:nq].detach())
    # LoRA checkpoint: merged export equals W + B·A·alpha/r, adapter-only export is PEFT shaped
    inject.inject_lora(m, rank=4, alpha=8, target_modules=("q_proj", "v_proj"))
    for mod in m.modules():
        if hasattr(mod, "lora"):
            for ad in mod.lora.values():
                torch.nn.init.normal_(ad.lora_B, std=0.05)
    (tmp_path / "lora").mkdir()
    torch.save({"policy_state_dict": {k: v.detach().clone() for k, v in m.state_dict().items()},
                "lora_config": {"rank": 4, "alpha": 8, "target_modules": ["q_proj", "v_proj"]}}, tmp_path / "lora" / "checkpoint.pt")
    export(str(tmp_path / "lora"), "random:tiny", str(tmp_path / "out_merged"))
    merged = load_file(str(tmp_path / "out_merged" / "model.safetensors"))
    ad = m.layers[0].lora["q_proj__default"]
    want = (m.layers[0].qkv_proj[:nq].float() + ad.lora_B.float() @ ad.lora_A.float() * ad.scaling).to(torch.bfloat16)
    torch.testing.assert_close(merged["model.layers.0.self_attn.q_proj.weight"].float(), want.float(), atol=1e-2, rtol=1e-2)
    assert export(str(tmp_path / "lora"), "random:tiny", str(tmp_path / "out_adapter"), adapter_only=True)["adapter"] == 1
    peft = load_file(str(tmp_path / "out_adapter" / "adapter_model.safetensors"))
    assert any(k.endswith("self_attn.q_proj.lora_A.default.weight") for k in peft)


def test_relative_interpolations():
    """``${.key}`` names a sibling, every further dot climbs one mapping (list entries count as a level), as in the recipes' schedulers
    (``num_timesteps: ${..num_inference_steps}``)."""
    from unirl_b200.config.node import ConfigNode, to_container

    c = ConfigNode({"n": 10, "s": {"steps": 4, "sched": {"num": "${..steps}", "same": "${.num}", "abs": "${n}", "lst": [{"k": "${....steps}", "j": "${.k}"}]}}})
    assert to_container(c)["s"]["sched"] == {"num": 4, "same": 4, "abs": 10, "lst": [{"k": 4, "j": 4}]}
    assert c.s.sched.num == 4 and c.s.sched.lst[0].j == 4
    import pytest

    with pytest.raises(KeyError):
        ConfigNode({"a": {"b": "${...x}"}}).a.b
