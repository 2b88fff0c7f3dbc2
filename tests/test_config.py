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
