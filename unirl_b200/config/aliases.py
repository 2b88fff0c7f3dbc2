"""Name tables for recipes written for the reference: pure data, importable without torch (the static recipe checker reads this file too).

``ALIASES``          whole targets that live elsewhere (``hydra.utils.*`` helpers).
``MODULE_ALIASES``   module paths of the reference that have no same-named module here → the module that holds the same names
                     (longest prefix first).  Paths are written after the ``unirl`` → ``unirl_b200`` package rename.
``NAME_ALIASES``     class names the reference spells differently.
"""

ALIASES = {
    "hydra.utils.get_class": "unirl_b200.config.instantiate.get_class",
    "hydra.utils.get_method": "unirl_b200.config.instantiate.get_method",
}

MODULE_ALIASES = tuple(sorted({
    **{f"unirl_b200.reward.local.{m}": "unirl_b200.reward.local.specs"
       for m in ("clip", "pickscore", "hpsv2", "hpsv3", "image_reward", "aesthetic", "ocr", "geneval2", "video", "video_pickscore", "registry")},
    "unirl_b200.reward.local.base": "unirl_b200.reward.base",
    # engines that drive external serving stacks in the reference: the native engines under the same class names
    **{f"unirl_b200.rollout.engine.{pkg}.{mod}": "unirl_b200.rollout.engine.compat" for pkg in ("sglang", "sglang_llm", "vllm_omni") for mod in ("engine", "config")},
    "unirl_b200.rollout.engine.composed.config": "unirl_b200.rollout.engine.compat",
    "unirl_b200.distributed.tensor.backend.transfer_queue.simple": "unirl_b200.distributed.tensor.backend.transfer_queue",
    "unirl_b200.distributed.tensor.backend.transfer_queue.mooncake": "unirl_b200.distributed.tensor.backend.transfer_queue",
}.items(), key=lambda kv: -len(kv[0])))

NAME_ALIASES = {"WAN21Bundle": "Wan21Bundle", "WAN21Pipeline": "Wan21Pipeline", "WAN21PipelineConfig": "Wan21PipelineConfig", "WAN21Conditions": "Wan21Conditions",
                "WAN22Bundle": "Wan22Bundle", "WAN22Pipeline": "Wan22Pipeline", "WAN22PipelineConfig": "Wan22PipelineConfig", "WAN22Conditions": "Wan22Conditions"}


def translate(path: str) -> str:
    """A target as written in a recipe → the dotted path to look up in this package."""
    if path in ALIASES:
        return ALIASES[path]
    if path == "unirl" or path.startswith("unirl."):
        path = "unirl_b200" + path[len("unirl"):]
    for old, new in MODULE_ALIASES:
        if path == old or path.startswith(old + "."):
            path = new + path[len(old):]
            break
    return ".".join(NAME_ALIASES.get(p, p) for p in path.split("."))
