"""Recipe/config system: flat YAML recipes with ``_target_`` nodes, env interpolation, CLI overrides."""
from unirl_b200.config.node import ConfigNode, to_container  # noqa: F401
from unirl_b200.config.loader import compose, load_recipe, main_entry, parse_cli  # noqa: F401
from unirl_b200.config.instantiate import get_class, get_method, instantiate, parse_cfg  # noqa: F401
from unirl_b200.config.require import require  # noqa: F401
