"""Typed configurations and the registries."""

from paged_kv_serving_b200.config.engine_config import DTYPES, EngineConfig
from paged_kv_serving_b200.config.model_config import CONFIG_FILE, ModelConfig
from paged_kv_serving_b200.config.registry import (
    architecture, known_architectures, known_parts, part, register_architecture, register_part,
)



def load_config(path):
    """Read ``config.json`` (a file or a model folder) into the typed configuration of the
    architecture it names: an architecture class may carry its own ``config_class`` (with
    ``from_dict``); without one the shared ``ModelConfig`` is used."""
    import json
    from pathlib import Path

    path = Path(path)
    if path.is_dir():
        path = path / CONFIG_FILE
    with open(path, encoding="utf-8") as handle:
        data = json.load(handle)
    if not isinstance(data, dict):
        raise ValueError(f"{path}: a model configuration must be a JSON object")
    name = data.get("architecture", "LlamaToyDecoder")
    config_class = getattr(architecture(name), "config_class", ModelConfig)
    return config_class.from_dict(data)


def write_config(config, path) -> None:
    """Write a configuration (of any architecture: it offers ``to_dict``) as ``config.json``."""
    import json
    from pathlib import Path

    path = Path(path)
    if path.is_dir():
        path = path / CONFIG_FILE
    path.write_text(json.dumps(config.to_dict(), indent=2, sort_keys=True) + "\n", encoding="utf-8")


__all__ = [
    "load_config", "write_config",
    "CONFIG_FILE", "DTYPES", "EngineConfig", "ModelConfig", "architecture", "known_architectures",
    "known_parts", "part", "register_architecture", "register_part",
]
