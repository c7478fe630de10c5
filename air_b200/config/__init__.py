from .model_config import ConfigError, Qwen2Config
from .bivizen_config import BivizenConfig
from .tomodra_config import TomodraConfig
from .pefivik_config import PefivikConfig
from .tabopel_config import TabopelConfig
from . import architectures  # registers the known architectures
import json
import os


def load_config(path_or_dict):
    """The typed configuration of a model folder (or of a config.json's contents): the class
    is chosen by the first entry of ``architectures`` through the registry."""
    from ..parts.registry import architecture
    folder = None
    if isinstance(path_or_dict, dict):
        d = path_or_dict
    else:
        path = path_or_dict
        if os.path.isdir(path):
            folder = path
            path = os.path.join(path, "config.json")
        try:
            with open(path) as f:
                d = json.load(f)
        except FileNotFoundError:
            raise ConfigError("data_error", f"no config.json at {path}") from None
        except json.JSONDecodeError as e:
            raise ConfigError("data_error", f"config.json is not valid JSON: {e}") from None
        if not isinstance(d, dict):
            raise ConfigError("data_error", "config.json must hold an object")
    # the design's name: the first entry of "architectures", or the string under "architecture"
    archs = d.get("architectures") or ([d["architecture"]] if isinstance(d.get("architecture"), str) else [])
    if not archs:
        raise ConfigError("data_error", "config.json lacks 'architectures'")
    config_class = architecture(archs[0]).config_class
    if getattr(config_class, "reads_shapes", False):
        # a design some of whose sizes are only the shapes of its tensors
        return config_class.from_dict(d, shapes=_tensor_shapes(folder) if folder else None)
    return config_class.from_dict(d)


def _tensor_shapes(folder):
    """name -> shape of the tensors of a model folder (headers only), or None if it has no model file."""
    from ..weights.loader import _open_files
    from ..weights.safetensors_io import SafetensorsError
    try:
        files = _open_files(folder)
    except SafetensorsError:
        return None
    return {name: tuple(f.info(name)[1]) for name, f in files.items()}
