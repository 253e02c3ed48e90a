"""The one registry from an architecture's name (config.json ``architectures``) to its config
class. The config class turns config.json into a ``ModelSpec``; the parts registry does the rest.

Adding an architecture: write a ``ModelConfig`` subclass with ``architecture``, ``from_dict``,
``to_dict`` and ``to_spec``, then ``register_architecture(YourConfig)``."""
from .config.base import ConfigError, read_config_json
from .config.qwen3 import Qwen3Config

_ARCHITECTURES = {}


def register_architecture(config_cls):
    if not config_cls.architecture:
        raise ValueError(f"{config_cls.__name__} does not name its architecture")
    _ARCHITECTURES[config_cls.architecture] = config_cls
    return config_cls


def architectures():
    return sorted(_ARCHITECTURES)


def config_class(name):
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(f"architecture {name!r} is not registered; known: {architectures()}") from None


def config_from_dict(d):
    archs = d.get("architectures")
    if not isinstance(archs, list) or len(archs) != 1 or not isinstance(archs[0], str):
        raise ConfigError(f"config.json: 'architectures' must be a list with one name, got {archs!r}")
    return config_class(archs[0]).from_dict(d)


def config_from_folder(folder):
    return config_from_dict(read_config_json(folder))


register_architecture(Qwen3Config)
