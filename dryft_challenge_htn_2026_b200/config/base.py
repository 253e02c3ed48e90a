"""Base of the architecture config classes: reading config.json and typed access to its keys."""
import json
import os


class ConfigError(ValueError):
    """A config.json that is missing a key, has a key of the wrong type, or asks for an option
    this library does not implement."""


_MISSING = object()


class ModelConfig:
    """Subclasses declare ``architecture`` (the name in config.json's ``architectures``), parse
    their keys in ``from_dict`` and build a ``ModelSpec`` in ``to_spec``. They can be written back
    with ``to_dict`` (the random-weights mode does)."""

    architecture = None

    @classmethod
    def from_dict(cls, d):
        raise NotImplementedError

    def to_dict(self):
        raise NotImplementedError

    def to_spec(self):
        raise NotImplementedError

    @classmethod
    def from_json(cls, path):
        return cls.from_dict(read_config_json(path))

    def save(self, folder):
        os.makedirs(folder, exist_ok=True)
        with open(os.path.join(folder, "config.json"), "w") as f:
            json.dump(self.to_dict(), f, indent=2)


def read_config_json(path):
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    try:
        with open(path) as f:
            d = json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"no config.json at {path}") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path} is not valid JSON: {e}") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: expected a JSON object")
    return d


def get(d, key, typ, default=_MISSING, positive=False):
    """d[key] checked against ``typ`` (int keys refuse bools and floats with a fraction)."""
    if key not in d or d[key] is None:
        if default is _MISSING:
            raise ConfigError(f"config.json: required key '{key}' is missing")
        return default
    v = d[key]
    if typ is int:
        if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v:
            raise ConfigError(f"config.json: '{key}' must be an integer, got {v!r}")
        v = int(v)
    elif typ is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"config.json: '{key}' must be a number, got {v!r}")
        v = float(v)
    elif typ is bool:
        if not isinstance(v, bool):
            raise ConfigError(f"config.json: '{key}' must be true or false, got {v!r}")
    elif not isinstance(v, typ):
        raise ConfigError(f"config.json: '{key}' must be {typ.__name__}, got {v!r}")
    if positive and not v > 0:
        raise ConfigError(f"config.json: '{key}' must be positive, got {v!r}")
    return v
