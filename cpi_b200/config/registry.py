"""One registry from an architecture's name (config.json `architectures[0]`) to its model.

The reference picks its safetensors engine by "the path is a folder with *.safetensors"
(src/main.cpp:169-174, src/app/main_helpers.cpp:464-486) and knows no names.
Here an architecture registers, under each name it answers to, a function that
reads config.json into its typed configuration and one that turns that
configuration into a `ModelSpec`.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable

import dataclasses

from .common import ConfigError, generation_stop_ids, read_config_json
from .spec import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable[[dict], Any]        # raw config.json dict -> typed configuration
    build_spec: Callable[[Any], ModelSpec]     # typed configuration -> ModelSpec
    # named sets of config.json keys that a command line or a caller may write over the file's
    presets: dict = dataclasses.field(default_factory=dict)
    # single config.json keys a command line may set: (flag, key, type or tuple of choices, help)
    cli_options: tuple = ()


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(arch: Architecture) -> None:
    _ARCHITECTURES[arch.name] = arch


def registered_architectures() -> list[str]:
    _ensure_builtin()
    return sorted(_ARCHITECTURES)


def get_architecture(name: str) -> Architecture:
    _ensure_builtin()
    if name not in _ARCHITECTURES:
        raise ConfigError(f"architecture '{name}' is not registered; registered: "
                          + ", ".join(sorted(_ARCHITECTURES)))
    return _ARCHITECTURES[name]


def architecture_of(raw_config: dict) -> Architecture:
    archs = raw_config.get("architectures")
    if not archs or not isinstance(archs, list):
        raise ConfigError("config.json: 'architectures' is missing or empty; registered: "
                          + ", ".join(registered_architectures()))
    return get_architecture(archs[0])


def apply_overrides(raw_config: dict, overrides: dict | None) -> dict:
    """A copy of a config.json dictionary with `overrides` written over its keys, in the nested
    `text_config` object when the file has one (that is where such a file keeps the decoder's keys).
    The way options of a command line (the reference's --rope-theta, src/app/main_cli.cpp:280-281)
    and named presets reach the typed configuration: as config.json keys, checked like the file's own."""
    if not overrides:
        return raw_config
    out = dict(raw_config)
    if isinstance(out.get("text_config"), dict):
        out["text_config"] = {**out["text_config"], **overrides}
    else:
        out.update(overrides)
    return out


def spec_from_model_dir(model_dir: str, overrides: dict | None = None):
    """(typed configuration, ModelSpec) of the model folder's config.json."""
    raw = apply_overrides(read_config_json(model_dir), overrides)
    arch = architecture_of(raw)
    cfg = arch.parse_config(raw)
    spec = arch.build_spec(cfg)
    spec.validate()
    more = tuple(t for t in generation_stop_ids(model_dir) if t not in spec.stop_token_ids)
    if more:
        spec = dataclasses.replace(spec, stop_token_ids=tuple(spec.stop_token_ids) + more)
    return cfg, spec


def cli_presets() -> dict:
    """{preset name: {config.json key: value}} over all registered architectures."""
    _ensure_builtin()
    out: dict = {}
    for arch in _ARCHITECTURES.values():
        for name, keys in arch.presets.items():
            if out.setdefault(name, keys) != keys:
                raise ConfigError(f"two architectures register different presets named '{name}'")
    return out


def cli_options() -> list:
    """The (flag, key, type or choices, help) options of all registered architectures, each flag once."""
    _ensure_builtin()
    seen, out = set(), []
    for arch in _ARCHITECTURES.values():
        for opt in arch.cli_options:
            if opt[0] not in seen:
                seen.add(opt[0])
                out.append(opt)
    return out


PLUGINS_ENV = "CPI_B200_PLUGINS"
_plugins_loaded = False


def _ensure_builtin() -> None:
    """The built-in architectures register themselves when the package of architectures is imported.  After
    them come the modules that the environment variable CPI_B200_PLUGINS names (comma separated, importable
    names): a module outside this package registers parts and architectures the same way, and every program
    of the package (the command lines, the replay tool) then knows them by their config.json name."""
    global _plugins_loaded
    from .. import models  # noqa: F401
    if _plugins_loaded:
        return
    _plugins_loaded = True
    import importlib
    import os
    for name in filter(None, (x.strip() for x in os.environ.get(PLUGINS_ENV, "").split(","))):
        try:
            importlib.import_module(name)
        except ImportError as e:
            raise ConfigError(f"{PLUGINS_ENV}: cannot import '{name}': {e}") from None
