"""What every architecture's configuration shares: the error type and the readers of a model folder's JSON files.

The reference never parses config.json in C++ (its engines carry their sizes as member defaults,
include/engine/llama4_cpu_engine.hpp:43-61); only its web server reads a handful of keys
(web/server/config.mjs:540-600).
"""
from __future__ import annotations

import json
import os


class ConfigError(ValueError):
    """A config.json value is missing, of the wrong type, or inconsistent."""


def _read_json_object(path: str) -> dict:
    with open(path, "r", encoding="utf-8") as f:
        try:
            raw = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return raw


def read_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in model folder '{model_dir}'")
    return _read_json_object(path)


def token_id_list(value, where: str) -> tuple:
    """An `eos_token_id`-style value (absent, one id, or a list of ids) as a tuple of ints."""
    if value is None:
        return ()
    items = value if isinstance(value, (list, tuple)) else [value]
    out = []
    for x in items:
        if isinstance(x, bool) or not isinstance(x, int):
            raise ConfigError(f"{where}: token ids must be integers, got {x!r}")
        out.append(int(x))
    return tuple(out)


def generation_stop_ids(model_dir: str) -> tuple:
    """The end tokens that a model folder's generation_config.json names (`eos_token_id`: one id or a list),
    or () when the folder has no such file.  The reference's engines stop on one compiled-in id
    (include/engine/llama4_cuda_engine.hpp:60) and its Python tool cuts at three ids of its own afterwards
    (tools/run_llama4_prompt.py:10, :76-81); here the ids come from the folder."""
    path = os.path.join(model_dir, "generation_config.json")
    if not os.path.isfile(path):
        return ()
    return token_id_list(_read_json_object(path).get("eos_token_id"), "generation_config.json: 'eos_token_id'")
