"""Typed configuration of the Llama4 text decoder, read from config.json keys.

The reference hard-codes every one of these values as a member default
(include/engine/llama4_cpu_engine.hpp:43-61, include/engine/llama4_cuda_engine.hpp:121-140)
and never parses config.json in C++; only its web server reads a handful of keys
(web/server/config.mjs:540-600).  Here every size and constant is a field that
comes from the model folder's config.json, and nothing below this module
carries a number of its own.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass
from typing import Any, Optional

from .common import ConfigError, read_config_json, token_id_list


@dataclass(frozen=True)
class RopeScaling:
    """llama3 frequency scaling (src/engine/llama4_cpu_engine.cpp:446-464)."""
    rope_type: str
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int


_KEYS_WITH_DEFAULTS = {
    # config.json key: default (None = required)
    "num_hidden_layers": None,
    "hidden_size": None,
    "num_attention_heads": None,
    "num_key_value_heads": None,
    "head_dim": "derived",
    "intermediate_size": None,
    "intermediate_size_mlp": "derived",
    "num_local_experts": None,
    "num_experts_per_tok": 1,
    "interleave_moe_layer_step": 1,
    "vocab_size": None,
    "rms_norm_eps": 1e-5,
    "rope_theta": 500000.0,
    "nope_layer_interval": 4,
    "attention_chunk_size": 8192,
    "use_qk_norm": True,
    "attn_temperature_tuning": True,
    "floor_scale": 8192,
    "attn_scale": 0.1,
    "tie_word_embeddings": False,
    "max_position_embeddings": 131072,
    "initializer_range": 0.02,
}

ROPE_PAIRINGS = ("half_split", "interleaved")
QK_NORM_ORDERS = ("after_rope", "before_rope")
QK_NORM_SCOPES = ("rope_layers", "all_layers")
ROUTER_GATES = ("sigmoid_input", "sigmoid_output", "none")

# Named sets of overrides.  "llama4": the library's defaults.  "reference_compat": what the reference's
# Llama4 engines compute (src/engine/llama4_cpu_engine.cpp:296-329): head norm before the rotation and on
# every layer, every layer rotates and sees all keys, no temperature on the queries, no gate value.
PRESETS = {
    "llama4": {"qk_norm_order": "after_rope", "qk_norm_scope": "rope_layers", "router_gate": "sigmoid_input"},
    "reference_compat": {"qk_norm_order": "before_rope", "qk_norm_scope": "all_layers", "router_gate": "none",
                         "nope_layer_interval": 0, "no_rope_layers": None, "layer_types": None,
                         "attention_chunk_size": 0, "attn_temperature_tuning": False},
}


# What a command line may set of this architecture besides its presets: (flag, config.json key, type or choices,
# help).  --rope-theta is the reference's own flag (src/app/main_cli.cpp:280-281).
CLI_OPTIONS = (
    ("--rope-theta", "rope_theta", float, "replaces config.json's rope_theta"),
    ("--rope-pairing", "rope_pairing", ROPE_PAIRINGS, "which elements of a head a rotation pairs"),
    ("--qk-norm-order", "qk_norm_order", QK_NORM_ORDERS, "head norm before or after the rotation"),
    ("--qk-norm-scope", "qk_norm_scope", QK_NORM_SCOPES, "head norm on the rotating layers or on all"),
    ("--router-gate", "router_gate", ROUTER_GATES, "where the router's sigmoid gate is applied"),
)


@dataclass(frozen=True)
class Llama4TextConfig:
    num_hidden_layers: int
    hidden_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int          # routed and shared expert width
    intermediate_size_mlp: int      # dense (non-MoE) layer width
    num_local_experts: int
    num_experts_per_tok: int
    interleave_moe_layer_step: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    rope_scaling: Optional[RopeScaling]
    nope_layer_interval: int
    attention_chunk_size: int       # 0 = no chunking
    use_qk_norm: bool
    attn_temperature_tuning: bool
    floor_scale: float
    attn_scale: float
    tie_word_embeddings: bool
    max_position_embeddings: int
    initializer_range: float
    bos_token_id: Optional[int] = None
    eos_token_ids: tuple = ()
    # per-layer overrides (lists of length num_hidden_layers) ---------------
    no_rope_layers: Optional[tuple] = None   # entry != 0: the layer uses RoPE
    moe_layers: Optional[tuple] = None       # indices of MoE layers
    # knobs that HF files do not carry; read from config.json when present ---
    rope_pairing: str = "half_split"
    qk_norm_order: str = "after_rope"
    qk_norm_scope: str = "rope_layers"
    router_gate: str = "sigmoid_input"
    architecture: str = "Llama4ForCausalLM"
    torch_dtype: str = "bfloat16"

    # ---- derived, per layer ------------------------------------------------
    def layer_is_moe(self, i: int) -> bool:
        if self.moe_layers is not None:
            return i in self.moe_layers
        return (i + 1) % self.interleave_moe_layer_step == 0

    def layer_uses_rope(self, i: int) -> bool:
        if self.no_rope_layers is not None:
            return bool(self.no_rope_layers[i])
        if self.nope_layer_interval <= 0:
            return True
        return (i + 1) % self.nope_layer_interval != 0

    def layer_has_qk_norm(self, i: int) -> bool:
        if not self.use_qk_norm:
            return False
        return self.qk_norm_scope == "all_layers" or self.layer_uses_rope(i)

    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    # ---- (de)serialisation -------------------------------------------------
    def to_json_dict(self) -> dict:
        d = asdict(self)
        arch = d.pop("architecture")
        eos = d.pop("eos_token_ids")
        rs = d.pop("rope_scaling")
        for k in ("no_rope_layers", "moe_layers"):
            if d[k] is None:
                d.pop(k)
            else:
                d[k] = list(d[k])
        if d["bos_token_id"] is None:
            d.pop("bos_token_id")
        if eos:
            d["eos_token_id"] = list(eos) if len(eos) > 1 else eos[0]
        d["rope_scaling"] = None if rs is None else dict(rs)
        d["model_type"] = "llama4_text"
        text = d
        if arch == "Llama4ForConditionalGeneration":
            return {"architectures": [arch], "model_type": "llama4", "text_config": text,
                    "tie_word_embeddings": text["tie_word_embeddings"]}
        return {"architectures": [arch], **text}

    @staticmethod
    def from_json_dict(raw: dict) -> "Llama4TextConfig":
        archs = raw.get("architectures") or []
        arch = archs[0] if archs else "Llama4ForCausalLM"
        d = raw
        if isinstance(raw.get("text_config"), dict):
            d = dict(raw["text_config"])
            for k in ("tie_word_embeddings", "bos_token_id", "eos_token_id", "torch_dtype"):
                if k not in d and k in raw:
                    d[k] = raw[k]
        vals: dict[str, Any] = {}
        for key, default in _KEYS_WITH_DEFAULTS.items():
            if key in d and d[key] is not None:
                vals[key] = d[key]
            elif default is None:
                raise ConfigError(f"config.json: required key '{key}' is missing")
            elif default != "derived":
                vals[key] = default
        if "head_dim" not in vals:
            _check_int("hidden_size", vals["hidden_size"])
            _check_int("num_attention_heads", vals["num_attention_heads"])
            if vals["hidden_size"] % vals["num_attention_heads"]:
                raise ConfigError("config.json: 'head_dim' is absent and 'hidden_size' is not a "
                                  "multiple of 'num_attention_heads'")
            vals["head_dim"] = vals["hidden_size"] // vals["num_attention_heads"]
        if "intermediate_size_mlp" not in vals:
            vals["intermediate_size_mlp"] = vals["intermediate_size"]
        if d.get("attention_chunk_size", 1) is None:
            vals["attention_chunk_size"] = 0
        rs = d.get("rope_scaling")
        scaling = None
        if rs is not None:
            if not isinstance(rs, dict):
                raise ConfigError("config.json: 'rope_scaling' must be an object or null")
            rope_type = rs.get("rope_type", rs.get("type"))
            if rope_type != "llama3":
                raise ConfigError(f"config.json: rope_scaling.rope_type '{rope_type}' is not supported "
                                  "(supported: 'llama3', or null for unscaled)")
            try:
                scaling = RopeScaling(
                    rope_type="llama3",
                    factor=float(rs["factor"]),
                    low_freq_factor=float(rs["low_freq_factor"]),
                    high_freq_factor=float(rs["high_freq_factor"]),
                    original_max_position_embeddings=int(rs["original_max_position_embeddings"]))
            except KeyError as e:
                raise ConfigError(f"config.json: rope_scaling is missing key {e}") from None
        eos_ids = token_id_list(d.get("eos_token_id"), "config.json: 'eos_token_id'")
        bos = d.get("bos_token_id")
        extras = {}
        for key, allowed in (("rope_pairing", ROPE_PAIRINGS), ("qk_norm_order", QK_NORM_ORDERS),
                             ("qk_norm_scope", QK_NORM_SCOPES), ("router_gate", ROUTER_GATES)):
            if key in d:
                if d[key] not in allowed:
                    raise ConfigError(f"config.json: '{key}' is '{d[key]}', expected one of {allowed}")
                extras[key] = d[key]
        nrl = d.get("no_rope_layers")
        if nrl is not None and len(nrl) == 0:
            nrl = None
        lt = d.get("layer_types")
        if nrl is None and lt:
            # per-layer attention kinds: "chunked_attention" layers rotate and see their chunk,
            # "full_attention" layers have no position encoding and see every key
            known = {"chunked_attention": 1, "full_attention": 0}
            for i, kind in enumerate(lt):
                if kind not in known:
                    raise ConfigError(f"config.json: 'layer_types'[{i}] is '{kind}', expected one of {sorted(known)}")
            nrl = [known[kind] for kind in lt]
        ml = d.get("moe_layers")
        cfg = Llama4TextConfig(
            rope_scaling=scaling,
            bos_token_id=None if bos is None else int(bos),
            eos_token_ids=eos_ids,
            no_rope_layers=None if nrl is None else tuple(int(x) for x in nrl),
            moe_layers=None if ml is None else tuple(int(x) for x in ml),
            architecture=arch,
            torch_dtype=str(d.get("torch_dtype", "bfloat16")),
            **vals, **extras)
        cfg.validate()
        return cfg

    @staticmethod
    def from_model_dir(path: str) -> "Llama4TextConfig":
        return Llama4TextConfig.from_json_dict(read_config_json(path))

    def validate(self) -> None:
        for key in ("num_hidden_layers", "hidden_size", "num_attention_heads", "num_key_value_heads",
                    "head_dim", "intermediate_size", "intermediate_size_mlp", "num_local_experts",
                    "num_experts_per_tok", "interleave_moe_layer_step", "vocab_size",
                    "max_position_embeddings"):
            _check_int(key, getattr(self, key))
            if getattr(self, key) < 1:
                raise ConfigError(f"config.json: '{key}' must be >= 1, got {getattr(self, key)}")
        for key in ("nope_layer_interval", "attention_chunk_size"):
            _check_int(key, getattr(self, key))
            if getattr(self, key) < 0:
                raise ConfigError(f"config.json: '{key}' must be >= 0, got {getattr(self, key)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError("config.json: 'num_attention_heads' (%d) is not a multiple of "
                              "'num_key_value_heads' (%d)" % (self.num_attention_heads,
                                                              self.num_key_value_heads))
        if self.head_dim % 2:
            raise ConfigError(f"config.json: 'head_dim' must be even, got {self.head_dim}")
        if self.num_experts_per_tok > self.num_local_experts:
            raise ConfigError("config.json: 'num_experts_per_tok' (%d) exceeds 'num_local_experts' (%d)"
                              % (self.num_experts_per_tok, self.num_local_experts))
        if not (self.rms_norm_eps > 0):
            raise ConfigError(f"config.json: 'rms_norm_eps' must be > 0, got {self.rms_norm_eps}")
        if not (self.rope_theta > 0):
            raise ConfigError(f"config.json: 'rope_theta' must be > 0, got {self.rope_theta}")
        if self.attn_temperature_tuning and not (self.floor_scale > 0):
            raise ConfigError(f"config.json: 'floor_scale' must be > 0, got {self.floor_scale}")
        if self.no_rope_layers is not None and len(self.no_rope_layers) != self.num_hidden_layers:
            raise ConfigError("config.json: 'no_rope_layers' has %d entries for %d layers"
                              % (len(self.no_rope_layers), self.num_hidden_layers))
        if self.moe_layers is not None:
            for i in self.moe_layers:
                if not 0 <= i < self.num_hidden_layers:
                    raise ConfigError(f"config.json: 'moe_layers' names layer {i} of "
                                      f"{self.num_hidden_layers}")
        if self.rope_scaling is not None:
            rs = self.rope_scaling
            if not rs.factor > 0 or rs.high_freq_factor == rs.low_freq_factor:
                raise ConfigError("config.json: rope_scaling needs factor > 0 and "
                                  "high_freq_factor != low_freq_factor")


def _check_int(key: str, v: Any) -> None:
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"config.json: '{key}' must be an integer, got {v!r}")
