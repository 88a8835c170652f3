"""Typed configuration, registry and spec."""
import json
import os
import tempfile

import pytest

import tiny
from cpi_b200.config.llama4 import Llama4TextConfig
from cpi_b200.config import (ConfigError, get_architecture, registered_architectures,
                             spec_from_model_dir, architecture_of, RunEntry)
from cpi_b200.models.llama4 import build_spec


def test_reads_flat_and_nested_configs():
    a = Llama4TextConfig.from_json_dict(tiny.config("A"))
    assert (a.num_hidden_layers, a.hidden_size, a.head_dim, a.q_size, a.kv_size) == (4, 64, 16, 64, 32)
    assert a.rope_scaling.factor == 16.0 and a.eos_token_ids == (3, 5)
    b = Llama4TextConfig.from_json_dict(tiny.config("B"))
    assert b.architecture == "Llama4ForConditionalGeneration" and b.tie_word_embeddings
    assert b.q_size == 192 and b.hidden_size == 96 and b.rope_scaling is None
    assert b.rope_pairing == "interleaved" and b.router_gate == "sigmoid_output" and b.eos_token_ids == (7,)


def test_layer_kinds():
    a = Llama4TextConfig.from_json_dict(tiny.config("A"))
    assert [a.layer_is_moe(i) for i in range(4)] == [True] * 4
    assert [a.layer_uses_rope(i) for i in range(4)] == [True, True, True, False]
    b = Llama4TextConfig.from_json_dict(tiny.config("B"))
    assert [b.layer_is_moe(i) for i in range(6)] == [False, True, False, True, False, True]
    assert [b.layer_uses_rope(i) for i in range(6)] == [True, True, False, True, True, False]
    c = tiny.config("A")
    c["no_rope_layers"] = [0, 1, 1, 1]
    c["moe_layers"] = [2]
    x = Llama4TextConfig.from_json_dict(c)
    assert [x.layer_uses_rope(i) for i in range(4)] == [False, True, True, True]
    assert [x.layer_is_moe(i) for i in range(4)] == [False, False, True, False]


def test_layer_types_list():
    c = tiny.config("A")
    c["layer_types"] = ["full_attention", "chunked_attention", "chunked_attention", "full_attention"]
    x = Llama4TextConfig.from_json_dict(c)
    assert [x.layer_uses_rope(i) for i in range(4)] == [False, True, True, False]
    c["layer_types"][1] = "sliding"
    with pytest.raises(ConfigError, match="layer_types"):
        Llama4TextConfig.from_json_dict(c)


def test_defaults_and_derived():
    c = tiny.config("A")
    for k in ("head_dim", "intermediate_size_mlp", "rms_norm_eps", "rope_theta", "num_experts_per_tok"):
        c.pop(k)
    x = Llama4TextConfig.from_json_dict(c)
    assert x.head_dim == 16 and x.intermediate_size_mlp == 128 and x.rms_norm_eps == 1e-5
    assert x.rope_theta == 500000.0 and x.num_experts_per_tok == 1
    c["attention_chunk_size"] = None
    assert Llama4TextConfig.from_json_dict(c).attention_chunk_size == 0


@pytest.mark.parametrize("key,value,word", [
    ("num_key_value_heads", 3, "num_key_value_heads"),
    ("head_dim", 15, "head_dim"),
    ("num_experts_per_tok", 9, "num_experts_per_tok"),
    ("hidden_size", 0, "hidden_size"),
    ("hidden_size", "64", "hidden_size"),
    ("rms_norm_eps", 0.0, "rms_norm_eps"),
    ("rope_pairing", "spiral", "rope_pairing"),
    ("no_rope_layers", [1, 0], "no_rope_layers"),
])
def test_errors_name_the_key(key, value, word):
    c = tiny.config("A")
    c[key] = value
    with pytest.raises(ConfigError) as e:
        Llama4TextConfig.from_json_dict(c)
    assert word in str(e.value)


def test_missing_key_and_bad_scaling():
    c = tiny.config("A")
    c.pop("vocab_size")
    with pytest.raises(ConfigError, match="vocab_size"):
        Llama4TextConfig.from_json_dict(c)
    c = tiny.config("A")
    c["rope_scaling"]["rope_type"] = "yarn"
    with pytest.raises(ConfigError, match="yarn"):
        Llama4TextConfig.from_json_dict(c)


def test_round_trip_through_json():
    for name in "AB":
        x = Llama4TextConfig.from_json_dict(tiny.config(name))
        y = Llama4TextConfig.from_json_dict(json.loads(json.dumps(x.to_json_dict())))
        assert x == y


def test_registry():
    assert "Llama4ForCausalLM" in registered_architectures()
    with pytest.raises(ConfigError, match="Llama4ForCausalLM"):
        get_architecture("GPT2LMHeadModel")
    with pytest.raises(ConfigError, match="architectures"):
        architecture_of({"hidden_size": 4})
    d = tempfile.mkdtemp()
    with pytest.raises(ConfigError, match="config.json"):
        spec_from_model_dir(d)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(tiny.config("B"), f)
    cfg, spec = spec_from_model_dir(d)
    assert spec.architecture == "Llama4ForConditionalGeneration" and len(spec.layers) == 6


def test_spec_of_config_a_and_b():
    sa = build_spec(Llama4TextConfig.from_json_dict(tiny.config("A")))
    assert [l.feed_forward.kind for l in sa.layers] == ["moe_swiglu"] * 4
    assert [l.mixer["position"].kind for l in sa.layers] == ["rope", "rope", "rope", "none"]
    assert [l.mixer["window"]["kind"] for l in sa.layers] == ["chunk", "chunk", "chunk", "full"]
    assert sa.layers[3].mixer["query_temperature"] == {"floor_scale": 32.0, "attn_scale": 0.1}
    assert sa.layers[0].mixer["query_temperature"] is None
    assert sa.layers[0].mixer["qk_norm"] and not sa.layers[3].mixer["qk_norm"]
    assert sa.head["weight"] == "lm_head.weight" and sa.stop_token_ids == (3, 5)
    sb = build_spec(Llama4TextConfig.from_json_dict(tiny.config("B")))
    assert [l.feed_forward.kind for l in sb.layers] == ["dense_swiglu", "moe_swiglu"] * 3
    assert sb.head["weight"] == sb.embedding["weight"] == "language_model.model.embed_tokens.weight"
    assert sb.layers[1].feed_forward["top_k"] == 2 and sb.layers[0].feed_forward["intermediate_size"] == 192
    assert sb.layers[0].mixer_norm["eps"] == 1e-6
    assert sb.ignored_tensor_prefixes == ("vision_model.", "multi_modal_projector.")


def test_run_order_validation():
    import dataclasses
    s = build_spec(Llama4TextConfig.from_json_dict(tiny.config("A")))
    ok = dataclasses.replace(s, run_order=(RunEntry(0), RunEntry(1), RunEntry(1), RunEntry(2, cache_of=0)))
    ok.validate()
    for bad in [(RunEntry(7),), (RunEntry(0, cache_of=0),), (RunEntry(0), RunEntry(1, cache_of=0), RunEntry(2, cache_of=1))]:
        with pytest.raises(ValueError):
            dataclasses.replace(s, run_order=bad).validate()


def test_overrides_and_presets():
    """Overrides are config.json keys written over the file's (inside text_config when the file nests them),
    and go through the same checks."""
    from cpi_b200.config.llama4 import PRESETS
    from cpi_b200.config.registry import apply_overrides, architecture_of
    for name in ("A", "B"):
        raw = tiny.config(name)
        arch = architecture_of(raw)
        assert apply_overrides(raw, None) is raw and apply_overrides(raw, {}) is raw
        new = apply_overrides(raw, {"rope_theta": 12345.0, **PRESETS["reference_compat"]})
        assert new is not raw and arch.parse_config(raw).rope_theta != 12345.0       # the input is not touched
        cfg = arch.parse_config(new)
        assert cfg.rope_theta == 12345.0 and cfg.router_gate == "none" and cfg.qk_norm_order == "before_rope"
        assert cfg.attention_chunk_size == 0 and not cfg.attn_temperature_tuning
        assert all(cfg.layer_uses_rope(i) and cfg.layer_has_qk_norm(i) == cfg.use_qk_norm
                   for i in range(cfg.num_hidden_layers))
        spec = arch.build_spec(cfg)
        assert all(l.mixer.params["window"]["kind"] == "full" for l in spec.layers)
        back = arch.parse_config(apply_overrides(new, PRESETS["llama4"]))
        assert (back.qk_norm_order, back.qk_norm_scope, back.router_gate) == ("after_rope", "rope_layers", "sigmoid_input")
        with pytest.raises(ConfigError, match="router_gate"):
            arch.parse_config(apply_overrides(raw, {"router_gate": "softmax"}))


def test_stop_ids_of_generation_config_json_join_the_models(tmp_path):
    """`eos_token_id` of generation_config.json (one id or a list) is added to config.json's; a folder without the
    file keeps config.json's alone; a value that is no id is an error that names the file."""
    import json as js
    from cpi_b200.config.common import generation_stop_ids
    d = tmp_path / "m"
    d.mkdir()
    (d / "config.json").write_text(js.dumps(tiny.config("A")))           # eos_token_id [3, 5]
    assert spec_from_model_dir(str(d))[1].stop_token_ids == (3, 5)
    (d / "generation_config.json").write_text(js.dumps({"eos_token_id": [5, 9, 11], "temperature": 0.6}))
    assert spec_from_model_dir(str(d))[1].stop_token_ids == (3, 5, 9, 11)
    (d / "generation_config.json").write_text(js.dumps({"eos_token_id": 7}))
    assert generation_stop_ids(str(d)) == (7,)
    (d / "generation_config.json").write_text(js.dumps({"eos_token_id": "</s>"}))
    with pytest.raises(ConfigError, match="generation_config.json"):
        spec_from_model_dir(str(d))
    (d / "generation_config.json").write_text(js.dumps({"temperature": 0.6}))
    assert spec_from_model_dir(str(d))[1].stop_token_ids == (3, 5)
