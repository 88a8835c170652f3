"""Llama4 text decoder as a `ModelSpec`: which parts each layer has, by configuration.

Tensor names follow what the reference loads
(src/engine/llama4_cpu_engine.cpp:419-443): prefix `language_model.model.` /
`language_model.lm_head.weight` for "Llama4ForConditionalGeneration"; for
"Llama4ForCausalLM" the same names without `language_model.`.

Layer kinds (the reference has one kind only; its forward is
src/engine/llama4_cpu_engine.cpp:293-333):
  * RoPE layer: rotary position encoding, optional weightless QK norm, attention
    restricted to the query's chunk of `attention_chunk_size` positions;
  * NoPE layer: no position encoding, causal attention over all keys, optional
    temperature scaling of the query;
  * feed-forward: routed experts plus a shared expert, or a dense SwiGLU MLP.
"""
from __future__ import annotations

from ..config.llama4 import CLI_OPTIONS, PRESETS, Llama4TextConfig
from ..config.registry import Architecture, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, RunEntry


def _position_spec(cfg: Llama4TextConfig, uses_rope: bool) -> PartSpec:
    if not uses_rope:
        return PartSpec("none", {})
    rs = cfg.rope_scaling
    return PartSpec("rope", {
        "head_dim": cfg.head_dim,
        "theta": float(cfg.rope_theta),
        "pairing": cfg.rope_pairing,
        "scaling": None if rs is None else {
            "rope_type": rs.rope_type, "factor": rs.factor,
            "low_freq_factor": rs.low_freq_factor, "high_freq_factor": rs.high_freq_factor,
            "original_max_position_embeddings": rs.original_max_position_embeddings},
    })


def build_spec(cfg: Llama4TextConfig) -> ModelSpec:
    if cfg.architecture == "Llama4ForConditionalGeneration":
        base, head_name = "language_model.model.", "language_model.lm_head.weight"
        ignored = ("vision_model.", "multi_modal_projector.")
    else:
        base, head_name = "model.", "lm_head.weight"
        ignored = ()
    layers = []
    for i in range(cfg.num_hidden_layers):
        uses_rope = cfg.layer_uses_rope(i)
        if uses_rope and cfg.attention_chunk_size > 0:
            window = {"kind": "chunk", "size": cfg.attention_chunk_size}
        else:
            window = {"kind": "full", "size": 0}
        temperature = None
        if (not uses_rope) and cfg.attn_temperature_tuning:
            temperature = {"floor_scale": float(cfg.floor_scale), "attn_scale": float(cfg.attn_scale)}
        mixer = PartSpec("attention", {
            "hidden_size": cfg.hidden_size,
            "num_heads": cfg.num_attention_heads,
            "num_kv_heads": cfg.num_key_value_heads,
            "head_dim": cfg.head_dim,
            "softmax_scale": float(cfg.head_dim) ** -0.5,
            "position": _position_spec(cfg, uses_rope),
            "qk_norm": cfg.layer_has_qk_norm(i),
            "qk_norm_eps": float(cfg.rms_norm_eps),
            "qk_norm_order": cfg.qk_norm_order,
            "window": window,
            "query_temperature": temperature,
        })
        if cfg.layer_is_moe(i):
            ffn = PartSpec("moe_swiglu", {
                "hidden_size": cfg.hidden_size,
                "num_experts": cfg.num_local_experts,
                "top_k": cfg.num_experts_per_tok,
                "expert_size": cfg.intermediate_size,
                "shared_size": cfg.intermediate_size,
                "router_gate": cfg.router_gate,
            })
        else:
            ffn = PartSpec("dense_swiglu", {
                "hidden_size": cfg.hidden_size,
                "intermediate_size": cfg.intermediate_size_mlp,
            })
        norm = {"size": cfg.hidden_size, "eps": float(cfg.rms_norm_eps)}
        layers.append(LayerSpec(
            prefix=f"{base}layers.{i}.",
            block=PartSpec("pre_norm", {}),
            mixer=mixer,
            feed_forward=ffn,
            mixer_norm=PartSpec("rmsnorm", {**norm, "weight": "input_layernorm.weight"}),
            feed_forward_norm=PartSpec("rmsnorm", {**norm, "weight": "post_attention_layernorm.weight"}),
        ))
    embed_name = base + "embed_tokens.weight"
    return ModelSpec(
        architecture=cfg.architecture,
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        embedding=PartSpec("token_embedding", {"weight": embed_name, "vocab_size": cfg.vocab_size,
                                               "hidden_size": cfg.hidden_size}),
        layers=tuple(layers),
        run_order=tuple(RunEntry(i) for i in range(cfg.num_hidden_layers)),
        final_norm=PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": float(cfg.rms_norm_eps),
                                        "weight": base + "norm.weight"}),
        head=PartSpec("linear_head", {"weight": embed_name if cfg.tie_word_embeddings else head_name,
                                      "vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size}),
        ignored_tensor_prefixes=ignored,
        bos_token_id=cfg.bos_token_id,
        stop_token_ids=tuple(cfg.eos_token_ids),
        max_position=cfg.max_position_embeddings,
        initializer_range=float(cfg.initializer_range),
    )


for _name in ("Llama4ForConditionalGeneration", "Llama4ForCausalLM"):
    register_architecture(Architecture(_name, Llama4TextConfig.from_json_dict, build_spec, PRESETS, CLI_OPTIONS))
