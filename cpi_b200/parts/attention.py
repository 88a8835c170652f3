"""Attention mixer: grouped-query attention over the paged cache, with a window and a position part.

Reference forward of one token (src/engine/llama4_cpu_engine.cpp:304-325): q, k, v projections
without bias, per-head weightless RMS norm of q and k, RoPE, cache write, causal softmax attention
with scale 1/sqrt(D), output projection added to the residual.  This part generalises it by
parameters: any head counts and head size, the position part (rotary or none), the norm on or off and
before or after the rotation, a window (all keys, the query's chunk, or the last n keys), and an
optional temperature on the query; and by batch: any mix of sequences and positions in one call.

params: hidden_size, num_heads, num_kv_heads, head_dim, softmax_scale, position (PartSpec), qk_norm,
qk_norm_eps, qk_norm_order ("before_rope" | "after_rope"), window {"kind", "size"},
query_temperature (None or {"floor_scale", "attn_scale"}).
Tensors under the prefix: self_attn.{q,k,v,o}_proj.weight  ([out, in]).
"""
from __future__ import annotations

import torch

from ..cache.manager import KVRequirement
from ..csrc import lib as K
from ..phases import phase
from ..weights.store import TensorReq
from .base import Mixer, RotaryEncoding, ScoreBias, build_part, register_mixer
from .linear import MODE_ADD, project


# set to False to run every attention through the general kernel (tests compare the two families)
use_tensor_core_kernels = True


@register_mixer("attention")
class AttentionMixer(Mixer):
    graph_safe = True
    def __init__(self, spec, prefix="", workspace=None, owns_cache=True):
        super().__init__(spec, prefix)
        p = spec.params
        self.has_kv = bool(owns_cache)      # False: every run entry of this layer reads another's cache
        self.hidden = int(p["hidden_size"])
        self.nh, self.nkv, self.d = int(p["num_heads"]), int(p["num_kv_heads"]), int(p["head_dim"])
        if self.nh % self.nkv:
            raise ValueError(f"attention: {self.nh} heads cannot be grouped over {self.nkv} key/value heads")
        if self.d % 16 or not 16 <= self.d <= 256:
            raise ValueError(f"attention: head size {self.d} is not supported (multiples of 16 from 16 to 256)")
        self.scale = float(p["softmax_scale"])
        self.position = build_part("position", p["position"])
        self.qk_norm = bool(p.get("qk_norm", False))
        self.qk_norm_eps = float(p.get("qk_norm_eps", 0.0))
        self.norm_before_rope = p.get("qk_norm_order", "after_rope") == "before_rope"
        w = p.get("window") or {"kind": "full", "size": 0}
        if w["kind"] not in K.WINDOW_KINDS:
            raise ValueError(f"attention: unknown window kind '{w['kind']}'")
        self.window_kind, self.window_size = w["kind"], int(w.get("size", 0))
        t = p.get("query_temperature")
        self.temperature = None if t is None else (float(t["floor_scale"]), float(t["attn_scale"]))
        self.ws = workspace
        self.w_qkv = self.w_o = None
        self.rotary = self.score_bias = None

    # ---- weights ---------------------------------------------------------------------------------
    def _names(self):
        a = self.prefix + "self_attn."
        return a + "q_proj.weight", a + "k_proj.weight", a + "v_proj.weight", a + "o_proj.weight"

    def requirements(self):
        q, k, v, o = self._names()
        reqs = [TensorReq(q, (self.nh * self.d, self.hidden)), TensorReq(o, (self.hidden, self.nh * self.d))]
        if self.has_kv:
            reqs += [TensorReq(k, (self.nkv * self.d, self.hidden)), TensorReq(v, (self.nkv * self.d, self.hidden))]
        return reqs

    def load(self, source, device):
        q, k, v, o = self._names()
        parts = [source.get(q, device)]
        if self.has_kv:
            parts += [source.get(k, device), source.get(v, device)]
        dt = torch.float32 if any(t.dtype == torch.float32 for t in parts) else torch.bfloat16
        self.w_qkv = torch.cat([t.to(dt) for t in parts], dim=0).contiguous()    # [Q + 2 KV, H]
        del parts
        self.w_o = source.get(o, device).contiguous()
        self.position.prepare(device)
        # what the position part is to this mixer: a rotation of q and k (done with the head norm and the cache
        # write, in one kernel), a bias on the scores (taken by the general attention kernel only), or nothing
        enc = self.position.encoding()
        self.rotary = enc if isinstance(enc, RotaryEncoding) else None
        self.score_bias = enc.table if isinstance(enc, ScoreBias) else None
        if enc is not None and self.rotary is None and self.score_bias is None:
            raise TypeError(f"attention: the position part '{self.position.spec.kind}' describes itself as "
                            f"{type(enc).__name__}; this mixer's kernels take RotaryEncoding, ScoreBias or None")
        if self.score_bias is not None and (self.score_bias.dim() != 2 or self.score_bias.shape[0] != self.nh
                                            or self.score_bias.dtype != torch.float32):
            raise ValueError(f"attention: a score bias must be float32 [{self.nh} heads, distances], got "
                             f"{tuple(self.score_bias.shape)} {self.score_bias.dtype}")

    # ---- cache -----------------------------------------------------------------------------------
    def kv_requirement(self):
        return KVRequirement(self.nkv, self.d, self.window_kind, self.window_size)

    # ---- step ------------------------------------------------------------------------------------
    def forward(self, h, residual, batch, cache):
        T = h.shape[0]
        dt = h.dtype
        qkv = self.ws.get("attn_qkv", (T, self.w_qkv.shape[0]), dt)
        with phase("qkv"):
            project(h, self.w_qkv, qkv)
        k_cache, v_cache, table, page_size = cache.kv()
        q = self.ws.get("attn_q", (T, self.nh * self.d), dt)
        with phase("kv_store"):          # head norm, rotation, temperature and the write into the cache: one kernel
            K.qkv_post(qkv, q, k_cache, v_cache, table, page_size, batch.token_seq, batch.token_pos,
                       batch.seq_slot, n_heads=self.nh, n_kv_heads=self.nkv, head_dim=self.d,
                       inv_freq=None if self.rotary is None else self.rotary.inv_freq,
                       interleaved=self.rotary is not None and self.rotary.interleaved,
                       qk_norm=self.qk_norm, norm_before_rope=self.norm_before_rope,
                       norm_eps=self.qk_norm_eps, temperature=self.temperature,
                       write_kv=self.has_kv and cache.owns)
        att = self.ws.get("attn_out", (T, self.nh * self.d), dt)
        with phase("attention"):
            self.attend(q, att, k_cache, v_cache, table, page_size, batch)
        with phase("wo"):
            project(att, self.w_o, residual, MODE_ADD)

    def attend(self, q, att, k_cache, v_cache, table, page_size, batch):
        wk = K.WINDOW_KINDS[self.window_kind]
        tensor_cores = use_tensor_core_kernels and self.score_bias is None     # those kernels add nothing to a score
        if (tensor_cores and batch.is_decode and q.dtype == torch.bfloat16
                and K.attention_decode_supported(self.nh, self.nkv, self.d, page_size)):
            # keys per sequence that the window lets through, at most (a bucketed bound: the split count
            # then stays the same from step to step, which a captured graph needs)
            longest = batch.ctx_bucket
            if self.window_kind != "full":
                longest = min(longest, self.window_size + page_size)
            pages = -(-longest // page_size)
            base = batch.n_tokens * self.nkv
            slots = K.attention_decode_blocks_per_sm(self.d) * K.sm_count()     # blocks that run at once
            if base <= slots:
                want = slots // base                                # one full wave and no more
            else:
                want = -(-4 * slots // base)                        # several waves of smaller blocks
            n_splits = max(1, min(want, pages // 4, K.MAX_DECODE_SPLITS))    # a block takes four pages or more
            K.attention_decode(q, att, k_cache, v_cache, table, page_size, batch.token_seq, batch.token_pos,
                               batch.seq_slot, n_heads=self.nh, n_kv_heads=self.nkv, head_dim=self.d,
                               window_kind=wk, window_size=self.window_size, scale=self.scale, n_splits=n_splits)
            return
        if (tensor_cores and not batch.is_decode and q.dtype == torch.bfloat16 and batch.n_q_tiles
                and K.attention_prefill_supported(self.nh, self.nkv, self.d, page_size)):
            K.attention_prefill(q, att, k_cache, v_cache, table, page_size, batch.token_seq, batch.token_pos,
                                batch.seq_slot, batch.tile_tok0, batch.tile_rows, n_heads=self.nh,
                                n_kv_heads=self.nkv, head_dim=self.d, window_kind=wk, window_size=self.window_size,
                                scale=self.scale)
            return
        K.attention_general(q, att, k_cache, v_cache, table, page_size, batch.token_seq, batch.token_pos,
                            batch.seq_slot, n_heads=self.nh, n_kv_heads=self.nkv, head_dim=self.d,
                            window_kind=K.WINDOW_KINDS[self.window_kind], window_size=self.window_size,
                            scale=self.scale, score_bias=self.score_bias)
