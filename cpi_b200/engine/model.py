"""A decoder built from a ModelSpec: layers of registered parts, run in the order the spec lists."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..config.spec import ModelSpec
from ..csrc import lib as K
from ..parts import base as parts_base
from ..parts import Workspace, build_part
from ..parts.linear import project
from ..phases import phase
from ..weights.store import TensorReq, check_source


@dataclass
class Layer:
    block: object
    mixer: object
    feed_forward: object
    mixer_norm: object
    feed_forward_norm: object

    def parts(self):
        return (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward)

    def all_parts(self):
        """Every object whose code runs in a step of this layer (the mixer's position encoding included)."""
        out = [self.block, *self.parts()]
        pos = getattr(self.mixer, "position", None)
        if pos is not None:
            out.append(pos)
        return out


class DecoderModel:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device, workspace: Workspace | None = None):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"activation dtype must be float32 or bfloat16, not {dtype}")
        spec.validate()
        self.spec, self.dtype, self.device = spec, dtype, torch.device(device)
        self.ws = workspace if workspace is not None else Workspace(self.device)
        owners = set()                      # layers that some run entry uses with a cache of its own
        for e in spec.run_order:
            if e.cache_of is None:
                owners.add(e.layer)
        self.layers = []
        for i, ls in enumerate(spec.layers):
            self.layers.append(Layer(
                block=build_part("block", ls.block, ls.prefix),
                mixer=build_part("mixer", ls.mixer, ls.prefix, workspace=self.ws, owns_cache=i in owners),
                feed_forward=build_part("feed_forward", ls.feed_forward, ls.prefix, workspace=self.ws),
                mixer_norm=build_part("norm", ls.mixer_norm, ls.prefix, workspace=self.ws, tag="norm_mixer"),
                feed_forward_norm=build_part("norm", ls.feed_forward_norm, ls.prefix, workspace=self.ws,
                                             tag="norm_ffn"),
            ))
        self.final_norm = build_part("norm", spec.final_norm, "", workspace=self.ws, tag="norm_final")
        self.embed_name = spec.embedding["weight"]
        self.head_name = spec.head["weight"]
        self.embedding = self.head = None
        self.err_flag = None

    # ---- weights ---------------------------------------------------------------------------------
    def all_parts(self) -> list:
        """Every part object of the model (layers' blocks, norms, mixers with their position encodings,
        feed-forwards, the final norm)."""
        out = [self.final_norm]
        for layer in self.layers:
            out += layer.all_parts()
        return out

    def requirements(self) -> list:
        V, H = self.spec.vocab_size, self.spec.hidden_size
        reqs = [TensorReq(self.embed_name, (V, H))]
        if self.head_name != self.embed_name:
            reqs.append(TensorReq(self.head_name, (V, H)))
        reqs += self.final_norm.requirements()
        for layer in self.layers:
            for p in layer.parts():
                reqs += p.requirements()
        return reqs

    def load(self, source) -> None:
        tolerated = ()
        if self.head_name == self.embed_name:      # a tied model may still store a head tensor
            tolerated = tuple(n for n in source.names() if n.endswith("lm_head.weight"))
        check_source(self.requirements(), source, self.spec.ignored_tensor_prefixes, tolerated)
        dev = self.device
        self.embedding = source.get(self.embed_name, dev).contiguous()
        self.head = self.embedding if self.head_name == self.embed_name else source.get(self.head_name, dev).contiguous()
        self.final_norm.load(source, dev)
        for layer in self.layers:
            for p in layer.parts():
                p.load(source, dev)
        # the word of the device's error flags that the embedding kernel sets for a token outside the table
        self.err_flag = K.device_error_flags(dev)[1:2] if torch.device(dev).type == "cuda" \
            else torch.zeros(1, dtype=torch.int32, device=dev)

    # ---- cache needs -----------------------------------------------------------------------------
    def cache_requirements(self):
        """({run entry: KVRequirement}, {run entry: [StateRequirement]}) for entries that own a cache."""
        kv, state = {}, {}
        for i, e in enumerate(self.spec.run_order):
            if e.cache_of is not None:
                continue
            m = self.layers[e.layer].mixer
            r = m.kv_requirement()
            if r is not None:
                kv[i] = r
            s = m.state_requirements()
            if s:
                state[i] = list(s)
        return kv, state

    # ---- forward ---------------------------------------------------------------------------------
    def run(self, batch, cache_manager) -> torch.Tensor:
        """Runs the step's tokens through every run entry; returns float32 logits [n_want, vocab]."""
        T, H = batch.n_tokens, self.spec.hidden_size
        x = self.ws.get("residual", (T, H), torch.float32)
        with phase("embedding"):
            K.embedding(batch.tokens, self.embedding, x, self.err_flag)
        for i, e in enumerate(self.spec.run_order):
            layer = self.layers[e.layer]
            owner = i if e.cache_of is None else e.cache_of
            view = parts_base.CacheView(cache_manager, owner, owns=e.cache_of is None)
            layer.block.run(layer, x, batch, view)
        R = batch.n_want
        logits = self.ws.get("logits", (R, self.spec.vocab_size), torch.float32)   # valid until the next step
        if R:
            with phase("rmsnorm"):
                xn = self.final_norm(x, self.dtype, rows=batch.want_rows)
            with phase("lm_head"):
                project(xn, self.head, logits)
        return logits


def tensor_requirements(spec: ModelSpec) -> list:
    """The tensors a model of this spec needs (names, shapes, random-init rule), without a device."""
    return DecoderModel(spec, torch.float32, "cpu").requirements()
