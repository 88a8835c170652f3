"""Feed-forward parts: a dense SwiGLU MLP, and routed experts with a shared expert.

Reference (src/engine/llama4_cpu_engine.cpp:252-291): router logits, the best expert, its
gate_up [H, 2I] and down [I, H] matrices applied as x @ W with a = silu(gate) * up, plus a shared
expert with ordinary [out, in] matrices, both added to the residual.  The reference takes one expert
and no gate value; top-k and the sigmoid gate (on the expert's input or output) are parameters here.

dense_swiglu  params: hidden_size, intermediate_size
              tensors: feed_forward.{gate,up,down}_proj.weight
moe_swiglu    params: hidden_size, num_experts, top_k, expert_size, shared_size (0 = no shared expert),
              router_gate ("sigmoid_input" | "sigmoid_output" | "none")
              tensors: feed_forward.router.weight [E, H], feed_forward.experts.gate_up_proj [E, H, 2I],
              feed_forward.experts.down_proj [E, I, H], feed_forward.shared_expert.{gate,up,down}_proj.weight

On load gate and up are stacked into one [2I, H] matrix, and the expert matrices are transposed to
[E, 2I, H] and [E, H, I], so that every contraction reads its weights along the reduction axis.
"""
from __future__ import annotations

import torch

from ..csrc import lib as K
from ..phases import active as phases_active, phase
from ..weights.store import TensorReq
from .base import FeedForward, register_feed_forward
from .linear import MODE_ADD, MODE_STORE, MODE_SWIGLU, project


def _stack(a, b):
    dt = torch.float32 if (a.dtype == torch.float32 or b.dtype == torch.float32) else torch.bfloat16
    return torch.cat([a.to(dt), b.to(dt)], dim=0).contiguous()


def _turned(t):
    """[E, in, out] as stored -> [E, out, in], contiguous (the library's transposing kernel on a GPU)."""
    if t.is_cuda and t.element_size() in (2, 4):
        return K.transpose_last2(t.contiguous())
    return t.transpose(1, 2).contiguous()


@register_feed_forward("dense_swiglu")
class DenseSwiGLU(FeedForward):
    graph_safe = True
    def __init__(self, spec, prefix="", workspace=None, names=("feed_forward.gate_proj.weight",
                                                                "feed_forward.up_proj.weight",
                                                                "feed_forward.down_proj.weight")):
        super().__init__(spec, prefix)
        self.hidden, self.inter = int(spec["hidden_size"]), int(spec["intermediate_size"])
        self.names = tuple(prefix + n for n in names)
        self.ws = workspace
        self.w_gate_up = self.w_down = None

    def requirements(self):
        g, u, d = self.names
        return [TensorReq(g, (self.inter, self.hidden)), TensorReq(u, (self.inter, self.hidden)),
                TensorReq(d, (self.hidden, self.inter))]

    def load(self, source, device):
        g, u, d = self.names
        self.w_gate_up = _stack(source.get(g, device), source.get(u, device))
        self.w_down = source.get(d, device).contiguous()

    def forward(self, h, residual, batch):
        a = self.ws.get("ffn_act", (h.shape[0], self.inter), h.dtype)
        with phase("mlp"):
            project(h, self.w_gate_up, a, MODE_SWIGLU)
            project(a, self.w_down, residual, MODE_ADD)


@register_feed_forward("moe_swiglu")
class MoESwiGLU(FeedForward):
    graph_safe = True
    def __init__(self, spec, prefix="", workspace=None):
        super().__init__(spec, prefix)
        p = spec.params
        self.hidden, self.n_experts, self.top_k = int(p["hidden_size"]), int(p["num_experts"]), int(p["top_k"])
        self.inter, self.shared_inter = int(p["expert_size"]), int(p.get("shared_size", 0))
        self.gate_mode = p.get("router_gate", "sigmoid_input")
        if self.gate_mode not in ("sigmoid_input", "sigmoid_output", "none"):
            raise ValueError(f"moe_swiglu: unknown router_gate '{self.gate_mode}'")
        if not 1 <= self.top_k <= self.n_experts:
            raise ValueError(f"moe_swiglu: top_k {self.top_k} of {self.n_experts} experts")
        if self.n_experts > 256:
            raise ValueError(f"moe_swiglu: {self.n_experts} experts (supported: up to 256)")
        self.ws = workspace
        f = prefix + "feed_forward."
        self.n_router, self.n_gate_up, self.n_down = f + "router.weight", f + "experts.gate_up_proj", f + "experts.down_proj"
        self.shared = None
        if self.shared_inter > 0:
            from ..config.spec import PartSpec
            self.shared = DenseSwiGLU(
                PartSpec("dense_swiglu", {"hidden_size": self.hidden, "intermediate_size": self.shared_inter}),
                prefix, workspace, names=("feed_forward.shared_expert.gate_proj.weight",
                                          "feed_forward.shared_expert.up_proj.weight",
                                          "feed_forward.shared_expert.down_proj.weight"))
        self.w_router = self.w_gate_up = self.w_down = None
        # The shared expert does not depend on the routing, so it runs on a second stream beside the routed
        # experts (fork after the norm).  The two must not add into the same residual rows at the same time:
        # either the routed outputs are stored and combined after the join, or (one expert per token, a step of
        # `join_early_tokens` tokens or more) the join comes before the routed down projection, which then adds
        # into the residual itself (measured at 2,048 tokens: 2.5 % of the step).
        self.overlap_shared = True
        self.join_early_tokens = 256
        self._side_stream = None
        self.capture = None        # a list: every forward appends a copy of its expert choices [T, k]

    def requirements(self):
        reqs = [TensorReq(self.n_router, (self.n_experts, self.hidden)),
                TensorReq(self.n_gate_up, (self.n_experts, self.hidden, 2 * self.inter)),
                TensorReq(self.n_down, (self.n_experts, self.inter, self.hidden))]
        if self.shared is not None:
            reqs += self.shared.requirements()
        return reqs

    def load(self, source, device):
        self.w_router = source.get(self.n_router, device).contiguous()
        self.w_gate_up = _turned(source.get(self.n_gate_up, device))          # [E, 2I, H]
        self.w_down = _turned(source.get(self.n_down, device))                # [E, H, I]
        if self.shared is not None:
            self.shared.load(source, device)

    def forward(self, h, residual, batch):
        T, E, Kk = h.shape[0], self.n_experts, self.top_k
        ws, i32, f32 = self.ws, torch.int32, torch.float32
        forked = None
        if self.shared is not None and self.overlap_shared and h.is_cuda and phases_active() is None:
            if self._side_stream is None:
                self._side_stream = torch.cuda.Stream(device=h.device)
            fork = torch.cuda.Event()
            fork.record(torch.cuda.current_stream())
            self._side_stream.wait_event(fork)
            with torch.cuda.stream(self._side_stream):
                self.shared.forward(h, residual, batch)
                forked = torch.cuda.Event()
                forked.record(self._side_stream)
        idx = ws.get("moe_topk_idx", (T, Kk), i32)
        gate = ws.get("moe_topk_gate", (T, Kk), f32)
        logits = ws.get("moe_router_logits", (T, E), f32)
        offsets = ws.get("moe_offsets", (E + 1,), i32)
        row_token = ws.get("moe_row_token", (T * Kk,), i32)
        row_scale = ws.get("moe_row_scale", (T * Kk,), f32)
        row_of_slot = ws.get("moe_row_of_slot", (T * Kk,), i32)
        M = T * Kk
        # rows sorted by expert, so that each expert reads a contiguous block (when rows are 16-byte multiples)
        sortable = (h.shape[1] * h.element_size()) % 16 == 0 and h.stride(0) * h.element_size() % 16 == 0
        sorted_h = ws.get("moe_in", (M, self.hidden), h.dtype) if sortable else None
        with phase("moe_router"):
            gathered = K.moe_route(h, self.w_router, idx, gate, logits, offsets, row_token, row_scale, row_of_slot,
                                   top_k=Kk, sigmoid_gate=self.gate_mode != "none", sorted_h=sorted_h)
        if self.capture is not None:
            self.capture.append(idx.clone())
        hint = max(1, -(-M // E))
        act = ws.get("moe_act", (M, self.inter), h.dtype)
        in_scale = row_scale if self.gate_mode == "sigmoid_input" else None
        with phase("moe_expert"):
            if sortable:
                if not gathered:
                    K.gather_rows(h, row_token, sorted_h)
                project(sorted_h, self.w_gate_up, act, MODE_SWIGLU, m_rows=M, row_scale=in_scale,
                        group_offsets=offsets, n_groups=E, rows_per_group_hint=hint)
            else:
                project(h, self.w_gate_up, act, MODE_SWIGLU, m_rows=M, a_rows=row_token, row_scale=in_scale,
                        group_offsets=offsets, n_groups=E, rows_per_group_hint=hint)
            out_scale = row_scale if self.gate_mode == "sigmoid_output" else None
            # One expert per token: the down projection can add straight into the residual rows.  Beside a shared
            # expert on the second stream that needs an order (two kernels adding into the same rows at once would
            # sum in whatever order they meet): in a step with many tokens the join comes before the down
            # projection (each product fills the GPU by itself, so nothing is lost by the wait, and the stored
            # outputs and the combine kernel go); in a step with few tokens the two chains run side by side to the
            # end and the combine adds the routed outputs after the join.
            join_early = forked is not None and Kk == 1 and T >= self.join_early_tokens
            if join_early:
                torch.cuda.current_stream().wait_event(forked)
            direct = Kk == 1 and (forked is None or join_early)
            if direct:
                project(act, self.w_down, residual, MODE_ADD, m_rows=M, out_rows=row_token, row_scale=out_scale,
                        group_offsets=offsets, n_groups=E, rows_per_group_hint=hint)
            else:
                y = ws.get("moe_y", (M, self.hidden), f32)
                project(act, self.w_down, y, MODE_STORE, m_rows=M, row_scale=out_scale,
                        group_offsets=offsets, n_groups=E, rows_per_group_hint=hint)
        if not direct:
            if forked is not None:
                torch.cuda.current_stream().wait_event(forked)
            with phase("moe_merge"):
                K.moe_combine(residual, y, row_of_slot, top_k=Kk)
        if forked is not None:
            return
        if self.shared is not None:
            self.shared.forward(h, residual, batch)
