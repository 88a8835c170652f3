"""Single kernels on small, self-contained workloads: for timing a kernel alone and for profiler captures.

    python -m cpi_b200.csrc.cases gemm --tokens 8 --out 8192 --in 5120 --mode swiglu --groups 16
    python -m cpi_b200.csrc.cases attention_decode --batch 8 --context 4096
    python -m cpi_b200.csrc.cases attention_prefill --tokens 2048
    python -m cpi_b200.csrc.cases step --layers 4 --batch 8 --context 4000 --decode

Each case holds a few GB at most, flushes the L2 between launches (a 256 MB write), times `--reps`
launches with CUDA events and prints the median with the bytes or flops the launch has to move.
"""
from __future__ import annotations

import argparse
import sys

import torch

from . import lib as K

DEV = "cuda:0"


def _graph_ms(body, reps: int) -> float:
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(reps):
            body()
    g.replay()
    torch.cuda.synchronize()
    times = []
    for _ in range(3):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    return sorted(times)[1]


def _timed(fn, reps: int, flush: torch.Tensor) -> float:
    """Microseconds per launch: a graph of `reps` x (L2 flush, kernel) minus a graph of `reps` flushes, so
    that neither the launch latency of Python nor the flush is counted."""
    fn()
    torch.cuda.synchronize()
    reps = max(reps, 5)
    both = _graph_ms(lambda: (flush.zero_(), fn()), reps)
    only = _graph_ms(lambda: flush.zero_(), reps)
    return (both - only) * 1e3 / reps


def case_gemm(a) -> None:
    T, N, Kd, G = a.tokens, a.out, a.inp, a.groups
    mode = {"store": K.MODE_STORE, "add": K.MODE_ADD, "swiglu": K.MODE_SWIGLU}[a.mode]
    rows = 2 * N if mode == K.MODE_SWIGLU else N
    g = torch.Generator(device=DEV).manual_seed(0)
    w = torch.empty((G, rows, Kd) if G else (rows, Kd), dtype=torch.bfloat16, device=DEV).normal_(0, 0.02, generator=g)
    x = torch.empty(T, Kd, dtype=torch.bfloat16, device=DEV).normal_(0, 1, generator=g)
    out = torch.zeros(T, N, dtype=torch.float32 if mode == K.MODE_ADD else torch.bfloat16, device=DEV)
    kw = {}
    touched = 1
    if G:
        # tokens spread over the groups as a uniform router would
        which = torch.randint(0, G, (T,), generator=torch.Generator().manual_seed(1)).sort().values
        counts = torch.bincount(which, minlength=G)
        touched = int((counts > 0).sum())
        offs = torch.zeros(G + 1, dtype=torch.int32)
        offs[1:] = counts.cumsum(0)
        kw = dict(m_rows=T, group_offsets=offs.to(DEV), n_groups=G)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=DEV)
    if a.persistent is not None:
        K.gemm_pair_persistent(a.persistent)
    fn = K.gemm_tc_pair if a.pair else K.gemm_tc
    if not fn(x, w, out, mode, **kw):
        sys.exit("this shape is outside what the tensor-core kernel takes")
    us = _timed(lambda: fn(x, w, out, mode, **kw), a.reps, flush)
    wbytes = touched * rows * Kd * 2
    flops = 2.0 * T * rows * Kd
    print(f"gemm{' (pair)' if a.pair else ''} tokens={T} out={N} in={Kd} mode={a.mode} groups={G} (touched {touched}): {us:.1f} us, "
          f"weights {wbytes / 1e6:.0f} MB -> {wbytes / us / 1e6:.2f} TB/s, {flops / us / 1e6:.1f} TFLOP/s")


def _paged(batch, context, NKV, D, page=64):
    blocks = -(-context // page)
    n_pages = batch * blocks
    g = torch.Generator(device=DEV).manual_seed(0)
    k = torch.empty(n_pages, NKV, page, D, dtype=torch.bfloat16, device=DEV).normal_(0, 1, generator=g)
    v = torch.empty_like(k).normal_(0, 1, generator=g)
    table = torch.randperm(n_pages).to(torch.int32).view(batch, blocks).to(DEV)
    return k, v, table


def case_attention_decode(a) -> None:
    B, ctx, NH, NKV, D = a.batch, a.context, a.heads, a.kv_heads, a.head_dim
    k, v, table = _paged(B, ctx, NKV, D)
    q = torch.randn(B, NH * D, device=DEV).bfloat16()
    out = torch.empty_like(q)
    seq = torch.arange(B, dtype=torch.int32, device=DEV)
    pos = torch.full((B,), ctx - 1, dtype=torch.int32, device=DEV)
    base, slots, pages = B * NKV, K.attention_decode_blocks_per_sm(D) * K.sm_count(), -(-ctx // 64)
    splits = a.splits or max(1, min(slots // base if base <= slots else -(-4 * slots // base),
                                    pages // 4, K.MAX_DECODE_SPLITS))
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=DEV)
    fn = lambda: K.attention_decode(q, out, k, v, table, 64, seq, pos, seq, n_heads=NH, n_kv_heads=NKV, head_dim=D,
                                    window_kind=0, window_size=0, scale=D ** -0.5, n_splits=splits)
    us = _timed(fn, a.reps, flush)
    nbytes = 2.0 * B * ctx * NKV * D * 2
    print(f"attention_decode batch={B} context={ctx} heads={NH}/{NKV} D={D} splits={splits}: {us:.1f} us, "
          f"cache {nbytes / 1e6:.0f} MB -> {nbytes / us / 1e6:.2f} TB/s")


def case_attention_prefill(a) -> None:
    T, NH, NKV, D = a.tokens, a.heads, a.kv_heads, a.head_dim
    k, v, table = _paged(1, T, NKV, D)
    q = torch.randn(T, NH * D, device=DEV).bfloat16()
    out = torch.empty_like(q)
    seq = torch.zeros(T, dtype=torch.int32, device=DEV)
    pos = torch.arange(T, dtype=torch.int32, device=DEV)
    slot = torch.zeros(1, dtype=torch.int32, device=DEV)
    R = K.PREFILL_TILE_ROWS
    tiles = [(t0, min(R, T - t0)) for t0 in range(0, T, R)][::-1]
    tok0 = torch.tensor([t[0] for t in tiles], dtype=torch.int32, device=DEV)
    rows = torch.tensor([t[1] for t in tiles], dtype=torch.int32, device=DEV)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=DEV)
    fn = lambda: K.attention_prefill(q, out, k, v, table, 64, seq, pos, slot, tok0, rows, n_heads=NH, n_kv_heads=NKV,
                                     head_dim=D, window_kind=0, window_size=0, scale=D ** -0.5)
    us = _timed(fn, a.reps, flush)
    flops = 4.0 * NH * D * T * (T + 1) / 2
    print(f"attention_prefill tokens={T} heads={NH}/{NKV} D={D}: {us:.1f} us, {flops / us / 1e6:.1f} TFLOP/s (causal)")


SCOUT_LAYER = {
    "architectures": ["Llama4ForCausalLM"], "hidden_size": 5120, "num_attention_heads": 40,
    "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 8192, "intermediate_size_mlp": 16384,
    "num_local_experts": 16, "num_experts_per_tok": 1, "interleave_moe_layer_step": 1, "vocab_size": 202048,
    "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 16.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "nope_layer_interval": 4, "attention_chunk_size": 8192, "use_qk_norm": True, "attn_temperature_tuning": True,
    "floor_scale": 8192, "attn_scale": 0.1, "tie_word_embeddings": False, "max_position_embeddings": 131072,
}


def case_step(a) -> None:
    """One whole engine step of a model with Scout-sized layers and random weights, bracketed by
    cudaProfilerStart/Stop (use `ncu --profile-from-start off`); graphs off, so every kernel is a launch."""
    from ..api import Model
    from ..engine import StepEntry
    cfg = dict(SCOUT_LAYER, num_hidden_layers=a.layers)
    m = Model.random(cfg, 0, dtype="bfloat16", max_batch=a.batch, max_context=a.context + 64)
    eng = m.engine
    eng.use_graphs = False
    g = torch.Generator().manual_seed(1)
    toks = lambda n: torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist()
    out = torch.empty(a.batch, dtype=torch.int32, device=DEV)
    slots = [eng.acquire_slot() for _ in range(a.batch)]
    if a.decode:
        eng.step([StepEntry(s, toks(a.context), []) for s in slots])

        def one():
            K.argmax(eng.step([StepEntry(s, toks(1), [0]) for s in slots]), out)
        for _ in range(3):
            one()
    else:
        def one():
            eng.step([StepEntry(s, toks(a.context), [a.context - 1]) for s in slots])
            for s in slots:
                eng.release_slot(s)
            slots[:] = [eng.acquire_slot() for _ in range(a.batch)]
        one()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.profiler.start()
    e0.record()
    one()
    e1.record()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    print(f"step layers={a.layers} batch={a.batch} context={a.context} {'decode' if a.decode else 'prefill'}: "
          f"{e0.elapsed_time(e1):.3f} ms")


def main() -> int:
    ap = argparse.ArgumentParser(prog="python -m cpi_b200.csrc.cases")
    sub = ap.add_subparsers(dest="case", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--tokens", type=int, default=8)
    g.add_argument("--out", type=int, default=8192)
    g.add_argument("--in", dest="inp", type=int, default=5120)
    g.add_argument("--mode", choices=["store", "add", "swiglu"], default="store")
    g.add_argument("--groups", type=int, default=0)
    g.add_argument("--pair", action="store_true", help="use the paired (two-SM) kernel")
    g.add_argument("--persistent", type=int, default=None, help="paired kernel: 2 a pair per SM pair works through the tiles, 0 a launch slot per tile, 1 by shape")
    d = sub.add_parser("attention_decode")
    d.add_argument("--batch", type=int, default=8)
    d.add_argument("--context", type=int, default=4096)
    d.add_argument("--splits", type=int, default=0)
    p = sub.add_parser("attention_prefill")
    p.add_argument("--tokens", type=int, default=2048)
    st = sub.add_parser("step")
    st.add_argument("--layers", type=int, default=4)
    st.add_argument("--batch", type=int, default=8)
    st.add_argument("--context", type=int, default=4000)
    st.add_argument("--decode", action="store_true", help="time a decode step after a prefill of --context tokens")
    for s in (g, d, p):
        s.add_argument("--reps", type=int, default=5)
    for s in (d, p):
        s.add_argument("--heads", type=int, default=40)
        s.add_argument("--kv-heads", type=int, default=8)
        s.add_argument("--head-dim", type=int, default=128)
    a = ap.parse_args()
    {"gemm": case_gemm, "attention_decode": case_attention_decode, "attention_prefill": case_attention_prefill,
     "step": case_step}[a.case](a)
    return 0


if __name__ == "__main__":
    sys.exit(main())
