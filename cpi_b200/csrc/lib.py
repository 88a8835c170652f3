"""ctypes bindings of the kernel library: torch tensors in, asynchronous launches on the current stream.

There is no CPU fallback and no library model code behind these functions: if the shared object
cannot be built or loaded, `load()` raises, and every function below raises with it.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_long, c_float, c_void_p

import torch

from . import build as _build

F32, BF16 = 0, 1
MODE_STORE, MODE_ADD, MODE_SWIGLU = 0, 1, 2
WINDOW_FULL, WINDOW_CHUNK, WINDOW_SLIDING = 0, 1, 2
WINDOW_KINDS = {"full": WINDOW_FULL, "chunk": WINDOW_CHUNK, "sliding": WINDOW_SLIDING}
MAX_DECODE_SPLITS = 256          # key splits that the combine kernel of decode attention takes
PREFILL_TILE_ROWS = 256          # most query rows of one sequence that a block of the prefill attention kernel takes

ABI_VERSION = 1                  # what cpi_abi_version() of a matching library answers

_lib = None
scratch_generation = 0    # grows whenever a scratch buffer of this module is (re)allocated
launch_count = 0          # kernels launched through this module since import (bench reports it)


class KernelError(RuntimeError):
    pass


def load():
    global _lib
    if _lib is None:
        path = _build.library_path()
        try:
            _lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"cpi_b200: cannot load the kernel library {path}: {e}") from None
        _lib.cpi_last_error.restype = ctypes.c_char_p
        if _lib.cpi_abi_version() != ABI_VERSION:
            raise KernelError(f"cpi_b200: {path} has ABI version {_lib.cpi_abi_version()}, this package "
                              f"wants {ABI_VERSION}")
    return _lib


def kernel_launches() -> int:
    """Kernels this library has launched from host code (graph replays are counted by the engine)."""
    load().cpi_launch_count.restype = c_long
    return int(load().cpi_launch_count())


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"cpi_b200 kernels take float32 or bfloat16, not {dt}")


def _p(t):
    return c_void_p(0 if t is None else t.data_ptr())


def _stream():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _call(name, *args):
    global launch_count
    rc = getattr(load(), name)(*args)
    if rc != 0:
        raise KernelError(load().cpi_last_error().decode())
    launch_count += 1


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise KernelError("cpi_b200 kernels run on CUDA tensors only (there is no CPU path)")


def _rowmajor(t, what):
    if t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"{what}: expected a 2-D tensor with contiguous rows, got shape "
                          f"{tuple(t.shape)} strides {t.stride()}")


# ------------------------------------------------------------------------------------------------
def embedding(tokens, table, out, err_flag):
    """out[t, :] = table[tokens[t], :] as float32; a token outside the table sets err_flag[0] = 1 + t."""
    _need_cuda(tokens, table, out, err_flag)
    T, H = out.shape
    assert tokens.dtype == torch.int32 and out.dtype == torch.float32 and out.is_contiguous()
    assert table.is_contiguous() and table.shape[1] == H
    _call("cpi_embedding", _p(tokens), _p(table), c_int(dtype_code(table.dtype)), _p(out), c_int(T), c_int(H),
          c_int(table.shape[0]), _p(err_flag), _stream())


def rmsnorm(x, weight, eps, out, rows=None):
    """out[r] = x[rows[r] or r] * rsqrt(mean(x^2) + eps) * weight; weight may be None."""
    _need_cuda(x, weight, out, rows)
    _rowmajor(x, "rmsnorm x"); _rowmajor(out, "rmsnorm out")
    n_rows, n = out.shape
    assert x.shape[1] == n and (rows is not None or x.shape[0] == n_rows)
    assert rows is None or rows.dtype == torch.int32
    assert weight is None or (weight.numel() == n and weight.is_contiguous())
    _call("cpi_rmsnorm", _p(x), c_int(dtype_code(x.dtype)), c_long(x.stride(0)), _p(rows), _p(weight),
          c_int(F32 if weight is None else dtype_code(weight.dtype)), _p(out), c_int(dtype_code(out.dtype)),
          c_long(out.stride(0)), c_int(n_rows), c_int(n), c_float(eps), _stream())


def gemm_simt(a, w, out, mode=MODE_STORE, *, n_out=None, m_rows=None, a_rows=None, out_rows=None,
              row_scale=None, group_offsets=None, n_groups=0, rows_per_group_hint=None):
    """out[m, n] (+)= sum_k a[a_rows[m] or m, k] * w[g(m)][n, k] on the FP32 pipe (see gemm_simt.cu).

    w is [N, K], or [2N, K] in SWIGLU mode, or [G, N or 2N, K] with group_offsets (int32 [G+1]).
    """
    _need_cuda(a, w, out, a_rows, out_rows, row_scale, group_offsets)
    _rowmajor(a, "gemm a"); _rowmajor(out, "gemm out")
    K = a.shape[1]
    if group_offsets is not None:
        assert w.dim() == 3 and w.is_contiguous() and w.shape[0] == n_groups
        rows_w, stride_g = w.shape[1], w.shape[1] * w.shape[2]
    else:
        _rowmajor(w, "gemm w")
        rows_w, stride_g = w.shape[0], 0
    assert w.shape[-1] == K, f"gemm: a has K={K}, w has K={w.shape[-1]}"
    N = n_out if n_out is not None else (rows_w // 2 if mode == MODE_SWIGLU else rows_w)
    assert rows_w == (2 * N if mode == MODE_SWIGLU else N)
    assert out.shape[1] == N
    M = m_rows if m_rows is not None else (a_rows.numel() if a_rows is not None else a.shape[0])
    ldw = w.stride(-2)
    hint = rows_per_group_hint if rows_per_group_hint is not None else M
    _call("cpi_gemm_simt", _p(a), c_int(dtype_code(a.dtype)), c_long(a.stride(0)), _p(a_rows),
          _p(w), c_int(dtype_code(w.dtype)), c_long(ldw), c_long(stride_g),
          _p(out), c_int(dtype_code(out.dtype)), c_long(out.stride(0)), _p(out_rows), _p(row_scale),
          _p(group_offsets), c_int(n_groups), c_int(M), c_int(N), c_int(K), c_int(mode), c_int(hint), _stream())


_errors = {}          # device index -> int32[2]: [0] a tensor-core kernel gave up a wait, [1] a token id out of range


def device_error_flags(device) -> torch.Tensor:
    """int32[2] on the device that kernels write when something went wrong: word 0 is set to 1 by a tensor-core
    kernel whose bounded barrier wait ran out, word 1 to 1 + t by the embedding kernel when token t of a step
    was outside the vocabulary.  The engine reads and clears them."""
    idx = torch.device(device).index or 0
    if idx not in _errors:
        _errors[idx] = torch.zeros(2, dtype=torch.int32, device=device)
    return _errors[idx]


def tc_error_flag(device) -> torch.Tensor:
    """int32[1] that a tensor-core kernel sets when one of its bounded waits ran out."""
    return device_error_flags(device)[0:1]


def sm_count() -> int:
    """Multiprocessors of the current CUDA device."""
    return int(load().cpi_sm_count())


def gemm_tc(a, w, out, mode=MODE_STORE, *, n_out=None, m_rows=None, a_rows=None, out_rows=None, row_scale=None,
            group_offsets=None, n_groups=0, rows_per_group_hint=None) -> bool:
    """The tcgen05 kernel for out[m, n] (+)= sum_k a[m, k] w[g(m)][n, k] in bfloat16 (see gemm_tc.cu).

    Returns False, having launched nothing, when the call is outside what the kernel takes (a row
    gather, K or a row stride that is no multiple of 8, unaligned operands, an output dtype the
    epilogue does not write); the caller then uses the FP32-pipe kernel."""
    if a_rows is not None or a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        return False
    if a.dim() != 2 or a.stride(1) != 1 or not w.is_contiguous() or out.stride(-1) != 1:
        return False
    K = a.shape[1]
    if K % 8 or a.stride(0) % 8 or a.data_ptr() % 16 or w.data_ptr() % 16 or w.shape[-1] != K:
        return False
    if mode == MODE_SWIGLU and out.dtype != torch.bfloat16:
        return False
    if mode == MODE_ADD and out.dtype != torch.float32:
        return False
    _need_cuda(a, w, out, out_rows, row_scale, group_offsets)
    grouped = group_offsets is not None
    rows_w = w.shape[-2]
    N = n_out if n_out is not None else (rows_w // 2 if mode == MODE_SWIGLU else rows_w)
    if rows_w != (2 * N if mode == MODE_SWIGLU else N) or out.shape[1] != N:
        raise KernelError(f"gemm_tc: weight rows {rows_w} do not match {N} outputs in mode {mode}")
    if grouped and (w.dim() != 3 or w.shape[0] != n_groups):
        raise KernelError("gemm_tc: grouped weights must be [groups, rows, K]")
    T = m_rows if m_rows is not None else a.shape[0]
    if T > a.shape[0]:
        raise KernelError("gemm_tc: more logical rows than activation rows")
    bn, splits, live_y = c_int(), c_int(), c_int()
    load().cpi_gemm_tc_plan(c_int(T), c_int(N), c_int(K), c_int(n_groups if grouped else 0),
                            c_int(int(mode == MODE_SWIGLU)), ctypes.byref(bn), ctypes.byref(splits),
                            ctypes.byref(live_y))
    _call("cpi_gemm_tc", _p(a), c_long(a.stride(0)), _p(w), _p(out), c_int(dtype_code(out.dtype)),
          c_long(out.stride(0)), _p(out_rows), _p(row_scale), _p(group_offsets), c_int(n_groups if grouped else 0),
          c_int(T), c_int(N), c_int(K), c_int(mode), c_int(bn.value), c_int(splits.value),
          _p(tc_error_flag(a.device)), _stream())
    return True


def gemm_tc_plan(T: int, N: int, K: int, n_groups: int = 0, swiglu: bool = False):
    """(token rows per tile, k splits) that `gemm_tc` uses for a product of these sizes on this device."""
    bn, splits, live_y = c_int(), c_int(), c_int()
    load().cpi_gemm_tc_plan(c_int(T), c_int(N), c_int(K), c_int(n_groups), c_int(int(swiglu)), ctypes.byref(bn),
                            ctypes.byref(splits), ctypes.byref(live_y))
    return bn.value, splits.value


def gemm_tc_wait_probe(spin_limit: int = 0, tx_extra: int = 0) -> None:
    """For the test of the give-up path of `gemm_tc`: launches from now on poll each barrier at most
    `spin_limit` times and expect `tx_extra` bytes more per stage than their loads bring, so that the wait runs
    out, the kernel raises the error flag and returns.  (0, 0) puts the ordinary values back."""
    load().cpi_gemm_tc_wait_probe(c_int(int(spin_limit)), c_int(int(tx_extra)))


def gemm_pair_persistent(mode) -> None:
    """Dense products of `gemm_tc_pair`: 2 / True = always one pair of CTAs per SM pair working through the
    tiles (the epilogue of one tile under the MMAs of the next), 0 / False = always a launch slot per tile,
    1 = the library's choice by shape (the default)."""
    load().cpi_gemm_tc_pair_persistent(c_int(2 if mode is True else 0 if mode is False else int(mode)))


def gemm_tc_pair(a, w, out, mode=MODE_STORE, *, m_rows=None, out_rows=None, row_scale=None, group_offsets=None,
                 n_groups=0, rows_per_group_hint=None) -> bool:
    """The paired (two-SM) tcgen05 kernel for products with many tokens, dense or grouped (see
    gemm_tc_pair.cu).  Returns False, having launched nothing, when the product is outside what it takes."""
    grouped = group_offsets is not None
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or a.dim() != 2 or w.dim() != (3 if grouped else 2):
        return False
    if a.stride(1) != 1 or not w.is_contiguous() or out.stride(-1) != 1:
        return False
    K = a.shape[1]
    T = m_rows if m_rows is not None else a.shape[0]
    rows_w = w.shape[-2]
    N = rows_w // 2 if mode == MODE_SWIGLU else rows_w
    if w.shape[-1] != K or out.shape[1] != N or a.stride(0) % 8 or a.data_ptr() % 16 or w.data_ptr() % 16:
        return False
    if grouped and w.shape[0] != n_groups:
        return False
    if (mode == MODE_SWIGLU and out.dtype != torch.bfloat16) or (mode == MODE_ADD and out.dtype != torch.float32):
        return False
    bn = load().cpi_gemm_tc_pair_plan(c_int(T), c_int(N), c_int(K), c_int(int(mode == MODE_SWIGLU)),
                                      c_int(n_groups if grouped else 0))
    if bn <= 0:
        return False
    _need_cuda(a, w, out, out_rows, row_scale, group_offsets)
    _call("cpi_gemm_tc_pair", _p(a), c_long(a.stride(0)), _p(w), _p(out), c_int(dtype_code(out.dtype)),
          c_long(out.stride(0)), _p(out_rows), _p(row_scale), _p(group_offsets), c_int(n_groups if grouped else 0),
          c_int(T), c_int(N), c_int(K), c_int(mode), c_int(bn), _p(tc_error_flag(a.device)), _stream())
    return True


# ---- load time ----------------------------------------------------------------------------------------------
def random_normal(out, start, seed, std, table):
    """out.view(-1)[k] = table[hash(seed, start + k)] * std, rounded to out's dtype (float32 or bfloat16), for a
    contiguous CUDA tensor; `table`: float32 [65536] on the same device."""
    _need_cuda(out, table)
    assert out.is_contiguous() and table.dtype == torch.float32 and table.numel() == 65536 and table.is_contiguous()
    rc = load().cpi_random_normal(_p(out), c_int(dtype_code(out.dtype)), c_long(int(start)), c_long(out.numel()),
                                  ctypes.c_ulonglong(int(seed) & 0xFFFFFFFFFFFFFFFF), c_float(std), _p(table), _stream())
    if rc:
        raise KernelError(load().cpi_last_error().decode())


def widen_f16(src, dst):
    """dst (float32) = src (float16), exactly; contiguous CUDA tensors of equal size."""
    _need_cuda(src, dst)
    assert src.dtype == torch.float16 and dst.dtype == torch.float32 and src.is_contiguous() and dst.is_contiguous()
    assert src.numel() == dst.numel()
    if load().cpi_widen_f16(_p(src), _p(dst), c_long(src.numel()), _stream()):
        raise KernelError(load().cpi_last_error().decode())


def transpose_last2(src, dst=None):
    """dst [..., c, r] = src [..., r, c] for a contiguous CUDA tensor of 2- or 4-byte elements."""
    _need_cuda(src, dst)
    assert src.is_contiguous() and src.dim() >= 2 and src.element_size() in (2, 4)
    r, c = src.shape[-2], src.shape[-1]
    g = src.numel() // (r * c) if src.numel() else 0
    if dst is None:
        dst = torch.empty(*src.shape[:-2], c, r, dtype=src.dtype, device=src.device)
    assert dst.is_contiguous() and dst.dtype == src.dtype and dst.numel() == src.numel()
    if load().cpi_transpose(_p(src), _p(dst), c_int(src.element_size()), c_long(g), c_int(r), c_int(c), _stream()):
        raise KernelError(load().cpi_last_error().decode())
    return dst


def gather_rows(src, rows, dst):
    """dst[r] = src[rows[r]] for 2-D tensors whose rows are multiples of 16 bytes."""
    _need_cuda(src, rows, dst)
    _rowmajor(src, "gather_rows src")
    assert dst.is_contiguous() and dst.dtype == src.dtype and dst.shape[1] == src.shape[1]
    assert rows.dtype == torch.int32
    n = dst.shape[0]
    _call("cpi_gather_rows", _p(src), c_long(src.stride(0) * src.element_size()), _p(rows), _p(dst), c_int(n),
          c_int(src.shape[1] * src.element_size()), _stream())


def qkv_post(qkv, q_out, k_cache, v_cache, page_table, page_size, token_seq, token_pos, seq_slot, *,
             n_heads, n_kv_heads, head_dim, inv_freq=None, interleaved=False, qk_norm=False,
             norm_before_rope=False, norm_eps=0.0, temperature=None, write_kv=True):
    """Norm / rotate / scale q and k per head, write q to q_out and k, v into the cache pages."""
    _need_cuda(qkv, q_out, k_cache, v_cache, page_table, token_seq, token_pos, seq_slot, inv_freq)
    _rowmajor(qkv, "qkv_post qkv")
    T = qkv.shape[0]
    assert q_out.is_contiguous() and q_out.dtype == qkv.dtype
    assert k_cache is None or k_cache.dtype == qkv.dtype
    assert inv_freq is None or (inv_freq.dtype == torch.float32 and inv_freq.numel() == head_dim // 2)
    fl, sc = (temperature if temperature is not None else (1.0, 0.0))
    _call("cpi_qkv_post", _p(qkv), c_long(qkv.stride(0)), _p(q_out), _p(k_cache), _p(v_cache),
          c_int(dtype_code(qkv.dtype)), _p(page_table), c_int(page_table.shape[1]), c_int(page_size),
          _p(token_seq), _p(token_pos), _p(seq_slot), _p(inv_freq), c_int(int(interleaved)),
          c_int(int(qk_norm)), c_int(int(norm_before_rope)), c_float(norm_eps),
          c_int(int(temperature is not None)), c_float(fl), c_float(sc), c_int(T), c_int(n_heads),
          c_int(n_kv_heads), c_int(head_dim), c_int(int(write_kv)), _stream())


def attention_general(q, out, k_cache, v_cache, page_table, page_size, token_seq, token_pos, seq_slot, *,
                      n_heads, n_kv_heads, head_dim, window_kind, window_size, scale, score_bias=None):
    """Attention of any head size and dtype over the paged cache.  `score_bias`: float32 [heads, n_dist] added
    to the scaled scores, indexed by the distance query position - key position (the last column for longer)."""
    _need_cuda(q, out, k_cache, v_cache, page_table, token_seq, token_pos, seq_slot, score_bias)
    assert q.is_contiguous() and out.is_contiguous() and q.dtype == out.dtype == k_cache.dtype
    assert score_bias is None or (score_bias.dtype == torch.float32 and score_bias.is_contiguous()
                                  and score_bias.dim() == 2 and score_bias.shape[0] == n_heads)
    T = q.shape[0]
    _call("cpi_attention_general", _p(q), _p(out), _p(k_cache), _p(v_cache), c_int(dtype_code(q.dtype)),
          _p(page_table), c_int(page_table.shape[1]), c_int(page_size), _p(token_seq), _p(token_pos),
          _p(seq_slot), c_int(T), c_int(n_heads), c_int(n_kv_heads), c_int(head_dim), c_int(window_kind),
          c_int(window_size), c_float(scale), _p(score_bias),
          c_int(0 if score_bias is None else score_bias.shape[1]), _stream())


_dec_scratch = {}


def attention_decode_supported(n_heads, n_kv_heads, head_dim, page_size) -> bool:
    return bool(load().cpi_attention_decode_supported(c_int(n_heads), c_int(n_kv_heads), c_int(head_dim),
                                                      c_int(page_size)))


def attention_decode(q, out, k_cache, v_cache, page_table, page_size, token_seq, token_pos, seq_slot, *,
                     n_heads, n_kv_heads, head_dim, window_kind, window_size, scale, n_splits):
    """bfloat16 attention of independent tokens against the paged cache, keys split over `n_splits` blocks."""
    _need_cuda(q, out, k_cache, v_cache, page_table, token_seq, token_pos, seq_slot)
    assert q.is_contiguous() and out.is_contiguous() and q.dtype == out.dtype == k_cache.dtype == torch.bfloat16
    T = q.shape[0]
    po = pml = None
    if n_splits > 1:
        idx = q.device.index or 0
        need = T * n_heads * n_splits * (head_dim + 2)
        buf = _dec_scratch.get(idx)
        if buf is None or buf.numel() < need:
            global scratch_generation
            buf = torch.empty(max(need, 1 << 20), dtype=torch.float32, device=q.device)
            _dec_scratch[idx] = buf
            scratch_generation += 1
        po, pml = buf, buf[T * n_heads * n_splits * head_dim:]
    assert k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.shape == v_cache.shape
    _call("cpi_attention_decode", _p(q), _p(out), _p(k_cache), _p(v_cache), c_long(k_cache.shape[0]), _p(page_table),
          c_int(page_table.shape[1]), c_int(page_size), _p(token_seq), _p(token_pos), _p(seq_slot), c_int(T),
          c_int(n_heads), c_int(n_kv_heads), c_int(head_dim), c_int(window_kind), c_int(window_size), c_float(scale),
          c_int(n_splits), _p(po), _p(pml), _p(tc_error_flag(q.device)), _stream())


def attention_decode_blocks_per_sm(head_dim: int) -> int:
    """Blocks of the decode attention kernel that share an SM."""
    return int(load().cpi_attention_decode_blocks_per_sm(c_int(head_dim)))


def attention_prefill_supported(n_heads, n_kv_heads, head_dim, page_size) -> bool:
    return bool(load().cpi_attention_prefill_supported(c_int(n_heads), c_int(n_kv_heads), c_int(head_dim),
                                                       c_int(page_size)))


def attention_prefill(q, out, k_cache, v_cache, page_table, page_size, token_seq, token_pos, seq_slot, tile_tok0,
                      tile_rows, *, n_heads, n_kv_heads, head_dim, window_kind, window_size, scale):
    """bfloat16 attention of query tiles (<= PREFILL_TILE_ROWS consecutive tokens of one sequence each) on tcgen05."""
    _need_cuda(q, out, k_cache, v_cache, page_table, token_seq, token_pos, seq_slot, tile_tok0, tile_rows)
    assert q.is_contiguous() and out.is_contiguous() and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert q.dtype == out.dtype == k_cache.dtype == torch.bfloat16
    _call("cpi_attention_prefill", _p(q), _p(out), _p(k_cache), _p(v_cache), c_long(k_cache.shape[0]), _p(page_table),
          c_int(page_table.shape[1]), c_int(page_size), _p(token_seq), _p(token_pos), _p(seq_slot), _p(tile_tok0),
          _p(tile_rows), c_int(tile_tok0.numel()), c_int(q.shape[0]), c_int(n_heads), c_int(n_kv_heads),
          c_int(head_dim), c_int(window_kind), c_int(window_size), c_float(scale), _p(tc_error_flag(q.device)),
          _stream())


def router_topk(h, w, topk_idx, topk_gate, *, top_k, sigmoid_gate, logits_out=None):
    _need_cuda(h, w, topk_idx, topk_gate, logits_out)
    _rowmajor(h, "router h")
    T, H = h.shape
    E = w.shape[0]
    assert w.is_contiguous() and w.shape[1] == H
    assert topk_idx.dtype == torch.int32 and topk_gate.dtype == torch.float32
    if logits_out is None:
        raise KernelError("router_topk: a float32 [tokens, experts] logits buffer is required")
    assert logits_out.dtype == torch.float32 and logits_out.is_contiguous() and logits_out.numel() >= T * E
    for t0 in range(0, T, 65535):            # the token axis is the grid's y dimension
        n = min(65535, T - t0)
        _call("cpi_router_topk", _p(h[t0:t0 + n]), c_int(dtype_code(h.dtype)), c_long(h.stride(0)), _p(w),
              c_int(dtype_code(w.dtype)), _p(logits_out[t0:t0 + n]), _p(topk_idx[t0:t0 + n]), _p(topk_gate[t0:t0 + n]),
              c_int(n), c_int(H), c_int(E), c_int(top_k), c_int(int(sigmoid_gate)), _stream())


def moe_route(h, w, topk_idx, topk_gate, logits, group_offsets, row_token, row_scale, row_of_slot, *, top_k,
              sigmoid_gate, sorted_h=None) -> bool:
    """Router logits, the top-k choice and the per-expert row lists of a step; returns whether
    `sorted_h` (the activation rows in expert order) was filled too.  A step with few tokens takes two
    launches (logits, then one kernel for the rest), a larger one the separate kernels; the results
    are the same."""
    _need_cuda(h, w, topk_idx, topk_gate, logits, group_offsets, row_token, row_scale, row_of_slot, sorted_h)
    _rowmajor(h, "router h")
    T, H = h.shape
    E = w.shape[0]
    if T <= 65535 and T * top_k <= 256 and T * E <= 4096:
        assert w.is_contiguous() and w.shape[1] == H and logits.dtype == torch.float32 and logits.is_contiguous()
        _call("cpi_router_topk", _p(h), c_int(dtype_code(h.dtype)), c_long(h.stride(0)), _p(w),
              c_int(dtype_code(w.dtype)), _p(logits), None, None, c_int(T), c_int(H), c_int(E), c_int(top_k),
              c_int(int(sigmoid_gate)), _stream())
        rc = load().cpi_moe_route_small(_p(logits), c_int(T), c_int(E), c_int(top_k), c_int(int(sigmoid_gate)),
                                        _p(topk_idx), _p(topk_gate), _p(group_offsets), _p(row_token), _p(row_scale),
                                        _p(row_of_slot), _p(h), c_long(h.stride(0) * h.element_size()), _p(sorted_h),
                                        c_int(H * h.element_size()), _stream())
        if rc == 0:
            global launch_count
            launch_count += 1
            return sorted_h is not None
        if rc > 0:
            raise KernelError(load().cpi_last_error().decode())
        # too large or unaligned for the one-launch kernel: select here, lists below
        _call("cpi_router_select", _p(logits), _p(topk_idx), _p(topk_gate), c_int(T), c_int(E), c_int(top_k),
              c_int(int(sigmoid_gate)), _stream())
    else:
        router_topk(h, w, topk_idx, topk_gate, top_k=top_k, sigmoid_gate=sigmoid_gate, logits_out=logits)
    moe_lists(topk_idx, topk_gate, group_offsets, row_token, row_scale, row_of_slot, n_tokens=T, top_k=top_k,
              n_experts=E)
    return False


def moe_lists(topk_idx, topk_gate, group_offsets, row_token, row_scale, row_of_slot, *, n_tokens, top_k,
              n_experts):
    _need_cuda(topk_idx, topk_gate, group_offsets, row_token, row_scale, row_of_slot)
    _call("cpi_moe_lists", _p(topk_idx), _p(topk_gate), _p(group_offsets), _p(row_token), _p(row_scale),
          _p(row_of_slot), c_int(n_tokens), c_int(top_k), c_int(n_experts), _stream())


def moe_combine(residual, y, row_of_slot, *, top_k):
    """residual[t] += y[row_of_slot[t, 0]] + ... + y[row_of_slot[t, top_k - 1]]."""
    _need_cuda(residual, y, row_of_slot)
    T, H = residual.shape
    assert residual.dtype == torch.float32 and residual.is_contiguous() and y.is_contiguous()
    _call("cpi_moe_combine", _p(residual), _p(y), c_int(dtype_code(y.dtype)), _p(row_of_slot), c_int(T),
          c_int(top_k), c_int(H), _stream())


def swiglu(gate_up, out):
    _need_cuda(gate_up, out)
    T, I = out.shape
    assert gate_up.shape == (T, 2 * I) and gate_up.is_contiguous() and out.is_contiguous()
    _call("cpi_swiglu", _p(gate_up), _p(out), c_int(dtype_code(out.dtype)), c_int(T), c_int(I), _stream())


def argmax(logits, out):
    _need_cuda(logits, out)
    _rowmajor(logits, "argmax logits")
    assert logits.dtype == torch.float32 and out.dtype == torch.int32
    R, V = logits.shape
    _call("cpi_argmax", _p(logits), c_long(logits.stride(0)), c_int(R), c_int(V), _p(out), _stream())


def sample(logits, work, temperature, top_k, top_p, uniform, out):
    _need_cuda(logits, work, temperature, top_k, top_p, uniform, out)
    _rowmajor(logits, "sample logits")
    R, V = logits.shape
    assert logits.dtype == torch.float32 and work.dtype == torch.float32 and work.numel() >= R * V
    assert temperature.dtype == torch.float32 and top_k.dtype == torch.int32 and top_p.dtype == torch.float32
    assert uniform.dtype == torch.float32 and out.dtype == torch.int32
    _call("cpi_sample", _p(logits), c_long(logits.stride(0)), _p(work), c_int(R), c_int(V), _p(temperature),
          _p(top_k), _p(top_p), _p(uniform), _p(out), _stream())


def repetition_penalty(logits, ids, id_offsets, penalty):
    _need_cuda(logits, ids, id_offsets, penalty)
    R, V = logits.shape
    _call("cpi_repetition_penalty", _p(logits), c_long(logits.stride(0)), c_int(R), c_int(V), _p(ids),
          _p(id_offsets), _p(penalty), _stream())


def ban_tokens(logits, ids, id_offsets):
    _need_cuda(logits, ids, id_offsets)
    R, V = logits.shape
    _call("cpi_ban_tokens", _p(logits), c_long(logits.stride(0)), c_int(R), c_int(V), _p(ids), _p(id_offsets),
          _stream())
