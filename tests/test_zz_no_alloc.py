"""The allocation-free decode attention entry point, called through its exported C symbol.

Some programs that embed the kernel library cannot hand it a scratch buffer: they have no device
allocator of their own, or their process has already given all device memory away.  For them the
library exports `cpi_attention_decode_noalloc`, which keeps the partial results of the key splits in
an array inside the library.  This test calls that symbol with ctypes, twice in a row with different
inputs (the array keeps what the previous call left in it), and checks each output against the ordinary
entry point, which takes its scratch from the caller.  It also checks that a request larger than the
built-in array is refused.  The file name sorts last on purpose: a run that stops at the first failure
has then already run every other test.
"""
from ctypes import c_float, c_int, c_long, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _case(seed, lengths, NH=40, NKV=8, D=128, page=64):
    g = torch.Generator().manual_seed(seed)
    blocks = [-(-l // page) for l in lengths]
    n_pages = sum(blocks) + 2
    perm = torch.randperm(n_pages, generator=g).tolist()
    table = torch.zeros(len(lengths) + 1, max(blocks) + 1, dtype=torch.int32)
    it = iter(perm)
    for s, b in enumerate(blocks):
        for i in range(b):
            table[s + 1, i] = next(it)
    mk = lambda *shape: torch.randn(*shape, generator=g).bfloat16().to(DEV)
    T = len(lengths)
    return dict(q=mk(T, NH * D), k=mk(n_pages, NKV, page, D), v=mk(n_pages, NKV, page, D), table=table.to(DEV),
                token_seq=torch.arange(T, dtype=torch.int32, device=DEV),
                token_pos=torch.tensor([l - 1 for l in lengths], dtype=torch.int32, device=DEV),
                seq_slot=torch.arange(1, T + 1, dtype=torch.int32, device=DEV), NH=NH, NKV=NKV, D=D, page=page)


def _call_noalloc(lib, c, out, n_splits, window=(0, 0)):
    fn = lib.cpi_attention_decode_noalloc
    fn.restype = c_int
    p = lambda t: c_void_p(t.data_ptr())
    return fn(p(c["q"]), p(out), p(c["k"]), p(c["v"]), c_long(c["k"].shape[0]), p(c["table"]),
              c_int(c["table"].shape[1]), c_int(c["page"]),
              p(c["token_seq"]), p(c["token_pos"]), p(c["seq_slot"]), c_int(c["q"].shape[0]), c_int(c["NH"]),
              c_int(c["NKV"]), c_int(c["D"]), c_int(window[0]), c_int(window[1]), c_float(c["D"] ** -0.5),
              c_int(n_splits), c_void_p(torch.cuda.current_stream().cuda_stream))


def test_noalloc_entry_point_matches_the_allocating_one_twice_in_a_row():
    from cpi_b200.csrc import lib as K
    lib = K.load()
    lib.cpi_attention_decode_noalloc_capacity.restype = c_long
    cap = lib.cpi_attention_decode_noalloc_capacity()
    assert cap == 2 << 20
    for seed, lengths, splits, window in [(1, [900, 64, 333, 2000], 7, (0, 0)), (2, [65, 1500, 7], 5, (1, 256))]:
        c = _case(seed, lengths)
        want = torch.empty_like(c["q"])
        K.attention_decode(c["q"], want, c["k"], c["v"], c["table"], c["page"], c["token_seq"], c["token_pos"],
                           c["seq_slot"], n_heads=c["NH"], n_kv_heads=c["NKV"], head_dim=c["D"],
                           window_kind=window[0], window_size=window[1], scale=c["D"] ** -0.5, n_splits=splits)
        got = torch.full_like(c["q"], float("nan"))
        rc = _call_noalloc(lib, c, got, splits, window)
        assert rc == 0, lib.cpi_last_error().decode()
        torch.cuda.synchronize()
        scale = float(want.float().abs().max())
        assert float((got.float() - want.float()).abs().max()) <= 1.5e-2 * max(1.0, scale)
        assert torch.equal(got, want)          # same kernels, same order of sums: the bits agree too


def test_noalloc_entry_point_refuses_more_than_its_array_holds():
    from cpi_b200.csrc import lib as K
    lib = K.load()
    c = _case(3, [100] * 64)
    out = torch.empty_like(c["q"])
    rc = _call_noalloc(lib, c, out, 64)                      # 64 * 40 * 64 * 130 floats > 2 Mi
    assert rc != 0
    msg = lib.cpi_last_error().decode()
    assert "scratch" in msg and "2097152" in msg
    assert _call_noalloc(lib, c, out, 1) == 0                # one split needs no scratch at all
    torch.cuda.synchronize()
