"""Cache bookkeeping on the host: slots and pages are never lost, held twice or freed twice."""
import random

import pytest
import torch

from cpi_b200.cache import CacheError, CacheFull, CacheManager, KVRequirement, PagePool, StateRequirement

FULL = KVRequirement(2, 16, "full", 0)
CHUNK = KVRequirement(2, 16, "chunk", 32)
SLIDE = KVRequirement(2, 16, "sliding", 20)


def manager(max_tokens=256, page=16, **kw):
    return CacheManager({0: CHUNK, 1: CHUNK, 2: FULL, 3: SLIDE}, {3: [StateRequirement("acc", (4,))]},
                        max_tokens=max_tokens, page_size=page, dtype=torch.float32, device="cpu", **kw)


def test_page_pool_rejects_double_free():
    p = PagePool(3)
    a, b, c = p.take(), p.take(), p.take()
    assert sorted([a, b, c]) == [0, 1, 2] and p.free_count == 0
    with pytest.raises(CacheFull):
        p.take()
    p.give_back(b)
    with pytest.raises(CacheError):
        p.give_back(b)
    with pytest.raises(CacheError):
        p.give_back(7)
    assert p.take() == b


def test_groups_by_requirement_have_storage_of_their_own():
    m = manager()
    assert sorted(len(g.entries) for g in m.groups) == [1, 1, 2]
    g = m.group_of_entry[0]
    assert g is m.group_of_entry[1] and g is not m.group_of_entry[2]
    assert g.k.shape == (2, 16, 2, 16, 16)
    k0, _, table, page = m.kv_view(0)
    k1, _, _, _ = m.kv_view(1)
    assert k0.data_ptr() != k1.data_ptr() and page == 16 and table.shape == (16, 16)


def test_slots_are_reused_and_double_release_is_an_error():
    m = manager()
    s = [m.acquire() for _ in range(m.max_slots)]
    assert len(set(s)) == m.max_slots
    with pytest.raises(CacheFull):
        m.acquire()
    m.release(s[3])
    with pytest.raises(CacheError):
        m.release(s[3])
    assert m.acquire() == s[3]
    m.check_consistency()


def test_pages_follow_lengths_and_windows():
    m = manager()
    s = m.acquire()
    assert m.prepare_step([s], [40]) == [0]
    m.commit_step([s], [40])
    full, chunk, slide = m.group_of_entry[2], m.group_of_entry[0], m.group_of_entry[3]
    assert sorted(full.blocks[s]) == [0, 1, 2] and sorted(chunk.blocks[s]) == [0, 1, 2]
    for _ in range(30):
        m.prepare_step([s], [1]); m.commit_step([s], [1])
    # length 70: the next position 69 -> chunk [64, 96) needs blocks from 4; sliding needs positions >= 50
    assert sorted(full.blocks[s]) == [0, 1, 2, 3, 4]
    assert sorted(chunk.blocks[s]) == [4]
    assert sorted(slide.blocks[s]) == [3, 4]
    assert full.table_host[s, 4] == full.blocks[s][4]
    m.check_consistency()
    m.release(s)
    assert all(g.pool.free_count == g.pool.n_pages for g in m.groups)


def test_state_is_zeroed_on_acquire():
    m = manager()
    s = m.acquire()
    m.state_view(3, "acc")[s] += 5
    m.release(s)
    assert m.acquire() == s and float(m.state_view(3, "acc")[s].abs().sum()) == 0


def test_capacity_errors():
    m = manager(max_tokens=64, page=16, max_seq_len=48)
    a, b = m.acquire(), m.acquire()
    with pytest.raises(CacheError, match="longest"):
        m.prepare_step([a], [49])
    m.prepare_step([a], [48]); m.commit_step([a], [48])
    with pytest.raises(CacheFull, match="full"):
        m.prepare_step([b], [17])
    with pytest.raises(CacheError, match="twice"):
        m.prepare_step([a, a], [1, 1])
    m.release(a); m.release(b)
    with pytest.raises(CacheError, match="not live"):
        m.prepare_step([a], [1])
    m.check_consistency()


def test_random_workload_never_loses_a_page():
    rng = random.Random(0)
    m = manager(max_tokens=512, page=16)
    live = {}
    for it in range(400):
        if live and rng.random() < 0.25:
            s = rng.choice(list(live))
            m.release(s); del live[s]
        elif len(live) < 6 and rng.random() < 0.4:
            s = m.acquire()
            n = rng.randint(1, 60)
            try:
                m.prepare_step([s], [n]); m.commit_step([s], [n]); live[s] = n
            except CacheFull:
                m.release(s)
        elif live:
            slots = list(live)
            try:
                m.prepare_step(slots, [1] * len(slots)); m.commit_step(slots, [1] * len(slots))
                for s in slots:
                    live[s] += 1
            except CacheFull:
                s = slots[0]
                m.release(s); del live[s]
        m.check_consistency()
        for s, n in live.items():
            assert m.lengths[s] == n
            full = m.group_of_entry[2]
            assert sorted(full.blocks[s]) == list(range(-(-n // 16)))
    for s in list(live):
        m.release(s)
    m.check_consistency()
    assert all(g.pool.free_count == g.pool.n_pages for g in m.groups) and m.free_slots == m.max_slots


def test_a_step_that_does_not_fit_takes_nothing():
    """A step either gets the pages of all its sequences or leaves the cache as it was; and a step that will run
    as several pieces is refused before its first piece."""
    m = CacheManager({0: KVRequirement(2, 16), 1: KVRequirement(2, 16, "chunk", 32)}, {}, max_tokens=64, max_seqs=3,
                     page_size=16, device="cpu", dtype=__import__("torch").float32)
    a, b, c = m.acquire(), m.acquire(), m.acquire()
    m.prepare_step([a], [20]); m.commit_step([a], [20])            # two of four pages
    held = [g.pages_held() for g in m.groups]
    with pytest.raises(CacheFull):
        m.prepare_step([b, c], [16, 17])                          # b would fit, c would not
    assert [g.pages_held() for g in m.groups] == held
    assert m.lengths[b] == 0 and m.lengths[c] == 0
    m.check_consistency()
    with pytest.raises(CacheFull):
        m.check_room([([b], [16]), ([c], [10]), ([c], [8])])      # the third piece would need a fifth page
    assert [g.pages_held() for g in m.groups] == held
    m.check_room([([b], [16]), ([c], [10]), ([c], [6])])
    with pytest.raises(CacheError, match="longest"):
        m.check_room([([b], [40]), ([b], [40])])
    # a windowed group gives pages back between pieces: 80 positions of one sequence pass through the chunk
    # group's four pages, but not through the group that keeps everything
    w = CacheManager({0: KVRequirement(2, 16, "chunk", 32)}, {}, max_tokens=64, max_seqs=1, max_seq_len=160,
                     page_size=16, device="cpu", dtype=__import__("torch").float32)
    s = w.acquire()
    w.check_room([([s], [40]), ([s], [40]), ([s], [40])])
    with pytest.raises(CacheFull):
        w.check_room([([s], [120])])                              # one piece holds all its pages at once


def test_a_group_stores_the_streams_its_requirement_names():
    """Keys and values of equal shape are only the default: a mixer may keep one compressed vector per position,
    or streams of unequal widths; its group stores exactly those, paged like any other."""
    import torch
    latent = KVRequirement(0, 0, streams=(("latent", 1, 24), ("rope_k", 1, 8)))
    m = CacheManager({0: KVRequirement(2, 16), 1: latent, 2: latent}, {}, max_tokens=64, max_seqs=2, page_size=16,
                     device="cpu", dtype=torch.float32)
    assert len(m.groups) == 2
    lat, table, page = m.stream_view(2, "latent")
    assert lat.shape == (4, 1, 16, 24) and page == 16 and m.stream_view(1, "rope_k")[0].shape == (4, 1, 16, 8)
    assert m.stream_view(1, "latent")[0].data_ptr() != lat.data_ptr()            # a layer of its own per run entry
    assert m.stream_view(0, "k")[0].shape == (4, 2, 16, 16) and m.kv_view(0)[0].shape == (4, 2, 16, 16)
    with pytest.raises(CacheError, match="latent"):
        m.kv_view(1)
    with pytest.raises(CacheError, match="'v'"):
        m.stream_view(1, "v")
    s = m.acquire()
    m.prepare_step([s], [20]); m.commit_step([s], [20])
    assert [g.pages_held() for g in m.groups] == [2, 2]
    m.release(s)
    m.check_consistency()
    with pytest.raises(CacheError, match="twice"):
        CacheManager({0: KVRequirement(0, 0, streams=(("a", 1, 4), ("a", 1, 4)))}, {}, max_tokens=16, page_size=16,
                     device="cpu", dtype=torch.float32)


def test_a_windowed_group_is_sized_for_its_window_and_one_step():
    """Told the most tokens a step brings, the cache gives a group with a window only the pages that a sequence can
    hold there at a time (the window and the step being added), not whole sequences; what the window has left behind
    is given back as a sequence grows, so a long sequence passes through."""
    import torch
    full, chunk = KVRequirement(2, 16), KVRequirement(2, 16, "chunk", 64)
    m = CacheManager({0: full, 1: chunk}, {}, max_tokens=8192, max_seqs=2, max_seq_len=4096, page_size=16,
                     device="cpu", dtype=torch.float32, max_step_tokens=32)
    g_full, g_chunk = (g for g in m.groups)
    assert g_full.pool.n_pages == 512
    assert g_chunk.pool.n_pages == 2 * (-(-(63 + 32) // 16) + 1) == 14
    a, b = m.acquire(), m.acquire()
    for _ in range(59):                                       # 1,888 positions each, 32 at a time
        m.prepare_step([a, b], [32, 32]); m.commit_step([a, b], [32, 32])
        assert g_chunk.pages_held() <= 14
    m.check_consistency()
    assert g_full.pages_held() == 2 * 118
    with pytest.raises(CacheFull, match="chunk"):             # a step larger than it was told does not fit the window's group
        m.prepare_step([a], [200])
    assert g_full.pages_held() == 2 * 118 and m.lengths[a] == 1888
    # without the figure every group holds whole sequences, as before
    n = CacheManager({0: full, 1: chunk}, {}, max_tokens=4096, max_seqs=2, page_size=16, device="cpu", dtype=torch.float32)
    assert [g.pool.n_pages for g in n.groups] == [256, 256]
