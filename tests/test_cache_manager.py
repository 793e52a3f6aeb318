"""The cache manager's ledger (no GPU): no page is lost, held twice or freed twice,
under random orders of requests; windows give pages back; prepare is all-or-nothing.
The reference tests its page table the same way, against a set oracle with seeded
random operations (tests/gpu_page_table_tests.cpp:226-285)."""
import random

import pytest
import torch

from mini_llm_runtime_b200.cache.manager import CacheError, CacheManager, GroupSpec, OutOfPages, OutOfSlots


def held_pages(cm, group, slot):
    return [p for p in cm.table_row(group, slot) if p >= 0]


def check_conservation(cm, live):
    """Every page id of every group is either free or held by exactly one request."""
    for g, spec in enumerate(cm.groups):
        held = []
        for slot in live:
            held += held_pages(cm, g, slot)
        assert len(held) == len(set(held)), f"group {g}: a page is held twice"
        assert all(0 <= p < spec.num_pages for p in held)
        assert len(held) + cm.free_pages(g) == spec.num_pages, f"group {g}: a page was lost or freed twice"


def test_growth_pages_and_reuse_order():
    cm = CacheManager([GroupSpec(None, 8)], page_size=4, max_requests=2, max_model_len=32)
    a = cm.open()
    cm.prepare([a], [5]); cm.commit()
    assert cm.length(a) == 5 and held_pages(cm, 0, a) == [0, 1] and cm.free_pages(0) == 6
    cm.prepare([a], [3]); cm.commit()           # 8 tokens: still two pages
    assert held_pages(cm, 0, a) == [0, 1]
    cm.prepare([a], [1]); cm.commit()
    assert held_pages(cm, 0, a) == [0, 1, 2]
    b = cm.open()
    cm.prepare([b], [4]); cm.commit()
    assert held_pages(cm, 0, b) == [3]
    cm.close(a)
    assert cm.free_pages(0) == 7
    c = cm.open()
    cm.prepare([c], [9]); cm.commit()
    # Freed pages are handed out again, last freed first.
    assert held_pages(cm, 0, c) == [2, 1, 0]
    check_conservation(cm, [b, c])


def test_prepare_is_all_or_nothing_and_discard_restores():
    cm = CacheManager([GroupSpec(None, 4)], page_size=4, max_requests=3, max_model_len=64)
    a, b = cm.open(), cm.open()
    cm.prepare([a], [8]); cm.commit()
    with pytest.raises(OutOfPages, match="needs 3 pages, 2 are free"):
        cm.prepare([a, b], [4, 8])
    assert cm.free_pages(0) == 2 and cm.length(a) == 8 and held_pages(cm, 0, b) == []
    cm.prepare([a, b], [1, 4])
    assert cm.free_pages(0) == 0
    cm.discard()
    assert cm.free_pages(0) == 2 and cm.length(a) == 8 and cm.length(b) == 0 and held_pages(cm, 0, b) == []
    cm.prepare([b], [4]); cm.commit()
    assert held_pages(cm, 0, b) == [2]          # the same page the discarded plan had taken first
    check_conservation(cm, [a, b])


def test_phase_and_argument_errors():
    cm = CacheManager([GroupSpec(None, 4)], page_size=4, max_requests=1, max_model_len=8)
    a = cm.open()
    with pytest.raises(OutOfSlots):
        cm.open()
    with pytest.raises(CacheError, match="without a prepared step"):
        cm.commit()
    with pytest.raises(CacheError, match="twice"):
        cm.prepare([a, a], [1, 1])
    with pytest.raises(CacheError, match="not open"):
        cm.prepare([3], [1])
    with pytest.raises(CacheError, match="maximum length"):
        cm.prepare([a], [9])
    cm.prepare([a], [2])
    with pytest.raises(CacheError, match="already prepared"):
        cm.prepare([a], [1])
    with pytest.raises(CacheError, match="while a step is prepared"):
        cm.close(a)
    cm.commit()
    cm.close(a)
    with pytest.raises(CacheError, match="not open"):
        cm.close(a)
    assert cm.free_pages(0) == 4 and cm.free_slots() == 1


def test_window_group_gives_pages_back_as_the_window_moves():
    # Group 0 keeps everything, group 1 the last 6 keys; pages of 4 tokens.
    cm = CacheManager([GroupSpec(None, 16), GroupSpec(6, 16)], page_size=4, max_requests=2, max_model_len=64)
    a = cm.open()
    cm.prepare([a], [10]); cm.commit()
    # The next query is at position 10 and reads keys 5..10: block 0 (keys 0..3) is gone.
    assert cm.table_row(1, a)[:3] == [-1, 1, 2] and len(held_pages(cm, 0, a)) == 3
    for _ in range(30):
        cm.prepare([a], [1]); cm.commit()
        n = cm.length(a)
        row = cm.table_row(1, a)
        lowest_block = max(0, n - 6 + 1) // 4
        assert all(p == -1 for p in row[:lowest_block])
        assert all(p >= 0 for p in row[lowest_block:(n + 3) // 4])
        assert len(held_pages(cm, 1, a)) <= cm.peak_pages(1, 64, 1)
        check_conservation(cm, [a])
    assert len(held_pages(cm, 0, a)) == 10
    cm.close(a)
    assert cm.free_pages(0) == 16 and cm.free_pages(1) == 16


def test_peak_pages_bounds_what_a_request_holds():
    for window, page, chunk in [(6, 4, 1), (6, 4, 5), (40, 16, 16), (17, 8, 3), (5, 4, 64)]:
        cm = CacheManager([GroupSpec(window, 64)], page_size=page, max_requests=1, max_model_len=256)
        a = cm.open()
        peak = 0
        bound = cm.peak_pages(0, 200, chunk)
        while cm.length(a) < 200:
            cm.prepare([a], [min(chunk, 200 - cm.length(a))])
            peak = max(peak, len(held_pages(cm, 0, a)))
            cm.commit()
        assert peak <= bound <= peak + 1, (window, page, chunk, peak, bound)
    cm = CacheManager([GroupSpec(None, 64)], page_size=16, max_requests=1, max_model_len=256)
    assert cm.peak_pages(0, 100, 7) == 7


def test_fill_table_writes_rows_in_request_order():
    cm = CacheManager([GroupSpec(None, 8)], page_size=2, max_requests=3, max_model_len=8)
    a, b = cm.open(), cm.open()
    cm.prepare([a, b], [3, 5]); cm.commit()
    out = torch.full((2, 6), 77, dtype=torch.int32)
    cm.fill_table(0, [b, a], out, columns=3)
    assert out[:, 3:].eq(77).all()
    assert out[0, :3].tolist() == held_pages(cm, 0, b) and out[1, :2].tolist() == held_pages(cm, 0, a) and out[1, 2] == -1
    with pytest.raises(CacheError):
        cm.fill_table(0, [a], torch.zeros((1, 2), dtype=torch.int64))


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_of_requests(seed):
    rng = random.Random(seed)
    page = rng.choice([1, 4, 16])
    groups = [GroupSpec(None, rng.randint(20, 60)), GroupSpec(rng.randint(3, 40), rng.randint(20, 60))]
    max_len = 96
    cm = CacheManager(groups, page_size=page, max_requests=5, max_model_len=max_len)
    lengths = {}                      # oracle: slot -> committed length
    for _ in range(3000):
        op = rng.random()
        if op < 0.15 and len(lengths) < 5:
            slot = cm.open()
            assert slot not in lengths
            lengths[slot] = 0
        elif op < 0.25 and lengths:
            slot = rng.choice(list(lengths))
            cm.close(slot)
            del lengths[slot]
        elif lengths:
            chosen = rng.sample(list(lengths), rng.randint(1, len(lengths)))
            chosen = [s for s in chosen if lengths[s] < max_len]
            if not chosen:
                continue
            counts = [rng.randint(1, min(20, max_len - lengths[s])) for s in chosen]
            before = [cm.free_pages(g) for g in range(2)]
            try:
                cm.prepare(chosen, counts)
            except OutOfPages:
                assert [cm.free_pages(g) for g in range(2)] == before
                check_conservation(cm, lengths)
                continue
            if rng.random() < 0.2:
                cm.discard()
                assert [cm.free_pages(g) for g in range(2)] == before
            else:
                # While the step runs every token of it has a page in every group.
                for s, c in zip(chosen, counts):
                    for g, spec in enumerate(groups):
                        row = cm.table_row(g, s)
                        lo = 0 if spec.window is None else max(0, lengths[s] - spec.window + 1)
                        for t in range(lo, lengths[s] + c):
                            assert row[t // page] >= 0, (g, s, t)
                cm.commit()
                for s, c in zip(chosen, counts):
                    lengths[s] += c
        for s, n in lengths.items():
            assert cm.length(s) == n
        check_conservation(cm, lengths)
    for s in list(lengths):
        cm.close(s)
    assert [cm.free_pages(g) for g in range(2)] == [g.num_pages for g in groups] and cm.free_slots() == 5
