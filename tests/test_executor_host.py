"""The native step function's host logic, without a GPU: `mlr_model_create(..., host_mode=1)`
makes the "device" buffers plain host memory and calls nothing of CUDA, and the program's ops
point at a recording function of the host library instead of kernels.  So what a step hands its
launches (row counts, metadata sections, block tables, plan fields), what it does to the page
ledger, and what a launch that fails in the middle of a step leaves behind can all be checked
here, on any machine (the reference tests its runtime's failure paths the same way, by making
wrapped calls fail on the host: tests/cuda_runtime_tests.cpp:15-49).
"""
import ctypes

import numpy as np
import pytest

from mini_llm_runtime_b200.cache.manager import CacheManager, GroupSpec
from mini_llm_runtime_b200.engine import executor as X
from mini_llm_runtime_b200.engine.builder import (K_FLOAT, K_IMM, K_META, K_PLAN, K_ROWS, K_SEGMENTS, K_TABLE, K_TABLE_STRIDE,
                                                  K_WANT, NEED_PLAN_FIELD, NEED_WANTED, OpRecord, PLAN_FIELDS)

PAGE = 4


def address_of(function) -> int:
    return ctypes.cast(function, ctypes.c_void_p).value


class Host:
    """A model in host mode over a real cache manager, with numpy arrays as its room."""

    def __init__(self, pages=16, window=None, max_requests=3, max_len=64):
        self.lib = X.library()
        self.cache = CacheManager([GroupSpec(window, pages)], PAGE, max_requests, max_len)
        self.handle = self.lib.mlr_model_create(self.cache._handle, 1, PAGE, max_len, 100, 148, 1)
        assert self.handle
        self.meta = np.zeros(4096, dtype=np.int32)
        self.pinned = [np.zeros(4096, dtype=np.int32) for _ in range(4)]
        self.logits = np.zeros((8, 100), dtype=np.float32)
        self.scratch = np.zeros(1 << 16, dtype=np.float32)
        self.counters = np.zeros(256, dtype=np.int32)
        pinned = (ctypes.c_void_p * 4)(*[p.ctypes.data for p in self.pinned])
        assert self.lib.mlr_model_set_room(self.handle, self.meta.ctypes.data, self.meta.size, pinned, 4096, self.logits.ctypes.data,
                                           8, 32, self.scratch.ctypes.data, self.scratch.size, self.counters.ctypes.data, 256) == 0
        self.plan = self.lib.mlr_model_add_plan(self.handle, (ctypes.c_int32 * 6)(4, 2, 0, 1, 64, 1))
        self.lib.mlr_test_recorded.argtypes = [ctypes.c_void_p, ctypes.c_longlong]
        self.lib.mlr_test_recorded.restype = ctypes.c_longlong

    def op(self, args, need=0, need_field=0):
        record = OpRecord()
        record.fn = address_of(self.lib.mlr_test_record)
        record.error_text = address_of(self.lib.mlr_test_record_error)
        record.n_args = len(args)
        record.need, record.need_plan, record.need_field = need, self.plan, need_field
        for k, (kind, aux, value) in enumerate(args):
            record.args[k].kind, record.args[k].aux = kind, aux
            if kind == K_FLOAT:
                record.args[k].f = value
            else:
                record.args[k].i = value
        return record

    def program(self, ops, lo=1, hi=32, want_lo=0, want_hi=8):
        array = (OpRecord * len(ops))(*ops)
        assert self.lib.mlr_model_add_program(self.handle, lo, hi, want_lo, want_hi, array, len(ops)) == 0, self.error()

    def error(self):
        return self.lib.mlr_exec_error().decode()

    def step(self, entries):
        """entries: (slot, tokens, want places)."""
        ints = lambda values: (ctypes.c_int32 * max(1, len(values)))(*values)
        tokens = np.asarray([t for _, ts, _ in entries for t in ts], dtype=np.int32)
        offsets, places = [0], []
        for _, _, want in entries:
            places += want
            offsets.append(len(places))
        info = X.StepInfo()
        code = self.lib.mlr_model_step(self.handle, len(entries), ints([s for s, _, _ in entries]), ints([len(t) for _, t, _ in entries]),
                                       tokens.ctypes.data, ints(offsets), ints(places), None, None, ctypes.byref(info))
        return code, info

    def recorded(self):
        out = (ctypes.c_int64 * 4096)()
        n = self.lib.mlr_test_recorded(out, 4096)
        values = list(out[:n])
        return [values[i:i + 9] for i in range(0, len(values), 9)]

    def ledger(self, slots):
        return self.cache.free_pages(0), self.cache.free_slots(), [self.cache.length(s) for s in slots]


def section(host, address, count):
    offset = (address - host.meta.ctypes.data) // 4
    return host.meta[offset:offset + count].tolist()


def test_a_step_hands_its_launches_what_the_step_knows():
    host = Host()
    a, b = host.cache.open(), host.cache.open()
    host.program([
        host.op([(K_ROWS, 0, 0), (K_WANT, 0, 0), (K_SEGMENTS, 0, 0), (K_META, 0, 0), (K_META, 1, 0), (K_META, 2, 0), (K_META, 3, 0),
                 (K_META, 5, 0), (K_FLOAT, 0, 0.25)]),
        host.op([(K_IMM, 0, 77), (K_TABLE, 0, 0), (K_TABLE_STRIDE, 0, 0), (K_PLAN, host.plan, PLAN_FIELDS["n_items"]),
                 (K_PLAN, host.plan, PLAN_FIELDS["items"]), (K_PLAN, host.plan, PLAN_FIELDS["n_tiles"]),
                 (K_PLAN, host.plan, PLAN_FIELDS["chunk"]), (K_PLAN, host.plan, PLAN_FIELDS["max_splits"])]),
        host.op([(K_IMM, 0, 5)], need=NEED_WANTED),
        host.op([(K_IMM, 0, 6)], need=NEED_PLAN_FIELD, need_field=PLAN_FIELDS["n_wide"]),
    ])
    code, info = host.step([(a, [5, 6, 7, 8, 9, 10], [5]), (b, [11], [0])])
    assert code == X.STEP_OK, host.error()
    first, second, wanted = host.recorded()            # the op that needs wide tiles was skipped: the step has none
    rows, want, segments, ids, positions, segment_of_row, info_at, want_rows, scaled = first
    assert (rows, want, segments, scaled) == (7, 2, 2, 250) and (info.rows, info.want) == (7, 2)
    assert section(host, ids, 7) == [5, 6, 7, 8, 9, 10, 11]
    assert section(host, positions, 7) == [0, 1, 2, 3, 4, 5, 0]
    assert section(host, segment_of_row, 7) == [0] * 6 + [1]
    assert section(host, info_at, 8) == [0, 6, 0, a, 6, 1, 0, b]
    assert section(host, want_rows, 2) == [5, 6]
    assert second[0] == 77 and second[2] == 2 and wanted[0] == 5         # two blocks of four tokens per table row
    table = section(host, second[1], 4)
    assert table[:2] == host.cache.table_row(0, a)[:2] and table[2] == host.cache.table_row(0, b)[0] and table[3] == -1
    # The plan: the single token of b goes to the split-KV kernel (listed, since a is not with it), a's six rows are one 64-row tile.
    assert second[3] == 1 and section(host, second[4], 1) == [1] and second[5] == 1 and second[7] == 1
    assert host.ledger([a, b]) == (16 - 3, 1, [6, 1])            # published: lengths advanced, three pages held
    # The next step continues where the cache is.
    code, _ = host.step([(b, [12, 13], []), (a, [1], [0])])
    assert code == X.STEP_OK
    first = host.recorded()[0]
    assert section(host, first[4], 3) == [1, 2, 6] and host.ledger([a, b])[2] == [7, 3]


def test_refusals_before_device_work_change_nothing():
    host = Host(pages=3)
    a = host.cache.open()
    host.program([host.op([(K_ROWS, 0, 0)])])
    assert host.step([(a, [1, 2, 3], [])])[0] == X.STEP_OK
    before = host.ledger([a])
    code, _ = host.step([(a, [1] * 12, [])])                       # 15 tokens need 4 pages, the pool has 3
    assert code == X.STEP_NO_PAGES and "pages" in host.error()
    for entries, words in (([(a, [], [])], "no tokens"), ([(a, [1], []), (a, [2], [])], "twice"), ([(2, [1], [])], "not open"),
                           ([(a, [100], [0])], "vocabulary"), ([(a, [1, 2], [2])], "place 2"), ([(a, [1] * 62, [])], "limit")):
        code, _ = host.step(entries)
        assert code == X.STEP_REFUSED and words in host.error(), (entries, host.error())
    assert host.ledger([a]) == before
    assert host.step([(a, [1] * 4, [0, 1, 2, 3])])[0] == X.STEP_OK
    # A step the room cannot hold (here: no program serves it) is told what it needs, and has changed nothing.
    host.lib.mlr_model_clear_programs(host.handle)
    before = host.ledger([a])
    code, info = host.step([(a, [3], [0])])
    assert code == X.STEP_NEEDS_ROOM and info.need_rows == 1 and info.need_want == 1 and host.ledger([a]) == before
    host.program([host.op([(K_ROWS, 0, 0)])], lo=1, hi=4, want_lo=0, want_hi=0)
    assert host.step([(a, [3], [0])])[0] == X.STEP_NEEDS_ROOM          # one row is wanted; that program serves none
    assert host.step([(a, [3], [])])[0] == X.STEP_OK


@pytest.mark.parametrize("nth", [0, 1, 2])
def test_a_launch_that_fails_rolls_the_ledger_back_and_poisons(nth):
    host = Host()
    a, b = host.cache.open(), host.cache.open()
    host.program([host.op([(K_IMM, 0, 1)]), host.op([(K_IMM, 0, 2)]), host.op([(K_IMM, 0, 3)])])
    assert host.step([(a, [1, 2, 3, 4, 5], []), (b, [1], [])])[0] == X.STEP_OK
    host.recorded()
    before = host.ledger([a, b])
    host.lib.mlr_exec_fail_after.argtypes = [ctypes.c_longlong]
    host.lib.mlr_exec_fail_after(nth)
    try:
        code, _ = host.step([(a, [6, 7, 8, 9], [3]), (b, [2], [0])])
    finally:
        host.lib.mlr_exec_fail_after(-1)
    assert code == X.STEP_FAILED and "injected failure" in host.error()
    assert [r[0] for r in host.recorded()] == [1, 2, 3][:nth]          # the launches before the failing one did run
    assert host.ledger([a, b]) == before, "pages or lengths of the failed step were kept"
    assert host.lib.mlr_model_poisoned(host.handle) == 1
    code, _ = host.step([(b, [3], [])])
    assert code == X.STEP_POISONED and "poisoned" in host.error()
    host.cache.close(a)
    host.cache.close(b)
    assert host.cache.free_pages(0) == 16 and host.cache.free_slots() == 3


def test_an_entry_point_that_refuses_its_arguments_fails_the_step():
    host = Host()
    a = host.cache.open()
    host.program([host.op([(K_IMM, 0, 1)]), host.op([(K_IMM, 0, -7)]), host.op([(K_IMM, 0, 3)])])     # -7: the recorder returns non-zero
    before = host.ledger([a])
    code, _ = host.step([(a, [1, 2], [1])])
    assert code == X.STEP_FAILED and "told to fail" in host.error() and host.ledger([a]) == before
    assert [r[0] for r in host.recorded()] == [1, -7]


def test_the_table_hook_sees_each_step_s_rows():
    host = Host()
    a = host.cache.open()
    host.program([host.op([(K_TABLE, 0, 0)])])
    host.step([(a, [1] * 9, [])])
    host.recorded()
    seen = []

    def hook(group, n, columns, rows):
        seen.append((group, n, columns, [rows[i] for i in range(n * columns)]))
        rows[0], rows[1] = rows[1], rows[0]

    keep = X.TABLE_HOOK(hook)
    host.lib.mlr_model_set_table_hook(host.handle, keep)
    assert host.step([(a, [2], [])])[0] == X.STEP_OK
    owned = host.cache.table_row(0, a)[:3]
    assert seen == [(0, 1, 3, owned)]
    assert section(host, host.recorded()[0][0], 3) == [owned[1], owned[0], owned[2]]


def test_plan_fields_that_say_whether_decoded_tokens_have_the_step_to_themselves():
    """`n_items_alone` / `n_items_beside` / `n_prompt_tiles`: a launch that stands for two others when a step has only
    decoded tokens depends on the first, the two others on the rest."""
    host = Host()
    a, b = host.cache.open(), host.cache.open()
    fields = [(K_PLAN, host.plan, PLAN_FIELDS[name]) for name in ("n_items", "n_items_alone", "n_items_beside", "n_prompt_tiles")]
    host.program([host.op(fields),
                  host.op([(K_IMM, 0, 1)], need=NEED_PLAN_FIELD, need_field=PLAN_FIELDS["n_items_alone"]),
                  host.op([(K_IMM, 0, 2)], need=NEED_PLAN_FIELD, need_field=PLAN_FIELDS["n_items_beside"]),
                  host.op([(K_IMM, 0, 3)], need=NEED_PLAN_FIELD, need_field=PLAN_FIELDS["n_prompt_tiles"])])
    assert host.step([(a, [5, 6, 7, 8, 9, 10], []), (b, [11], [0])])[0] == X.STEP_OK       # a prompt portion beside a token
    recorded = host.recorded()
    assert recorded[0][:4] == [1, 0, 1, 1] and [r[0] for r in recorded[1:]] == [2, 3]
    assert host.step([(a, [1], [0]), (b, [2, 3], [1])])[0] == X.STEP_OK                    # tokens only
    recorded = host.recorded()
    assert recorded[0][:4] == [2, 2, 0, 0] and [r[0] for r in recorded[1:]] == [1]


def test_the_few_row_route_is_left_to_matrices_whose_units_fill_their_rounds():
    """`units_balance`: 16 rows of a matrix at a time, one block per SM.  256 or 384 units over 148 SMs fill 86 % of
    their rounds; 320 units (a width of 5120) fill 72 % and are routed to the products that cut K across the SMs."""
    from mini_llm_runtime_b200.engine.runtime import units_balance
    assert units_balance(4096, 148) == pytest.approx(256 / 296) and units_balance(6144, 148) == pytest.approx(384 / 444)
    assert units_balance(5120, 148) == pytest.approx(320 / 444) and units_balance(5120, 148) < 0.8 <= units_balance(4096, 148)
    assert units_balance(1024, 148) == 1.0 and units_balance(16 * 148, 148) == 1.0 and units_balance(16 * 149, 148) == pytest.approx(149 / 296)
    assert units_balance(151936, 148) > 0.98
