"""Python face of the native step executor (`csrc/host/executor.cpp`).

`NativeStepper` owns what the executor needs around a model whose parts all compile into
programs: the workspace the programs' buffers are cut from, the metadata, logits and scratch
buffers, one program per range of row counts (built on first use by asking the parts to
`emit` into a `ProgramBuilder`), and the call `mlr_model_step` that runs a step.  Buffers grow
to the largest step seen and are then reused: a step in the steady state allocates nothing
(`allocations` counts the growths, `bench.py` asserts that none happens in its timed steps).
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..csrc import build
from .builder import OpRecord, ProgramBuilder, SplitRows

STEP_OK, STEP_REFUSED, STEP_NO_PAGES, STEP_NEEDS_ROOM, STEP_FAILED, STEP_POISONED = range(6)
_PINNED = 4


class StepInfo(ctypes.Structure):
    _fields_ = [("rows", ctypes.c_int32), ("want", ctypes.c_int32), ("graphed", ctypes.c_int32), ("captured", ctypes.c_int32),
                ("h2d_bytes", ctypes.c_int64), ("launches", ctypes.c_int64), ("need_rows", ctypes.c_int64),
                ("need_want", ctypes.c_int64), ("need_meta_ints", ctypes.c_int64), ("need_scratch_floats", ctypes.c_int64),
                ("need_counters", ctypes.c_int64)]


TABLE_HOOK = ctypes.CFUNCTYPE(None, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_int32))


def library():
    lib = build.load("host")
    if not getattr(lib, "_mlr_exec_bound", False):
        c_int, c_ll, p = ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p
        ip = ctypes.POINTER(ctypes.c_int32)
        lib.mlr_exec_error.restype = ctypes.c_char_p
        lib.mlr_exec_launch_count.restype = c_ll
        lib.mlr_exec_reset_launch_count.restype = None
        lib.mlr_library_set_workspace.argtypes = [p, c_ll]
        lib.mlr_plan_attention.argtypes = [ip, c_int, ip, ip, c_int, c_int, ip, ctypes.POINTER(c_ll), ip, c_int, ctypes.POINTER(c_int)]
        lib.mlr_k_splits.argtypes = [c_int, c_int, c_int]
        lib.mlr_model_create.argtypes = [p, c_int, c_int, c_int, c_int, c_int, c_int]
        lib.mlr_model_create.restype = p
        lib.mlr_model_destroy.argtypes = [p]
        lib.mlr_model_destroy.restype = None
        lib.mlr_model_add_plan.argtypes = [p, ip]
        lib.mlr_model_set_room.argtypes = [p, p, c_ll, ctypes.POINTER(p), c_ll, p, c_ll, c_ll, p, c_ll, p, c_ll]
        lib.mlr_model_clear_programs.argtypes = [p]
        lib.mlr_model_clear_programs.restype = None
        lib.mlr_model_add_program.argtypes = [p, c_int, c_int, c_int, c_int, ctypes.POINTER(OpRecord), c_int]
        lib.mlr_model_has_program.argtypes = [p, c_int, c_int]
        lib.mlr_model_set_graphs.argtypes = [p, c_int, c_int, c_int, c_int]
        lib.mlr_model_set_graphs.restype = None
        lib.mlr_model_graph_count.argtypes = [p]
        lib.mlr_model_set_table_hook.argtypes = [p, TABLE_HOOK]
        lib.mlr_model_set_table_hook.restype = None
        lib.mlr_model_poisoned.argtypes = [p]
        lib.mlr_model_poison_reason.argtypes = [p]
        lib.mlr_model_poison_reason.restype = ctypes.c_char_p
        lib.mlr_model_poison.argtypes = [p, ctypes.c_char_p]
        lib.mlr_model_poison.restype = None
        lib.mlr_model_step.argtypes = [p, c_int, p, p, p, p, p, p, p, ctypes.POINTER(StepInfo)]
        lib._mlr_exec_bound = True
    return lib


def k_splits_for(rows: int, K: int, sms: int) -> int:
    """How many ranges to cut K into for a few-row product over a weight matrix of `rows` rows."""
    return library().mlr_k_splits(rows, K, sms)


def plan_attention(spec: Sequence[int], segments: Sequence[Tuple[int, int]], context_bound: int, sm_count: int) -> Dict[str, object]:
    """The attention launch plan of a step (see `plan_attention` in the executor): counts, split
    sizes and, under "lists", the int32 lists that `*_offset` index."""
    lib = library()
    n = len(segments)
    ints = lambda values: (ctypes.c_int32 * len(values))(*values)
    out = (ctypes.c_int32 * 9)()
    scratch = ctypes.c_longlong(0)
    capacity = 2 * sum(-(-c // 64) for _, c in segments) + n + 8
    extra = (ctypes.c_int32 * capacity)()
    used = ctypes.c_int(0)
    if lib.mlr_plan_attention(ints(list(spec)), n, ints([s for s, _ in segments]), ints([c for _, c in segments]), context_bound,
                              sm_count, out, ctypes.byref(scratch), extra, capacity, ctypes.byref(used)) != 0:
        raise RuntimeError(lib.mlr_exec_error().decode())
    names = ("n_items", "items_offset", "chunk", "max_splits", "n_tiles", "tiles_offset", "n_wide", "wide_offset", "counters")
    values = dict(zip(names, list(out)))
    values["scratch_floats"] = scratch.value
    values["lists"] = list(extra[:used.value])
    return values


class NativeStepper:
    def __init__(self, model):
        self.model = model
        self.lib = library()
        rt, cfg = model.rt, model.cache_config
        self.handle = self.lib.mlr_model_create(model.cache._handle, len(model.group_windows), cfg.page_size, cfg.max_model_len,
                                                model.plan.vocab_size, rt.sm_count, 0)
        if not self.handle:
            raise RuntimeError(self.lib.mlr_exec_error().decode())
        self.plans: List[tuple] = []
        self._plans_sent = 0
        self.capacity_rows = 0
        self.allocations = 0             # times a buffer had to grow
        self.programs = {}               # (rows lo, hi, wanted lo, hi) -> the entry points of the program, in order
        self.workspace = self.logits = self.scratch = self.counters = self.device_meta = None
        self.pinned: List[torch.Tensor] = []
        self._hook = None
        self.last_info = StepInfo()
        self.graph_launches = 0
        self._routing_version = rt.routing_version

    def __del__(self):
        handle, self.handle = getattr(self, "handle", None), None
        if handle:
            self.lib.mlr_model_destroy(handle)

    # ---- room
    def _send_room(self) -> None:
        ptr = lambda t: t.data_ptr() if t is not None else None
        pinned = (ctypes.c_void_p * _PINNED)(*[t.data_ptr() for t in self.pinned])
        self.lib.mlr_model_set_room(
            self.handle, ptr(self.device_meta), self.device_meta.numel(), pinned, self.pinned[0].numel(), ptr(self.logits),
            self.logits.shape[0] if self.logits is not None else 0, self.capacity_rows, ptr(self.scratch),
            self.scratch.numel() if self.scratch is not None else 0, ptr(self.counters), self.counters.numel())

    def _grow(self, info: StepInfo) -> None:
        device = self.model.rt.device
        vocab = self.model.plan.vocab_size
        changed = False
        if self.device_meta is None or info.need_meta_ints > self.device_meta.numel():
            # The executor copies from the pinned buffers itself, so the allocator does not know when a copy
            # out of an old buffer has finished: wait for the stream before the old buffers are let go.
            torch.cuda.current_stream(device).synchronize()
            size = max(1 << 16, 2 * info.need_meta_ints)
            self.device_meta = torch.empty(size, dtype=torch.int32, device=device)
            self.pinned = [torch.empty(size, dtype=torch.int32).pin_memory() for _ in range(_PINNED)]
            changed = True
        if self.logits is None or info.need_want > self.logits.shape[0]:
            rows = max(self.model.cache.max_requests, info.need_want + info.need_want // 2)
            self.logits = None
            self.logits = torch.empty((rows, vocab), dtype=torch.float32, device=device)
            self._clear_programs()       # buffers of the wanted rows were laid out for the old count
            changed = True
        if info.need_scratch_floats > (self.scratch.numel() if self.scratch is not None else 0):
            self.scratch = torch.empty(2 * info.need_scratch_floats, dtype=torch.float32, device=device)
            changed = True
        if self.counters is None or info.need_counters > self.counters.numel():
            self.counters = torch.zeros(max(1 << 14, 2 * info.need_counters), dtype=torch.int32, device=device)
            changed = True
        if info.need_rows > self.capacity_rows:
            self.capacity_rows = max(64, 1 << (int(info.need_rows) - 1).bit_length())
            self._clear_programs()
            changed = True
        if changed:
            self.allocations += 1
            self._send_room()
        if not self.lib.mlr_model_has_program(self.handle, int(info.need_rows), int(info.need_want)):
            self._build_program(int(info.need_rows), int(info.need_want))

    def _clear_programs(self) -> None:
        self.programs.clear()
        self.lib.mlr_model_clear_programs(self.handle)

    # ---- programs
    def _build_program(self, rows: int, want: int) -> None:
        """The program for steps of `rows` rows of which `want` are wanted: the widest ranges of both
        counts around them over which every routing decision of the parts comes out the same."""
        model = self.model
        lo, hi, want_lo, want_hi = 1, self.capacity_rows, 0, self.logits.shape[0]
        while True:
            try:
                base = self.workspace.data_ptr() if self.workspace is not None else 0
                builder = ProgramBuilder(model.rt, lo, hi, want_lo, want_hi, base, model.cache_config.page_size,
                                         model.status.data_ptr(), self.plans)
                builder.begin()
                model.emit_program(builder)
            except SplitRows as cut:
                if cut.wanted:
                    want_lo, want_hi = (cut.at, want_hi) if want >= cut.at else (want_lo, cut.at - 1)
                else:
                    lo, hi = (cut.at, hi) if rows >= cut.at else (lo, cut.at - 1)
                continue
            need = builder.workspace_bytes()
            if self.workspace is None or need > self.workspace.numel():
                # The workspace moves: programs built before point into the old one.
                self.workspace = None
                self._clear_programs()
                self.workspace = torch.empty(need + need // 8, dtype=torch.uint8, device=model.rt.device)
                self.allocations += 1
                continue
            break
        for spec in self.plans[self._plans_sent:]:
            self.lib.mlr_model_add_plan(self.handle, (ctypes.c_int32 * 6)(*spec))
        self._plans_sent = len(self.plans)
        ops = builder.finish()
        self.programs[(lo, hi, want_lo, want_hi)] = list(builder.names)
        if self.lib.mlr_model_add_program(self.handle, lo, hi, want_lo, want_hi, ops, len(ops)) != 0:
            raise RuntimeError(self.lib.mlr_exec_error().decode())

    # ---- settings
    def set_graphs(self, use: bool, graph_after: int, bucket_blocks: int, max_graphs: int) -> None:
        self.lib.mlr_model_set_graphs(self.handle, int(use), graph_after, bucket_blocks, max_graphs)

    def graph_count(self) -> int:
        return self.lib.mlr_model_graph_count(self.handle)

    def set_table_hook(self, hook) -> None:
        if hook is None:
            self._hook = None
            self.lib.mlr_model_set_table_hook(self.handle, ctypes.cast(None, TABLE_HOOK))
            return

        def call(group, n, columns, rows):
            table = torch.from_numpy(np.ctypeslib.as_array(rows, shape=(n, columns)))
            hook(group, None, table)

        self._hook = TABLE_HOOK(call)
        self.lib.mlr_model_set_table_hook(self.handle, self._hook)

    def poison(self, why: str) -> None:
        self.lib.mlr_model_poison(self.handle, why.encode())

    # ---- the step
    def step(self, slots: Sequence[int], counts: Sequence[int], tokens: Optional[np.ndarray], want_offsets: Sequence[int],
             want_places: Sequence[int], device_tokens: Optional[torch.Tensor], stream: int):
        """Returns (code, message, logits or None)."""
        n = len(slots)
        if self._routing_version != self.model.rt.routing_version:      # programs recorded under other routing settings
            self._routing_version = self.model.rt.routing_version
            self._clear_programs()
        ints = lambda values: (ctypes.c_int32 * max(1, len(values)))(*values)
        c_slots, c_counts, c_offsets, c_places = ints(slots), ints(counts), ints(want_offsets), ints(want_places)
        token_ptr = tokens.ctypes.data if tokens is not None else None
        device_ptr = device_tokens.data_ptr() if device_tokens is not None else None
        info = self.last_info
        for _ in range(6):
            code = self.lib.mlr_model_step(self.handle, n, c_slots, c_counts, token_ptr, c_offsets, c_places, device_ptr, stream,
                                           ctypes.byref(info))
            if code != STEP_NEEDS_ROOM:
                break
            self._grow(info)
        if code != STEP_OK:
            return code, self.lib.mlr_exec_error().decode(), None
        if info.graphed:
            self.graph_launches += info.launches
        return code, "", (self.logits[:info.want] if info.want else None)
