"""How parts say what they launch.

A built-in part describes its work once, in `emit(builder, ...)`: which kernel entry points
it calls with which arguments, on buffers it asks the builder for.  Two builders exist.

* `EagerBuilder` belongs to one step that Python runs: the row count is a number, buffers are
  torch tensors, and every `launch` happens at once.  `Part.forward` uses it, so a part that is
  called by hand (a test, a model that also holds parts written in Python) runs the very
  same description.
* `ProgramBuilder` records: the row count is a symbol that stands for a RANGE of row counts,
  buffers are addresses in the model's workspace, and `launch` appends an op to a program that
  the native executor (`csrc/host/executor.cpp`) walks at every step of that range without
  coming back to Python.  A decision that depends on a row count (`le`, `ge`)
  must come out the same for the whole range; if it does not, the builder raises `SplitRows`
  and the model cuts the range in two.

The reference's layer executor is a fixed C++ list of enqueues (src/minillm/cuda/layer.cpp:21-72);
here the list is made by the parts, so another mixer or feed-forward adds its own.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple, Union

import torch

from ..ops import native

# Sections of a step's metadata on the device (all int32).
META = {"token_ids": 0, "positions": 1, "segment_of_row": 2, "segment_info": 3, "slots": 4, "want_rows": 5}
# Fields of an attention launch plan (PlanField in the executor).
PLAN_FIELDS = {"items": 0, "n_items": 1, "chunk": 2, "max_splits": 3, "scratch": 4, "counters": 5,
               "tiles": 6, "n_tiles": 7, "wide_tiles": 8, "n_wide": 9,
               # derived: the split-KV items when the step has no prompt tiles / when it has some; all prompt tiles
               "n_items_alone": 10, "n_items_beside": 11, "n_prompt_tiles": 12}

K_IMM, K_FLOAT, K_ROWS, K_WANT, K_SEGMENTS, K_META, K_TABLE, K_TABLE_STRIDE, K_PLAN, K_STREAM, K_LOGITS = range(11)
NEED_ALWAYS, NEED_WANTED, NEED_PLAN_FIELD = 0, 1, 2
MAX_ARGS = 30


class SplitRows(Exception):
    """A routing decision differs within the range of row counts (`wanted` False) or of wanted-row
    counts (`wanted` True) that a program is being built for; the range has to be cut so that `at`
    starts a new one."""

    def __init__(self, at: int, wanted: bool = False):
        super().__init__(f"the program's range must be cut at {at}")
        self.at, self.wanted = at, wanted


@dataclass(frozen=True)
class Sym:
    """A value only the step knows, as an op argument: (kind, aux, i)."""
    kind: int
    aux: int = 0
    i: int = 0


Count = Union[int, Sym]


@dataclass
class Buf:
    """A row-major device buffer [rows, width] with row stride `ld` (elements); with `slices`,
    float32 partial sums [slices][rows][width] that a reader adds up, `slice_stride` apart."""
    ptr: int
    rows: Count
    width: int
    dtype: torch.dtype
    ld: int
    slices: int = 0
    slice_stride: int = 0
    tensor: Optional[torch.Tensor] = None
    # A norm that has not been launched: `ptr` is None and this holds (stream Buf, weight tensor, eps,
    # wanted rows only, what a product prepared of it or None).  A product that can norm its own input takes
    # it as it is; anyone else asks the runtime to `materialize` it first.
    norm: Optional[tuple] = None

    @property
    def is_bf16(self) -> int:
        return native.is_bf16_dtype(self.dtype)


class PlanRef:
    """The attention launch plan of a step for one (head grouping, window): fields by name."""

    def __init__(self, values: Dict[str, object]):
        self.__dict__.update(values)


def _element_size(dtype: torch.dtype) -> int:
    return torch.empty((), dtype=dtype).element_size()


# --------------------------------------------------------------------------- eager
class _NormHints:
    """What parts tell one another through the builder about the norm that reads the residual stream next.

    `norm_ahead`: set by whoever arranges the parts (a block, the model) before a part that adds into the stream
    is described: what `Norm.foldable()` of the next norm returned, or None.  A product that adds into the stream
    may then prepare that norm (`Runtime.linear_delta`) and says so in `prepared`; the norm's `emit` takes it."""
    norm_ahead = None
    norm_after_block = None
    prepared = None


class EagerBuilder(_NormHints):
    """Runs a part's description at once, for one step that Python drives."""
    recording = False

    def __init__(self, step, want_rows: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None):
        self.step = step
        self.rt = step.rt
        self.rows: Count = step.num_rows
        self._want_rows = want_rows
        self.want: Count = 0 if want_rows is None else int(want_rows.shape[0])
        self.residual: Optional[Buf] = self.wrap(residual) if residual is not None else None
        self.page_size = step.page_size
        self.status = step.status.data_ptr()
        self.stream = native.stream()
        self.table_stride_of = lambda group: step.tables[group].stride(0)

    # ---- decisions on a row count (the step's rows, or the wanted rows that a head works on)
    def le(self, count: Count, n: int) -> bool:
        return count <= n

    def ge(self, count: Count, n: int) -> bool:
        return count >= n

    def need_for(self, count: Count):
        """The `need` of a launch over `count` rows (nothing to add when the count is a number)."""
        return None

    # ---- buffers
    def wrap(self, t: Optional[torch.Tensor]) -> Optional[Buf]:
        if t is None:
            return None
        if t.dim() == 3:
            return Buf(t.data_ptr(), t.shape[1], t.shape[2], t.dtype, t.stride(1), t.shape[0], t.stride(0), t)
        return Buf(t.data_ptr(), t.shape[0], t.shape[1], t.dtype, t.stride(0), tensor=t)

    def temp(self, rows: Count, width: int, dtype: torch.dtype, slices: int = 0) -> Buf:
        shape = (slices, rows, width) if slices else (rows, width)
        return self.wrap(torch.empty(shape, dtype=dtype, device=self.rt.device))

    def logits(self, vocab: int) -> Buf:
        return self.temp(self.want, vocab, torch.float32)

    # ---- what the step knows
    def meta(self, name: str) -> int:
        if name == "want_rows":
            return 0 if self._want_rows is None else self._want_rows.data_ptr()
        return getattr(self.step, name).data_ptr()

    def table(self, group: int) -> int:
        return self.step.tables[group].data_ptr()

    def table_stride(self, group: int) -> int:
        return self.step.tables[group].stride(0)

    @property
    def segments(self) -> int:
        return len(self.step.segments)

    def plan(self, spec: Tuple[int, int, int, int, int, int]) -> PlanRef:
        """spec: (query heads per kv head, kv heads, window, wide tiles allowed, head size, small allowed)."""
        key = ("attention_plan",) + tuple(spec)
        found = self.step.scratch.get(key)
        if found is not None:
            return found
        from . import executor
        values = executor.plan_attention(spec, [(s.start, s.count) for s in self.step.segments], self.step.context_bound or 0,
                                         self.rt.sm_count)
        lists = values.pop("lists")
        device = self.rt.device
        held = torch.tensor(lists, dtype=torch.int32).to(device) if lists else None
        at = lambda offset: 0 if offset < 0 else held.data_ptr() + 4 * offset
        scratch = None
        if values["scratch_floats"]:
            scratch = torch.empty(values["scratch_floats"], dtype=torch.float32, device=device)
        counters = self.rt.split_counters(max(1, values["counters"]))
        plan = PlanRef({"items": at(values["items_offset"]), "n_items": values["n_items"], "chunk": values["chunk"],
                        "max_splits": values["max_splits"], "scratch": scratch.data_ptr() if scratch is not None else 0,
                        "counters": counters.data_ptr(), "tiles": at(values["tiles_offset"]), "n_tiles": values["n_tiles"],
                        "wide_tiles": at(values["wide_offset"]), "n_wide": values["n_wide"], "_held": (held, scratch, counters)})
        prompt_tiles = values["n_tiles"] + values["n_wide"]
        plan.n_prompt_tiles = prompt_tiles
        plan.n_items_alone = 0 if prompt_tiles else values["n_items"]
        plan.n_items_beside = values["n_items"] if prompt_tiles else 0
        self.step.scratch[key] = plan
        return plan

    # ---- launching
    def launch(self, module: str, function: str, *args, need=None) -> None:
        if need is not None:
            if need == "want":
                if not self.want:
                    return
            elif not need:
                return
        native.call(module, function, *args)


# --------------------------------------------------------------------------- recording
class _Arg(ctypes.Structure):
    _fields_ = [("kind", ctypes.c_int32), ("aux", ctypes.c_int32), ("i", ctypes.c_int64), ("f", ctypes.c_double)]


class OpRecord(ctypes.Structure):
    _fields_ = [("fn", ctypes.c_void_p), ("error_text", ctypes.c_void_p), ("n_args", ctypes.c_int32), ("need", ctypes.c_int32),
                ("need_plan", ctypes.c_int32), ("need_field", ctypes.c_int32), ("args", _Arg * MAX_ARGS)]


class _PlanField(Sym):
    pass


class ProgramBuilder(_NormHints):
    """Records a part's description as ops for a range [lo, hi] of row counts.  Buffers are cut
    from a workspace at `base` (two alternating banks after a fixed part, see `next_bank`)."""
    recording = True

    def __init__(self, rt, lo: int, hi: int, want_lo: int, want_hi: int, base: int, page_size: int, status_ptr: int,
                 plans: List[tuple]):
        self.rt = rt
        self.lo, self.hi = lo, hi
        self.want_lo, self.want_hi = want_lo, want_hi
        self.rows: Count = Sym(K_ROWS)
        self.want: Count = Sym(K_WANT)
        self.base = base
        self.page_size = page_size
        self.status = status_ptr
        self.stream = Sym(K_STREAM)
        self.segments = Sym(K_SEGMENTS)
        self.residual: Optional[Buf] = None
        self.ops: List[OpRecord] = []
        self.names: List[str] = []          # the entry point of each op, for whoever wants to read a program
        self.plans = plans                   # specs registered with the native model, by index
        self._fixed_top = 0                  # bytes of buffers that live for the whole step
        self._bank_top = [0, 0]
        self._bank = 0
        self._in_banks = False
        self.bank_bytes = [0, 0]

    # ---- decisions on a row count: they must hold for the program's whole range
    def _range(self, count: Count):
        if isinstance(count, int):
            return count, count, False
        if count.kind == K_ROWS:
            return self.lo, self.hi, False
        return self.want_lo, self.want_hi, True

    def le(self, count: Count, n: int) -> bool:
        lo, hi, wanted = self._range(count)
        if hi <= n:
            return True
        if lo > n:
            return False
        raise SplitRows(n + 1, wanted)

    def ge(self, count: Count, n: int) -> bool:
        lo, hi, wanted = self._range(count)
        if lo >= n:
            return True
        if hi < n:
            return False
        raise SplitRows(n, wanted)

    def need_for(self, count: Count):
        """The `need` of a launch over `count` rows: one over the wanted rows is skipped when a step wants none."""
        return "want" if isinstance(count, Sym) and count.kind == K_WANT else None

    # ---- buffers
    def _bound(self, rows: Count) -> int:
        if isinstance(rows, int):
            return rows
        return self.hi if rows.kind == K_ROWS else max(1, self.want_hi)

    def _cut(self, nbytes: int) -> int:
        nbytes = (nbytes + 255) // 256 * 256
        if not self._in_banks:
            offset = self._fixed_top
            self._fixed_top += nbytes
            return offset
        offset = self._bank_top[self._bank]
        self._bank_top[self._bank] += nbytes
        self.bank_bytes[self._bank] = max(self.bank_bytes[self._bank], self._bank_top[self._bank])
        return ("bank", self._bank, offset)

    def start_banks(self) -> None:
        """From here on buffers live for one run of a layer: they are cut from two banks that
        alternate (`next_bank`), so what a run leaves for the next one is not overwritten by it."""
        self._in_banks = True

    def next_bank(self) -> None:
        self._bank ^= 1
        self._bank_top[self._bank] = 0

    def temp(self, rows: Count, width: int, dtype: torch.dtype, slices: int = 0) -> Buf:
        bound = self._bound(rows)
        size = _element_size(dtype)
        where = self._cut(max(1, slices) * bound * width * size)
        return Buf(_Where(where), rows, width, dtype, width, slices, bound * width if slices else 0)

    def logits(self, vocab: int) -> Buf:
        return Buf(Sym(K_LOGITS), self.want, vocab, torch.float32, vocab)

    def wrap(self, t):
        raise RuntimeError("a program is built from the parts' own buffers, not from tensors")

    # ---- what the step knows
    def meta(self, name: str) -> Sym:
        return Sym(K_META, META[name])

    def table(self, group: int) -> Sym:
        return Sym(K_TABLE, group)

    def table_stride(self, group: int) -> Sym:
        return Sym(K_TABLE_STRIDE)

    def plan(self, spec) -> PlanRef:
        spec = tuple(int(v) for v in spec)
        if spec not in self.plans:
            self.plans.append(spec)
        index = self.plans.index(spec)
        return PlanRef({name: _PlanField(K_PLAN, index, field) for name, field in PLAN_FIELDS.items()})

    # ---- launching
    def launch(self, module: str, function: str, *args, need=None) -> None:
        if len(args) > MAX_ARGS:
            raise ValueError(f"{function} has {len(args)} arguments, an op takes {MAX_ARGS}")
        op = OpRecord()
        fn, error_text = native.entry_points(module, function)
        op.fn, op.error_text, op.n_args = fn, error_text, len(args)
        if need == "want":
            op.need = NEED_WANTED
        elif isinstance(need, _PlanField):
            op.need, op.need_plan, op.need_field = NEED_PLAN_FIELD, need.aux, need.i
        elif need is not None:
            raise ValueError("a recorded op can depend on the wanted rows or on a field of a plan")
        for k, value in enumerate(args):
            a = op.args[k]
            if isinstance(value, Sym):
                a.kind, a.aux, a.i = value.kind, value.aux, value.i
            elif isinstance(value, _Where):
                a.kind, a.i = K_IMM, 0
                self._patches.append((len(self.ops), k, value.where))
            elif isinstance(value, float):
                a.kind, a.f = K_FLOAT, value
            elif value is None:
                a.kind, a.i = K_IMM, 0
            elif isinstance(value, (int, bool)):
                a.kind, a.i = K_IMM, int(value)
            else:
                raise TypeError(f"{function}: argument {k} of type {type(value).__name__} cannot be recorded")
        self.ops.append(op)
        self.names.append(function)

    _patches: List[tuple]

    def begin(self) -> None:
        self._patches = []

    def workspace_bytes(self) -> int:
        return self._fixed_top + self.bank_bytes[0] + self.bank_bytes[1]

    def finish(self):
        """Resolves buffer addresses (fixed part, then bank 0, then bank 1) and returns the ops
        as a ctypes array."""
        bank_base = [self._fixed_top, self._fixed_top + self.bank_bytes[0]]
        for op_index, arg_index, where in self._patches:
            if isinstance(where, tuple):
                address = self.base + bank_base[where[1]] + where[2]
            else:
                address = self.base + where
            self.ops[op_index].args[arg_index].i = address
        return (OpRecord * len(self.ops))(*self.ops)


class _Where:
    """A workspace address that is known once the whole program has been laid out."""

    def __init__(self, where):
        self.where = where

    def __add__(self, nbytes: int):
        if isinstance(self.where, tuple):
            return _Where(("bank", self.where[1], self.where[2] + nbytes))
        return _Where(self.where + nbytes)

    def __mod__(self, n: int) -> int:          # alignment checks: every cut is 256-byte aligned
        offset = self.where[2] if isinstance(self.where, tuple) else self.where
        return offset % n

    def __bool__(self) -> bool:
        return True
