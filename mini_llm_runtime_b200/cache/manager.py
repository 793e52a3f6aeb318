"""Cache manager: the host-side ledger of pages, block tables and state slots.

The ledger itself is native code (`csrc/host/cache_manager.cpp`); this class is its
Python face and adds nothing to its decisions.  It owns no device memory: the pools
that the page ids index are allocated by the model (`engine/model.py`, `allocate_cache`).

Layers are grouped by what they keep: group `g` keeps every key (`window` None) or
only the last `window` keys.  Each group has `num_pages` page ids and one block
table; a request's row of that table maps block index (position // page_size) to a
page id, -1 where the request holds none (not reached yet, or released because the
window has moved past it).

A request is opened (it gets a slot, which is also the index of its fixed-size
state), grows step by step, and is closed (all its pages and the slot return).  A
step is `prepare` (takes the pages of all requests of the step, or none and raises
`OutOfPages`), then `commit` or `discard`.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from ..csrc import build

_OK, _BAD_ARGUMENT, _NO_PAGES, _NO_SLOT, _BAD_PHASE, _TOO_LONG = range(6)


class CacheError(RuntimeError):
    pass


class OutOfPages(CacheError):
    """A step needs more pages than a group has free; nothing was changed."""


class OutOfSlots(CacheError):
    """Every request slot is taken."""


@dataclass(frozen=True)
class GroupSpec:
    window: Optional[int]   # None: all keys are kept
    num_pages: int


def _library():
    lib = build.load("host")
    if not getattr(lib, "_mlr_cache_bound", False):
        i, p = ctypes.c_int, ctypes.c_void_p
        ip = ctypes.POINTER(ctypes.c_int)
        lib.mlr_cache_create.argtypes = [i, ip, ip, i, i, i]
        lib.mlr_cache_create.restype = p
        lib.mlr_cache_destroy.argtypes = [p]
        lib.mlr_cache_destroy.restype = None
        lib.mlr_cache_error.argtypes = [p]
        lib.mlr_cache_error.restype = ctypes.c_char_p
        lib.mlr_cache_max_blocks.argtypes = [p]
        lib.mlr_cache_open.argtypes = [p, ip]
        lib.mlr_cache_close.argtypes = [p, i]
        lib.mlr_cache_length.argtypes = [p, i]
        lib.mlr_cache_free_pages.argtypes = [p, i]
        lib.mlr_cache_free_slots.argtypes = [p]
        lib.mlr_cache_peak_pages.argtypes = [p, i, i, i]
        lib.mlr_cache_prepare.argtypes = [p, i, ip, ip]
        lib.mlr_cache_commit.argtypes = [p]
        lib.mlr_cache_discard.argtypes = [p]
        lib.mlr_cache_fill_table.argtypes = [p, i, i, ip, i, ctypes.c_void_p, i]
        lib._mlr_cache_bound = True
    return lib


def _ints(values: Sequence[int]):
    return (ctypes.c_int * len(values))(*values)


class CacheManager:
    def __init__(self, groups: Sequence[GroupSpec], page_size: int, max_requests: int, max_model_len: int):
        if page_size <= 0 or max_requests <= 0 or max_model_len <= 0:
            raise CacheError("page size, request count and maximum length must be positive")
        for g in groups:
            if g.num_pages <= 0 or (g.window is not None and g.window <= 0):
                raise CacheError(f"bad cache group {g}")
        self.groups = list(groups)
        self.page_size = page_size
        self.max_requests = max_requests
        self.max_model_len = max_model_len
        self._lib = _library()
        windows = _ints([g.window or 0 for g in groups])
        pages = _ints([g.num_pages for g in groups])
        self._handle = self._lib.mlr_cache_create(len(groups), windows, pages, page_size, max_requests, max_model_len)
        if not self._handle:
            raise CacheError("the cache manager refused its configuration")
        self.max_blocks = self._lib.mlr_cache_max_blocks(self._handle)

    def __del__(self):
        handle, self._handle = getattr(self, "_handle", None), None
        if handle:
            self._lib.mlr_cache_destroy(handle)

    def _check(self, code: int) -> None:
        if code == _OK:
            return
        message = self._lib.mlr_cache_error(self._handle).decode()
        if code == _NO_PAGES:
            raise OutOfPages(message)
        if code == _NO_SLOT:
            raise OutOfSlots(message)
        raise CacheError(message)

    # ---- requests
    def open(self) -> int:
        slot = ctypes.c_int(-1)
        self._check(self._lib.mlr_cache_open(self._handle, ctypes.byref(slot)))
        return slot.value

    def close(self, slot: int) -> None:
        self._check(self._lib.mlr_cache_close(self._handle, slot))

    def length(self, slot: int) -> int:
        n = self._lib.mlr_cache_length(self._handle, slot)
        if n < 0:
            raise CacheError(f"slot {slot} is not open")
        return n

    def free_slots(self) -> int:
        return self._lib.mlr_cache_free_slots(self._handle)

    # ---- pages
    def free_pages(self, group: int) -> int:
        n = self._lib.mlr_cache_free_pages(self._handle, group)
        if n < 0:
            raise CacheError(f"no cache group {group}")
        return n

    def peak_pages(self, group: int, total_tokens: int, max_step_tokens: int) -> int:
        """The most pages a request of `total_tokens` holds at once in `group` when no
        step gives it more than `max_step_tokens` tokens."""
        n = self._lib.mlr_cache_peak_pages(self._handle, group, total_tokens, max_step_tokens)
        if n < 0:
            raise CacheError(f"no cache group {group}")
        return n

    # ---- steps
    def prepare(self, slots: Sequence[int], new_tokens: Sequence[int]) -> None:
        if len(slots) != len(new_tokens):
            raise CacheError("prepare() wants one token count per slot")
        self._check(self._lib.mlr_cache_prepare(self._handle, len(slots), _ints(slots), _ints(new_tokens)))

    def commit(self) -> None:
        self._check(self._lib.mlr_cache_commit(self._handle))

    def discard(self) -> None:
        self._check(self._lib.mlr_cache_discard(self._handle))

    def fill_table(self, group: int, slots: Sequence[int], out: torch.Tensor, columns: Optional[int] = None) -> None:
        """Writes the block-table rows of `slots` into the CPU int32 tensor `out`
        [len(slots), >= columns]."""
        if out.dtype is not torch.int32 or out.is_cuda or out.dim() != 2 or out.stride(1) != 1 or out.shape[0] < len(slots):
            raise CacheError("fill_table() wants a CPU int32 matrix with a row per slot")
        columns = out.shape[1] if columns is None else columns
        if columns > out.shape[1]:
            raise CacheError("fill_table() asked for more columns than the output has")
        self._check(self._lib.mlr_cache_fill_table(self._handle, group, len(slots), _ints(slots), columns,
                                                   out.data_ptr(), out.stride(0)))

    def table_row(self, group: int, slot: int) -> List[int]:
        out = torch.empty((1, self.max_blocks), dtype=torch.int32)
        self.fill_table(group, [slot], out)
        return out[0].tolist()
