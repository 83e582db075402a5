"""Cache manager: pages, block tables and request slots (host side, C++ underneath).

See ``csrc/host/cache_manager.cpp`` for the rules.  This wrapper adds typed errors and numpy
views of the block tables; it holds no device memory (the engine owns the pages and the state slabs).
"""

from __future__ import annotations

import ctypes
import dataclasses
from ctypes import POINTER, c_int, c_int32, c_longlong, c_void_p

import numpy as np

from ..kernels import build

KEEP_ALL, KEEP_CHUNK, KEEP_WINDOW = 0, 1, 2


class CacheError(RuntimeError):
    """Misuse of the cache manager (an unknown slot, a second release, a length that is not reserved)."""


class OutOfPages(CacheError):
    """A reservation that the pools cannot serve now; nothing was taken."""


class OutOfSlots(CacheError):
    pass


@dataclasses.dataclass(frozen=True)
class Retention:
    """Which keys a group's layers can still read: all, those of the query's chunk, or a window."""

    kind: int = KEEP_ALL
    size: int = 0

    @staticmethod
    def all() -> "Retention":
        return Retention(KEEP_ALL, 0)

    @staticmethod
    def chunk(size: int) -> "Retention":
        return Retention(KEEP_CHUNK, int(size))

    @staticmethod
    def window(size: int) -> "Retention":
        return Retention(KEEP_WINDOW, int(size))


_lib = None


def _host() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        lib = ctypes.CDLL(str(build.ensure_built(["host"])["host"]))
        lib.cm_create.restype = c_void_p
        lib.cm_create.argtypes = [c_int, c_int, c_int]
        lib.cm_destroy.argtypes = [c_void_p]
        lib.cm_add_group.argtypes = [c_void_p, c_int, c_int, c_int]
        for f in ("cm_num_groups", "cm_free_slot_count", "cm_alloc_slot", "cm_check"):
            getattr(lib, f).argtypes = [c_void_p]
        for f in ("cm_free_pages", "cm_num_pages"):
            getattr(lib, f).argtypes = [c_void_p, c_int]
        lib.cm_table.restype = POINTER(c_int32)
        lib.cm_table.argtypes = [c_void_p, c_int]
        for f in ("cm_committed", "cm_reserved"):
            getattr(lib, f).restype = c_longlong
            getattr(lib, f).argtypes = [c_void_p, c_int]
        lib.cm_pages_needed.argtypes = [c_void_p, c_int, c_longlong]
        lib.cm_reserve.argtypes = [c_void_p, c_int, c_longlong]
        lib.cm_commit.argtypes = [c_void_p, c_int, c_longlong]
        lib.cm_release.argtypes = [c_void_p, c_int]
        lib.cm_pages_held.argtypes = [c_void_p, c_int, c_int]
        lib.cm_pack_step.restype = c_longlong
        lib.cm_pack_step.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                     c_int, c_int, c_void_p]
        _lib = lib
    return _lib


class CacheManager:
    """Pools of pages for groups of layers, a block table per request and group, and request slots."""

    def __init__(self, page_size: int, max_slots: int, max_pages_per_request: int):
        self._lib = _host()
        self.page_size, self.max_slots, self.max_pages_per_request = page_size, max_slots, max_pages_per_request
        self._h = self._lib.cm_create(page_size, max_slots, max_pages_per_request)
        if not self._h:
            raise CacheError(f"bad cache sizes: page_size={page_size} max_slots={max_slots} "
                             f"max_pages_per_request={max_pages_per_request}")
        self.groups: list[Retention] = []
        self._tables: list[np.ndarray] = []

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.cm_destroy(self._h)
            self._h = None

    # ------------------------------------------------------------------ set-up
    def add_group(self, retention: Retention, num_pages: int) -> int:
        g = self._lib.cm_add_group(self._h, retention.kind, retention.size, num_pages)
        if g < 0:
            raise CacheError(f"bad group: {retention} with {num_pages} pages")
        self.groups.append(retention)
        ptr = self._lib.cm_table(self._h, g)
        self._tables.append(np.ctypeslib.as_array(ptr, shape=(self.max_slots, self.max_pages_per_request)))
        return g

    # ---------------------------------------------------------------- requests
    def alloc_slot(self) -> int:
        s = self._lib.cm_alloc_slot(self._h)
        if s < 0:
            raise OutOfSlots(f"all {self.max_slots} request slots are in use")
        return s

    def pages_needed(self, slot: int, new_len: int) -> int:
        n = self._lib.cm_pages_needed(self._h, slot, new_len)
        if n == -1:
            raise CacheError(f"slot {slot} is not live")
        if n == -2:
            raise CacheError(f"length {new_len} exceeds the block table ({self.max_pages_per_request} pages of {self.page_size})")
        return n

    def can_reserve(self, slot: int, new_len: int) -> bool:
        n = self.pages_needed(slot, new_len)
        return all(self.free_pages(g) >= n for g in range(len(self.groups)))

    def reserve(self, slot: int, new_len: int) -> None:
        rc = self._lib.cm_reserve(self._h, slot, new_len)
        if rc == 1:
            raise OutOfPages(f"not enough free pages for slot {slot} to reach {new_len} tokens "
                             f"(free per group: {[self.free_pages(g) for g in range(len(self.groups))]})")
        if rc == -1:
            raise CacheError(f"slot {slot} is not live")
        if rc == -2:
            raise CacheError(f"length {new_len} exceeds the block table ({self.max_pages_per_request} pages of {self.page_size})")

    def commit(self, slot: int, new_len: int) -> int:
        rc = self._lib.cm_commit(self._h, slot, new_len)
        if rc == -1:
            raise CacheError(f"slot {slot} is not live")
        if rc == -3:
            raise CacheError(f"slot {slot}: cannot commit length {new_len} (committed {self.committed(slot)}, "
                             f"reserved {self.reserved(slot)})")
        return rc

    def release(self, slot: int) -> int:
        rc = self._lib.cm_release(self._h, slot)
        if rc < 0:
            raise CacheError(f"slot {slot} is not live (released twice?)")
        return rc

    # ------------------------------------------------------------------- state
    def committed(self, slot: int) -> int:
        n = self._lib.cm_committed(self._h, slot)
        if n < 0:
            raise CacheError(f"slot {slot} is not live")
        return n

    def reserved(self, slot: int) -> int:
        n = self._lib.cm_reserved(self._h, slot)
        if n < 0:
            raise CacheError(f"slot {slot} is not live")
        return n

    def free_pages(self, group: int) -> int:
        return self._lib.cm_free_pages(self._h, group)

    def num_pages(self, group: int) -> int:
        return self._lib.cm_num_pages(self._h, group)

    def free_slots(self) -> int:
        return self._lib.cm_free_slot_count(self._h)

    def pages_held(self, slot: int, group: int) -> int:
        return self._lib.cm_pages_held(self._h, slot, group)

    def table(self, group: int) -> np.ndarray:
        """Live view [max_slots, max_pages_per_request] of a group's block table."""
        return self._tables[group]

    def check(self) -> None:
        rc = self._lib.cm_check(self._h)
        if rc:
            names = {1: "a page id out of range", 2: "a page on the free stack twice", 3: "a page both free and held",
                     4: "a dead slot holds a page", 5: "a page held twice", 6: "a held page not marked held",
                     7: "a page lost (neither free nor held)", 8: "a bad free-slot list", 9: "a slot lost"}
            raise CacheError("cache manager invariant broken: " + names.get(rc, str(rc)))

    # -------------------------------------------------------------- descriptor
    @staticmethod
    def packed_size(n_groups: int, N_pad: int, R_pad: int, M_pad: int, width: int) -> int:
        return 3 * N_pad + (R_pad + 1) + 3 * R_pad + M_pad + n_groups * R_pad * width

    def pack_step(self, slot_ids: np.ndarray, n_tokens: np.ndarray, tokens: np.ndarray, want_offsets: np.ndarray,
                  want: np.ndarray, width: int, N_pad: int, R_pad: int, M_pad: int, out: np.ndarray) -> int:
        """Writes the step descriptor (see cm_pack_step) into the int32 array ``out``."""
        need = self.packed_size(len(self.groups), N_pad, R_pad, M_pad, width)
        if out.size < need or out.dtype != np.int32:
            raise CacheError("pack_step: output buffer too small or not int32")
        rc = self._lib.cm_pack_step(self._h, len(slot_ids), slot_ids.ctypes.data, n_tokens.ctypes.data,
                                    tokens.ctypes.data, want_offsets.ctypes.data, want.ctypes.data, width, N_pad, R_pad,
                                    M_pad, out.ctypes.data)
        if rc < 0:
            why = {-1: "a request's slot is not live", -2: "a request's new positions were not reserved",
                   -3: "a wanted place lies outside the request's tokens", -4: "block-table width too small",
                   -5: "padded sizes smaller than the batch"}
            raise CacheError("pack_step: " + why.get(int(rc), str(rc)))
        return int(rc)
