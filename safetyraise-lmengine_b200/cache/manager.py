"""Python face of the native cache manager, plus the device memory it indexes.

``CacheGroupSpec`` says what one group of cache entries needs: pages of keys
and values (all of them, or a window), or a fixed-size state per request.  The
native manager (csrc/host/cache_manager.cpp) does the page and slot accounting;
this module allocates one pool of device memory per group and hands out views.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..errors import ConfigError, ResourceExhausted

PAGED_ALL, PAGED_WINDOW, FIXED_STATE = "paged_all", "paged_window", "fixed_state"


@dataclass(frozen=True)
class CacheGroupSpec:
    """What the cache entries of one group need.

    paged groups: ``entries`` cache entries (one per run step that writes), each with
    ``kv_heads * head_dim`` keys and values per token.  fixed_state groups: one tensor of
    ``state_shape`` per request and entry.
    """
    name: str
    kind: str
    entries: Tuple[int, ...]                 # cache entry ids (RunStep.cache) of this group
    kv_heads: int = 0
    head_dim: int = 0
    window: Optional[int] = None
    state_shape: Tuple[int, ...] = ()
    state_dtype: torch.dtype = torch.float32

    def bytes_per_token(self, dtype: torch.dtype) -> int:
        if self.kind == FIXED_STATE:
            return 0
        return 2 * len(self.entries) * self.kv_heads * self.head_dim * (4 if dtype == torch.float32 else 2)

    def bytes_per_request(self, dtype: torch.dtype, context: int, page_size: int = 1) -> int:
        """What one request of ``context`` tokens holds in this group at most: its keys and values (of a
        window group only those the window still covers, in whole pages), or its fixed-size state.
        Counterpart of state_bytes (src/model/spec.rs:491-522)."""
        if self.kind == FIXED_STATE:
            n = 1
            for d in self.state_shape:
                n *= d
            return len(self.entries) * n * self.state_dtype.itemsize
        tokens = context
        if self.kind == PAGED_WINDOW and self.window:
            tokens = min(context, self.window + page_size)
        return self.bytes_per_token(dtype) * -(-tokens // page_size) * page_size


_runtime = None


def runtime():
    global _runtime
    if _runtime is None:
        from ..csrc.build import build_runtime
        lib = C.CDLL(build_runtime())
        lib.srlm_cache_create.restype = C.c_void_p
        lib.srlm_cache_create.argtypes = [C.c_int, C.c_int] + [C.POINTER(C.c_int)] * 4
        lib.srlm_sched_create.restype = C.c_void_p
        lib.srlm_sched_create.argtypes = [C.c_void_p] + [C.c_int] * 5
        for name in ("open", "close", "reserve", "fit_tokens", "commit", "truncate", "length", "reserved",
                     "generation", "free_pages", "audit"):
            fn = getattr(lib, "srlm_cache_" + name)
            fn.restype = C.c_int
            fn.argtypes = [C.c_void_p] + [C.c_int] * {"open": 0, "audit": 0, "close": 1, "length": 1,
                                                        "reserved": 1, "generation": 1,
                                                        "free_pages": 1}.get(name, 2)
        lib.srlm_cache_table.restype = C.c_int
        lib.srlm_cache_table.argtypes = [C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_int32), C.c_int]
        lib.srlm_cache_destroy.argtypes = [C.c_void_p]
        lib.srlm_cache_reuse_counts.argtypes = [C.c_void_p, C.POINTER(C.c_int64), C.POINTER(C.c_int64)]
        lib.srlm_sched_destroy.argtypes = [C.c_void_p]
        lib.srlm_sched_submit.argtypes = [C.c_void_p, C.c_int64, C.c_int, C.c_int]
        lib.srlm_sched_plan.argtypes = [C.c_void_p, C.POINTER(C.c_int64), C.c_int, C.POINTER(C.c_int64),
                                        C.POINTER(C.c_int)]
        lib.srlm_sched_advance.argtypes = [C.c_void_p, C.c_int64, C.c_int]
        for name in ("rollback", "append_token", "retract_token", "finish"):
            getattr(lib, "srlm_sched_" + name).argtypes = [C.c_void_p, C.c_int64]
        lib.srlm_sched_has_work.argtypes = [C.c_void_p]
        lib.srlm_sched_counters.argtypes = [C.c_void_p, C.POINTER(C.c_int64)]
        _runtime = lib
    return _runtime


class CacheManager:
    """Pages, block tables and state slots for up to ``max_requests`` live requests.

    ``device=None`` makes the accounting only (no device memory), which is all the
    CPU tests and the scheduler need.
    """

    def __init__(self, groups: Sequence[CacheGroupSpec], page_size: int, num_pages: int,
                 max_requests: int, dtype: torch.dtype = torch.bfloat16, device=None):
        if page_size <= 0 or num_pages <= 0 or max_requests <= 0:
            raise ConfigError("page_size, num_pages and max_requests must be positive")
        self.groups = list(groups)
        self.page_size, self.num_pages, self.max_requests = page_size, num_pages, max_requests
        self.dtype, self.device = dtype, device
        self._paged = [g for g in self.groups if g.kind in (PAGED_ALL, PAGED_WINDOW)]
        self._paged_index = {g.name: i for i, g in enumerate(self._paged)}
        n = len(self._paged)
        arr = lambda vals: (C.c_int * max(n, 1))(*vals) if n else (C.c_int * 1)()
        lib = runtime()
        self._lib = lib
        self._h = lib.srlm_cache_create(
            max_requests, n,
            arr([1 if g.kind == PAGED_WINDOW else 0 for g in self._paged]),
            arr([page_size] * n), arr([num_pages] * n),
            arr([g.window or 0 for g in self._paged]))
        if not self._h:
            raise ConfigError("the cache manager refused its configuration")
        # device memory: per paged group [entries, 2, num_pages, kv_heads, page_size, head_dim]:
        # one KV head's share of a page is contiguous, which is what the attention kernels stream
        self.kv_pools: Dict[str, torch.Tensor] = {}
        self.state_pools: Dict[str, torch.Tensor] = {}
        self.entry_home: Dict[int, Tuple[str, int]] = {}
        for g in self.groups:
            for i, e in enumerate(g.entries):
                if e in self.entry_home:
                    raise ConfigError(f"cache entry {e} is in two groups")
                self.entry_home[e] = (g.name, i)
            if device is None:
                continue
            if g.kind == FIXED_STATE:
                self.state_pools[g.name] = torch.zeros((len(g.entries), max_requests) + tuple(g.state_shape),
                                                       dtype=g.state_dtype, device=device)
            else:
                self.kv_pools[g.name] = torch.zeros((len(g.entries), 2, num_pages, g.kv_heads, page_size,
                                                     g.head_dim), dtype=dtype, device=device)
        self._table_buf = (C.c_int32 * (num_pages + 1))()

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.srlm_cache_destroy(h)

    # ---- accounting ---------------------------------------------------------
    def open_request(self) -> int:
        slot = self._lib.srlm_cache_open(self._h)
        if slot < 0:
            raise ResourceExhausted(f"all {self.max_requests} request slots are taken")
        return slot          # the engine zeroes the slot's fixed-size state when it first runs the new occupant

    def close_request(self, slot: int) -> None:
        if self._lib.srlm_cache_close(self._h, slot) != 0:
            raise ValueError(f"slot {slot} is not open (closed twice?)")

    def reserve(self, slot: int, new_len: int) -> bool:
        r = self._lib.srlm_cache_reserve(self._h, slot, new_len)
        if r < 0:
            raise ValueError(f"reserve(slot={slot}, new_len={new_len}) is invalid ({r})")
        return r == 1

    def fit_tokens(self, slot: int, want_len: int) -> int:
        return self._lib.srlm_cache_fit_tokens(self._h, slot, want_len)

    def commit(self, slot: int, new_len: int) -> None:
        r = self._lib.srlm_cache_commit(self._h, slot, new_len)
        if r != 0:
            raise ValueError(f"commit(slot={slot}, new_len={new_len}) is invalid ({r})")

    def truncate(self, slot: int, length: int) -> None:
        r = self._lib.srlm_cache_truncate(self._h, slot, length)
        if r != 0:
            raise ValueError(f"truncate(slot={slot}, len={length}) is invalid ({r})")

    def length(self, slot: int) -> int:
        return self._lib.srlm_cache_length(self._h, slot)

    def generation(self, slot: int) -> int:
        return self._lib.srlm_cache_generation(self._h, slot)

    def table(self, group: str, slot: int) -> List[int]:
        n = self._lib.srlm_cache_table(self._h, self._paged_index[group], slot, self._table_buf,
                                       len(self._table_buf))
        if n < 0:
            raise ValueError(f"slot {slot} is not open")
        return list(self._table_buf[:n])

    def table_into(self, group: str, slot: int, out) -> int:
        """Writes the slot's block table into ``out`` (a contiguous int32 numpy array) and returns its
        length (entries beyond len(out) are not written)."""
        n = self._lib.srlm_cache_table(self._h, self._paged_index[group], slot,
                                       out.ctypes.data_as(C.POINTER(C.c_int32)), len(out))
        if n < 0:
            raise ValueError(f"slot {slot} is not open")
        return n

    def free_pages(self, group: Optional[str] = None) -> int:
        return self._lib.srlm_cache_free_pages(self._h, self._paged_index[group] if group else 0)

    def audit(self) -> int:
        return self._lib.srlm_cache_audit(self._h)

    def reuse_counts(self) -> Tuple[int, int]:
        a, b = C.c_int64(), C.c_int64()
        self._lib.srlm_cache_reuse_counts(self._h, C.byref(a), C.byref(b))
        return a.value, b.value

    @property
    def paged_groups(self) -> List[CacheGroupSpec]:
        return self._paged

    @property
    def handle(self):
        return self._h

    # ---- device views ---------------------------------------------------------
    def kv_of_entry(self, entry: int) -> Tuple[torch.Tensor, torch.Tensor, str]:
        """(K pool, V pool, group name) of one cache entry: [num_pages, kv_heads, page_size, head_dim]."""
        name, i = self.entry_home[entry]
        pool = self.kv_pools[name]
        return pool[i, 0], pool[i, 1], name

    def state_of_entry(self, entry: int) -> torch.Tensor:
        """[max_requests, *state_shape]: the fixed-size state of every slot for one cache entry."""
        name, i = self.entry_home[entry]
        return self.state_pools[name][i]

    def bytes_per_page(self) -> int:
        return sum(g.bytes_per_token(self.dtype) for g in self._paged) * self.page_size
