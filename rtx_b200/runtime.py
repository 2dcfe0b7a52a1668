"""Runtime glue of the Python frontends (rtx/runtime.py:62-269): environment
check, the bounded LRU that owns launch workspaces, cache limits from the
environment, and cache release."""

from __future__ import annotations

import os
from collections.abc import MutableMapping
from importlib import import_module
from threading import RLock


def validate_runtime_environment(*, require_device: bool = False) -> dict[str, object]:
    """Check what the sm_100a path needs: a CUDA build of PyTorch, the in-tree
    native library, and (when `require_device`) a compute-capability 10.x GPU.
    Returns the facts it checked; raises RuntimeError with the reason otherwise."""
    import torch

    from . import _native

    facts: dict[str, object] = {"torch": torch.__version__, "torch_cuda": torch.version.cuda,
                                "library": _native.LIB_PATH}
    if torch.version.cuda is None:
        raise RuntimeError("rtx_b200 needs a CUDA build of PyTorch")
    if not os.path.exists(_native.LIB_PATH):
        raise RuntimeError(f"{_native.LIB_PATH} is missing: run `python -m rtx_b200.build`")
    facts["abi_version"] = _native.load().rtxb_version()
    if require_device:
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device is visible")
        major, minor = torch.cuda.get_device_capability()
        facts["capability"] = (major, minor)
        if major != 10:
            raise RuntimeError(f"the native kernels are built for sm_100a (B200); got capability {(major, minor)}")
    return facts


class BoundedCache(MutableMapping):
    """LRU table for the launch objects that own GPU workspaces (same name, mapping protocol and
    `stats()` keys as the reference's runner cache, rtx/runtime.py:134-206).

    Built on the insertion order of a plain dict: the first key is always the least recently used,
    a lookup re-inserts its key at the end.  `max_entries == 0` stores nothing, so a value lives only
    as long as the caller's own reference.  Counters: `hits` / `misses` count `cache[key]` lookups,
    `evictions` counts values dropped for space (a value refused by a zero-sized cache counts)."""

    def __init__(self, max_entries: int) -> None:
        capacity = int(max_entries)
        if capacity < 0:
            raise ValueError("cache size cannot be negative")
        self.max_entries = capacity
        self.hits = 0
        self.misses = 0
        self.evictions = 0
        self._table: dict = {}
        self._guard = RLock()

    def _touch(self, key):
        """Value of `key`, made the most recent entry; KeyError if absent.  Caller holds the lock."""
        value = self._table.pop(key)
        self._table[key] = value
        return value

    def __getitem__(self, key):
        with self._guard:
            if key in self._table:
                self.hits += 1
                return self._touch(key)
            self.misses += 1
        raise KeyError(key)

    def __contains__(self, key) -> bool:       # membership tests do not count as lookups
        with self._guard:
            return key in self._table

    def get(self, key, default=None):
        with self._guard:
            if key in self._table:
                self.hits += 1
                return self._touch(key)
            self.misses += 1
            return default

    def __setitem__(self, key, value) -> None:
        with self._guard:
            if self.max_entries == 0:
                self.evictions += 1
                return
            self._table.pop(key, None)
            self._table[key] = value
            overflow = len(self._table) - self.max_entries
            for oldest in list(self._table)[:max(overflow, 0)]:
                del self._table[oldest]
                self.evictions += 1

    def __delitem__(self, key) -> None:
        with self._guard:
            del self._table[key]

    def __iter__(self):
        with self._guard:
            snapshot = list(self._table)
        return iter(snapshot)

    def __len__(self) -> int:
        with self._guard:
            return len(self._table)

    def clear(self) -> None:
        with self._guard:
            self._table = {}

    def stats(self) -> dict[str, int]:
        with self._guard:
            return dict(entries=len(self._table), max_entries=self.max_entries, hits=self.hits,
                        misses=self.misses, evictions=self.evictions)


def runner_cache_limit(kind: str, default: int = 8, *, namespace: str = "MXFP8") -> int:
    """Entries a frontend's cache may hold: the environment's RTX_<NAMESPACE>_<KIND>_CACHE_ENTRIES if
    set, else RTX_<NAMESPACE>_RUNNER_CACHE_ENTRIES, else `default` (the reference's variable names,
    rtx/runtime.py:209-225).  Non-integers and negative values are refused."""
    names = (f"RTX_{namespace}_{kind.upper()}_CACHE_ENTRIES", f"RTX_{namespace}_RUNNER_CACHE_ENTRIES")
    for name in names:
        text = os.environ.get(name)
        if text is None:
            continue
        try:
            limit = int(text)
        except ValueError:
            raise ValueError(f"{name} must be an integer, got {text!r}") from None
        if limit < 0:
            raise ValueError(f"{name} cannot be negative")
        return limit
    return default


_CACHING_FRONTENDS = ("fp8", "fp8_bwd", "fp4")


def clear_runtime_caches(*, synchronize: bool = True, device=None) -> dict[str, object]:
    """Drop every workspace the frontends hold (rtx/runtime.py:250-269).  Kernels may still be reading
    those buffers, so by default the device is synchronised first.  Returns what each frontend
    reported releasing."""
    import torch

    if synchronize and torch.cuda.is_available():
        torch.cuda.synchronize(device)
    report: dict[str, object] = {}
    for name in _CACHING_FRONTENDS:
        hook = getattr(import_module(f"{__package__}.{name}"), "_clear_runtime_caches", None)
        if callable(hook):
            report[name] = hook()
    return report


__all__ = ["BoundedCache", "clear_runtime_caches", "runner_cache_limit", "validate_runtime_environment"]
