"""Runtime glue of the Python frontends (rtx/runtime.py:62-269): environment
check, the bounded LRU that owns launch workspaces, cache limits from the
environment, and cache release."""

from __future__ import annotations

import os
from collections import OrderedDict
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
    """Small thread-safe LRU for launchers that retain GPU workspaces.  A size of
    zero keeps nothing (the value stays alive for the caller's invocation only)."""

    def __init__(self, max_entries: int) -> None:
        if max_entries < 0:
            raise ValueError("cache size cannot be negative")
        self.max_entries = int(max_entries)
        self._values: OrderedDict = OrderedDict()
        self._lock = RLock()
        self.hits = self.misses = self.evictions = 0

    def __getitem__(self, key):
        with self._lock:
            try:
                value = self._values.pop(key)
            except KeyError:
                self.misses += 1
                raise
            self._values[key] = value
            self.hits += 1
            return value

    def get(self, key, default=None):
        try:
            return self[key]
        except KeyError:
            return default

    def __setitem__(self, key, value) -> None:
        with self._lock:
            self._values.pop(key, None)
            if self.max_entries == 0:
                self.evictions += 1
                return
            self._values[key] = value
            while len(self._values) > self.max_entries:
                self._values.popitem(last=False)
                self.evictions += 1

    def __delitem__(self, key) -> None:
        with self._lock:
            del self._values[key]

    def __iter__(self):
        with self._lock:
            return iter(tuple(self._values))

    def __len__(self) -> int:
        with self._lock:
            return len(self._values)

    def clear(self) -> None:
        with self._lock:
            self._values.clear()

    def stats(self) -> dict[str, int]:
        with self._lock:
            return {"entries": len(self._values), "max_entries": self.max_entries, "hits": self.hits,
                    "misses": self.misses, "evictions": self.evictions}


def runner_cache_limit(kind: str, default: int = 8, *, namespace: str = "MXFP8") -> int:
    """RTX_<NAMESPACE>_<KIND>_CACHE_ENTRIES, else RTX_<NAMESPACE>_RUNNER_CACHE_ENTRIES, else `default`."""
    specific = f"RTX_{namespace}_{kind.upper()}_CACHE_ENTRIES"
    raw = os.getenv(specific, os.getenv(f"RTX_{namespace}_RUNNER_CACHE_ENTRIES", str(default)))
    try:
        value = int(raw)
    except ValueError as exc:
        raise ValueError(f"{specific} must be an integer, got {raw!r}") from exc
    if value < 0:
        raise ValueError(f"{specific} cannot be negative")
    return value


def clear_runtime_caches(*, synchronize: bool = True, device=None) -> dict[str, object]:
    """Release the workspaces the frontends cache; launches are asynchronous, so the
    default synchronises first."""
    if synchronize:
        import torch

        if torch.cuda.is_available():
            torch.cuda.synchronize(device)
    released: dict[str, object] = {}
    for name in ("fp8", "fp8_bwd", "fp4"):
        module = import_module(f".{name}", __package__)
        clear = getattr(module, "_clear_runtime_caches", None)
        if clear is not None:
            released[name] = clear()
    return released


__all__ = ["BoundedCache", "clear_runtime_caches", "runner_cache_limit", "validate_runtime_environment"]
