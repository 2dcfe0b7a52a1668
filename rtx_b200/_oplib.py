"""Operator registration for the `rtx::` custom ops.

`torch.library.custom_op` wraps every call of the device implementation in several Python layers (an
aliasing check, a compile-disable frame, an autograd trampoline even for ops without a backward): tens of
microseconds per call, more than a whole decode step takes on the device.  The ops here are declared with
the dispatcher directly instead — same inferred schema, same `pt2_compliant` tag, fake and autograd
registrations through the same `torch.library` functions — so an eager call costs one dispatch.
The returned handle offers the part of the `custom_op` object's interface the package uses.
"""

from __future__ import annotations

from typing import Callable, Optional

import torch

_LIB = torch.library.Library("rtx", "FRAGMENT")


class OpHandle:
    """Callable handle of one registered op (`torch.ops.rtx.<name>.default`)."""

    def __init__(self, qualname: str, fn: Callable):
        namespace, name = qualname.split("::")
        self.qualname = qualname
        self.fn = fn                                  # the device implementation, for direct in-package calls
        self.overload = getattr(getattr(torch.ops, namespace), name).default
        self.__name__ = getattr(fn, "__name__", name)
        self.__doc__ = fn.__doc__

    def __call__(self, *args, **kwargs):
        return self.overload(*args, **kwargs)

    def register_fake(self, fn: Callable) -> Callable:
        torch.library.register_fake(self.qualname, fn, lib=_LIB)
        return fn

    def register_autograd(self, backward: Callable, *, setup_context: Optional[Callable] = None) -> None:
        torch.library.register_autograd(self.qualname, backward, setup_context=setup_context, lib=_LIB)


def custom_op(qualname: str, *, mutates_args=(), device_types: str = "cuda") -> Callable[[Callable], OpHandle]:
    """Decorator with the call signature of `torch.library.custom_op` (schema inferred from the annotations)."""
    if device_types != "cuda":
        raise ValueError("the rtx:: ops have CUDA implementations only")

    def register(fn: Callable) -> OpHandle:
        schema = torch.library.infer_schema(fn, mutates_args=mutates_args)
        torch.library.define(qualname, schema, lib=_LIB, tags=(torch.Tag.pt2_compliant_tag,))
        torch.library.impl(qualname, "CUDA", fn, lib=_LIB)
        return OpHandle(qualname, fn)

    return register
