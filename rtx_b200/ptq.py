"""Model conversion frontends: swap the BF16 `nn.Linear` layers of a model for the block-scaled
modules, for training (the BF16 master weight stays, same `Parameter` object) or for inference
(the weight is packed once and the BF16 copy is dropped).

Same functions and policy dataclasses as the reference (rtx/ptq.py:34-93 policies, :212-289
training conversion, :292-384 `quantize_`, which follows TorchAO's `quantize_` convention).
A conversion is all-or-nothing: every selected layer is validated and every replacement is
built before the module tree is touched.
"""

from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Callable, Dict, List, Optional, Tuple

import torch
from torch import nn

ModuleFilter = Callable[[nn.Module, str], bool]


@dataclass(frozen=True)
class MXFP8TrainingConfig:
    """What `convert_to_mxfp8_training` passes to every `MXFP8Linear` it builds."""
    forward_config: object = None
    dynamic_config: object = None
    backward_config: object = None
    backend: str = "auto"
    autotune: object = None
    tuning_policy: object = None
    autotune_cache_dir: "Path | str | None" = None


@dataclass(frozen=True)
class NVFP4TrainingConfig:
    """What `convert_to_nvfp4_training` passes to every `NVFP4Linear` it builds."""
    scale_config: object = None
    backward_config: object = None
    scaling: Optional[str] = None
    scale_region_rows: Optional[int] = None
    x_scale_region_rows: Optional[int] = None
    weight_scale_region_rows: Optional[int] = None
    backend: str = "auto"
    autotune: object = None
    tuning_policy: object = None
    autotune_cache_dir: "Path | str | None" = None
    dynamic_config: object = None


@dataclass(frozen=True)
class MXFP8WeightOnlyConfig:
    """Packed MXFP8 weights; activations are still quantized to MXFP8 on the fly at run time
    ("weight only" describes what the checkpoint holds)."""
    dynamic_config: object = None
    autotune: object = None
    tuning_policy: object = None
    autotune_cache_dir: "Path | str | None" = None


@dataclass(frozen=True)
class NVFP4WeightOnlyConfig:
    """Packed NVFP4 weights, BF16 activations quantized on the fly."""
    scaling: str = "current"
    quant_config: object = None
    weight_prequant_config: object = None
    fully_prequant_config: object = None
    autotune: object = None
    tuning_policy: object = None
    autotune_cache_dir: "Path | str | None" = None

    def __post_init__(self) -> None:
        if self.scaling not in ("current", "block"):
            raise ValueError("packed NVFP4 PTQ scaling must be current or block")


class _Swap:
    """One conversion, planned before anything is touched: which modules are replaced and under which
    qualified names each of them hangs in the tree (a shared module hangs under several)."""

    def __init__(self, model: nn.Module, wanted: Optional[ModuleFilter], device, needs_cuda: bool):
        if not isinstance(model, nn.Module):
            raise TypeError(f"model must be an nn.Module, got {type(model).__name__}")
        if device is not None:
            model.to(device=device)
        self.model = model
        # torch walks the tree for us; with remove_duplicate=False every alias path is reported
        paths: Dict[int, List[str]] = {}
        modules: Dict[int, nn.Module] = {}
        for path, module in model.named_modules(remove_duplicate=False):
            modules[id(module)] = module
            paths.setdefault(id(module), []).append(path)
        self.targets: List[Tuple[nn.Module, List[str]]] = []
        for key, module in modules.items():
            where = paths[key]
            if wanted is None:
                picked = [isinstance(module, nn.Linear)] * len(where)
            else:
                picked = [bool(wanted(module, path)) for path in where]
            if True not in picked:
                continue
            shown = [path if path else "<root>" for path in where]
            if False in picked:
                raise ValueError("filter selected only some aliases of one shared module: " + ", ".join(shown))
            self._check(module, shown[0], needs_cuda)
            self.targets.append((module, where))

    @staticmethod
    def _check(module: nn.Module, shown: str, needs_cuda: bool) -> None:
        if not isinstance(module, nn.Linear):
            raise TypeError(f"RTX conversion can only replace nn.Linear modules; filter selected {type(module).__name__}")
        if module.bias is not None:
            raise NotImplementedError(f"RTX linear layers do not support bias; selected {shown} has bias")
        weight = module.weight
        if weight.dtype is not torch.bfloat16:
            raise TypeError(f"RTX conversion requires a BF16 weight; {shown} has {weight.dtype}")
        if needs_cuda and not weight.is_cuda:
            raise ValueError(f"RTX PTQ requires CUDA weights; {shown} is on {weight.device}")

    def apply(self, make: Callable[[nn.Linear], nn.Module]) -> nn.Module:
        """Build every replacement (any failure leaves the model untouched), then hang each one under
        every path of the module it replaces.  Returns the root, which may itself have been replaced."""
        replacements = [(make(module), where) for module, where in self.targets]
        root = self.model
        for new, where in replacements:
            for path in where:
                if not path:
                    root = new
                    continue
                owner_path, _, leaf = path.rpartition(".")
                self.model.get_submodule(owner_path)._modules[leaf] = new
        return root

    def cuda_devices(self):
        return {module.weight.device for module, _ in self.targets if module.weight.is_cuda}


def _adopt(new: nn.Module, old: nn.Linear) -> nn.Module:
    """Training swap: the replacement takes over the very `Parameter` object and the mode flag."""
    new.weight = old.weight
    new.train(old.training)
    return new


def convert_to_mxfp8_training(model: nn.Module, *, module_filter_fn: Optional[ModuleFilter] = None,
                              config: Optional[MXFP8TrainingConfig] = None, device=None) -> nn.Module:
    """BF16 linears -> `MXFP8Linear` (dynamic weights).  The original `Parameter` objects are kept, so
    optimizer references, weight sharing, state-dict keys and `requires_grad` carry over."""
    from .fp8 import MXFP8Linear

    policy = config if config is not None else MXFP8TrainingConfig()
    options = dict(forward_config=policy.forward_config, dynamic_config=policy.dynamic_config,
                   backward_config=policy.backward_config, backend=policy.backend, autotune=policy.autotune,
                   tuning_policy=policy.tuning_policy, autotune_cache_dir=policy.autotune_cache_dir)

    def make(old: nn.Linear) -> nn.Module:
        return _adopt(MXFP8Linear(old.in_features, old.out_features, bias=False, device=old.weight.device,
                                  dtype=torch.bfloat16, **options), old)

    return _Swap(model, module_filter_fn, device, needs_cuda=False).apply(make)


def convert_to_nvfp4_training(model: nn.Module, *, module_filter_fn: Optional[ModuleFilter] = None,
                              config: Optional[NVFP4TrainingConfig] = None, device=None) -> nn.Module:
    """BF16 linears -> `NVFP4Linear` (NVFP4 forward, MXFP8 backward), parameters kept as above."""
    from .fp4 import NVFP4Linear

    policy = config if config is not None else NVFP4TrainingConfig()
    options = dict(scale_config=policy.scale_config, backward_config=policy.backward_config, scaling=policy.scaling,
                   scale_region_rows=policy.scale_region_rows, x_scale_region_rows=policy.x_scale_region_rows,
                   weight_scale_region_rows=policy.weight_scale_region_rows, backend=policy.backend,
                   autotune=policy.autotune, tuning_policy=policy.tuning_policy,
                   autotune_cache_dir=policy.autotune_cache_dir, dynamic_config=policy.dynamic_config)

    def make(old: nn.Linear) -> nn.Module:
        return _adopt(NVFP4Linear(old.in_features, old.out_features, bias=False, device=old.weight.device,
                                  dtype=torch.bfloat16, **options), old)

    return _Swap(model, module_filter_fn, device, needs_cuda=False).apply(make)


def quantize_(model: nn.Module, config, filter_fn: Optional[ModuleFilter] = None, device=None) -> nn.Module:
    """Post-training quantization: pack the weights of the selected no-bias BF16 linears (which must be on a
    CUDA device) and replace the layers by inference-only packed modules.  Children are replaced in place;
    the (possibly replaced) root is returned."""
    if isinstance(config, MXFP8WeightOnlyConfig):
        from .fp8 import MXFP8Linear, quantize_mxfp8

        def make(old: nn.Linear) -> nn.Module:
            return MXFP8Linear(old.in_features, old.out_features, bias=False, device=old.weight.device,
                               dtype=torch.bfloat16, dynamic_config=config.dynamic_config, autotune=config.autotune,
                               tuning_policy=config.tuning_policy, autotune_cache_dir=config.autotune_cache_dir,
                               packed_weight=quantize_mxfp8(old.weight.detach()))
    elif isinstance(config, NVFP4WeightOnlyConfig):
        from .fp4 import NVFP4Linear, quantize_nvfp4

        def make(old: nn.Linear) -> nn.Module:
            # the block policy has no outer scale: its tensor scale is exactly one
            unit = torch.ones((), dtype=torch.float32, device=old.weight.device) if config.scaling == "block" else None
            packed = quantize_nvfp4(old.weight.detach(), tensor_scale=unit, config=config.quant_config)
            return NVFP4Linear(old.in_features, old.out_features, bias=False, device=old.weight.device,
                               dtype=torch.bfloat16, scaling=config.scaling, autotune=config.autotune,
                               tuning_policy=config.tuning_policy, autotune_cache_dir=config.autotune_cache_dir,
                               weight_prequant_config=config.weight_prequant_config,
                               fully_prequant_config=config.fully_prequant_config, packed_weight=packed)
    else:
        if not isinstance(model, nn.Module):
            raise TypeError(f"model must be an nn.Module, got {type(model).__name__}")
        raise TypeError("rtx.quantize_ requires MXFP8WeightOnlyConfig or NVFP4WeightOnlyConfig; "
                        f"got {type(config).__name__}")
    swap = _Swap(model, filter_fn, device, needs_cuda=True)
    root = swap.apply(make)
    # packing was only enqueued: let it finish before the caller drops the BF16 masters
    for dev in swap.cuda_devices():
        torch.cuda.current_stream(dev).synchronize()
    return root


__all__ = ["MXFP8TrainingConfig", "MXFP8WeightOnlyConfig", "ModuleFilter", "NVFP4TrainingConfig",
           "NVFP4WeightOnlyConfig", "convert_to_mxfp8_training", "convert_to_nvfp4_training", "quantize_"]
