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
# (parent or None for the root, attribute name, module, fully qualified name)
_Site = Tuple[Optional[nn.Module], Optional[str], nn.Module, str]


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


def _is_linear(module: nn.Module, fqn: str) -> bool:
    return isinstance(module, nn.Linear)


def _sites(root: nn.Module) -> List[_Site]:
    """Every place a module is referenced from, aliases of shared modules included; a shared
    module's children are walked once."""
    found: List[_Site] = [(None, None, root, "")]
    seen = {id(root)}
    stack = [(root, "")]
    while stack:
        parent, prefix = stack.pop()
        for name, child in list(parent._modules.items()):
            if child is None:
                continue
            fqn = f"{prefix}.{name}" if prefix else name
            found.append((parent, name, child, fqn))
            if id(child) not in seen:
                seen.add(id(child))
                stack.append((child, fqn))
    return found


def _select(model: nn.Module, filter_fn: Optional[ModuleFilter], require_cuda: bool):
    """[(linear, its sites)] for the layers the filter picks, validated."""
    keep = filter_fn or _is_linear
    by_module: Dict[int, List[_Site]] = {}
    for site in _sites(model):
        by_module.setdefault(id(site[2]), []).append(site)
    chosen = []
    for sites in by_module.values():
        votes = [bool(keep(module, fqn)) for _, _, module, fqn in sites]
        if not any(votes):
            continue
        names = [fqn or "<root>" for _, _, _, fqn in sites]
        if not all(votes):
            raise ValueError("filter selected only some aliases of one shared module: " + ", ".join(names))
        module = sites[0][2]
        if not isinstance(module, nn.Linear):
            raise TypeError(f"RTX conversion can only replace nn.Linear modules; filter selected {type(module).__name__}")
        if module.bias is not None:
            raise NotImplementedError(f"RTX linear layers do not support bias; selected {names[0]} has bias")
        if module.weight.dtype is not torch.bfloat16:
            raise TypeError(f"RTX conversion requires a BF16 weight; {names[0]} has {module.weight.dtype}")
        if require_cuda and module.weight.device.type != "cuda":
            raise ValueError(f"RTX PTQ requires CUDA weights; {names[0]} is on {module.weight.device}")
        chosen.append((module, sites))
    return chosen


def _install(model: nn.Module, chosen, built: Dict[int, nn.Module]) -> nn.Module:
    for module, sites in chosen:
        for parent, name, _, _ in sites:
            if parent is not None:
                parent._modules[name] = built[id(module)]
    return built.get(id(model), model)


def _prepare(model: nn.Module, device) -> None:
    if not isinstance(model, nn.Module):
        raise TypeError(f"model must be an nn.Module, got {type(model).__name__}")
    if device is not None:
        model.to(device=device)


def convert_to_mxfp8_training(model: nn.Module, *, module_filter_fn: Optional[ModuleFilter] = None,
                              config: Optional[MXFP8TrainingConfig] = None, device=None) -> nn.Module:
    """BF16 linears -> `MXFP8Linear` (dynamic weights).  The original `Parameter` objects are kept, so
    optimizer references, weight sharing, state-dict keys and `requires_grad` carry over."""
    from .fp8 import MXFP8Linear

    _prepare(model, device)
    chosen = _select(model, module_filter_fn, require_cuda=False)
    policy = config or MXFP8TrainingConfig()
    built: Dict[int, nn.Module] = {}
    for module, _ in chosen:
        new = MXFP8Linear(module.in_features, module.out_features, bias=False, device=module.weight.device,
                          dtype=torch.bfloat16, forward_config=policy.forward_config,
                          dynamic_config=policy.dynamic_config, backward_config=policy.backward_config,
                          backend=policy.backend, autotune=policy.autotune, tuning_policy=policy.tuning_policy,
                          autotune_cache_dir=policy.autotune_cache_dir)
        new.weight = module.weight
        new.train(module.training)
        built[id(module)] = new
    return _install(model, chosen, built)


def convert_to_nvfp4_training(model: nn.Module, *, module_filter_fn: Optional[ModuleFilter] = None,
                              config: Optional[NVFP4TrainingConfig] = None, device=None) -> nn.Module:
    """BF16 linears -> `NVFP4Linear` (NVFP4 forward, MXFP8 backward), parameters kept as above."""
    from .fp4 import NVFP4Linear

    _prepare(model, device)
    chosen = _select(model, module_filter_fn, require_cuda=False)
    policy = config or NVFP4TrainingConfig()
    built: Dict[int, nn.Module] = {}
    for module, _ in chosen:
        new = NVFP4Linear(module.in_features, module.out_features, bias=False, device=module.weight.device,
                          dtype=torch.bfloat16, scale_config=policy.scale_config,
                          backward_config=policy.backward_config, scaling=policy.scaling,
                          scale_region_rows=policy.scale_region_rows,
                          x_scale_region_rows=policy.x_scale_region_rows,
                          weight_scale_region_rows=policy.weight_scale_region_rows, backend=policy.backend,
                          autotune=policy.autotune, tuning_policy=policy.tuning_policy,
                          autotune_cache_dir=policy.autotune_cache_dir, dynamic_config=policy.dynamic_config)
        new.weight = module.weight
        new.train(module.training)
        built[id(module)] = new
    return _install(model, chosen, built)


def quantize_(model: nn.Module, config, filter_fn: Optional[ModuleFilter] = None, device=None) -> nn.Module:
    """Post-training quantization: pack the weights of the selected no-bias BF16 linears (which must be on a
    CUDA device) and replace the layers by inference-only packed modules.  Children are replaced in place;
    the (possibly replaced) root is returned."""
    _prepare(model, device)
    if not isinstance(config, (MXFP8WeightOnlyConfig, NVFP4WeightOnlyConfig)):
        raise TypeError("rtx.quantize_ requires MXFP8WeightOnlyConfig or NVFP4WeightOnlyConfig; "
                        f"got {type(config).__name__}")
    chosen = _select(model, filter_fn, require_cuda=True)
    built: Dict[int, nn.Module] = {}
    if isinstance(config, MXFP8WeightOnlyConfig):
        from .fp8 import MXFP8Linear, quantize_mxfp8

        for module, _ in chosen:
            packed = quantize_mxfp8(module.weight.detach())
            built[id(module)] = MXFP8Linear(module.in_features, module.out_features, bias=False,
                                            device=module.weight.device, dtype=torch.bfloat16,
                                            dynamic_config=config.dynamic_config, autotune=config.autotune,
                                            tuning_policy=config.tuning_policy,
                                            autotune_cache_dir=config.autotune_cache_dir, packed_weight=packed)
    else:
        from .fp4 import NVFP4Linear, quantize_nvfp4

        for module, _ in chosen:
            scale = (torch.ones((), dtype=torch.float32, device=module.weight.device)
                     if config.scaling == "block" else None)
            packed = quantize_nvfp4(module.weight.detach(), tensor_scale=scale, config=config.quant_config)
            built[id(module)] = NVFP4Linear(module.in_features, module.out_features, bias=False,
                                            device=module.weight.device, dtype=torch.bfloat16,
                                            scaling=config.scaling, autotune=config.autotune,
                                            tuning_policy=config.tuning_policy,
                                            autotune_cache_dir=config.autotune_cache_dir,
                                            weight_prequant_config=config.weight_prequant_config,
                                            fully_prequant_config=config.fully_prequant_config,
                                            packed_weight=packed)
    # the packing launches are asynchronous: finish them before the BF16 masters can be freed
    for dev in {m.weight.device for m, _ in chosen if m.weight.device.type == "cuda"}:
        torch.cuda.current_stream(dev).synchronize()
    return _install(model, chosen, built)


__all__ = ["MXFP8TrainingConfig", "MXFP8WeightOnlyConfig", "ModuleFilter", "NVFP4TrainingConfig",
           "NVFP4WeightOnlyConfig", "convert_to_mxfp8_training", "convert_to_nvfp4_training", "quantize_"]
