"""Swap fake-quant linears for packed ones, and load packed checkpoints.

``convert_arcq_linear_to_packed`` / ``count_packed_linear`` keep the reference's names and
behaviour (methods/fair_qat_framework/fair_qat/arcq_packed_convert.py:8-28): children are
matched by the class *name* ``QuantLinearPCARCQ`` plus the three attributes, and replaced with
``setattr``.  ``to_on_the_fly`` is the second swap the reference benchmark performs
(scripts/benchmark_arcq_on_the_fly.py:151-173).  ``load_packed_state_dict`` is new: the
reference writes packed state-dicts (scripts/convert_arcq_to_packed.py:90) but has no code
that reads one back without the original QAT model.
"""
from __future__ import annotations

from typing import Dict

import torch
import torch.nn as nn

from .packed_linear import ARCQPackedLinear, ARCQPackedLinearOnTheFly
from .staging import attach_weight_stager


def _is_pcarcq_linear(module: nn.Module) -> bool:
    return (module.__class__.__name__ == "QuantLinearPCARCQ" and hasattr(module, "linear")
            and hasattr(module, "act_quant") and hasattr(module, "weight_quant"))


def convert_arcq_linear_to_packed(model: nn.Module, runtime_code_format: str = "packed") -> nn.Module:
    """Recursively replace QuantLinearPCARCQ modules with ARCQPackedLinear."""
    for name, child in list(model.named_children()):
        if _is_pcarcq_linear(child):
            setattr(model, name, ARCQPackedLinear(child, runtime_code_format=runtime_code_format))
        else:
            convert_arcq_linear_to_packed(child, runtime_code_format=runtime_code_format)
    return model


def count_packed_linear(model: nn.Module) -> int:
    return sum(1 for m in model.modules() if isinstance(m, (ARCQPackedLinear, ARCQPackedLinearOnTheFly)))


def _swap_to_on_the_fly(model: nn.Module) -> None:
    for name, child in list(model.named_children()):
        if isinstance(child, ARCQPackedLinear):
            setattr(model, name, ARCQPackedLinearOnTheFly.from_packed(child))
        else:
            _swap_to_on_the_fly(child)


def to_on_the_fly(model: nn.Module) -> nn.Module:
    """Replace every ARCQPackedLinear by an ARCQPackedLinearOnTheFly sharing its buffers, and give the new
    layers a common weight stager (staging.py) so that each layer's weight is unpacked while the previous
    layer computes."""
    _swap_to_on_the_fly(model)
    attach_weight_stager(model)
    return model


def packed_prefixes(state_dict: Dict[str, torch.Tensor]):
    """Module paths (with trailing dot) that hold a packed linear in a state-dict."""
    return sorted(k[: -len("packed_weight_codes")] for k in state_dict if k.endswith("packed_weight_codes"))


def load_packed_state_dict(model: nn.Module, state_dict: Dict[str, torch.Tensor], on_the_fly: bool = True,
                           strict: bool = True) -> nn.Module:
    """Install a packed checkpoint into a float model skeleton.

    Every ``<path>.packed_weight_codes`` entry turns the module at ``<path>`` (whatever it is) into
    a packed linear built from the checkpoint's buffers; all remaining keys are loaded as
    ordinary parameters/buffers.
    """
    prefixes = packed_prefixes(state_dict)
    used = set()
    for pre in prefixes:
        path = pre[:-1].split(".")
        parent = model
        for part in path[:-1]:
            parent = getattr(parent, part)
        layer = ARCQPackedLinear.from_state_dict(state_dict, pre)
        setattr(parent, path[-1], ARCQPackedLinearOnTheFly.from_packed(layer) if on_the_fly else layer)
        used.update(k for k in state_dict if k.startswith(pre))
    rest = {k: v for k, v in state_dict.items() if k not in used}
    own = {k for k in model.state_dict() if not any(k.startswith(p) for p in prefixes)}
    missing = sorted(own - set(rest))
    unexpected = sorted(set(rest) - own)
    if strict and (missing or unexpected):
        raise KeyError(f"packed checkpoint mismatch: missing={missing[:5]} unexpected={unexpected[:5]}")
    model.load_state_dict({k: v for k, v in rest.items() if k in own}, strict=False)
    if on_the_fly:
        attach_weight_stager(model)
    return model
