"""Run the reference's own code (installed by ``baseline/install_ref.py``) as a baseline.

Two baselines, both built around this repository's plain-PyTorch DeiT skeleton (the reference takes the
surrounding model from timm, which is not part of its tree):

* ``reference_cpu_model``: the reference's fake-quant layer ``QuantLinearPCARCQ``
  (fair_qat/quant_backends.py:282-322, quantizer quant/dcarcq.py:512-578) in the qkv / proj / fc1 / fc2 slots,
  fp32 on the host cores.  This is the CPU baseline the headline ratio is quoted against.
* ``reference_triton_model``: the reference's ``ARCQPackedLinearOnTheFly`` (fair_qat/arcq_packed_on_the_fly.py)
  with its Triton kernels, given the packed buffers of an already packed model, one shared fp16 weight buffer
  as in scripts/benchmark_arcq_on_the_fly.py:186-191.  This is the path the B200 back end replaces.

Baseline infrastructure only: nothing in the package imports this file.
"""
from __future__ import annotations

import sys
import types
from pathlib import Path

import torch
import torch.nn as nn

HERE = Path(__file__).resolve().parent
REF = HERE / "_ref"


def available() -> bool:
    sys.path.insert(0, str(HERE))
    try:
        import install_ref
        return install_ref.is_installed(REF)
    finally:
        sys.path.pop(0)


def _import_reference():
    """Import the installed files; the CUDA extension the packed module imports at the top is replaced by the
    NumPy packer exactly as the reference's scripts/convert_arcq_to_packed.py:56-59 does."""
    if str(REF) not in sys.path:
        sys.path.insert(0, str(REF))
    from fair_qat.arcq_packed_py import pack_codes_py, unpack_codes_py
    if "fair_qat.arcq_infer_cuda" not in sys.modules:
        stub = types.ModuleType("fair_qat.arcq_infer_cuda")
        for n in ("arcq_linear_forward", "arcq_linear_forward_u8", "quantize_activation", "quantize_activation_dequant",
                  "quantize_activation_u8", "unpack_codes"):
            setattr(stub, n, None)
        stub.pack_codes, stub.unpack_codes_u8 = pack_codes_py, unpack_codes_py
        sys.modules["fair_qat.arcq_infer_cuda"] = stub
    from fair_qat.quant_backends import QuantLinearPCARCQ
    return QuantLinearPCARCQ


def _get(model, path):
    for part in path.split("."):
        model = getattr(model, part)
    return model


def _set(model, path, new):
    parts = path.split(".")
    setattr(_get(model, ".".join(parts[:-1])) if len(parts) > 1 else model, parts[-1], new)


@torch.no_grad()
def reference_cpu_model(pkg, model_name: str, bits: int, calib_images: torch.Tensor, seed: int = 0):
    """fp32 CPU DeiT with the reference's QuantLinearPCARCQ in the four linear slots of every block, codebooks
    compiled on ``calib_images`` by one calibrating forward and then frozen (compile_steps emptied, as
    scripts/benchmark_arcq_packed_inference.py:135-139 does)."""
    QuantLinearPCARCQ = _import_reference()
    m = pkg.create_vit(model_name, seed=seed).float()
    for name in pkg.quantised_linear_names(m):
        lin = _get(m, name)
        q = QuantLinearPCARCQ(lin.in_features, lin.out_features, lin.bias is not None, bits, bits, group_size=64)
        q.linear.weight.copy_(lin.weight)
        if lin.bias is not None:
            q.linear.bias.copy_(lin.bias)
        _set(m, name, q)
    m.eval()
    m(calib_images.float())                      # the calibrating forward compiles every codebook
    for mod in m.modules():
        if hasattr(mod, "compile_steps"):
            mod.compile_steps = set()
    return m


@torch.no_grad()
def reference_triton_model(pkg, packed_model: nn.Module):
    """Swap the reference's Triton-backed on-the-fly linear into a packed model (same packed buffers)."""
    _import_reference()
    from fair_qat.arcq_packed_on_the_fly import ARCQPackedLinearOnTheFly as RefOTF
    layers, max_w = [], 0
    for name in pkg.quantised_linear_names(packed_model):
        l = _get(packed_model, name)
        r = RefOTF(l.in_features, l.out_features, l.bias_tensor.numel() > 0, l.packed_weight_codes, l.weight_codebook,
                   l.weight_center, l.weight_scale, l.weight_code_sum, l.activation_codebook, l.activation_thresholds,
                   l.bits, l.group_size, l.bias_tensor if l.bias_tensor.numel() else None)
        _set(packed_model, name, r)
        layers.append(r)
        max_w = max(max_w, l.in_features * l.out_features)
    dev = layers[0].packed_weight_codes.device
    buf = torch.zeros(max_w, dtype=torch.float16, device=dev)
    for r in layers:
        r._weight_buffer = buf                   # one shared scratch, as the reference benchmark does
    return packed_model.eval()
