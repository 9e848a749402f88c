"""Packed ARCQ linear modules: the drop-in boundary.

Two ``nn.Module``s with the constructor signatures, buffer names and ``forward(x)``
contract of the reference's packed layers:

* ``ARCQPackedLinear(source, runtime_code_format)`` --
  methods/fair_qat_framework/fair_qat/arcq_packed_linear.py:56-241.  Built from a trained
  fake-quant layer (anything exposing ``.linear``, ``.act_quant``, ``.weight_quant`` with compiled
  codebooks); owns the packed state-dict format; ``forward`` returns fp32.
* ``ARCQPackedLinearOnTheFly(...buffers...)`` --
  methods/fair_qat_framework/fair_qat/arcq_packed_on_the_fly.py:93-169.  Built from buffers;
  ``forward`` returns fp16 ("half chain").

Both forwards are launches behind the C ABI: the activation quantizer (packed codes + per-group
statistics, or the fp16 reconstruction) and a tcgen05 GEMM -- with the weight rebuilt inside the
kernel, or unpacked by a third launch on a side stream while the previous layer runs (``staging.py``);
the routes give the same bits.  There is no Triton, no cuBLAS and no CPU path; without the built
library the forward raises.

Added on this side of the boundary (the reference never loads its own packed
checkpoints back): ``ARCQPackedLinear.from_state_dict`` / ``from_buffers``.
"""
from __future__ import annotations

import os

import math
from typing import Optional, Tuple

import torch
import torch.nn as nn

from . import ops
from .packing import pack_codes, unpack_codes_u8

_FORMATS = ("packed", "u8", "dequant_gemm")


def _vector(name: str, value) -> torch.Tensor:
    if not isinstance(value, torch.Tensor) or value.numel() == 0:
        raise ValueError(f"{name} is missing; load a checkpoint with compiled ARCQ codebooks first")
    return value.detach().float().flatten().contiguous()


@torch.no_grad()
def quantize_weight(weight: torch.Tensor, thresholds: torch.Tensor, codebook: torch.Tensor, group_size: int,
                    eps: float = 1e-6) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Weight codes and per-(row, group) statistics at conversion time.

    Same arithmetic as the reference's ``_quantize_weight_reference``
    (arcq_packed_linear.py:27-53): fp32 torch ops on whatever device the weight is on.
    Returns (codes int64 [N,K], center, scale, code_sum fp32 [N,G]).
    """
    if weight.dim() != 2:
        raise ValueError(f"ARCQPackedLinear expects 2D linear weight, got shape={tuple(weight.shape)}")
    N, K = weight.shape
    if K % group_size != 0:
        raise ValueError(f"in_features={K} must be divisible by group_size={group_size}")
    w3 = weight.detach().float().contiguous().reshape(N, K // group_size, group_size)
    center = w3.mean(dim=-1)
    resid = w3 - center.unsqueeze(-1)
    scale = (resid.square().mean(dim=-1) + float(eps)).sqrt()
    codes = torch.bucketize(resid / scale.unsqueeze(-1), thresholds.to(resid))
    code_sum = codebook.to(resid)[codes].sum(dim=-1)
    return codes.reshape(N, K).to(torch.int64), center, scale, code_sum


class _KeepsFp32Metadata(nn.Module):
    """``model.half()`` must not touch the fp32 metadata buffers the kernels read (the reference
    benchmark restores them after the cast, scripts/benchmark_arcq_on_the_fly.py:63-85): let the
    cast or move happen, then put any fp32 buffer that changed dtype back, on its new device."""

    def _apply(self, fn, *args, **kwargs):
        keep = {n: b for n, b in self._buffers.items() if b is not None and b.dtype == torch.float32}
        super()._apply(fn, *args, **kwargs)
        for n, old in keep.items():
            new = self._buffers[n]
            if new.dtype != torch.float32:
                self._buffers[n] = old.to(device=new.device)
        return self


class ARCQPackedLinear(_KeepsFp32Metadata):
    """Inference-only packed ARCQ linear: low-bit weight indices + per-group metadata, no float weight."""

    def __init__(self, source: nn.Module, runtime_code_format: str = "packed"):
        super().__init__()
        if runtime_code_format not in _FORMATS:
            raise ValueError("runtime_code_format must be 'packed', 'u8', or 'dequant_gemm', "
                             f"got {runtime_code_format}")
        linear = getattr(source, "linear", None)
        if linear is None or not hasattr(linear, "weight"):
            raise TypeError("ARCQPackedLinear source must expose source.linear.weight")
        act_q, w_q = getattr(source, "act_quant", None), getattr(source, "weight_quant", None)
        if act_q is None or w_q is None:
            raise TypeError("ARCQPackedLinear source must expose act_quant and weight_quant")
        bits = int(getattr(w_q, "bits", 4))
        a_bits = int(getattr(act_q, "bits", bits))
        if bits != a_bits:
            raise ValueError(f"packed kernel currently requires W bits == A bits, got W{bits} A{a_bits}")
        group_size = int(getattr(w_q, "group_size", 64))
        eps = float(getattr(w_q, "eps", getattr(act_q, "eps", 1.0e-6)))
        a_cb = _vector("act_quant._pc_cb", getattr(act_q, "_pc_cb", None))
        a_th = _vector("act_quant._pc_thresholds", getattr(act_q, "_pc_thresholds", None))
        w_cb = _vector("weight_quant._pc_cb", getattr(w_q, "_pc_cb", None))
        w_th = _vector("weight_quant._pc_thresholds", getattr(w_q, "_pc_thresholds", None))
        self._validate(int(linear.weight.shape[1]), bits, group_size, a_cb, w_cb)
        dev = linear.weight.device
        codes, center, scale, code_sum = quantize_weight(linear.weight, w_th.to(dev), w_cb.to(dev), group_size, eps)
        bias = None if linear.bias is None else linear.bias.detach()
        self._install(runtime_code_format, bits, group_size, pack_codes(codes, bits), center, scale, code_sum,
                      w_cb.to(dev), a_cb.to(dev), a_th.to(dev), bias, codes=codes)

    # ------------------------------------------------------------------ construction helpers
    @staticmethod
    def _validate(in_features: int, bits: int, group_size: int, a_cb: torch.Tensor, w_cb: torch.Tensor) -> None:
        if bits not in (2, 3, 4):
            raise ValueError(f"packed kernel supports bits 2/3/4, got {bits}")
        if in_features % group_size != 0:
            raise ValueError(f"in_features={in_features} must be divisible by group_size={group_size}")
        if a_cb.numel() != 2 ** bits or w_cb.numel() != 2 ** bits:
            raise ValueError(f"codebook size must be {2 ** bits}, got A={a_cb.numel()} W={w_cb.numel()}")

    def _install(self, fmt, bits, group_size, packed, center, scale, code_sum, w_cb, a_cb, a_th, bias, codes=None):
        dev = packed.device
        N, G = center.shape
        self.runtime_code_format = fmt
        self.bits, self.act_bits, self.group_size = bits, bits, group_size
        self.in_features, self.out_features = G * group_size, N
        f32 = lambda t: t.detach().to(device=dev, dtype=torch.float32).contiguous()  # noqa: E731
        self.register_buffer("packed_weight_codes", packed.contiguous())
        if fmt == "u8":
            u8 = unpack_codes_u8(packed, bits, self.in_features).contiguous()
        else:
            u8 = torch.empty(0, device=dev, dtype=torch.uint8)
        self.register_buffer("weight_codes_u8", u8)
        if fmt == "dequant_gemm":
            if codes is None:
                codes = unpack_codes_u8(packed, bits, self.in_features).long()
            vals = f32(w_cb)[codes.to(dev)].reshape(N, G, group_size)
            wd = f32(center).unsqueeze(-1) + f32(scale).unsqueeze(-1) * (vals - f32(code_sum).unsqueeze(-1) / group_size)
            wd = wd.reshape(N, self.in_features).to(torch.float16).contiguous()
        else:
            wd = torch.empty(0, device=dev, dtype=torch.float16)
        self.register_buffer("weight_dequant", wd)
        self.register_buffer("weight_center", f32(center))
        self.register_buffer("weight_scale", f32(scale))
        self.register_buffer("weight_code_sum", f32(code_sum))
        self.register_buffer("weight_codebook", f32(w_cb))
        self.register_buffer("activation_codebook", f32(a_cb))
        self.register_buffer("activation_thresholds", f32(a_th))
        self.register_buffer("product_table", (f32(a_cb).view(-1, 1) * f32(w_cb).view(1, -1)).contiguous())
        self.register_buffer("bias", torch.empty(0, device=dev, dtype=torch.float32) if bias is None or bias.numel() == 0
                             else f32(bias))
        self.packed_weight_bytes = int(self.packed_weight_codes.numel())
        self.weight_meta_floats = int(3 * self.weight_center.numel())

    @classmethod
    def from_buffers(cls, packed_weight_codes, weight_center, weight_scale, weight_code_sum, weight_codebook,
                     activation_codebook, activation_thresholds, bias=None,
                     runtime_code_format: str = "packed") -> "ARCQPackedLinear":
        """Build from packed buffers.  bits, group size and K are not stored in the format; they
        follow from the shapes: bits = log2(levels), G = center.shape[1], K = packed_cols*8/bits."""
        if runtime_code_format not in _FORMATS:
            raise ValueError(f"bad runtime_code_format {runtime_code_format}")
        self = cls.__new__(cls)
        nn.Module.__init__(self)
        levels = int(weight_codebook.numel())
        bits = int(round(math.log2(levels)))
        if 2 ** bits != levels:
            raise ValueError(f"codebook size {levels} is not a power of two")
        G = int(weight_center.shape[1])
        pc = int(packed_weight_codes.shape[1])
        if (pc * 8) % bits != 0 or (pc * 8 // bits) % G != 0:
            raise ValueError(f"packed row of {pc} bytes does not hold a whole number of {bits}-bit groups x {G}")
        K = pc * 8 // bits
        cls._validate(K, bits, K // G, activation_codebook.flatten(), weight_codebook.flatten())
        self._install(runtime_code_format, bits, K // G, packed_weight_codes, weight_center, weight_scale,
                      weight_code_sum, weight_codebook.flatten(), activation_codebook.flatten(),
                      activation_thresholds.flatten(), bias)
        return self

    @classmethod
    def from_state_dict(cls, state_dict, prefix: str = "", runtime_code_format: str = "packed") -> "ARCQPackedLinear":
        """Rebuild a layer from the packed checkpoint entries ``<prefix>packed_weight_codes`` etc."""
        g = lambda k: state_dict[prefix + k]  # noqa: E731
        return cls.from_buffers(g("packed_weight_codes"), g("weight_center"), g("weight_scale"), g("weight_code_sum"),
                                g("weight_codebook"), g("activation_codebook"), g("activation_thresholds"),
                                state_dict.get(prefix + "bias"), runtime_code_format)

    # ------------------------------------------------------------------ forward
    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, bits={self.bits}, "
                f"group_size={self.group_size}, runtime_code_format={self.runtime_code_format}, "
                f"packed_weight_bytes={self.packed_weight_bytes}")

    def _run(self, x2: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        packed_x, mu, sg, cs = ops.quantize_activation(x2, self.activation_thresholds, self.activation_codebook,
                                                       self.bits, self.group_size)
        return ops.arcq_linear_forward(packed_x, mu, sg, cs, self.packed_weight_codes, self.weight_center,
                                       self.weight_scale, self.weight_code_sum, self.activation_codebook,
                                       self.weight_codebook, self.bias if self.bias.numel() else None, self.bits,
                                       self.group_size, self.in_features, self.out_features, out_dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        if shape[-1] != self.in_features:
            raise ValueError(f"expected last dim {self.in_features}, got {shape[-1]}")
        x2 = x.reshape(-1, self.in_features).to(device=self.packed_weight_codes.device)
        if x2.dtype not in (torch.float32, torch.float16, torch.bfloat16):
            x2 = x2.float()
        return self._run(x2.contiguous(), torch.float32).reshape(*shape[:-1], self.out_features)

    def estimated_storage_bytes(self) -> int:
        meta = sum(b.numel() for b in (self.weight_center, self.weight_scale, self.weight_code_sum,
                                       self.weight_codebook, self.activation_codebook, self.activation_thresholds,
                                       self.product_table, self.bias)) * 4
        return int(self.packed_weight_codes.numel() + meta)

    def runtime_cache_bytes(self) -> int:
        return int(self.weight_codes_u8.numel() * self.weight_codes_u8.element_size()
                   + self.weight_dequant.numel() * self.weight_dequant.element_size())


class ARCQPackedLinearOnTheFly(_KeepsFp32Metadata):
    """Buffers-only packed linear of the fp16 chain; same constructor as the reference class."""

    def __init__(self, in_features: int, out_features: int, bias: bool, packed_weight_codes: torch.Tensor,
                 weight_codebook: torch.Tensor, weight_center: torch.Tensor, weight_scale: torch.Tensor,
                 weight_code_sum: torch.Tensor, activation_codebook: torch.Tensor,
                 activation_thresholds: torch.Tensor, bits: int, group_size: int,
                 bias_tensor: Optional[torch.Tensor]):
        super().__init__()
        if bits not in (2, 3, 4):
            raise ValueError(f"packed kernel supports bits 2/3/4, got {bits}")
        if in_features % group_size != 0:
            raise ValueError(f"in_features={in_features} must be divisible by group_size={group_size}")
        self.in_features, self.out_features = in_features, out_features
        self.bits, self.group_size, self.groups = bits, group_size, in_features // group_size
        f32 = lambda t: t.detach().float().contiguous()  # noqa: E731  metadata stays fp32 in the half chain
        self.register_buffer("packed_weight_codes", packed_weight_codes.contiguous())
        self.register_buffer("weight_codebook", f32(weight_codebook))
        self.register_buffer("weight_center", f32(weight_center))
        self.register_buffer("weight_scale", f32(weight_scale))
        self.register_buffer("weight_code_sum", f32(weight_code_sum))
        self.register_buffer("activation_codebook", f32(activation_codebook))
        self.register_buffer("activation_thresholds", f32(activation_thresholds))
        if bias and bias_tensor is not None and bias_tensor.numel() > 0:
            self.register_buffer("bias_tensor", f32(bias_tensor))
        else:
            self.register_buffer("bias_tensor", torch.empty(0))

    @classmethod
    def from_packed(cls, m: ARCQPackedLinear) -> "ARCQPackedLinearOnTheFly":
        """Share the buffers of an ``ARCQPackedLinear`` (what the reference benchmark does,
        scripts/benchmark_arcq_on_the_fly.py:151-173)."""
        return cls(m.in_features, m.out_features, m.bias.numel() > 0, m.packed_weight_codes, m.weight_codebook,
                   m.weight_center, m.weight_scale, m.weight_code_sum, m.activation_codebook,
                   m.activation_thresholds, m.bits, m.group_size, m.bias if m.bias.numel() > 0 else None)

    # the module can apply the GELU that precedes it in an MLP block while it quantises its input
    supports_pre_gelu = True

    # How the weight reaches the tensor cores.
    #   "staged": unpacked into one of two fp16 scratch matrices on a side stream while the previous layer runs
    #             (the reference's own data flow, arcq_packed_on_the_fly.py:147-160, with its `_weight_buffer`),
    #             then read by TMA.  Needs a WeightStager on the model (attached by this package's converters).
    #   "packed": rebuilt from the codes inside the GEMM kernel, never in HBM.
    #   "dense":  unpacked on the layer's own stream right before the GEMM (no overlap, no stager needed).
    #   "auto":   staged when the model has a stager and the GEMM has at least WeightStager.min_rows rows, else packed.
    # The three forms produce the same bits: the unpack kernel writes exactly the fp16 values the packed-weight
    # kernels rebuild on chip.
    weight_form = os.environ.get("ARCQ_WEIGHT_FORM", "auto")
    _scratch: dict = {}

    def _weight_scratch(self) -> torch.Tensor:
        """fp16 scratch of at least N*K elements: the caller's `_weight_buffer` if one was attached (as
        scripts/benchmark_arcq_on_the_fly.py:189-191 does), else one buffer per (device, stream) shared by all
        layers -- they run one after the other on that stream."""
        need = self.out_features * self.in_features
        buf = getattr(self, "_weight_buffer", None)
        if buf is not None and buf.is_cuda and buf.dtype == torch.float16 and buf.is_contiguous() and buf.numel() >= need:
            return buf
        dev = self.packed_weight_codes.device
        key = (dev.index, torch.cuda.current_stream(dev).cuda_stream)
        buf = ARCQPackedLinearOnTheFly._scratch.get(key)
        if buf is None or buf.numel() < need:
            buf = torch.empty(need, dtype=torch.float16, device=dev)
            ARCQPackedLinearOnTheFly._scratch[key] = buf
        return buf

    def _weight_route(self, rows: int) -> str:
        form = self.weight_form
        stager = getattr(self, "_stager", None)
        if form == "auto":
            return "staged" if stager is not None and rows >= stager.min_rows else "packed"
        if form == "staged" and stager is None:
            return "dense"
        return form

    def takes_reconstructed_input(self) -> bool:
        """True if ``forward(x_hat, pre_quantized=True)`` is available: the layer runs the two-kernel route whose
        GEMM reads the reconstructed activation, so a caller may produce that activation itself
        (``ops.add_layernorm_quant`` with this layer's ``activation_thresholds`` / ``activation_codebook``)."""
        return (self.group_size == 64 and self.in_features <= 1024
                and ops.packed_weight_gemm_supported(self.in_features, self.out_features, self.bits, self.group_size))

    def forward(self, x: torch.Tensor, pre_gelu: bool = False, pre_quantized: bool = False) -> torch.Tensor:
        """``pre_gelu=True``: x is the pre-activation of the GELU in front of this layer; the result
        equals ``forward(F.gelu(x))`` with the GELU fused into the activation quantizer.
        ``pre_quantized=True``: x is already this layer's reconstructed activation (see
        ``takes_reconstructed_input``); the quantizer is skipped."""
        if pre_quantized and (pre_gelu or not self.takes_reconstructed_input()):
            raise ValueError("pre_quantized input is not available for this layer / combination")
        shape = x.shape
        if shape[-1] != self.in_features:
            raise ValueError(f"expected last dim {self.in_features}, got {shape[-1]}")
        x2 = x.reshape(-1, self.in_features).to(device=self.packed_weight_codes.device, dtype=torch.float16).contiguous()
        bias = self.bias_tensor if self.bias_tensor.numel() else None
        if ops.packed_weight_gemm_supported(self.in_features, self.out_features, self.bits, self.group_size):
            # the reference's own data flow: fp16 activation quantised and reconstructed (its step 2),
            # then weight unpack + contraction + bias (its steps 3-5) in one persistent kernel
            route = self._weight_route(x2.shape[0])
            if route == "staged":
                w16, ready, prefetch = self._stager.stage(self)     # also arranges the next layer's unpack
            x_hat = x2 if pre_quantized else ops.quantize_activation_dequant(
                x2, self.activation_thresholds, self.activation_codebook, self.bits, self.group_size, torch.float16, pre_gelu)
            if route == "staged":
                if ready is not None:
                    torch.cuda.current_stream(x2.device).wait_event(ready)
                y = ops.dense_weight_gemm(x_hat, w16, bias, torch.float16, prefetch=prefetch)
                self._stager.done(self)
            elif route == "dense":
                w16 = ops.unpack_weight_f16(self.packed_weight_codes, self.weight_center, self.weight_scale,
                                            self.weight_code_sum, self.weight_codebook, self.bits, self.group_size,
                                            out=self._weight_scratch())
                y = ops.dense_weight_gemm(x_hat, w16, bias, torch.float16)
            else:
                y = ops.packed_weight_gemm(x_hat, self.packed_weight_codes, self.weight_center, self.weight_scale,
                                           self.weight_code_sum, self.weight_codebook, bias, self.bits,
                                           self.group_size, torch.float16)
        else:
            # shapes the persistent kernel does not take (e.g. 3-bit rows of 72 bytes): packed codes both sides
            packed_x, mu, sg, cs = ops.quantize_activation(x2, self.activation_thresholds, self.activation_codebook,
                                                           self.bits, self.group_size, True, pre_gelu)
            y = ops.arcq_linear_forward(packed_x, mu, sg, cs, self.packed_weight_codes, self.weight_center,
                                        self.weight_scale, self.weight_code_sum, self.activation_codebook,
                                        self.weight_codebook, bias, self.bits, self.group_size, self.in_features,
                                        self.out_features, torch.float16)
        return y.reshape(*shape[:-1], self.out_features)

    def estimated_persistent_mb(self) -> float:
        return sum(b.numel() * b.element_size() for b in self.buffers()) / 1024 / 1024
