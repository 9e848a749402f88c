"""CPU fake-quant DeiT: the whole-model oracle and the timed CPU baseline.  TEST INFRASTRUCTURE ONLY.

Restates, on host cores in fp32, what the reference's CPU path computes for a DeiT whose
qkv / proj / fc1 / fc2 linears are ``QuantLinearPCARCQ`` (methods/fair_qat_framework/fair_qat/
quant_backends.py:282-322): both operands fake-quantised by the group-residual quantizer
(quant/dcarcq.py:512-578) and contracted with the host BLAS in fp32.  The quantizer is the C
restatement in ``arcq_oracle.c`` (fixed summation order), the floating-point glue (patch
embedding, LayerNorm, softmax attention, GELU, head) uses torch CPU ops in fp32.  The
surrounding ViT follows the architecture facts of DeiT (the reference takes it from timm, which
is not part of its tree); weights come from a state-dict with timm-style names.

Parity status: the per-layer quantizer is pinned to the reference through the golden fixtures;
the ViT glue has no reference counterpart in the tree to pin against.
"""
from __future__ import annotations

from typing import Dict, Optional

import numpy as np
import torch
import torch.nn.functional as F

from . import arcq_oracle as O


class OracleViT:
    def __init__(self, state_dict: Dict[str, torch.Tensor], dim: int, heads: int, depth: int, bits: int,
                 group_size: int = 64, patch: int = 16, cache_weights: bool = True, fp16_operands: bool = False):
        self.sd = {k: v.detach().float().cpu() for k, v in state_dict.items()}
        self.dim, self.heads, self.depth, self.bits, self.gs, self.patch = dim, heads, depth, bits, group_size, patch
        # the reference fake-quantises the weight again on every forward (quant_backends.py:320);
        # cache_weights=False does the same (for timing), True keeps the identical result (for tests)
        self.cache_weights = cache_weights
        # True: both fake-quantised operands are rounded to fp16 before the fp32 contraction (what any half-precision
        # tensor-core path does to them); everything else unchanged.  Used to measure how far a rounding-only change
        # moves the logits of this model.
        self.fp16_operands = fp16_operands
        self.codebooks: Dict[str, Dict[str, np.ndarray]] = {}
        self._w_hat: Dict[str, np.ndarray] = {}

    def layer_names(self):
        out = []
        for i in range(self.depth):
            out += [f"blocks.{i}.attn.qkv", f"blocks.{i}.attn.proj", f"blocks.{i}.mlp.fc1", f"blocks.{i}.mlp.fc2"]
        return out

    # -- one quantised linear -------------------------------------------------------------
    def _qlinear(self, name: str, x: torch.Tensor, capture: Optional[dict]) -> torch.Tensor:
        W = self.sd[name + ".weight"].numpy()
        b = self.sd[name + ".bias"].numpy() if name + ".bias" in self.sd else None
        x2 = x.reshape(-1, x.shape[-1]).numpy()
        if name not in self.codebooks:          # the calibrating (first) forward: compile both codebooks
            a_cb, a_th = O.calibrate(x2, self.bits, self.gs)
            w_cb, w_th = O.calibrate(W, self.bits, self.gs)
            self.codebooks[name] = dict(act_cb=a_cb, act_th=a_th, w_cb=w_cb, w_th=w_th)
        c = self.codebooks[name]
        if name not in self._w_hat or not self.cache_weights:
            Wf = np.ascontiguousarray(W, np.float32)
            self._w_hat[name] = O.fake_quant(Wf, c["w_th"], c["w_cb"], self.gs)   # Wf + (W_hat - Wf)
        ca, mu, sg, _ = O.quantize(x2, c["act_th"], c["act_cb"], self.gs)
        xf = np.ascontiguousarray(x2, np.float32)
        x_hat = xf + (O.dequant(ca, mu, sg, c["act_cb"], self.gs) - xf)
        xt, wt = torch.from_numpy(x_hat), torch.from_numpy(self._w_hat[name])
        if self.fp16_operands:
            xt, wt = xt.half().float(), wt.half().float()
        y = xt @ wt.T
        if b is not None:
            y = y + torch.from_numpy(b)
        if capture is not None:
            capture[name] = dict(x=x2.copy(), act_codes=ca, y=y.numpy().copy())
        return y.reshape(*x.shape[:-1], -1)

    # -- whole model ----------------------------------------------------------------------
    @torch.no_grad()
    def forward(self, images: torch.Tensor, capture: Optional[dict] = None) -> torch.Tensor:
        sd = self.sd
        x = F.conv2d(images.float(), sd["patch_embed.proj.weight"], sd["patch_embed.proj.bias"], stride=self.patch)
        x = x.flatten(2).transpose(1, 2)
        x = torch.cat([sd["cls_token"].expand(x.shape[0], -1, -1), x], dim=1) + sd["pos_embed"]
        B, T, C = x.shape
        hd = C // self.heads
        for i in range(self.depth):
            p = f"blocks.{i}."
            h = F.layer_norm(x, (C,), sd[p + "norm1.weight"], sd[p + "norm1.bias"], 1e-6)
            qkv = self._qlinear(p + "attn.qkv", h, capture).reshape(B, T, 3, self.heads, hd).permute(2, 0, 3, 1, 4)
            att = torch.softmax((qkv[0] @ qkv[1].transpose(-2, -1)) * hd ** -0.5, dim=-1) @ qkv[2]
            x = x + self._qlinear(p + "attn.proj", att.transpose(1, 2).reshape(B, T, C), capture)
            h = F.layer_norm(x, (C,), sd[p + "norm2.weight"], sd[p + "norm2.bias"], 1e-6)
            h = F.gelu(self._qlinear(p + "mlp.fc1", h, capture))
            x = x + self._qlinear(p + "mlp.fc2", h, capture)
        x = F.layer_norm(x, (C,), sd["norm.weight"], sd["norm.bias"], 1e-6)
        return x[:, 0] @ sd["head.weight"].T + sd["head.bias"]

    __call__ = forward

    def codebooks_as_torch(self):
        return {n: {k: torch.from_numpy(v) for k, v in c.items()} for n, c in self.codebooks.items()}
