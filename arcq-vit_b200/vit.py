"""Plain-PyTorch DeiT / ViT skeleton that hosts the packed linears (whole-model caller).

The reference builds its models with ``timm.create_model`` (third party, not part of the
reference tree: methods/fair_qat_framework/fair_qat/timm_quant_models.py:163-167) and then swaps
the linears.  This file is an independent skeleton with the same architecture facts --
16x16 patch embedding, class token, learned position embedding, pre-LayerNorm blocks of
multi-head self-attention and a GELU MLP, final LayerNorm, linear head -- and the parameter
names the reference's tools rely on (``blocks.<i>.attn.qkv``, ``blocks.<i>.attn.proj``,
``blocks.<i>.mlp.fc1``, ``blocks.<i>.mlp.fc2``, ``head``).  Only the four linears of each block
are quantised; patch embedding, LayerNorm, softmax attention, GELU and the head stay in
floating point (ordinary PyTorch ops).
"""
from __future__ import annotations

import os
from typing import Callable, Dict, List, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import codebook as cbk
from .packed_linear import ARCQPackedLinear, ARCQPackedLinearOnTheFly
from .staging import attach_weight_stager

# name -> (embed dim, heads, depth); MLP hidden = 4 * dim; 224x224 input, patch 16, 1000 classes
DEIT_CONFIGS: Dict[str, Tuple[int, int, int]] = {
    "deit_tiny": (192, 3, 12),
    "deit_small": (384, 6, 12),
    "deit_base": (768, 12, 12),
}


class Attention(nn.Module):
    # "kernel": this package's attention kernel (heads of 64, at most 256 tokens, fp16 on a GPU), which also runs
    # proj's activation quantizer when proj can take a reconstructed input; "sdpa": the library attention.
    implementation = os.environ.get("ARCQ_ATTENTION", "sdpa")

    def __init__(self, dim: int, heads: int):
        super().__init__()
        self.num_heads = heads
        self.qkv = nn.Linear(dim, 3 * dim)
        self.proj = nn.Linear(dim, dim)

    def forward(self, x: torch.Tensor, pre_quantized: bool = False) -> torch.Tensor:
        B, T, C = x.shape
        qkv = self.qkv(x, pre_quantized=True) if pre_quantized else self.qkv(x)
        if (self.implementation == "kernel" and qkv.is_cuda and qkv.dtype == torch.float16 and C == 64 * self.num_heads
                and T <= 256):
            from . import ops
            proj = self.proj
            if isinstance(proj, ARCQPackedLinearOnTheFly) and proj.takes_reconstructed_input():
                xh = ops.attention(qkv, B, T, self.num_heads, proj.activation_thresholds, proj.activation_codebook,
                                   proj.bits, proj.group_size)
                return proj(xh.reshape(B, T, C), pre_quantized=True)
            return proj(ops.attention(qkv, B, T, self.num_heads).reshape(B, T, C))
        qkv = qkv.reshape(B, T, 3, self.num_heads, C // self.num_heads).permute(2, 0, 3, 1, 4)
        o = F.scaled_dot_product_attention(qkv[0], qkv[1], qkv[2])
        return self.proj(o.transpose(1, 2).reshape(B, T, C))


class Mlp(nn.Module):
    def __init__(self, dim: int, hidden: int):
        super().__init__()
        self.fc1 = nn.Linear(dim, hidden)
        self.fc2 = nn.Linear(hidden, dim)

    def forward(self, x: torch.Tensor, pre_quantized: bool = False) -> torch.Tensor:
        h = self.fc1(x, pre_quantized=True) if pre_quantized else self.fc1(x)
        if getattr(self.fc2, "supports_pre_gelu", False) and h.dtype == torch.float16:
            return self.fc2(h, pre_gelu=True)       # GELU fused into fc2's activation quantizer
        return self.fc2(F.gelu(h))


class Block(nn.Module):
    def __init__(self, dim: int, heads: int):
        super().__init__()
        self.norm1 = nn.LayerNorm(dim, eps=1e-6)
        self.attn = Attention(dim, heads)
        self.norm2 = nn.LayerNorm(dim, eps=1e-6)
        self.mlp = Mlp(dim, 4 * dim)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = x + self.attn(self.norm1(x))
        return x + self.mlp(self.norm2(x))


class PatchEmbed(nn.Module):
    def __init__(self, dim: int, patch: int = 16):
        super().__init__()
        self.proj = nn.Conv2d(3, dim, kernel_size=patch, stride=patch)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        # Non-overlapping patches: the convolution is a matrix product over flattened patches.  Written that
        # way (one gather copy + one GEMM) because the library convolution picked for this shape is slow.
        B, C, H, W = x.shape
        p = self.proj.kernel_size[0]
        gh, gw = H // p, W // p
        if x.is_cuda and x.dtype == torch.float16 and p % 8 == 0 and H % p == 0 and W % p == 0:
            from . import ops
            patches = ops.patchify(x.contiguous(), p)          # the same matrix, gathered with 16-byte accesses
        else:
            patches = x.reshape(B, C, gh, p, gw, p).permute(0, 2, 4, 1, 3, 5).reshape(B, gh * gw, C * p * p)
        return F.linear(patches, self.proj.weight.reshape(self.proj.out_channels, -1), self.proj.bias)


class VisionTransformer(nn.Module):
    # The LayerNorm in front of qkv / fc1 also runs that layer's activation quantizer (one kernel instead of two, the
    # LayerNorm output never leaves the SM): "auto" / "1" wherever the merged kernel is built (rows of 192, 384 or 768
    # values), "0" never.  The merged kernel gives the same bits as the two separate kernels, so the switch changes
    # timing only (DeiT-S batch 64: 1.96 -> 1.85 ms; batch 1: 0.525 -> 0.509 ms).  The library picks a low-latency form
    # of the kernel for inputs of less than one 128-group tile per SM.
    fuse_norm_quant = os.environ.get("ARCQ_LN_QUANT", "auto")

    def __init__(self, dim: int, heads: int, depth: int, num_classes: int = 1000, img_size: int = 224,
                 patch: int = 16):
        super().__init__()
        self.embed_dim, self.num_heads, self.depth = dim, heads, depth
        n_tokens = (img_size // patch) ** 2 + 1
        self.patch_embed = PatchEmbed(dim, patch)
        self.cls_token = nn.Parameter(torch.zeros(1, 1, dim))
        self.pos_embed = nn.Parameter(torch.zeros(1, n_tokens, dim))
        self.blocks = nn.ModuleList(Block(dim, heads) for _ in range(depth))
        self.norm = nn.LayerNorm(dim, eps=1e-6)
        self.head = nn.Linear(dim, num_classes)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = self.patch_embed(x)
        if x.is_cuda and x.dtype == torch.float16 and x.shape[-1] % 8 == 0 and self.cls_token.dtype == torch.float16:
            from . import ops
            x = ops.assemble_tokens(x, self.cls_token, self.pos_embed)     # cat + add in one pass, same bits
        else:
            x = torch.cat([self.cls_token.expand(x.shape[0], -1, -1), x], dim=1) + self.pos_embed
        if x.is_cuda and x.dtype == torch.float16 and x.shape[-1] % 8 == 0 and x.shape[-1] <= 2048:
            return self._forward_fused_glue(x)
        for blk in self.blocks:
            x = blk(x)
        return self.head(self.norm(x)[:, 0])

    def _forward_fused_glue(self, x: torch.Tensor) -> torch.Tensor:
        """Same computation as the loop over blocks, with every residual add merged into the LayerNorm
        that follows it (one kernel instead of two): x += attn(norm1(x)); x += mlp(norm2(x))."""
        from . import ops

        def norm_into(x, y, norm, lin):
            """(x + y, input of `lin`, whether that input is already quantised): the LayerNorm in front of a packed
            linear also runs that linear's activation quantizer when the layer can take the result."""
            mode = self.fuse_norm_quant
            mode = "1" if mode is True else "0" if mode is False else str(mode)
            width = x.shape[-1]
            fuse = mode in ("1", "auto") and width in (192, 384, 768)
            if fuse and isinstance(lin, ARCQPackedLinearOnTheFly) and lin.takes_reconstructed_input():
                s, xh = ops.add_layernorm_quant(x, y, norm, lin.activation_thresholds, lin.activation_codebook,
                                                lin.bits, lin.group_size)
                return s, xh, True
            s, h = ops.add_layernorm(x, y, norm)
            return s, h, False

        n = len(self.blocks)
        _, h, q = norm_into(x, None, self.blocks[0].norm1, self.blocks[0].attn.qkv)
        for i, blk in enumerate(self.blocks):
            a = blk.attn(h, pre_quantized=True) if q else blk.attn(h)
            x, h, q = norm_into(x, a, blk.norm2, blk.mlp.fc1)
            m = blk.mlp(h, pre_quantized=True) if q else blk.mlp(h)
            if i + 1 < n:
                x, h, q = norm_into(x, m, self.blocks[i + 1].norm1, self.blocks[i + 1].attn.qkv)
            else:
                x, h = ops.add_layernorm(x, m, self.norm)
        return self.head(h[:, 0])


def create_vit(name: str, seed: int = 0, num_classes: int = 1000) -> VisionTransformer:
    """Random-init model: truncated-normal(0.02) linear / embedding weights, zero biases except a
    small normal(0.01) bias on the quantised linears (so the bias path is exercised), ones/zeros
    LayerNorm.  No pretrained weights exist offline; every measurement uses this recipe."""
    dim, heads, depth = DEIT_CONFIGS[name]
    g = torch.Generator().manual_seed(seed)
    m = VisionTransformer(dim, heads, depth, num_classes)
    with torch.no_grad():
        for n, p in m.named_parameters():
            if p.dim() >= 2 or n in ("cls_token", "pos_embed"):
                p.copy_(torch.empty_like(p).normal_(0.0, 0.02, generator=g).clamp_(-0.04, 0.04))
            elif "norm" in n:
                p.fill_(1.0 if n.endswith("weight") else 0.0)
            elif any(k in n for k in ("qkv", "proj", "fc1", "fc2")) and "patch_embed" not in n:
                p.copy_(torch.empty_like(p).normal_(0.0, 0.01, generator=g))
            else:
                p.zero_()
    return m.eval()


def quantised_linear_names(model: nn.Module) -> List[str]:
    """Paths of the quantised linears: qkv / proj / fc1 / fc2 of every block, forward order."""
    out = []
    for i, _ in enumerate(model.blocks):
        out += [f"blocks.{i}.attn.qkv", f"blocks.{i}.attn.proj", f"blocks.{i}.mlp.fc1", f"blocks.{i}.mlp.fc2"]
    return out


def _get(model: nn.Module, path: str) -> nn.Module:
    for part in path.split("."):
        model = getattr(model, part)
    return model


def _set(model: nn.Module, path: str, new: nn.Module) -> None:
    parts = path.split(".")
    setattr(_get(model, ".".join(parts[:-1])) if len(parts) > 1 else model, parts[-1], new)


class _FloatSource(nn.Module):
    """Minimal stand-in for a trained fake-quant layer: what ``ARCQPackedLinear(source)`` reads."""

    class _Q(nn.Module):
        def __init__(self, bits, group_size, cb, th):
            super().__init__()
            self.bits, self.group_size, self.eps = bits, group_size, 1e-6
            self._pc_cb, self._pc_thresholds = cb, th

    def __init__(self, linear: nn.Linear, bits: int, group_size: int, a_cb, a_th, w_cb, w_th):
        super().__init__()
        self.linear = linear
        self.act_quant = self._Q(bits, group_size, a_cb, a_th)
        self.weight_quant = self._Q(bits, group_size, w_cb, w_th)


def pack_linear(linear: nn.Linear, bits: int, act_codebook, act_thresholds, w_codebook=None, w_thresholds=None,
                group_size: int = 64, on_the_fly: bool = True) -> nn.Module:
    """nn.Linear + codebooks -> packed linear.  Without weight codebooks, fit them to the weight."""
    if w_codebook is None:
        w_codebook, w_thresholds = cbk.calibrate_codebook(linear.weight, bits, group_size)
    src = _FloatSource(linear, bits, group_size, act_codebook, act_thresholds, w_codebook, w_thresholds)
    packed = ARCQPackedLinear(src, "packed")
    return ARCQPackedLinearOnTheFly.from_packed(packed) if on_the_fly else packed


class _CalibratingLinear(nn.Module):
    """First forward: fit the activation codebook on the incoming tensor and the weight codebook
    on the weight (the reference's step-0 codebook compile, quant/dcarcq.py:540-547), build the
    packed layer, run it.  Later forwards just run it."""

    def __init__(self, linear: nn.Linear, bits: int, group_size: int, on_the_fly: bool):
        super().__init__()
        self.linear, self.bits, self.group_size, self.on_the_fly = linear, bits, group_size, on_the_fly
        self.packed = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.packed is None:
            a_cb, a_th = cbk.calibrate_codebook(x.reshape(-1, x.shape[-1]), self.bits, self.group_size)
            self.packed = pack_linear(self.linear, self.bits, a_cb, a_th, group_size=self.group_size,
                                      on_the_fly=self.on_the_fly)
        return self.packed(x)


@torch.no_grad()
def quantise_model(model: VisionTransformer, calib_images: torch.Tensor, bits: int, group_size: int = 64,
                   on_the_fly: bool = True) -> VisionTransformer:
    """Float model (already on its device / dtype) -> packed model, codebooks calibrated on one batch
    layer by layer in forward order and then frozen."""
    names = quantised_linear_names(model)
    for n in names:
        _set(model, n, _CalibratingLinear(_get(model, n), bits, group_size, on_the_fly))
    model(calib_images)
    for n in names:
        _set(model, n, _get(model, n).packed)
    if on_the_fly:
        attach_weight_stager(model)
    return model


@torch.no_grad()
def pack_model_with_codebooks(model: VisionTransformer, codebooks: Dict[str, Dict[str, torch.Tensor]], bits: int,
                              group_size: int = 64, on_the_fly: bool = True) -> VisionTransformer:
    """Float model + given codebooks per layer path ({'act_cb','act_th','w_cb','w_th'}) -> packed model."""
    for n in quantised_linear_names(model):
        c = codebooks[n]
        _set(model, n, pack_linear(_get(model, n), bits, c["act_cb"], c["act_th"], c["w_cb"], c["w_th"], group_size,
                                   on_the_fly))
    if on_the_fly:
        attach_weight_stager(model)
    return model


class GraphedModel:
    """Whole-model CUDA-graph replay for a fixed batch shape (the reference captures the model the
    same way at batch 1, scripts/benchmark_arcq_on_the_fly.py:223-231)."""

    def __init__(self, model: nn.Module, example: torch.Tensor, warmup: int = 3):
        self.static_in = example.clone()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(warmup):
                model(self.static_in)
        torch.cuda.current_stream().wait_stream(side)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph), torch.no_grad():
            self.static_out = model(self.static_in)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        self.static_in.copy_(x, non_blocking=True)
        self.graph.replay()
        return self.static_out


class HostPipeline:
    """Feeds pinned host batches to a model (or a ``GraphedModel``) and returns the logits in pinned host
    memory.  Batch i+1 is copied to the device on a second stream while batch i computes, and the caller reads
    the logits of batch i-1 meanwhile; every batch still pays its own host-to-device copy and its own
    device-to-host read.  Two device staging buffers and two host result buffers alternate."""

    def __init__(self, runner, example_host: torch.Tensor, out_shape, device=None, out_dtype=torch.float16):
        device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        self.runner = runner
        self.copy_stream = torch.cuda.Stream(device=device)
        self.stage = [torch.empty(example_host.shape, dtype=example_host.dtype, device=device) for _ in range(2)]
        self.out_host = [torch.empty(tuple(out_shape), dtype=out_dtype).pin_memory() for _ in range(2)]
        self.h2d_done = [torch.cuda.Event() for _ in range(2)]
        self.slot_free = [torch.cuda.Event() for _ in range(2)]
        self.out_done = [torch.cuda.Event() for _ in range(2)]

    def run(self, host_batches, on_result=None) -> int:
        """Process an iterable of pinned host tensors; ``on_result(logits_host)`` is called once per batch,
        in order, when that batch's logits have arrived.  Returns the number of batches."""
        cur = torch.cuda.current_stream()
        prev, n = None, 0
        for hb in host_batches:
            s = n & 1
            with torch.cuda.stream(self.copy_stream):
                self.copy_stream.wait_event(self.slot_free[s])      # the step that read this buffer is over
                self.stage[s].copy_(hb, non_blocking=True)
                self.h2d_done[s].record(self.copy_stream)
            cur.wait_event(self.h2d_done[s])
            with torch.no_grad():
                y = self.runner(self.stage[s])
            self.slot_free[s].record(cur)
            self.out_host[s].copy_(y, non_blocking=True)
            self.out_done[s].record(cur)
            if prev is not None:
                self.out_done[prev].synchronize()
                if on_result is not None:
                    on_result(self.out_host[prev])
            prev = s
            n += 1
        if prev is not None:
            self.out_done[prev].synchronize()
            if on_result is not None:
                on_result(self.out_host[prev])
        return n

