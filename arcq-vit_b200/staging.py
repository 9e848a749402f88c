"""Weight staging for the on-the-fly linears: unpack layer L+1 while layer L computes.

The reference's on-the-fly layer unpacks its weight into a shared fp16 scratch matrix and then calls a dense
GEMM (fair_qat/arcq_packed_on_the_fly.py:147-160, scratch attached by
scripts/benchmark_arcq_on_the_fly.py:189-191).  Here the unpack of the next layer's weight goes into the other of
two scratch matrices while the current layer computes, so that by the time the next layer's activations are
quantised its weight is already in L2 and the GEMM reads both operands by TMA.  Two ways of running that unpack
(``WeightStager.mode``): "stream" (default) -- its own kernel on a side stream, ordered by events; "inline" -- the
epilogue warps of the current layer's GEMM kernel do it before their first accumulator is ready, no extra launch,
stream or event.  Same bits either way; the inline form measured slower at every batch size (DeiT-S batch 1 / 8 / 64:
0.534 / 0.742 / 1.849 ms against 0.506 / 0.727 / 1.817 ms): the side stream hides the unpack completely, inside the
GEMM it delays the first tile's drain.
Nothing but the packed codes is kept between forwards; the scratch is two matrices of the largest layer.

The order of the layers is their registration order in the model (timm's and this package's ViT register
qkv, proj, fc1, fc2 block by block, which is the order they run in).  A layer that is called out of that
order, or on its own, simply unpacks its weight when it is called.

A stager belongs to one model and keeps per-forward state (which layer each scratch matrix holds, the events that
order the two streams): one forward of that model at a time.  Concurrent forwards of the same model from several host
threads need one model copy (and stager) per thread; the packed buffers can be shared.
"""
from __future__ import annotations

import os
from typing import List, Optional, Tuple

import torch
import torch.nn as nn

from . import ops


class WeightStager:
    #: a GEMM with fewer rows than this keeps the packed-weight kernel.  1: always stage -- the hidden unpack plus the
    #: dense pair GEMM measured faster than the fused kernels at every batch size (DeiT-S batch 1 / 8 / 64:
    #: 0.55 / 0.74 / 2.00 ms against 0.67 / 0.91 / 2.24 ms)
    min_rows = 1
    #: "stream": the next layer's weight is unpacked by its own kernel on a side stream; "inline": by the epilogue
    #: warps of this layer's GEMM kernel (measured slower, kept as a tested option)
    mode = os.environ.get("ARCQ_STAGER_MODE", "stream")

    def __init__(self, model: nn.Module, layer_type: type):
        self.layers: List[nn.Module] = [m for m in model.modules() if isinstance(m, layer_type)]
        for i, m in enumerate(self.layers):
            m._stager, m._stage_index = self, i
        self._side: Optional[torch.cuda.Stream] = None
        self._scratch: List[Optional[torch.Tensor]] = [None, None]
        self._reset()
        model.register_forward_pre_hook(self._begin)
        model.register_forward_hook(self._end)

    # ---- per-forward state: which layer each scratch matrix holds, and the events that order the two streams
    def _reset(self) -> None:
        self._holds: List[Optional[int]] = [None, None]
        self._ready: List[Optional[torch.cuda.Event]] = [None, None]     # unpack into scratch b finished
        self._free: List[Optional[torch.cuda.Event]] = [None, None]      # the GEMM that read scratch b finished
        self._side_used = False                                          # the side stream has work of this forward

    def _begin(self, module, args) -> None:
        self._reset()

    def _end(self, module, args, output) -> None:
        if self._side_used:
            torch.cuda.current_stream().wait_stream(self._side)     # nothing of the side stream outlives the forward
        self._reset()

    def _buffer(self, b: int, layer: nn.Module) -> torch.Tensor:
        need = max(m.in_features * m.out_features for m in self.layers)
        buf = self._scratch[b]
        dev = layer.packed_weight_codes.device
        if buf is None or buf.numel() < need or buf.device != dev:
            buf = torch.empty(need, dtype=torch.float16, device=dev)
            self._scratch[b] = buf
            self._holds[b] = None
        return buf

    def _unpack(self, i: int, cur: torch.cuda.Stream) -> None:
        layer, b = self.layers[i], i & 1
        buf = self._buffer(b, layer)
        if self._side is None or self._side.device != buf.device:
            self._side = torch.cuda.Stream(device=buf.device)
        if self._free[b] is not None:
            self._side.wait_event(self._free[b])          # the previous reader of this scratch matrix is done
        else:
            self._side.wait_stream(cur)                   # first use in this forward: order after everything so far
        ops.unpack_weight_f16(layer.packed_weight_codes, layer.weight_center, layer.weight_scale, layer.weight_code_sum,
                              layer.weight_codebook, layer.bits, layer.group_size, out=buf, stream=self._side)
        ev = torch.cuda.Event()
        ev.record(self._side)
        self._ready[b], self._holds[b] = ev, i
        self._side_used = True

    def _unpack_here(self, i: int) -> None:
        """Unpack layer i on the current stream (inline mode: the first layer of a forward, or a layer called out of
        the registered order).  Stream order alone makes this safe: everything that read the matrix was launched
        before."""
        layer, b = self.layers[i], i & 1
        buf = self._buffer(b, layer)
        ops.unpack_weight_f16(layer.packed_weight_codes, layer.weight_center, layer.weight_scale, layer.weight_code_sum,
                              layer.weight_codebook, layer.bits, layer.group_size, out=buf)
        self._ready[b], self._holds[b] = None, i

    def stage(self, layer: nn.Module):
        """(fp16 weight [N, K] of ``layer``, event to wait for before reading it or None, prefetch argument for the
        layer's GEMM or None).  Starts the unpack of the layer registered after it ("stream" mode) or describes it
        for the GEMM to do ("inline" mode).  Call before the layer's activation quantizer is launched."""
        cur = torch.cuda.current_stream(layer.packed_weight_codes.device)
        i = layer._stage_index
        b = i & 1
        inline = self.mode == "inline"
        if self._holds[b] != i:
            self._unpack_here(i) if inline else self._unpack(i, cur)
        prefetch = None
        if i + 1 < len(self.layers) and self._holds[(i + 1) & 1] != i + 1:
            if inline:
                nxt = self.layers[i + 1]
                prefetch = (nxt.packed_weight_codes, nxt.weight_center, nxt.weight_scale, nxt.weight_code_sum,
                            nxt.weight_codebook, nxt.bits, nxt.group_size, self._buffer((i + 1) & 1, nxt))
                self._ready[(i + 1) & 1], self._holds[(i + 1) & 1] = None, i + 1      # done by this layer's GEMM
            else:
                self._unpack(i + 1, cur)
        w16 = self._scratch[b][: layer.out_features * layer.in_features].view(layer.out_features, layer.in_features)
        return w16, self._ready[b], prefetch

    def done(self, layer: nn.Module) -> None:
        """Call after the GEMM that reads the layer's staged weight has been launched."""
        if self.mode == "inline":
            return
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(layer.packed_weight_codes.device))
        self._free[layer._stage_index & 1] = ev

    def scratch_bytes(self) -> int:
        return sum(b.numel() * 2 for b in self._scratch if b is not None)


def attach_weight_stager(model: nn.Module) -> Optional[WeightStager]:
    """Give the on-the-fly linears of ``model`` a common stager (idempotent); None if the model has none."""
    from .packed_linear import ARCQPackedLinearOnTheFly
    old = getattr(model, "_arcq_weight_stager", None)
    layers = [m for m in model.modules() if isinstance(m, ARCQPackedLinearOnTheFly)]
    if old is not None and old.layers == layers:
        return old
    if not layers:
        return None
    if old is not None:
        raise RuntimeError("the model's packed layers changed after a weight stager was attached")
    stager = WeightStager(model, ARCQPackedLinearOnTheFly)
    object.__setattr__(model, "_arcq_weight_stager", stager)
    return stager
