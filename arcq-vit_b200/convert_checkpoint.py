"""Convert a trained ARCQ fake-quant checkpoint into packed checkpoints.

    python arcq-vit_b200/convert_checkpoint.py --model deit_small --bits 4 \
        --checkpoint runs/.../best.pt --output-dir runs/arcq_packed [--formats packed,dequant_gemm]

Counterpart of the reference's ``scripts/convert_arcq_to_packed.py`` (:29-97).  The checkpoint is the
state-dict of a model whose quantised linears are ``QuantLinearPCARCQ`` modules
(methods/fair_qat_framework/fair_qat/quant_backends.py:282-322): per linear ``<path>.linear.weight``,
``<path>.linear.bias`` and the compiled codebooks ``<path>.act_quant._pc_cb`` / ``._pc_thresholds``,
``<path>.weight_quant._pc_cb`` / ``._pc_thresholds`` (quant/dcarcq.py:452-453, :485-486).  Every such linear
becomes an ``ARCQPackedLinear`` (same buffers and key names as the reference's packed module, so the files
are interchangeable with the reference's); everything else in the checkpoint is copied through.

Differences from the reference script, all of them fixes:
  * each requested format is converted from a fresh copy of the float model -- the reference converts one model
    object in place twice, so its second file holds the first format again (:64-77);
  * the file name comes from ``--model`` and ``--bits`` instead of being fixed to one model (:88), and both
    options are used: ``--bits`` is checked against the codebook sizes found in the checkpoint;
  * a linear without compiled codebooks in the checkpoint is an error, not a silently unconverted layer;
  * no dependency on the training stack: the model skeleton is this package's plain-PyTorch DeiT with the same
    parameter names, and packing runs on the CPU through the NumPy packer.
"""
from __future__ import annotations

import argparse
import copy
import importlib.util
import sys
from pathlib import Path
from typing import Dict, List

import torch
import torch.nn as nn

PKG_DIR = Path(__file__).resolve().parent
PKG_NAME = "arcq_vit_b200"


def _package():
    """This directory as the package ``arcq_vit_b200`` (its name on disk has a hyphen)."""
    if PKG_NAME in sys.modules:
        return sys.modules[PKG_NAME]
    spec = importlib.util.spec_from_file_location(PKG_NAME, PKG_DIR / "__init__.py", submodule_search_locations=[str(PKG_DIR)])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[PKG_NAME] = mod
    spec.loader.exec_module(mod)
    return mod


def read_state(path: Path) -> Dict[str, torch.Tensor]:
    """The model state-dict inside a checkpoint file (bare, or under 'model' / 'state_dict' / 'model_state')."""
    obj = torch.load(path, map_location="cpu", weights_only=False)
    for key in ("model", "state_dict", "model_state", "model_state_dict"):
        if isinstance(obj, dict) and key in obj and isinstance(obj[key], dict):
            obj = obj[key]
            break
    if not isinstance(obj, dict):
        raise ValueError(f"{path}: no state-dict found")
    return {k[len("module."):] if k.startswith("module.") else k: v for k, v in obj.items() if isinstance(v, torch.Tensor)}


def quantised_paths(state: Dict[str, torch.Tensor]) -> List[str]:
    """Paths of the fake-quant linears in a checkpoint: those with a ``.linear.weight`` and a weight quantizer."""
    return sorted(k[: -len(".linear.weight")] for k in state
                  if k.endswith(".linear.weight") and state[k].dim() == 2
                  and any(q.startswith(k[: -len("linear.weight")] + "weight_quant.") for q in state))


def build_packed_model(state: Dict[str, torch.Tensor], model_name: str, bits: int, runtime_code_format: str) -> nn.Module:
    """Float skeleton + checkpoint -> model with packed linears (a fresh model object on every call)."""
    pkg = _package()
    from arcq_vit_b200.vit import _FloatSource, _get, _set
    model = pkg.create_vit(model_name, seed=0)
    paths = quantised_paths(state)
    if not paths:
        raise ValueError("the checkpoint holds no fake-quant linear (no '<path>.linear.weight' with a weight quantizer)")
    used = set()
    for path in paths:
        need = {n: f"{path}.{n}" for n in ("linear.weight", "act_quant._pc_cb", "act_quant._pc_thresholds",
                                             "weight_quant._pc_cb", "weight_quant._pc_thresholds")}
        for n, k in need.items():
            if k not in state or state[k].numel() == 0:
                raise KeyError(f"{path}: the checkpoint has no compiled '{n}' (was the codebook compile step reached?)")
        levels = state[need["act_quant._pc_cb"]].numel()
        if levels != 2 ** bits or state[need["weight_quant._pc_cb"]].numel() != 2 ** bits:
            raise ValueError(f"{path}: codebooks of {levels} / {state[need['weight_quant._pc_cb']].numel()} entries "
                             f"do not match --bits {bits}")
        w = state[need["linear.weight"]].float()
        b = state.get(f"{path}.linear.bias")
        lin = nn.Linear(w.shape[1], w.shape[0], bias=b is not None)
        with torch.no_grad():
            lin.weight.copy_(w)
            if b is not None:
                lin.bias.copy_(b.float())
        gs = int(state[f"{path}.act_quant.group_size"]) if f"{path}.act_quant.group_size" in state else 64
        src = _FloatSource(lin, bits, gs, state[need["act_quant._pc_cb"]].float(), state[need["act_quant._pc_thresholds"]].float(),
                           state[need["weight_quant._pc_cb"]].float(), state[need["weight_quant._pc_thresholds"]].float())
        try:
            _get(model, path)
        except AttributeError:
            raise KeyError(f"{path}: no such module in the {model_name} skeleton")
        _set(model, path, pkg.ARCQPackedLinear(src, runtime_code_format))
        used.update(k for k in state if k.startswith(path + "."))
    rest = {k: v for k, v in state.items() if k not in used}
    own = {k: v for k, v in model.state_dict().items() if not any(k.startswith(p + ".") for p in paths)}
    missing = sorted(set(own) - set(rest))
    if missing:
        raise KeyError(f"the checkpoint lacks {len(missing)} tensors of the {model_name} skeleton, e.g. {missing[:4]}")
    model.load_state_dict({k: rest[k] for k in own}, strict=False)
    model.ignored_checkpoint_keys = sorted(set(rest) - set(own))
    return model.eval()


def convert(checkpoint: Path, model_name: str, bits: int, output_dir: Path, formats: List[str]) -> List[Path]:
    pkg = _package()
    state = read_state(checkpoint)
    output_dir.mkdir(parents=True, exist_ok=True)
    written = []
    for fmt in formats:
        model = build_packed_model(copy.copy(state), model_name, bits, fmt)       # a fresh model per format
        mb = 1024 * 1024
        params = sum(p.numel() * p.element_size() for p in model.parameters()) / mb
        bufs = sum(b.numel() * b.element_size() for b in model.buffers()) / mb
        out = output_dir / f"{model_name}_w{bits}a{bits}_packed_{fmt}.pt"
        torch.save(model.state_dict(), out)
        print(f"[{fmt}] packed_layers={pkg.count_packed_linear(model)} params={params:.1f}MB buffers={bufs:.1f}MB "
              f"file={out.stat().st_size / mb:.1f}MB -> {out}")
        if model.ignored_checkpoint_keys:
            print(f"  ignored {len(model.ignored_checkpoint_keys)} checkpoint tensors without a place in the skeleton, "
                  f"e.g. {model.ignored_checkpoint_keys[:3]}")
        written.append(out)
    return written


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", default="deit_small", choices=["deit_tiny", "deit_small", "deit_base"])
    ap.add_argument("--bits", type=int, default=4, choices=[2, 3, 4])
    ap.add_argument("--checkpoint", type=Path, required=True)
    ap.add_argument("--output-dir", type=Path, required=True)
    ap.add_argument("--formats", default="packed,dequant_gemm", help="comma-separated runtime_code_format values")
    a = ap.parse_args(argv)
    formats = [f for f in a.formats.split(",") if f]
    for f in formats:
        if f not in ("packed", "u8", "dequant_gemm"):
            ap.error(f"unknown format {f}")
    convert(a.checkpoint, a.model, a.bits, a.output_dir, formats)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
