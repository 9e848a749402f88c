"""Generate the golden fixtures in this directory from the reference implementation.

Run where the reference checkout is available:

    python tests/golden/make_golden.py --reference /path/to/ARCQ-ViT

It imports, unmodified, the reference's quantizer (``quant/dcarcq.py``), its
fake-quant linear (``fair_qat/quant_backends.py::QuantLinearPCARCQ``), its
NumPy bit packer (``fair_qat/arcq_packed_py.py``) and its packed-linear
constructor (``fair_qat/arcq_packed_linear.py::ARCQPackedLinear``; the CUDA
extension that module imports is replaced by the NumPy packer exactly as the
reference's own ``scripts/convert_arcq_to_packed.py:56-59`` does), runs them on
CPU in fp32 on seeded inputs and stores their outputs as ``.npz`` files.

Inputs come from ``numpy.random.default_rng(seed)`` rather than from torch's
generator so that they are reproduced bit for bit on any host; each fixture
stores a SHA-256 of its inputs and tests re-create the inputs with
``golden_inputs`` below and check the hash before using the fixture.

The reference's tests hold no golden vectors (there is no test suite), so these
fixtures are the pin between the oracle under ``oracle/`` and the reference.
"""
from __future__ import annotations

import argparse
import hashlib
import sys
import types
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent

# name -> (M, K, N, bits, seed, outliers)
CASES = {
    # the single-linear configuration: X [8*197, 384] ~ N(0,1) with 4 channels x20, W [1536,384] ~ N(0,0.02)
    "c1_w4a4": dict(M=8 * 197, K=384, N=1536, bits=4, seed=0, outliers=4),
    "c1_w3a3": dict(M=8 * 197, K=384, N=1536, bits=3, seed=0, outliers=4),
    # ragged / small cases: one group, odd row count; 3-bit rows of 72 bytes (K=192)
    "edge_k64_w4a4": dict(M=5, K=64, N=8, bits=4, seed=11, outliers=1),
    "edge_k192_w3a3": dict(M=197, K=192, N=72, bits=3, seed=12, outliers=2),
    "edge_k1536_w4a4": dict(M=67, K=1536, N=384, bits=4, seed=13, outliers=4),
}


def golden_inputs(M: int, K: int, N: int, seed: int, outliers: int):
    """Seeded inputs of a fixture: X, W, bias as fp32 arrays."""
    rng = np.random.default_rng(seed)
    X = rng.standard_normal((M, K), dtype=np.float32)
    cols = rng.permutation(K)[:outliers]
    X[:, cols] *= np.float32(20.0)
    W = (rng.standard_normal((N, K), dtype=np.float32) * np.float32(0.02)).astype(np.float32)
    b = (rng.standard_normal((N,), dtype=np.float32) * np.float32(0.01)).astype(np.float32)
    return X, W, b


def input_hash(X, W, b) -> str:
    h = hashlib.sha256()
    for a in (X, W, b):
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def _import_reference(root: Path):
    sys.path.insert(0, str(root / "methods" / "fair_qat_framework"))
    from fair_qat.arcq_packed_py import pack_codes_py, unpack_codes_py
    stub = types.ModuleType("fair_qat.arcq_infer_cuda")
    for n in ("arcq_linear_forward", "arcq_linear_forward_u8", "quantize_activation",
              "quantize_activation_dequant", "quantize_activation_u8", "unpack_codes"):
        setattr(stub, n, None)
    stub.pack_codes, stub.unpack_codes_u8 = pack_codes_py, unpack_codes_py
    sys.modules["fair_qat.arcq_infer_cuda"] = stub
    import fair_qat.arcq_packed_linear as dpl
    from fair_qat.quant_backends import QuantLinearPCARCQ
    return dpl, QuantLinearPCARCQ, pack_codes_py, unpack_codes_py


def make_case(name: str, spec: dict, ref) -> None:
    import torch
    dpl, QuantLinearPCARCQ, pack_codes_py, unpack_codes_py = ref
    M, K, N, bits = spec["M"], spec["K"], spec["N"], spec["bits"]
    X, W, b = golden_inputs(M, K, N, spec["seed"], spec["outliers"])
    torch.manual_seed(0)
    lin = QuantLinearPCARCQ(K, N, True, bits, bits, group_size=64)
    with torch.no_grad():
        lin.linear.weight.copy_(torch.from_numpy(W))
        lin.linear.bias.copy_(torch.from_numpy(b))
        xt = torch.from_numpy(X)
        lin(xt)                                   # the calibrating forward: compiles both codebooks
        for q in (lin.act_quant, lin.weight_quant):
            q.compile_steps = set()               # freeze, as mark_arcq_codebooks_ready does
        y_ref = lin(xt).numpy()
        x_fq = lin.act_quant(xt).numpy()
    aq, wq = lin.act_quant, lin.weight_quant
    a_codes, a_mu, a_sigma, a_cs = dpl._quantize_weight_reference(xt, aq._pc_thresholds, aq._pc_cb, 64, 1e-6)
    packed = dpl.ARCQPackedLinear(lin, "packed")
    sd = {k: v.numpy() for k, v in packed.state_dict().items()}
    w_codes = unpack_codes_py(packed.packed_weight_codes, bits, K).numpy().astype(np.uint8)
    out = dict(
        input_sha256=np.array(input_hash(X, W, b)),
        spec=np.array([M, K, N, bits, spec["seed"], spec["outliers"], 64], np.int64),
        act_codebook=aq._pc_cb.numpy(), act_thresholds=aq._pc_thresholds.numpy(),
        w_codebook=wq._pc_cb.numpy(), w_thresholds=wq._pc_thresholds.numpy(),
        act_packed=pack_codes_py(a_codes, bits).numpy(),
        act_mu=a_mu.numpy(), act_sigma=a_sigma.numpy(), act_code_sum=a_cs.numpy(),
        w_codes_sha256=np.array(hashlib.sha256(w_codes.tobytes()).hexdigest()),
        x_fq_sha256=np.array(hashlib.sha256(np.ascontiguousarray(x_fq).tobytes()).hexdigest()),
        x_fq_head=x_fq[:16].copy(),
        y_ref_sub=y_ref[::16, ::4].copy(),
        y_ref_rms=np.array(float(np.sqrt(np.mean(y_ref.astype(np.float64) ** 2)))),
        state_dict_keys=np.array(list(sd.keys())),
    )
    for k, v in sd.items():
        out["sd." + k] = v
    np.savez_compressed(HERE / f"{name}.npz", **out)
    print(f"{name}: wrote {(HERE / (name + '.npz')).stat().st_size / 1024:.0f} KiB")


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project (ARCQ-ViT)")
    ap.add_argument("--only", default="")
    args = ap.parse_args()
    ref = _import_reference(Path(args.reference))
    for name, spec in CASES.items():
        if args.only and name not in args.only.split(","):
            continue
        make_case(name, spec, ref)


if __name__ == "__main__":
    main()
