"""Install the reference's own implementation of the path next to this repository, unmodified.

    python baseline/install_ref.py --reference /path/to/ARCQ-ViT

copies the handful of reference files that implement the packed on-the-fly inference path and its
fake-quant oracle into ``baseline/_ref/`` (git-ignored; byte-for-byte copies, checked by SHA-256 and
listed in ``baseline/_ref/MANIFEST.json``):

    fair_qat/arcq_packed_on_the_fly.py   the module whose forward this repository replaces (Triton back end)
    fair_qat/arcq_packed_triton.py       its two Triton kernels
    fair_qat/arcq_packed_linear.py       the packed module / state-dict writer (extension-backed)
    fair_qat/arcq_packed_py.py           NumPy bit packer
    fair_qat/arcq_packed_convert.py      model converter
    fair_qat/quant_backends.py           QuantLinearPCARCQ, the fake-quant layer
    quant/dcarcq.py                      the quantizer

``bench.py`` times them as baselines when they are present (``baseline/ref_runner.py``): the fake-quant model
on the host cores and the Triton path on the GPU.  Nothing under ``baseline/_ref`` is part of the product
and nothing in the package imports it.  The reference is a plain Python tree (no build step, no
``setup.py``), so "installing" it is this copy.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import shutil
from pathlib import Path

HERE = Path(__file__).resolve().parent
DEST = HERE / "_ref"
FQ = Path("methods") / "fair_qat_framework"
FILES = [
    "fair_qat/__init__.py",
    "fair_qat/arcq_packed_on_the_fly.py",
    "fair_qat/arcq_packed_triton.py",
    "fair_qat/arcq_packed_linear.py",
    "fair_qat/arcq_packed_py.py",
    "fair_qat/arcq_packed_convert.py",
    "fair_qat/quant_backends.py",
    "quant/__init__.py",
    "quant/dcarcq.py",
]


def _sha(p: Path) -> str:
    return hashlib.sha256(p.read_bytes()).hexdigest()


def install(reference: Path, dest: Path = DEST) -> dict:
    src_root = reference / FQ
    if not src_root.is_dir():
        raise FileNotFoundError(f"{src_root} not found: --reference must point at an ARCQ-ViT checkout")
    manifest = {}
    for rel in FILES:
        src, dst = src_root / rel, dest / rel
        dst.parent.mkdir(parents=True, exist_ok=True)
        shutil.copyfile(src, dst)
        if _sha(src) != _sha(dst):
            raise RuntimeError(f"copy of {rel} differs from its source")
        manifest[rel] = _sha(dst)
    (dest / "MANIFEST.json").write_text(json.dumps({"source": str(FQ), "files": manifest}, indent=1))
    return manifest


def is_installed(dest: Path = DEST) -> bool:
    m = dest / "MANIFEST.json"
    if not m.exists():
        return False
    try:
        files = json.loads(m.read_text())["files"]
    except (ValueError, KeyError):
        return False
    return all((dest / rel).exists() and _sha(dest / rel) == h for rel, h in files.items()) and set(files) == set(FILES)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", type=Path, required=True, help="root of an ARCQ-ViT checkout")
    a = ap.parse_args()
    m = install(a.reference)
    print(f"installed {len(m)} reference files into {DEST}")
