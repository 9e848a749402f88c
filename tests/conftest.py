import json
import os
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import __graft_entry__ as entry  # noqa: E402

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def pkg():
    entry.build()
    return entry.import_package()


@pytest.fixture(scope="session")
def oracle():
    o = entry.import_oracle()
    o.build()
    return o


def _load_golden(name: str):
    """Fixture file + its regenerated inputs (hash-checked)."""
    sys.path.insert(0, str(GOLDEN))
    import make_golden
    g = dict(np.load(GOLDEN / f"{name}.npz", allow_pickle=False))
    M, K, N, bits, seed, outliers, gs = (int(v) for v in g["spec"])
    X, W, b = make_golden.golden_inputs(M, K, N, seed, outliers)
    assert make_golden.input_hash(X, W, b) == str(g["input_sha256"]), "golden inputs are not reproduced on this host"
    g.update(X=X, W=W, b=b, M=M, K=K, N=N, bits=bits, gs=gs)
    return g


_cache = {}


@pytest.fixture(scope="session")
def golden():
    def get(name):
        if name not in _cache:
            _cache[name] = _load_golden(name)
        return _cache[name]
    return get


GOLDEN_CASES = ["c1_w4a4", "c1_w3a3", "edge_k64_w4a4", "edge_k192_w3a3", "edge_k1536_w4a4"]


def ulp_diff(a: np.ndarray, b: np.ndarray) -> int:
    """Largest distance in units in the last place between two positive fp32 arrays."""
    return int(np.abs(a.view(np.int32).astype(np.int64) - b.view(np.int32).astype(np.int64)).max())


@pytest.fixture(scope="session")
def cuda_device():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


@pytest.fixture(scope="session")
def report(tmp_path_factory):
    """Append one JSON record per call to ``parity_report.jsonl`` in the directory named by the environment
    variable ARCQ_REPORT_DIR, or in pytest's temporary directory when it is unset."""
    d = os.environ.get("ARCQ_REPORT_DIR")
    out = Path(d) if d else tmp_path_factory.getbasetemp()
    out.mkdir(parents=True, exist_ok=True)

    def write(name, **kw):
        with open(out / "parity_report.jsonl", "a") as f:
            f.write(json.dumps(dict(test=name, **kw)) + "\n")
    return write
