"""Host-side wiring of the weight stager (no GPU): which layers it adopts, in which order, idempotence, and the route
an on-the-fly layer reports with and without one."""
import numpy as np
import pytest
import torch


def _packed_toy_model(pkg):
    """Two packed on-the-fly linears inside a plain module tree, built on the CPU from hand-made buffers."""
    def layer(n, k, seed):
        g = torch.Generator().manual_seed(seed)
        G = k // 64
        cb = torch.sort(torch.randn(16, generator=g))[0]
        th = (cb[:-1] + cb[1:]) / 2
        codes = torch.randint(0, 256, (n, k // 2), generator=g, dtype=torch.uint8)
        stats = lambda: torch.randn(n, G, generator=g)  # noqa: E731
        return pkg.ARCQPackedLinearOnTheFly(k, n, True, codes, cb, stats(), stats().abs() + 0.1, stats(), cb, th, 4, 64,
                                            torch.zeros(n))
    class Toy(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.a = layer(128, 64, 1)
            self.mid = torch.nn.Sequential(torch.nn.Identity(), layer(64, 128, 2))
            self.plain = torch.nn.Linear(4, 4)
    return Toy()


def test_stager_adopts_the_packed_layers_in_registration_order(pkg):
    model = _packed_toy_model(pkg)
    assert model.a._weight_route(5000) == "packed"             # no stager yet
    stager = pkg.attach_weight_stager(model)
    assert stager is not None and stager.layers == [model.a, model.mid[1]]
    assert [m._stage_index for m in stager.layers] == [0, 1] and all(m._stager is stager for m in stager.layers)
    assert pkg.attach_weight_stager(model) is stager            # idempotent
    assert model.a._weight_route(1) == "staged" and model.a._weight_route(5000) == "staged"
    saved = pkg.ARCQPackedLinearOnTheFly.weight_form
    try:
        pkg.ARCQPackedLinearOnTheFly.weight_form = "packed"
        assert model.a._weight_route(5000) == "packed"
        pkg.ARCQPackedLinearOnTheFly.weight_form = "dense"
        assert model.a._weight_route(5000) == "dense"
    finally:
        pkg.ARCQPackedLinearOnTheFly.weight_form = saved
    assert stager.scratch_bytes() == 0                           # nothing is allocated before the first forward
    # a model whose packed layers changed after the stager was attached is refused instead of silently mis-ordered
    model.b = _packed_toy_model(pkg).a
    with pytest.raises(RuntimeError):
        pkg.attach_weight_stager(model)


def test_model_without_packed_layers_gets_no_stager(pkg):
    assert pkg.attach_weight_stager(torch.nn.Sequential(torch.nn.Linear(3, 3))) is None
    lone = _packed_toy_model(pkg).a
    assert lone._weight_route(4096) == "packed"
    saved = pkg.ARCQPackedLinearOnTheFly.weight_form
    try:
        pkg.ARCQPackedLinearOnTheFly.weight_form = "staged"      # asked for, but there is no stager: unpack in place
        assert lone._weight_route(4096) == "dense"
    finally:
        pkg.ARCQPackedLinearOnTheFly.weight_form = saved
