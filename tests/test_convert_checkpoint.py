"""The checkpoint converter: a fake-quant (QAT-style) state-dict in, packed checkpoints out, and back in."""
import importlib.util

import pytest
import torch

from conftest import ROOT


def _converter():
    spec = importlib.util.spec_from_file_location("_arcq_convert_checkpoint", ROOT / "arcq-vit_b200" / "convert_checkpoint.py")
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    return m


def fake_qat_checkpoint(pkg, model_name="deit_tiny", bits=4, depth=2, seed=3):
    """A state-dict laid out like a trained QuantLinearPCARCQ model: '<path>.linear.*' plus compiled codebooks."""
    m = pkg.create_vit(model_name, seed=seed)
    m.blocks = torch.nn.ModuleList(list(m.blocks)[:depth])
    g = torch.Generator().manual_seed(seed)
    state = {}
    q = set(pkg.quantised_linear_names(m))
    for k, v in m.state_dict().items():
        path = k.rsplit(".", 1)[0]
        if path in q:
            state[f"{path}.linear.{k.rsplit('.', 1)[1]}"] = v.clone()
        else:
            state[k] = v.clone()
    for path in q:
        w = state[f"{path}.linear.weight"]
        w_cb, w_th = pkg.codebook.calibrate_codebook(w, bits, 64)
        a_cb, a_th = pkg.codebook.calibrate_codebook(torch.randn(64, w.shape[1], generator=g), bits, 64)
        state[f"{path}.act_quant._pc_cb"], state[f"{path}.act_quant._pc_thresholds"] = a_cb, a_th
        state[f"{path}.weight_quant._pc_cb"], state[f"{path}.weight_quant._pc_thresholds"] = w_cb, w_th
        state[f"{path}.act_quant._pc_step"] = torch.tensor(7)          # training bookkeeping the converter ignores
    return state, depth


def test_converter_writes_one_distinct_file_per_format_and_they_load_back(pkg, tmp_path):
    cc = _converter()
    state, depth = fake_qat_checkpoint(pkg)
    ck = tmp_path / "best.pt"
    torch.save({"model": state, "epoch": 3}, ck)
    # a skeleton of the same depth: the converter builds the full model, so give it a full-depth checkpoint view
    import arcq_vit_b200.vit as vit
    full = pkg.create_vit("deit_tiny", seed=3)
    assert len(full.blocks) == 12
    orig = vit.create_vit
    try:
        def shallow(name, seed=0, num_classes=1000):
            m = orig(name, seed, num_classes)
            m.blocks = torch.nn.ModuleList(list(m.blocks)[:depth])
            return m
        vit.create_vit = shallow
        pkg.create_vit = shallow
        files = cc.convert(ck, "deit_tiny", 4, tmp_path / "out", ["packed", "dequant_gemm"])
        assert [f.name for f in files] == ["deit_tiny_w4a4_packed_packed.pt", "deit_tiny_w4a4_packed_dequant_gemm.pt"]
        a, b = (torch.load(f, map_location="cpu") for f in files)
        k = "blocks.0.attn.qkv.weight_dequant"
        assert a[k].numel() == 0 and b[k].numel() == 192 * 576            # the second file really is the second format
        assert torch.equal(a["blocks.1.mlp.fc2.packed_weight_codes"], b["blocks.1.mlp.fc2.packed_weight_codes"])
        assert not any(".linear." in key or "_pc_" in key for key in a)
        # wrong --bits is caught, and so is a layer without compiled codebooks
        with pytest.raises(ValueError):
            cc.convert(ck, "deit_tiny", 3, tmp_path / "out3", ["packed"])
        broken = dict(state)
        broken["blocks.0.attn.proj.act_quant._pc_cb"] = torch.empty(0)
        torch.save(broken, tmp_path / "broken.pt")
        with pytest.raises(KeyError):
            cc.convert(tmp_path / "broken.pt", "deit_tiny", 4, tmp_path / "outb", ["packed"])
        # the packed file loads into a float skeleton without the QAT model
        skel = shallow("deit_tiny", seed=0)
        loaded = pkg.load_packed_state_dict(skel, a, on_the_fly=True)
        assert pkg.count_packed_linear(loaded) == 4 * depth
        assert torch.equal(loaded.blocks[1].mlp.fc1.packed_weight_codes, a["blocks.1.mlp.fc1.packed_weight_codes"])
        assert torch.equal(loaded.norm.weight, state["norm.weight"])
    finally:
        vit.create_vit = orig
        pkg.create_vit = orig


@pytest.mark.gpu
def test_a_converted_checkpoint_loads_and_runs_like_the_directly_packed_model(pkg, cuda_device, tmp_path):
    cc = _converter()
    state, _ = fake_qat_checkpoint(pkg, depth=12)
    ck = tmp_path / "best.pt"
    torch.save(state, ck)
    (f,) = cc.convert(ck, "deit_tiny", 4, tmp_path / "out", ["packed"])
    loaded = pkg.load_packed_state_dict(pkg.create_vit("deit_tiny", seed=0), torch.load(f, map_location="cpu")).half().to(cuda_device)
    direct = cc.build_packed_model(state, "deit_tiny", 4, "packed")
    direct = pkg.to_on_the_fly(direct).half().to(cuda_device)
    x = torch.randn(8, 3, 224, 224, generator=torch.Generator().manual_seed(2)).half().to(cuda_device)
    with torch.no_grad():
        ya, yb = loaded(x), direct(x)
    assert torch.isfinite(ya).all() and ya.shape == (8, 1000)
    assert torch.equal(ya, yb)
    assert pkg.ops.device_status() == 0
