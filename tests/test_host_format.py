"""Host-side format layer and module boundary (no GPU)."""
import re

import numpy as np
import pytest
import torch

from conftest import GOLDEN_CASES, ROOT, ulp_diff


@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("length", [1, 7, 8, 63, 64, 192, 385])
def test_pack_unpack_agree_with_oracle(pkg, oracle, bits, length):
    rng = np.random.default_rng(bits * 1000 + length)
    codes = rng.integers(0, 2 ** bits, size=(5, length), dtype=np.uint8)
    packed = pkg.packing.pack_codes(torch.from_numpy(codes).long(), bits)
    assert packed.dtype == torch.uint8 and tuple(packed.shape) == (5, (length * bits + 7) // 8)
    assert np.array_equal(packed.numpy(), oracle.pack(codes, bits))
    assert np.array_equal(pkg.packing.unpack_codes_u8(packed, bits, length).numpy(), codes)
    assert pkg.packing.unpack_codes(packed, bits, length).dtype == torch.int64


def test_pack_rejects_bad_arguments(pkg):
    with pytest.raises(ValueError):
        pkg.packing.pack_codes(torch.zeros(4, 8, dtype=torch.long), 5)
    with pytest.raises(ValueError):
        pkg.packing.pack_codes(torch.zeros(8, dtype=torch.long), 4)


def _source(pkg, g):
    from arcq_vit_b200.vit import _FloatSource
    lin = torch.nn.Linear(g["K"], g["N"])
    with torch.no_grad():
        lin.weight.copy_(torch.from_numpy(g["W"]))
        lin.bias.copy_(torch.from_numpy(g["b"]))
    t = torch.from_numpy
    return _FloatSource(lin, g["bits"], g["gs"], t(g["act_codebook"]), t(g["act_thresholds"]), t(g["w_codebook"]),
                        t(g["w_thresholds"]))


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_packed_state_dict_equals_reference(pkg, golden, name):
    g = golden(name)
    layer = pkg.ARCQPackedLinear(_source(pkg, g), "packed")
    sd = layer.state_dict()
    assert list(sd.keys()) == [str(k) for k in g["state_dict_keys"]]
    for k, v in sd.items():
        ref = g["sd." + k]
        assert tuple(v.shape) == ref.shape and str(v.numpy().dtype) == str(ref.dtype), k
        if k == "weight_scale":
            assert ulp_diff(v.numpy(), ref) <= 1
        else:
            assert np.array_equal(v.numpy(), ref), k
    assert layer.in_features == g["K"] and layer.out_features == g["N"] and layer.bits == g["bits"]
    assert layer.packed_weight_bytes == g["N"] * g["K"] * g["bits"] // 8
    assert layer.estimated_storage_bytes() > layer.packed_weight_bytes and layer.runtime_cache_bytes() == 0


def test_round_trip_through_state_dict_and_formats(pkg, golden):
    g = golden("edge_k192_w3a3")
    layer = pkg.ARCQPackedLinear(_source(pkg, g), "packed")
    sd = {"blocks.0.attn.qkv." + k: v for k, v in layer.state_dict().items()}
    again = pkg.ARCQPackedLinear.from_state_dict(sd, "blocks.0.attn.qkv.")
    assert (again.bits, again.group_size, again.in_features, again.out_features) == (3, 64, 192, 72)
    for k, v in layer.state_dict().items():
        assert torch.equal(v, again.state_dict()[k]), k
    u8 = pkg.ARCQPackedLinear(_source(pkg, g), "u8")
    assert tuple(u8.weight_codes_u8.shape) == (72, 192) and u8.runtime_cache_bytes() == 72 * 192
    dq = pkg.ARCQPackedLinear(_source(pkg, g), "dequant_gemm")
    assert dq.weight_dequant.dtype == torch.float16 and tuple(dq.weight_dequant.shape) == (72, 192)
    otf = pkg.ARCQPackedLinearOnTheFly.from_packed(layer)
    assert otf.groups == 3 and otf.estimated_persistent_mb() > 0
    assert otf.packed_weight_codes.data_ptr() == layer.packed_weight_codes.data_ptr()   # buffers are shared


def test_constructor_and_forward_errors(pkg, golden):
    g = golden("edge_k64_w4a4")
    src = _source(pkg, g)
    with pytest.raises(ValueError):
        pkg.ARCQPackedLinear(src, "int8")
    with pytest.raises(TypeError):
        pkg.ARCQPackedLinear(torch.nn.Linear(64, 8))
    src.act_quant.bits = 3
    with pytest.raises(ValueError):
        pkg.ARCQPackedLinear(src)
    src.act_quant.bits = 4
    src.act_quant._pc_cb = torch.empty(0)
    with pytest.raises(ValueError):
        pkg.ARCQPackedLinear(src)
    layer = pkg.ARCQPackedLinear(_source(pkg, g))
    with pytest.raises(ValueError):
        layer(torch.zeros(2, 32))
    # no CPU fallback: a CPU tensor cannot be run
    with pytest.raises(RuntimeError):
        layer(torch.zeros(2, 64))


def test_half_cast_keeps_fp32_metadata(pkg, golden):
    g = golden("edge_k64_w4a4")
    holder = torch.nn.Sequential(pkg.ARCQPackedLinearOnTheFly.from_packed(pkg.ARCQPackedLinear(_source(pkg, g))),
                                 torch.nn.LayerNorm(8))
    holder.half()
    assert holder[1].weight.dtype == torch.float16
    for n, b in holder[0].named_buffers():
        assert b.dtype == (torch.uint8 if n == "packed_weight_codes" else torch.float32), n


def test_convert_matches_by_class_name(pkg, golden):
    g = golden("edge_k64_w4a4")
    src = _source(pkg, g)
    QuantLinearPCARCQ = type("QuantLinearPCARCQ", (torch.nn.Module,), {})
    q = QuantLinearPCARCQ()
    q.linear, q.act_quant, q.weight_quant = src.linear, src.act_quant, src.weight_quant
    model = torch.nn.ModuleDict({"attn": torch.nn.ModuleDict({"qkv": q}), "other": torch.nn.Linear(8, 8)})
    pkg.convert_arcq_linear_to_packed(model, "packed")
    assert isinstance(model["attn"]["qkv"], pkg.ARCQPackedLinear) and isinstance(model["other"], torch.nn.Linear)
    assert pkg.count_packed_linear(model) == 1
    pkg.to_on_the_fly(model)
    assert isinstance(model["attn"]["qkv"], pkg.ARCQPackedLinearOnTheFly)


def test_load_packed_checkpoint_into_skeleton(pkg):
    m = pkg.create_vit("deit_tiny", seed=3)
    cb = torch.linspace(-2.5, 2.5, 16)
    th = (cb[:-1] + cb[1:]) / 2
    books = {n: dict(act_cb=cb, act_th=th, w_cb=cb, w_th=th) for n in pkg.quantised_linear_names(m)}
    packed = pkg.pack_model_with_codebooks(pkg.create_vit("deit_tiny", seed=3), books, 4, on_the_fly=False)
    sd = packed.state_dict()
    assert pkg.count_packed_linear(packed) == 48 and "blocks.11.mlp.fc2.packed_weight_codes" in sd
    fresh = pkg.load_packed_state_dict(pkg.create_vit("deit_tiny", seed=9), sd)
    assert pkg.count_packed_linear(fresh) == 48
    a, b = fresh.state_dict(), {k: v for k, v in sd.items()}
    assert torch.equal(a["blocks.5.attn.qkv.packed_weight_codes"], b["blocks.5.attn.qkv.packed_weight_codes"])
    assert torch.equal(a["head.weight"], b["head.weight"])
    # packed DeiT-T: 5.3 M weights at 4 bit + 3 floats per (row, group)
    n_packed = sum(v.numel() for k, v in sd.items() if k.endswith("packed_weight_codes"))
    assert n_packed == 12 * (576 * 192 + 192 * 192 + 768 * 192 + 192 * 768) // 2


def test_codebook_fit_agrees_with_oracle_and_reference(pkg, oracle, golden):
    for name in ("c1_w4a4", "c1_w3a3"):
        g = golden(name)
        cb, th = pkg.codebook.calibrate_codebook(torch.from_numpy(g["X"]), g["bits"], g["gs"])
        # the package's fit reproduces the reference's fitted codebook and thresholds exactly
        assert np.array_equal(cb.numpy(), g["act_codebook"])
        assert np.array_equal(th.numpy(), g["act_thresholds"])
        cbo, _ = oracle.calibrate(g["X"], g["bits"], g["gs"])     # the oracle's independent numpy restatement
        assert np.abs(cb.numpy() - cbo).max() < 2e-3


def test_library_exports_every_declared_symbol(pkg):
    header = (ROOT / "include" / "arcq_b200.h").read_text()
    declared = sorted(set(re.findall(r"\b(arcq_[a-z0-9_]+)\s*\(", header)))
    assert declared, "no declarations found"
    lib = pkg._cabi.load()
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/arcq_b200.h but not exported"
    assert sorted(pkg._cabi.EXPORTS) == declared
    assert lib.arcq_version() == 100


def test_c_abi_rejects_bad_arguments_before_any_launch(pkg):
    lib = pkg._cabi.load()
    import ctypes
    buf = ctypes.create_string_buffer(4096)
    p = ctypes.cast(buf, ctypes.c_void_p)
    E_ARG, E_SHAPE, E_UNSUP = -1, -2, -3
    assert lib.arcq_act_quant(None, 0, 1, 64, p, p, 4, 64, p, p, p, p, None, 0, None) == E_ARG
    assert "null" in pkg._cabi.last_error()
    assert lib.arcq_act_quant(p, 0, 1, 64, p, p, 5, 64, p, p, p, p, None, 0, None) == E_ARG
    assert lib.arcq_act_quant(p, 0, 1, 100, p, p, 4, 64, p, p, p, p, None, 0, None) == E_SHAPE
    assert lib.arcq_act_quant(p, 0, 1, 64, p, p, 4, 32, p, p, p, p, None, 0, None) == E_UNSUP
    assert lib.arcq_act_quant(p, 7, 1, 64, p, p, 4, 64, p, p, p, p, None, 0, None) == E_ARG
    args = [p] * 11
    assert lib.arcq_packed_gemm(*args, 4, 64, 1, 12, 64, p, 1, None) == E_SHAPE      # N % 8
    assert lib.arcq_packed_gemm(*args, 4, 64, 1, 16, 96, p, 1, None) == E_SHAPE      # K % 64
    assert lib.arcq_packed_gemm(*args, 4, 64, 1, 16, 64, p, 2, None) == E_ARG        # bf16 out not built
    a7 = [p] * 7
    assert lib.arcq_packed_weight_gemm(*a7, 4, 64, 1, 24, 64, p, 1, None) == E_UNSUP      # N % 16
    assert lib.arcq_packed_weight_gemm(*a7, 3, 64, 1, 64, 192, p, 1, None) == E_UNSUP     # 72-byte packed rows
    assert lib.arcq_packed_weight_gemm(*a7, 4, 64, 1, 64, 100, p, 1, None) == E_SHAPE
    assert lib.arcq_packed_weight_gemm(None, *a7[1:], 4, 64, 1, 64, 64, p, 1, None) == E_ARG
    assert lib.arcq_unpack_codes(p, 1, 8, 7, p, None) == E_ARG
    assert lib.arcq_pack_codes(None, 1, 8, 4, p, None) == E_ARG
    assert lib.arcq_dequant(p, p, p, p, p, 4, 64, 1, 100, p, 1, None) == E_SHAPE
    # empty inputs are a successful no-op
    assert lib.arcq_act_quant(p, 0, 0, 64, p, p, 4, 64, p, p, p, p, None, 0, None) == 0
    assert lib.arcq_unpack_codes(p, 0, 8, 4, p, None) == 0
