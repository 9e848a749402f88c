"""The oracle against the reference's own outputs (fixtures made by tests/golden/make_golden.py)."""
import hashlib

import numpy as np
import pytest

from conftest import GOLDEN_CASES, ulp_diff


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_activation_quantizer_matches_reference(oracle, golden, name):
    g = golden(name)
    codes, mu, sg, cs = oracle.quantize(g["X"], g["act_thresholds"], g["act_codebook"], g["gs"])
    ref_codes = oracle.unpack(g["act_packed"], g["bits"], g["K"])
    assert np.array_equal(codes, ref_codes), "activation codes differ from the reference quantizer"
    assert np.array_equal(oracle.pack(codes, g["bits"]), g["act_packed"])
    assert np.array_equal(mu, g["act_mu"])
    assert np.array_equal(cs, g["act_code_sum"])
    # the reference's CPU square root (the host math library's vector sqrt) is not correctly
    # rounded: it is one unit in the last place off in under 1 % of groups; the oracle is IEEE
    assert ulp_diff(sg, g["act_sigma"]) <= 1
    assert (sg != g["act_sigma"]).mean() < 0.02


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_weight_quantizer_and_packing_match_reference(oracle, golden, name):
    g = golden(name)
    codes, mu, sg, cs = oracle.quantize(g["W"], g["w_thresholds"], g["w_codebook"], g["gs"])
    assert hashlib.sha256(codes.tobytes()).hexdigest() == str(g["w_codes_sha256"])
    assert np.array_equal(oracle.pack(codes, g["bits"]), g["sd.packed_weight_codes"])
    assert np.array_equal(oracle.unpack(g["sd.packed_weight_codes"], g["bits"], g["K"]), codes)
    assert np.array_equal(mu, g["sd.weight_center"])
    assert np.array_equal(cs, g["sd.weight_code_sum"])
    assert ulp_diff(sg, g["sd.weight_scale"]) <= 1


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_fake_quant_linear_matches_reference(oracle, golden, name):
    g = golden(name)
    y, inter = oracle.fake_quant_linear(g["X"], g["W"], g["b"], g["act_thresholds"], g["act_codebook"],
                                        g["w_thresholds"], g["w_codebook"], g["gs"])
    rms = float(g["y_ref_rms"])
    assert np.abs(y[::16, ::4] - g["y_ref_sub"]).max() / rms < 1e-4
    # the reference's fake-quant activation (first rows); only groups whose sigma is 1 ulp apart may differ
    head = oracle.fake_quant(g["X"][:16], g["act_thresholds"], g["act_codebook"], g["gs"])
    assert np.abs(head - g["x_fq_head"]).max() <= 1e-5 * np.abs(g["x_fq_head"]).max()
    # the code-sum form of the packed kernel is the same number
    y2 = oracle.linear_codesum(inter["act_codes"], inter["act_mu"], inter["act_sigma"], inter["act_code_sum"],
                               inter["w_codes"], inter["w_mu"], inter["w_sigma"], inter["w_code_sum"],
                               g["act_codebook"], g["w_codebook"], g["b"], g["gs"])
    assert np.abs(y2 - y).max() / rms < 1e-4


def test_codebook_fit_matches_reference(oracle, golden):
    for name in ("c1_w4a4", "c1_w3a3"):
        g = golden(name)
        cb, th = oracle.calibrate(g["X"], g["bits"], g["gs"])
        assert np.abs(cb - g["act_codebook"]).max() < 2e-3
        assert np.abs(th - g["act_thresholds"]).max() < 2e-3
        cbw, _ = oracle.calibrate(g["W"], g["bits"], g["gs"])
        assert np.abs(cbw - g["w_codebook"]).max() < 2e-3
        assert cb[cb == 0].size == 1 and np.all(np.diff(cb) > 0)


def test_summation_order_is_torch_cpu_order(oracle):
    import torch
    x = torch.randn(4096, 64, generator=torch.Generator().manual_seed(3)) * 3 + 0.25
    assert np.array_equal(oracle.row_sums(x.numpy()), x.sum(-1).numpy())


def test_pack_layout_small_known_answers(oracle):
    # 4-bit: byte = c[2k] + (c[2k+1] << 4); 3-bit: 8 codes <-> 3 bytes, LSB first
    c4 = np.array([[1, 2, 3, 4]], np.uint8)
    assert oracle.pack(c4, 4).tolist() == [[0x21, 0x43]]
    c3 = np.array([[1, 2, 3, 4, 5, 6, 7, 0]], np.uint8)
    bits = sum(int(v) << (3 * i) for i, v in enumerate(c3[0]))
    assert oracle.pack(c3, 3).tolist() == [[bits & 255, (bits >> 8) & 255, (bits >> 16) & 255]]
    ragged = np.array([[3, 1, 2], [0, 3, 3]], np.uint8)           # length*bits not a multiple of 8
    assert oracle.pack(ragged, 3).shape == (2, 2)
    assert np.array_equal(oracle.unpack(oracle.pack(ragged, 3), 3, 3), ragged)
