"""Parity of the CUDA kernels with the oracle and the golden fixtures, through the C ABI."""
import json
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN_CASES, ROOT, ulp_diff

pytestmark = pytest.mark.gpu


def _t(a, dev, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    return t if dtype is None else t.to(dtype)




def _near_threshold(oracle, X, th, cb, gs, rows, cols):
    """|t - nearest threshold| for the listed elements: tells a 1-ulp tie from a bug."""
    t = oracle.normalized_groups(X, gs).reshape(X.shape)
    return [float(np.abs(th - t[r, c]).min()) for r, c in zip(rows[:8], cols[:8])]


# ------------------------------------------------------------------ activation quantizer
@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_act_quant_bit_exact_vs_reference_fixture(pkg, oracle, golden, cuda_device, name):
    g = golden(name)
    th, cb = _t(g["act_thresholds"], cuda_device), _t(g["act_codebook"], cuda_device)
    packed, mu, sg, cs = pkg.ops.quantize_activation(_t(g["X"], cuda_device), th, cb, g["bits"], g["gs"])
    assert pkg.ops.device_status() == 0
    packed = packed.cpu().numpy()
    if not np.array_equal(packed, g["act_packed"]):
        mine = oracle.unpack(packed, g["bits"], g["K"])
        ref = oracle.unpack(g["act_packed"], g["bits"], g["K"])
        r, c = np.nonzero(mine != ref)
        pytest.fail(f"{r.size} activation codes differ from the reference; first at {list(zip(r[:8], c[:8]))}, "
                    f"|t-threshold| there = {_near_threshold(oracle, g['X'], g['act_thresholds'], g['act_codebook'], g['gs'], r, c)}")
    assert np.array_equal(mu.cpu().numpy(), g["act_mu"])
    assert np.array_equal(cs.cpu().numpy(), g["act_code_sum"])
    _, o_mu, o_sg, o_cs = oracle.quantize(g["X"], g["act_thresholds"], g["act_codebook"], g["gs"])
    assert np.array_equal(sg.cpu().numpy(), o_sg)                    # IEEE sqrt on both sides
    assert ulp_diff(sg.cpu().numpy(), g["act_sigma"]) <= 1           # reference CPU sqrt is 1 ulp off at times


@pytest.mark.parametrize("bits", [4, 3, 2])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(1, 64), (3, 192), (197, 384), (130, 1536)])
def test_act_quant_matches_oracle_all_dtypes(pkg, oracle, cuda_device, bits, dtype, shape):
    rng = np.random.default_rng(hash((bits, shape)) % 2 ** 31)
    X = rng.standard_normal(shape, dtype=np.float32) * rng.uniform(0.1, 4.0, size=(shape[0], 1)).astype(np.float32)
    X[:, ::37] *= 15.0
    x = torch.from_numpy(X).to(dtype)
    Xr = x.float().numpy()                                  # the values the kernel sees
    L = 2 ** bits
    cb = np.sort(rng.uniform(-2.8, 2.8, L)).astype(np.float32)
    th = ((cb[:-1] + cb[1:]) / np.float32(2)).astype(np.float32)
    codes, mu, sg, cs = oracle.quantize(Xr, th, cb, 64)
    p, m, s, c = pkg.ops.quantize_activation(x.to(cuda_device), _t(th, cuda_device), _t(cb, cuda_device), bits, 64)
    assert np.array_equal(p.cpu().numpy(), oracle.pack(codes, bits))
    assert np.array_equal(m.cpu().numpy(), mu) and np.array_equal(s.cpu().numpy(), sg)
    assert np.array_equal(c.cpu().numpy(), cs)
    # reconstruction output mode == oracle dequant, rounded to the output type
    xh = pkg.ops.quantize_activation_dequant(x.to(cuda_device), _t(th, cuda_device), _t(cb, cuda_device), bits, 64,
                                             torch.float32)
    assert np.array_equal(xh.cpu().numpy(), oracle.dequant(codes, mu, sg, cb, 64))
    xh16 = pkg.ops.quantize_activation_dequant(x.to(cuda_device), _t(th, cuda_device), _t(cb, cuda_device), bits, 64,
                                               torch.float16)
    assert torch.equal(xh16.cpu(), torch.from_numpy(oracle.dequant(codes, mu, sg, cb, 64)).half())
    assert pkg.ops.device_status() == 0


def test_act_quant_ties_go_to_the_lower_code(pkg, cuda_device):
    # a value exactly on a threshold takes the lower code (count of thresholds strictly below)
    cb = np.arange(-8, 8, dtype=np.float32) * 0.25
    th = ((cb[:-1] + cb[1:]) / 2).astype(np.float32)
    x = np.zeros((1, 64), np.float32)
    x[0, :32], x[0, 32:] = -1.0, 1.0                # mean 0, scale sqrt(1+1e-6) -> t = +-0.9999995
    t_pos = np.float32(1.0) / np.sqrt(np.float32(1.0) + np.float32(1e-6), dtype=np.float32)
    th[11] = t_pos                                    # 0.625 < t_pos < 1.125: still sorted, exactly at t
    assert np.all(np.diff(th) > 0)
    p, *_ = pkg.ops.quantize_activation(_t(x, cuda_device), _t(th, cuda_device), _t(cb, cuda_device), 4, 64)
    codes = pkg.ops.unpack_codes_u8(p, 4, 64).cpu().numpy()[0]
    assert int(codes[63]) == int((th < t_pos).sum()) == 11      # not 12: the tie stays below
    th[11] = np.nextafter(t_pos, np.float32(0))                 # one ulp lower: now strictly below t
    p, *_ = pkg.ops.quantize_activation(_t(x, cuda_device), _t(th, cuda_device), _t(cb, cuda_device), 4, 64)
    assert int(pkg.ops.unpack_codes_u8(p, 4, 64).cpu().numpy()[0, 63]) == 12


def test_act_quant_full_size_properties(pkg, cuda_device):
    # the headline size (DeiT-S fc2 input at batch 64): too slow for the scalar oracle in full, so check
    # properties: each row's result is independent of the batch it sits in, and requantising the
    # reconstruction with the same codebook reproduces the codes of a sample checked elsewhere.
    M, K = 64 * 197, 1536
    gen = torch.Generator(device="cpu").manual_seed(5)
    x = torch.randn(M, K, generator=gen).half().to(cuda_device)
    cb = torch.linspace(-2.6, 2.6, 16, device=cuda_device)
    th = (cb[:-1] + cb[1:]) / 2
    p, mu, sg, cs = pkg.ops.quantize_activation(x, th, cb, 4, 64)
    perm = torch.randperm(M, generator=gen).to(cuda_device)
    p2, mu2, sg2, cs2 = pkg.ops.quantize_activation(x[perm].contiguous(), th, cb, 4, 64)
    assert torch.equal(p[perm], p2) and torch.equal(mu[perm], mu2) and torch.equal(sg[perm], sg2)
    p3, *_ = pkg.ops.quantize_activation(x[1000:1197].contiguous(), th, cb, 4, 64)
    assert torch.equal(p[1000:1197], p3)
    codes = pkg.ops.unpack_codes_u8(p, 4, K)
    assert int(codes.max()) <= 15 and torch.equal(pkg.ops.pack_codes(codes, 4), p)
    # the code sum equals the sum of looked-up levels (fp32, any order within 1e-5)
    want = cb[codes.long()].reshape(M, K // 64, 64).sum(-1)
    assert torch.allclose(cs, want, atol=2e-5)
    assert pkg.ops.device_status() == 0


def test_act_quant_argument_errors(pkg, cuda_device):
    cb = torch.linspace(-2, 2, 16, device=cuda_device)
    th = (cb[:-1] + cb[1:]) / 2
    with pytest.raises(RuntimeError):
        pkg.ops.quantize_activation(torch.zeros(2, 100, device=cuda_device), th, cb, 4, 64)     # K % gs
    with pytest.raises(RuntimeError):
        pkg.ops.quantize_activation(torch.zeros(2, 64), th, cb, 4, 64)                          # CPU tensor
    with pytest.raises(RuntimeError):
        pkg.ops.quantize_activation(torch.zeros(2, 64, device=cuda_device), th, cb, 3, 64)      # codebook size
    with pytest.raises(RuntimeError):
        pkg.ops.quantize_activation(torch.zeros(2, 64, device=cuda_device), th, cb, 4, 32)      # group size not built
    p, mu, sg, cs = pkg.ops.quantize_activation(torch.zeros(0, 64, device=cuda_device), th, cb, 4, 64)
    assert p.shape == (0, 32) and mu.shape == (0, 1)


# ------------------------------------------------------------------ pack / unpack / reconstruct
@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("shape", [(1, 8), (5, 63), (72, 192), (384, 1536)])
def test_pack_unpack_kernels(pkg, oracle, cuda_device, bits, shape):
    rng = np.random.default_rng(bits + shape[1])
    codes = rng.integers(0, 2 ** bits, size=shape, dtype=np.uint8)
    packed = pkg.ops.pack_codes(_t(codes, cuda_device), bits)
    assert np.array_equal(packed.cpu().numpy(), oracle.pack(codes, bits))
    assert np.array_equal(pkg.ops.unpack_codes_u8(packed, bits, shape[1]).cpu().numpy(), codes)
    assert pkg.ops.unpack_codes(packed, bits, shape[1]).dtype == torch.int64


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_unpacked_weight_indices_bit_exact(pkg, oracle, golden, cuda_device, name):
    g = golden(name)
    got = pkg.ops.unpack_codes_u8(_t(g["sd.packed_weight_codes"], cuda_device), g["bits"], g["K"]).cpu().numpy()
    want, *_ = oracle.quantize(g["W"], g["w_thresholds"], g["w_codebook"], g["gs"])
    assert np.array_equal(got, want)
    # weights quantised on the device by the same kernel give the same packed bytes as the reference
    p, mu, sg, cs = pkg.ops.quantize_activation(_t(g["W"], cuda_device), _t(g["w_thresholds"], cuda_device),
                                                _t(g["w_codebook"], cuda_device), g["bits"], g["gs"])
    assert np.array_equal(p.cpu().numpy(), g["sd.packed_weight_codes"])
    assert np.array_equal(mu.cpu().numpy(), g["sd.weight_center"])
    # reconstruction kernel == oracle dequant
    w = pkg.ops.dequant(_t(g["sd.packed_weight_codes"], cuda_device), mu, sg, cs, _t(g["w_codebook"], cuda_device),
                        g["bits"], g["gs"], torch.float32)
    assert np.array_equal(w.cpu().numpy(), oracle.dequant(want, mu.cpu().numpy(), sg.cpu().numpy(), g["w_codebook"], g["gs"]))


# ------------------------------------------------------------------ packed GEMM
TOL = 2e-2      # max |dy| relative to the RMS of the reference output (the bar for linear outputs)


def _gemm_case(pkg, oracle, dev, X, W, b, a_th, a_cb, w_th, w_cb, bits, out_dtype):
    y_ref, it = oracle.fake_quant_linear(X, W, b, a_th, a_cb, w_th, w_cb, 64)
    pa = oracle.pack(it["act_codes"], bits)
    pw = oracle.pack(it["w_codes"], bits)
    y = pkg.ops.arcq_linear_forward(
        _t(pa, dev), _t(it["act_mu"], dev), _t(it["act_sigma"], dev), _t(it["act_code_sum"], dev),
        _t(pw, dev), _t(it["w_mu"], dev), _t(it["w_sigma"], dev), _t(it["w_code_sum"], dev),
        _t(a_cb, dev), _t(w_cb, dev), None if b is None else _t(b, dev), bits, 64, X.shape[1], W.shape[0], out_dtype)
    assert pkg.ops.device_status() == 0, "a bounded wait in the GEMM kernel ran out"
    rms = float(np.sqrt((y_ref.astype(np.float64) ** 2).mean()))
    return y, y_ref, rms


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_packed_gemm_vs_fake_quant_reference(pkg, oracle, golden, cuda_device, name, out_dtype, report):
    g = golden(name)
    y, y_ref, rms = _gemm_case(pkg, oracle, cuda_device, g["X"], g["W"], g["b"], g["act_thresholds"],
                               g["act_codebook"], g["w_thresholds"], g["w_codebook"], g["bits"], out_dtype)
    assert y.dtype == out_dtype
    yn = y.float().cpu().numpy()
    err = float(np.abs(yn - y_ref).max() / rms)
    err_ref = float(np.abs(yn[::16, ::4] - g["y_ref_sub"]).max() / float(g["y_ref_rms"]))
    report("packed_gemm", case=name, out=str(out_dtype), max_abs_over_rms=err, vs_reference_fixture=err_ref)
    assert err < TOL, f"max|dy|/rms = {err:.3e}"
    assert err_ref < TOL


@pytest.mark.parametrize("bits", [4, 3, 2])
@pytest.mark.parametrize("M,K,N", [(1, 64, 8), (5, 64, 16), (129, 128, 24), (197, 192, 576), (300, 384, 1152),
                                   (64, 768, 72), (257, 1536, 384)])
def test_packed_gemm_shapes_and_edges(pkg, oracle, cuda_device, bits, M, K, N, report):
    rng = np.random.default_rng(M * 7 + K + N + bits)
    X = rng.standard_normal((M, K), dtype=np.float32)
    X[:, rng.permutation(K)[:2]] *= 20
    W = (rng.standard_normal((N, K), dtype=np.float32) * 0.02).astype(np.float32)
    b = (rng.standard_normal(N, dtype=np.float32) * 0.01).astype(np.float32) if (M + N) % 2 else None
    a_cb, a_th = oracle.calibrate(X, bits)
    w_cb, w_th = oracle.calibrate(W, bits)
    y, y_ref, rms = _gemm_case(pkg, oracle, cuda_device, X, W, b, a_th, a_cb, w_th, w_cb, bits, torch.float32)
    err = float(np.abs(y.cpu().numpy() - y_ref).max() / rms)
    report("packed_gemm_shapes", bits=bits, M=M, K=K, N=N, max_abs_over_rms=err)
    assert err < TOL, f"max|dy|/rms = {err:.3e}"


def test_packed_gemm_row_results_do_not_depend_on_the_batch(pkg, oracle, golden, cuda_device):
    g = golden("c1_w4a4")
    dev = cuda_device
    th, cb = _t(g["act_thresholds"], dev), _t(g["act_codebook"], dev)
    wt = [_t(g["sd." + k], dev) for k in ("packed_weight_codes", "weight_center", "weight_scale", "weight_code_sum")]
    wcb, bias = _t(g["sd.weight_codebook"], dev), _t(g["sd.bias"], dev)

    def run(x):
        p, mu, sg, cs = pkg.ops.quantize_activation(x, th, cb, 4, 64)
        return pkg.ops.arcq_linear_forward(p, mu, sg, cs, *wt, cb, wcb, bias, 4, 64, g["K"], g["N"], torch.float16)

    x = _t(g["X"], dev)
    full = run(x)
    part = run(x[197:2 * 197].contiguous())
    assert torch.equal(full[197:2 * 197], part)        # bit-identical: tiling does not change a row's sum
    one = run(x[5:6].contiguous())
    assert torch.equal(full[5:6], one)
    assert pkg.ops.device_status() == 0


def test_packed_gemm_full_size_properties(pkg, cuda_device, report):
    # DeiT-S fc1 at batch 64 (M=12608, K=384, N=1536): bias enters linearly and exactly once, and
    # a permutation of the rows permutes the output.
    M, K, N = 64 * 197, 384, 1536
    dev = cuda_device
    gen = torch.Generator().manual_seed(11)
    cb = torch.linspace(-2.6, 2.6, 16, device=dev)
    th = (cb[:-1] + cb[1:]) / 2
    x = torch.randn(M, K, generator=gen).half().to(dev)
    w = (torch.randn(N, K, generator=gen) * 0.02).to(dev)
    bias = (torch.randn(N, generator=gen) * 0.01).to(dev)
    pw, mw, sw, cw = pkg.ops.quantize_activation(w, th, cb, 4, 64)
    pa, ma, sa, ca = pkg.ops.quantize_activation(x, th, cb, 4, 64)
    f = lambda b, p=pa, m=ma, s=sa, c=ca: pkg.ops.arcq_linear_forward(p, m, s, c, pw, mw, sw, cw, cb, cb, b, 4, 64, K, N,  # noqa: E731
                                                                    torch.float32)
    y0, yb = f(None), f(bias)
    assert torch.allclose(yb - y0, bias.expand_as(y0), atol=1e-5)
    perm = torch.randperm(M, generator=gen).to(dev)
    yp = f(None, pa[perm].contiguous(), ma[perm].contiguous(), sa[perm].contiguous(), ca[perm].contiguous())
    assert torch.equal(yp, y0[perm])
    # against a plain fp32 contraction of the reconstructed operands (torch, on the device)
    xa = pkg.ops.dequant(pa, ma, sa, ca, cb, 4, 64, torch.float32)
    wa = pkg.ops.dequant(pw, mw, sw, cw, cb, 4, 64, torch.float32)
    ref = xa.double() @ wa.double().T
    err = float((y0.double() - ref).abs().max() / ref.pow(2).mean().sqrt())
    report("packed_gemm_full_size", M=M, K=K, N=N, max_abs_over_rms=err)
    assert err < TOL
    assert pkg.ops.device_status() == 0


# ------------------------------------------------------------------ packed-weight GEMM (fp16 activation operand)
def _pw_case(pkg, oracle, dev, X, W, b, a_th, a_cb, w_th, w_cb, bits, out_dtype):
    y_ref, it = oracle.fake_quant_linear(X, W, b, a_th, a_cb, w_th, w_cb, 64)
    xh = pkg.ops.quantize_activation_dequant(_t(X, dev), _t(a_th, dev), _t(a_cb, dev), bits, 64, torch.float16)
    assert torch.equal(xh.cpu(), torch.from_numpy(oracle.dequant(it["act_codes"], it["act_mu"], it["act_sigma"],
                                                               a_cb, 64)).half())
    y = pkg.ops.packed_weight_gemm(xh, _t(oracle.pack(it["w_codes"], bits), dev), _t(it["w_mu"], dev),
                                   _t(it["w_sigma"], dev), _t(it["w_code_sum"], dev), _t(w_cb, dev),
                                   None if b is None else _t(b, dev), bits, 64, out_dtype)
    assert pkg.ops.device_status() == 0, "a bounded wait in the persistent GEMM ran out"
    rms = float(np.sqrt((y_ref.astype(np.float64) ** 2).mean()))
    return y, y_ref, rms


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("name", ["c1_w4a4", "c1_w3a3", "edge_k1536_w4a4"])
def test_packed_weight_gemm_vs_fake_quant_reference(pkg, oracle, golden, cuda_device, name, out_dtype, report):
    g = golden(name)
    y, y_ref, rms = _pw_case(pkg, oracle, cuda_device, g["X"], g["W"], g["b"], g["act_thresholds"], g["act_codebook"],
                             g["w_thresholds"], g["w_codebook"], g["bits"], out_dtype)
    yn = y.float().cpu().numpy()
    err = float(np.abs(yn - y_ref).max() / rms)
    err_ref = float(np.abs(yn[::16, ::4] - g["y_ref_sub"]).max() / float(g["y_ref_rms"]))
    report("packed_weight_gemm", case=name, out=str(out_dtype), max_abs_over_rms=err, vs_reference_fixture=err_ref)
    assert err < TOL and err_ref < TOL, f"max|dy|/rms = {err:.3e}"


@pytest.mark.parametrize("bits", [4, 3, 2])
@pytest.mark.parametrize("M,K,N", [(1, 64, 16), (5, 128, 32), (129, 128, 48), (197, 192, 576), (300, 384, 1152),
                                   (1000, 384, 384), (64, 768, 2304), (257, 1536, 384), (700, 3072, 768)])
def test_packed_weight_gemm_shapes(pkg, oracle, cuda_device, bits, M, K, N, report):
    if not pkg.ops.packed_weight_gemm_supported(K, N, bits, 64):
        pytest.skip("shape is routed to the packed-codes kernel")
    rng = np.random.default_rng(M * 5 + K + N + bits)
    X = rng.standard_normal((M, K), dtype=np.float32)
    X[:, rng.permutation(K)[:2]] *= 20
    W = (rng.standard_normal((N, K), dtype=np.float32) * 0.02).astype(np.float32)
    b = (rng.standard_normal(N, dtype=np.float32) * 0.01).astype(np.float32) if (M + N) % 2 else None
    a_cb, a_th = oracle.calibrate(X, bits)
    w_cb, w_th = oracle.calibrate(W, bits)
    y, y_ref, rms = _pw_case(pkg, oracle, cuda_device, X, W, b, a_th, a_cb, w_th, w_cb, bits, torch.float16)
    err = float(np.abs(y.float().cpu().numpy() - y_ref).max() / rms)
    report("packed_weight_gemm_shapes", bits=bits, M=M, K=K, N=N, max_abs_over_rms=err)
    assert err < TOL, f"max|dy|/rms = {err:.3e}"


def test_packed_weight_gemm_full_size_properties(pkg, cuda_device, report):
    # DeiT-S at batch 64: fc1 (weights stay resident in shared memory) and fc2 (weights stream)
    dev = cuda_device
    gen = torch.Generator().manual_seed(13)
    cb = torch.linspace(-2.6, 2.6, 16, device=dev)
    th = (cb[:-1] + cb[1:]) / 2
    for (M, K, N) in [(64 * 197, 384, 1536), (64 * 197, 1536, 384), (64 * 197, 384, 1152)]:
        x = torch.randn(M, K, generator=gen).half().to(dev)
        w = (torch.randn(N, K, generator=gen) * 0.02).to(dev)
        bias = (torch.randn(N, generator=gen) * 0.01).to(dev)
        pw, mw, sw, cw = pkg.ops.quantize_activation(w, th, cb, 4, 64)
        xh = pkg.ops.quantize_activation_dequant(x, th, cb, 4, 64, torch.float16)
        f = lambda a, b: pkg.ops.packed_weight_gemm(a, pw, mw, sw, cw, cb, b, 4, 64, torch.float32)  # noqa: E731
        y0, yb = f(xh, None), f(xh, bias)
        assert torch.allclose(yb - y0, bias.expand_as(y0), atol=1e-5)
        perm = torch.randperm(M, generator=gen).to(dev)
        assert torch.equal(f(xh[perm].contiguous(), None), y0[perm])          # rows do not depend on their tile
        assert torch.equal(f(xh[300:497].contiguous(), None), y0[300:497])    # nor on the batch size
        wa = pkg.ops.dequant(pw, mw, sw, cw, cb, 4, 64, torch.float32)
        ref = xh.double() @ wa.double().T
        err = float((y0.double() - ref).abs().max() / ref.pow(2).mean().sqrt())
        report("packed_weight_gemm_full_size", M=M, K=K, N=N, max_abs_over_rms=err)
        assert err < 5e-3                                                       # only W^ rounding to fp16 differs
        assert pkg.ops.device_status() == 0


def test_gelu_fused_into_the_quantizer(pkg, oracle, cuda_device):
    # small input (8-lane kernel) and large input (one-thread-per-group kernel)
    for M, K in [(197, 1536), (40 * 197, 1536)]:
        gen = torch.Generator().manual_seed(M)
        pre = (torch.randn(M, K, generator=gen) * 1.5).half().to(cuda_device)
        cb = torch.linspace(-2.6, 2.6, 16, device=cuda_device)
        th = (cb[:-1] + cb[1:]) / 2
        act = torch.nn.functional.gelu(pre)                       # what the separate kernel would store (fp16)
        want = pkg.ops.quantize_activation(act, th, cb, 4, 64)
        got = pkg.ops.quantize_activation(pre, th, cb, 4, 64, True, True)
        # the fused GELU is rounded to fp16 like the stored tensor; allow the rare 1-ulp erf difference
        same = float((want[0] == got[0]).float().mean())
        assert same > 0.9999, same
        if M == 197:
            a = act.float().cpu().numpy()
            codes, mu, sg, cs = oracle.quantize(a, th.cpu().numpy(), cb.cpu().numpy(), 64)
            assert (pkg.ops.unpack_codes_u8(got[0], 4, K).cpu().numpy() == codes).mean() > 0.9999
        xh_want = pkg.ops.quantize_activation_dequant(act, th, cb, 4, 64, torch.float16)
        xh_got = pkg.ops.quantize_activation_dequant(pre, th, cb, 4, 64, torch.float16, True)
        assert float((xh_want == xh_got).float().mean()) > 0.999
    assert pkg.ops.device_status() == 0


@pytest.mark.parametrize("M,K", [(1, 192), (197, 384), (64 * 197, 384), (1000, 768), (33, 2048)])
def test_add_layernorm_matches_torch(pkg, cuda_device, M, K):
    gen = torch.Generator().manual_seed(M + K)
    x = (torch.randn(M, K, generator=gen) * 2 + 0.5).half().to(cuda_device)
    y = torch.randn(M, K, generator=gen).half().to(cuda_device)
    ln = torch.nn.LayerNorm(K, eps=1e-6).to(cuda_device)
    with torch.no_grad():
        ln.weight.copy_(1 + 0.1 * torch.randn(K, generator=gen))
        ln.bias.copy_(0.1 * torch.randn(K, generator=gen))
    ln = ln.half()
    with torch.no_grad():
        s_ref = x + y
        h_ref = ln(s_ref)
        s, h = pkg.ops.add_layernorm(x, y, ln)
        assert torch.equal(s, s_ref)                                   # fp16 sum, same rounding
        # fp32 reference of the normalisation on the same fp16 sum; the result may differ from torch's by
        # one fp16 unit in the last place where the two fp32 evaluations round differently
        f = torch.nn.functional.layer_norm(s_ref.float(), (K,), ln.weight.float(), ln.bias.float(), 1e-6)
        assert float((h.float() - f).abs().max()) <= 2e-3 * max(1.0, float(f.abs().max()))
        assert float((h == h_ref).float().mean()) > 0.99
        x0, h0 = pkg.ops.add_layernorm(x, None, ln)
        assert x0 is x and float((h0 == ln(x)).float().mean()) > 0.99
    with pytest.raises(RuntimeError):
        pkg.ops.add_layernorm(torch.zeros(2, 12, dtype=torch.float16, device=cuda_device), None,
                              torch.nn.LayerNorm(12).half().to(cuda_device))


@pytest.mark.parametrize("bits", [4, 3, 2])
@pytest.mark.parametrize("dtype", [torch.float16, torch.float32, torch.bfloat16])
def test_staged_quantizer_kernel_matches_oracle_and_the_parallel_kernel(pkg, oracle, cuda_device, bits, dtype):
    """Inputs with >= 37 888 groups take the one-thread-per-group kernel (staged loads, division-free exact
    threshold test, uniform-grid first guess); smaller ones the 8-lanes-per-group kernel.  Both must give
    the oracle's codes and statistics bit for bit."""
    import os
    M, K = 2048, 1536                                        # 49 152 groups
    rng = np.random.default_rng(bits * 7 + 1)
    X = rng.standard_normal((M, K), dtype=np.float32) * rng.uniform(0.05, 6.0, size=(M, 1)).astype(np.float32)
    X[:, ::29] *= 12.0
    x = torch.from_numpy(X).to(dtype)
    Xr = x.float().numpy()
    L = 2 ** bits
    if bits == 4:                                             # shape of a fitted codebook: two ramps around zero
        cb = np.concatenate([-np.linspace(0, 2.6, 8)[1:][::-1], [0.0], np.linspace(0, 2.58, 9)[1:]]).astype(np.float32)
    else:
        cb = np.sort(rng.uniform(-2.8, 2.8, L)).astype(np.float32)
    th = ((cb[:-1] + cb[1:]) / np.float32(2)).astype(np.float32)
    codes, mu, sg, cs = oracle.quantize(Xr, th, cb, 64)
    xd = x.to(cuda_device)
    p, m, s, c = pkg.ops.quantize_activation(xd, _t(th, cuda_device), _t(cb, cuda_device), bits, 64)
    assert np.array_equal(p.cpu().numpy(), oracle.pack(codes, bits))
    assert np.array_equal(m.cpu().numpy(), mu) and np.array_equal(s.cpu().numpy(), sg)
    assert np.array_equal(c.cpu().numpy(), cs)
    with pkg._cabi.option("ARCQ_ACT_QUANT_V1", 1):           # same input through the other kernel
        p1, m1, s1, c1 = pkg.ops.quantize_activation(xd, _t(th, cuda_device), _t(cb, cuda_device), bits, 64)
    assert torch.equal(p, p1) and torch.equal(m, m1) and torch.equal(s, s1) and torch.equal(c, c1)
    if dtype != torch.float32:                              # and through the two-lanes-per-group form
        with pkg._cabi.option("ARCQ_ACT_QUANT_V2", 2):
            p2, m2, s2, c2 = pkg.ops.quantize_activation(xd, _t(th, cuda_device), _t(cb, cuda_device), bits, 64)
            xh2 = pkg.ops.quantize_activation_dequant(xd, _t(th, cuda_device), _t(cb, cuda_device), bits, 64, dtype)
        assert torch.equal(p, p2) and torch.equal(m, m2) and torch.equal(s, s2) and torch.equal(c, c2)
        assert torch.equal(xh2, pkg.ops.quantize_activation_dequant(xd, _t(th, cuda_device), _t(cb, cuda_device), bits, 64, dtype))
    # reconstruction output: the reference's three rounded fp32 steps in every kernel variant -> the same bits
    xh = pkg.ops.quantize_activation_dequant(xd, _t(th, cuda_device), _t(cb, cuda_device), bits, 64, dtype)
    want = torch.from_numpy(oracle.dequant(codes, mu, sg, cb, 64)).to(dtype)
    assert torch.equal(xh.cpu(), want)
    with pkg._cabi.option("ARCQ_ACT_QUANT_V1", 1):           # and the small-input kernel agrees bit for bit
        assert torch.equal(pkg.ops.quantize_activation_dequant(xd, _t(th, cuda_device), _t(cb, cuda_device), bits, 64, dtype), xh)
    assert pkg.ops.device_status() == 0


def test_staged_quantizer_with_close_thresholds_falls_back_to_the_search(pkg, oracle, cuda_device):
    # two thresholds closer than a grid cell: the first-guess table is not valid, the search must be used
    cb = np.array([-2.5, -2.0, -1.5, -1.0, -0.6, -0.3, -0.1, 0.0, 0.004, 0.008, 0.3, 0.7, 1.1, 1.6, 2.1, 2.6], np.float32)
    th = ((cb[:-1] + cb[1:]) / np.float32(2)).astype(np.float32)
    rng = np.random.default_rng(5)
    X = (rng.standard_normal((1024, 2560), dtype=np.float32) * 0.8).astype(np.float32)      # 40 960 groups
    codes, mu, sg, cs = oracle.quantize(X, th, cb, 64)
    p, m, s, c = pkg.ops.quantize_activation(_t(X, cuda_device), _t(th, cuda_device), _t(cb, cuda_device), 4, 64)
    assert np.array_equal(p.cpu().numpy(), oracle.pack(codes, 4))
    assert np.array_equal(c.cpu().numpy(), cs)


def _dequant_with_stats(pkg, x, th, cb, bits, pre_gelu=False):
    """arcq_act_quant through the C ABI with no packed output: reconstruction plus the three statistics."""
    lib = pkg._cabi.load()
    M, K = x.shape
    G = K // 64
    out = torch.empty_like(x)
    mu, sg, cs = (torch.empty((M, G), dtype=torch.float32, device=x.device) for _ in range(3))
    dt = {torch.float32: pkg._cabi.DT_F32, torch.float16: pkg._cabi.DT_F16, torch.bfloat16: pkg._cabi.DT_BF16}[x.dtype]
    fn = lib.arcq_gelu_act_quant if pre_gelu else lib.arcq_act_quant
    rc = fn(x.data_ptr(), dt, M, K, th.data_ptr(), cb.data_ptr(), bits, 64, None, mu.data_ptr(), sg.data_ptr(),
            cs.data_ptr(), out.data_ptr(), dt, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.arcq_last_error_string()
    return out, mu, sg, cs


@pytest.mark.parametrize("bits", [4, 3, 2])
@pytest.mark.parametrize("dtype", [torch.float16, torch.float32, torch.bfloat16])
def test_reconstruction_with_statistics_and_no_packed_output(pkg, oracle, cuda_device, bits, dtype):
    """The call the on-the-fly linear makes, plus the statistics: no packed output.  Statistics must be the
    oracle's bit for bit through both quantizer kernels, also with a ragged number of groups."""
    import os
    M, K = 1021, 2560                                        # 40 840 groups, not a multiple of a block
    rng = np.random.default_rng(bits * 11 + 3)
    X = rng.standard_normal((M, K), dtype=np.float32) * rng.uniform(0.05, 6.0, size=(M, 1)).astype(np.float32)
    X[:, ::31] *= 9.0
    x = torch.from_numpy(X).to(dtype)
    L = 2 ** bits
    if bits == 4:
        cb = np.concatenate([-np.linspace(0, 2.6, 8)[1:][::-1], [0.0], np.linspace(0, 2.58, 9)[1:]]).astype(np.float32)
    else:
        cb = np.sort(rng.uniform(-2.8, 2.8, L)).astype(np.float32)
    th = ((cb[:-1] + cb[1:]) / np.float32(2)).astype(np.float32)
    codes, mu, sg, cs = oracle.quantize(x.float().numpy(), th, cb, 64)
    xd, thd, cbd = x.to(cuda_device), _t(th, cuda_device), _t(cb, cuda_device)
    xh, m, s, c = _dequant_with_stats(pkg, xd, thd, cbd, bits)
    assert np.array_equal(m.cpu().numpy(), mu) and np.array_equal(s.cpu().numpy(), sg)
    assert np.array_equal(c.cpu().numpy(), cs)               # equal code sums <=> equal codes, group by group
    with pkg._cabi.option("ARCQ_ACT_QUANT_V1", 1):           # same call through the 8-lanes-per-group kernel
        xh1, m1, s1, c1 = _dequant_with_stats(pkg, xd, thd, cbd, bits)
    assert torch.equal(c, c1) and torch.equal(m, m1) and torch.equal(s, s1)
    if dtype == torch.float32:
        assert float((xh - xh1).abs().max()) <= 4e-6 * float(xh1.abs().max())
    else:
        assert float((xh == xh1).float().mean()) > 0.999
    assert pkg.ops.device_status() == 0


def test_quantizer_with_a_threshold_at_zero_and_with_close_thresholds(pkg, oracle, cuda_device):
    """A threshold that is exactly zero keeps the division-free test (its boundary is half the smallest
    subnormal); two thresholds closer than a first-guess cell fall back to the search.  GELU fused in front."""
    rng = np.random.default_rng(17)
    X = (rng.standard_normal((1024, 2560), dtype=np.float32) * 0.8).astype(np.float32)      # 40 960 groups
    X[5, :64] = 0.0                                                                          # an all-zero group
    X[6, :64] = np.float32(1e-30)
    for cb in (np.array([-2.5, -2.0, -1.5, -1.0, -0.6, -0.3, -0.1, 0.0, 0.004, 0.008, 0.3, 0.7, 1.1, 1.6, 2.1, 2.6], np.float32),
               np.array([-2.4, -1.9, -1.4, -1.0, -0.7, -0.45, -0.25, -0.1, 0.1, 0.25, 0.45, 0.7, 1.0, 1.4, 1.9, 2.4], np.float32)):
        th = ((cb[:-1] + cb[1:]) / np.float32(2)).astype(np.float32)      # second codebook: th[7] == 0 exactly
        codes, mu, sg, cs = oracle.quantize(X, th, cb, 64)
        xh, m, s, c = _dequant_with_stats(pkg, _t(X, cuda_device), _t(th, cuda_device), _t(cb, cuda_device), 4)
        assert np.array_equal(c.cpu().numpy(), cs) and np.array_equal(s.cpu().numpy(), sg)
        p = pkg.ops.quantize_activation(_t(X, cuda_device), _t(th, cuda_device), _t(cb, cuda_device), 4, 64)[0]
        assert np.array_equal(p.cpu().numpy(), oracle.pack(codes, 4))
        want = oracle.dequant(codes, mu, sg, cb, 64)
        assert float(np.abs(xh.cpu().numpy() - want).max()) <= 4e-6 * float(np.abs(want).max())
    # GELU in front: same as quantising the stored fp16 activation
    pre = (torch.randn(600, 1536, generator=torch.Generator().manual_seed(3)) * 1.5).half().to(cuda_device)
    cbt = torch.linspace(-2.6, 2.6, 16, device=cuda_device)
    tht = (cbt[:-1] + cbt[1:]) / 2
    act = torch.nn.functional.gelu(pre)
    want = _dequant_with_stats(pkg, act, tht, cbt, 4)[0]
    got = _dequant_with_stats(pkg, pre, tht, cbt, 4, pre_gelu=True)[0]
    assert float((want == got).float().mean()) > 0.999
    assert pkg.ops.device_status() == 0


def test_fused_gelu_over_every_fp16_input(pkg, cuda_device, report):
    """The fused GELU must store what a separate fp16 GELU kernel stores.  Every finite fp16 value goes through
    it (shuffled, so small and large arguments share warps) and the reconstruction is compared with the one
    computed from torch's GELU output."""
    vals = torch.arange(65536, dtype=torch.int32).to(torch.int16).view(torch.float16)
    vals = vals[torch.isfinite(vals)]
    gen = torch.Generator().manual_seed(11)
    reps = 20                                                     # 63 488 values x 40 = 39 680 groups
    by_size = torch.argsort(vals.float().abs(), stable=True)      # groups of like magnitude: small values count
    idx = torch.cat([torch.randperm(vals.numel(), generator=gen) for _ in range(reps)] + [by_size] * reps)
    pre = vals[idx].reshape(-1, 2560).to(cuda_device)
    pre = torch.where(pre.abs() > 30000, pre.sign() * 30000, pre)  # keep group statistics finite
    cb = torch.linspace(-2.6, 2.55, 16, device=cuda_device)
    th = (cb[:-1] + cb[1:]) / 2
    act = torch.nn.functional.gelu(pre)
    want = pkg.ops.quantize_activation_dequant(act, th, cb, 4, 64, torch.float16)
    got = pkg.ops.quantize_activation_dequant(pre, th, cb, 4, 64, torch.float16, True)
    groups_equal = float((want.view(-1, 64) == got.view(-1, 64)).all(dim=1).float().mean())
    report("fused_gelu_all_fp16_inputs", groups_equal=groups_equal)
    # a differing GELU value changes its whole group's statistics; 3 such inputs in 63 488 can touch 0.3 % of groups
    assert groups_equal > 0.99, groups_equal
    assert pkg.ops.device_status() == 0


@pytest.mark.parametrize("out_dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("M,K,N", [(1, 64, 16), (129, 128, 48), (197, 384, 1152), (300, 1536, 384), (1000, 768, 2304),
                                   (64 * 197, 1536, 384), (64 * 197, 384, 1536)])
def test_dense_weight_gemm_matches_an_fp64_product(pkg, cuda_device, M, K, N, out_dtype):
    """The persistent kernel with an fp16 weight matrix as its second operand (sub-tiles by TMA, nothing
    rebuilt): against the fp64 product of the same fp16 operands."""
    gen = torch.Generator().manual_seed(M + K + N)
    x = torch.randn(M, K, generator=gen).half().to(cuda_device)
    w = (torch.randn(N, K, generator=gen) * 0.05).half().to(cuda_device)
    b = torch.randn(N, generator=gen).to(cuda_device)
    y = pkg.ops.dense_weight_gemm(x, w, b, out_dtype)
    ref = x.double() @ w.double().t() + b.double()
    err = float((y.double() - ref).abs().max() / ref.pow(2).mean().sqrt())
    assert y.dtype == out_dtype and err < (2e-3 if out_dtype == torch.float16 else 2e-5), err
    y0 = pkg.ops.dense_weight_gemm(x, w, None, out_dtype)
    assert float((y0.double() - (ref - b.double())).abs().max() / ref.pow(2).mean().sqrt()) < 2e-3
    assert pkg.ops.device_status() == 0


def test_dense_route_of_the_linear_equals_the_packed_route(pkg, oracle, golden, cuda_device):
    """Unpack into scratch + dense GEMM (the reference's data flow) against the in-kernel rebuild: the two weight
    forms differ only in how W^ is rounded to fp16, so outputs agree far inside the parity tolerance."""
    rng = np.random.default_rng(21)
    M, K, N, bits = 2100, 1536, 384, 4
    X = rng.standard_normal((M, K), dtype=np.float32)
    W = (rng.standard_normal((N, K), dtype=np.float32) * 0.03).astype(np.float32)
    cb = np.concatenate([-np.linspace(0, 2.6, 8)[1:][::-1], [0.0], np.linspace(0, 2.58, 9)[1:]]).astype(np.float32)
    th = ((cb[:-1] + cb[1:]) / np.float32(2)).astype(np.float32)
    thd, cbd = _t(th, cuda_device), _t(cb, cuda_device)
    pw, mw, sw, cw = pkg.ops.quantize_activation(_t(W, cuda_device), thd, cbd, bits, 64)
    xh = pkg.ops.quantize_activation_dequant(_t(X, cuda_device).half(), thd, cbd, bits, 64, torch.float16)
    y_packed = pkg.ops.packed_weight_gemm(xh, pw, mw, sw, cw, cbd, None, bits, 64, torch.float16)
    scratch = torch.empty(N * K + 100, dtype=torch.float16, device=cuda_device)
    w16 = pkg.ops.dequant(pw, mw, sw, cw, cbd, bits, 64, torch.float16, out=scratch)
    assert w16.data_ptr() == scratch.data_ptr() and tuple(w16.shape) == (N, K)
    codes, mu, sg, cs = oracle.quantize(W, th, cb, 64)
    assert float((w16.float().cpu() - torch.from_numpy(oracle.dequant(codes, mu, sg, cb, 64))).abs().max()) < 1e-3
    y_dense = pkg.ops.dense_weight_gemm(xh, w16, None, torch.float16)
    rms = float(y_packed.float().pow(2).mean().sqrt())
    assert float((y_dense.float() - y_packed.float()).abs().max()) < 1e-2 * rms
    assert pkg.ops.device_status() == 0


def test_two_lane_quantizer_search_and_zero_threshold_paths(pkg, oracle, cuda_device):
    """The two-lanes-per-group form on codebooks that leave the first-guess path (close thresholds -> search) or
    have a threshold at zero, fp16 and bf16 inputs, ragged group count, all three outputs."""
    import os
    rng = np.random.default_rng(23)
    X = (rng.standard_normal((1023, 2560), dtype=np.float32) * 0.8).astype(np.float32)      # 40 920 groups
    X[7, :64] = 0.0
    with pkg._cabi.option("ARCQ_ACT_QUANT_V2", 2):
        for dtype in (torch.float16, torch.bfloat16):
            x = torch.from_numpy(X).to(dtype)
            xr = x.float().numpy()
            for cb in (np.array([-2.5, -2.0, -1.5, -1.0, -0.6, -0.3, -0.1, 0.0, 0.004, 0.008, 0.3, 0.7, 1.1, 1.6, 2.1, 2.6], np.float32),
                       np.array([-2.4, -1.9, -1.4, -1.0, -0.7, -0.45, -0.25, -0.1, 0.1, 0.25, 0.45, 0.7, 1.0, 1.4, 1.9, 2.4], np.float32)):
                th = ((cb[:-1] + cb[1:]) / np.float32(2)).astype(np.float32)
                codes, mu, sg, cs = oracle.quantize(xr, th, cb, 64)
                p, m, s, c = pkg.ops.quantize_activation(x.to(cuda_device), _t(th, cuda_device), _t(cb, cuda_device), 4, 64)
                assert np.array_equal(p.cpu().numpy(), oracle.pack(codes, 4))
                assert np.array_equal(m.cpu().numpy(), mu) and np.array_equal(s.cpu().numpy(), sg)
                assert np.array_equal(c.cpu().numpy(), cs)
            # 3-bit and 2-bit packing of the swapped half-words
            for bits in (3, 2):
                cb = np.sort(rng.uniform(-2.8, 2.8, 2 ** bits)).astype(np.float32)
                th = ((cb[:-1] + cb[1:]) / np.float32(2)).astype(np.float32)
                codes, mu, sg, cs = oracle.quantize(xr, th, cb, 64)
                p = pkg.ops.quantize_activation(x.to(cuda_device), _t(th, cuda_device), _t(cb, cuda_device), bits, 64)[0]
                assert np.array_equal(p.cpu().numpy(), oracle.pack(codes, bits))
    assert pkg.ops.device_status() == 0
