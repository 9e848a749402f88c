"""The CTA-pair form of the packed-weight GEMM (tcgen05 cta_group::2): equal, bit for bit, to the one-CTA
kernel on the same operands, for every slab width / stage configuration it can be given; the one-CTA
kernel's epilogue with odd step counts; and the path a bounded wait takes when it runs out."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _operands(pkg, dev, M, K, N, bits, seed):
    gen = torch.Generator().manual_seed(seed)
    cb = torch.sort(torch.randn(2 ** bits, generator=gen) * 1.2)[0].to(dev)
    th = (cb[:-1] + cb[1:]) / 2
    x = torch.randn(M, K, generator=gen).half().to(dev)
    w = (torch.randn(N, K, generator=gen) * 0.02).to(dev)
    bias = (torch.randn(N, generator=gen) * 0.01).to(dev)
    pw, mw, sw, cw = pkg.ops.quantize_activation(w, th, cb, bits, 64)
    xh = pkg.ops.quantize_activation_dequant(x, th, cb, bits, 64, torch.float16)
    return xh, pw, mw, sw, cw, cb, bias


def _run(pkg, ops_args, bits, out_dtype, **options):
    xh, pw, mw, sw, cw, cb, bias = ops_args
    saved = {k: pkg._cabi.get_option(k) for k in options}
    try:
        for k, v in options.items():
            pkg._cabi.set_option(k, v)
        y = pkg.ops.packed_weight_gemm(xh, pw, mw, sw, cw, cb, bias, bits, 64, out_dtype)
        assert pkg.ops.device_status() == 0, f"a bounded wait ran out with {options}"
        return y
    finally:
        for k, v in saved.items():
            pkg._cabi.set_option(k, v)


def _fp64(pkg, ops_args, bits):
    xh, pw, mw, sw, cw, cb, bias = ops_args
    wa = pkg.ops.dequant(pw, mw, sw, cw, cb, bits, 64, torch.float16)
    return xh.double() @ wa.double().T + bias.double()


@pytest.mark.parametrize("out_dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("bits", [4, 3, 2])
@pytest.mark.parametrize("M,K,N", [(256, 64, 64), (300, 384, 192), (1024, 384, 384), (2049, 192, 576), (64 * 197, 384, 1536),
                                   (64 * 197, 1536, 384), (3000, 768, 2304), (1500, 3072, 768)])
def test_pair_kernel_equals_the_one_cta_kernel(pkg, cuda_device, M, K, N, bits, out_dtype):
    if not pkg.ops.packed_weight_gemm_supported(K, N, bits, 64):
        pytest.skip("shape is routed to the packed-codes kernel")
    a = _operands(pkg, cuda_device, M, K, N, bits, seed=M + K + N + bits)
    y_pair = _run(pkg, a, bits, out_dtype, ARCQ_PAIR=1, ARCQ_PAIR_MIN_M=1)
    y_one = _run(pkg, a, bits, out_dtype, ARCQ_PAIR=0)
    assert torch.equal(y_pair, y_one)
    ref = _fp64(pkg, a, bits)
    err = float((y_pair.double() - ref).abs().max() / ref.pow(2).mean().sqrt())
    assert err < (6e-3 if bits > 2 else 1.2e-2), f"max|dy|/rms = {err:.3e}"   # only the fp16 rounding of the rebuilt weight differs


@pytest.mark.parametrize("options", [
    dict(ARCQ_PAIR_BN=32), dict(ARCQ_PAIR_BN=64), dict(ARCQ_PAIR_BN=96), dict(ARCQ_PAIR_BN=128), dict(ARCQ_PAIR_BN=192),
    dict(ARCQ_PAIR_KS=1), dict(ARCQ_PAIR_KS=2), dict(ARCQ_PAIR_KS=3), dict(ARCQ_PAIR_KS=6, ARCQ_PAIR_SA=2),
    dict(ARCQ_PAIR_SA=2), dict(ARCQ_PAIR_SA=3, ARCQ_PAIR_KS=1), dict(ARCQ_PAIR_LUT=4), dict(ARCQ_PAIR_LUT=5, ARCQ_PAIR_SA=2),
    dict(ARCQ_PAIR_PAIRS=5), dict(ARCQ_PAIR_PAIRS=1), dict(ARCQ_PDL=0),
    dict(ARCQ_PAIR_STATIONARY=0), dict(ARCQ_PAIR_STATIONARY=0, ARCQ_PAIR_NBB=1), dict(ARCQ_PAIR_STATIONARY=0, ARCQ_PAIR_WS=2),
    dict(ARCQ_PAIR_STATIONARY=0, ARCQ_PAIR_WS=6, ARCQ_PAIR_KS=3), dict(ARCQ_PAIR_STATIONARY=0, ARCQ_PAIR_KS=1, ARCQ_PAIR_WS=3),
])
def test_pair_kernel_configurations_agree(pkg, cuda_device, options):
    """Slab widths, stage shapes, ring depths, grid sizes: the result does not depend on them."""
    M, K, N, bits = 4000, 384, 576, 4
    a = _operands(pkg, cuda_device, M, K, N, bits, seed=5)
    base = _run(pkg, a, bits, torch.float16, ARCQ_PAIR=0)
    y = _run(pkg, a, bits, torch.float16, ARCQ_PAIR=1, ARCQ_PAIR_MIN_M=1, **options)
    assert torch.equal(y, base), options


def test_pair_kernel_rows_do_not_depend_on_batch_or_order(pkg, cuda_device):
    M, K, N, bits = 64 * 197, 384, 1152, 4
    xh, pw, mw, sw, cw, cb, bias = _operands(pkg, cuda_device, M, K, N, bits, seed=9)
    f = lambda x: pkg.ops.packed_weight_gemm(x, pw, mw, sw, cw, cb, bias, bits, 64, torch.float16)  # noqa: E731
    y = f(xh)
    perm = torch.randperm(M, generator=torch.Generator().manual_seed(1)).to(cuda_device)
    assert torch.equal(f(xh[perm].contiguous()), y[perm])
    assert torch.equal(f(xh[1000:1197].contiguous()), y[1000:1197])       # one image's rows alone (one-CTA kernel)
    assert torch.equal(f(xh[:5000].contiguous()), y[:5000])
    assert pkg.ops.device_status() == 0


@pytest.mark.parametrize("out_dtype,bn", [(torch.float16, 96), (torch.float16, 32), (torch.float32, 48), (torch.float32, 16)])
def test_one_cta_kernel_epilogue_with_an_odd_number_of_store_steps(pkg, cuda_device, out_dtype, bn):
    """Slab widths whose tile takes an odd number of 64-byte store steps, with several tiles per CTA: the two
    staging blocks must keep alternating from one tile to the next."""
    M, K, bits = 40 * 128 + 17, 384, 4
    N = 3 * bn
    a = _operands(pkg, cuda_device, M, K, N, bits, seed=bn)
    y = _run(pkg, a, bits, out_dtype, ARCQ_PAIR=0, ARCQ_WS_BN=bn, ARCQ_WS_GRID=3)     # 41 row tiles on one CTA per slab
    ref = _fp64(pkg, a, bits)
    err = float((y.double() - ref).abs().max() / ref.pow(2).mean().sqrt())
    assert err < 6e-3, f"max|dy|/rms = {err:.3e}"


def test_a_wait_that_runs_out_sets_the_status_word_and_returns(pkg, cuda_device):
    lib = pkg._cabi.load()
    assert pkg.ops.device_status() == 0
    assert lib.arcq_debug_wait_timeout(200, torch.cuda.current_stream().cuda_stream) == 0
    assert pkg.ops.device_status() == 0x7E57            # the wait gave up and said so
    assert pkg.ops.device_status() == 0                 # reading clears the word
    assert lib.arcq_debug_wait_timeout(1 << 20, None) != 0      # long limits are refused before any launch
    # the device is fine: a GEMM right after is correct
    a = _operands(pkg, cuda_device, 2000, 384, 384, 4, seed=3)
    y = _run(pkg, a, 4, torch.float16)
    ref = _fp64(pkg, a, 4)
    assert float((y.double() - ref).abs().max() / ref.pow(2).mean().sqrt()) < 6e-3

