"""The entry point that owns its weight scratch (`arcq_packed_linear_static_scratch`), called through the C
ABI.  Collected last, and written to pass both on its own and after every other GPU test: it depends on no
state but the library's static array, whose content it never assumes."""

import pytest
import torch

pytestmark = pytest.mark.gpu

STATIC_ELEMS = 768 * 3072
E_TOO_LARGE = -6


def _problem(pkg, dev, M, K, N, bits, seed):
    gen = torch.Generator().manual_seed(seed)
    L = 2 ** bits
    cb = torch.linspace(-2.6, 2.55, L, device=dev)
    th = (cb[:-1] + cb[1:]) / 2
    x = torch.randn(M, K, generator=gen).half().to(dev)
    w = (torch.randn(N, K, generator=gen) * 0.03).to(dev)
    bias = torch.randn(N, generator=gen).to(dev)
    pw, mu, sg, cs = pkg.ops.quantize_activation(w, th, cb, bits, 64)
    xh = pkg.ops.quantize_activation_dequant(x, th, cb, bits, 64, torch.float16)
    return xh, pw, mu, sg, cs, cb, bias


def _static(lib, xh, pw, mu, sg, cs, cb, bias, bits, y):
    M, K = xh.shape
    N = pw.shape[0]
    return lib.arcq_packed_linear_static_scratch(
        xh.data_ptr(), pw.data_ptr(), mu.data_ptr(), sg.data_ptr(), cs.data_ptr(), cb.data_ptr(),
        bias.data_ptr() if bias is not None else None, bits, 64, M, N, K, y.data_ptr(),
        1 if y.dtype == torch.float16 else 0, torch.cuda.current_stream().cuda_stream)


def _caller_scratch(lib, xh, pw, mu, sg, cs, cb, bias, bits, y):
    """The existing route: arcq_dequant into a buffer of the caller, then arcq_dense_weight_gemm."""
    M, K = xh.shape
    N = pw.shape[0]
    w16 = torch.empty(N, K, dtype=torch.float16, device=xh.device)
    st = torch.cuda.current_stream().cuda_stream
    rc = lib.arcq_dequant(pw.data_ptr(), mu.data_ptr(), sg.data_ptr(), cs.data_ptr(), cb.data_ptr(), bits, 64, N, K,
                          w16.data_ptr(), 1, st)
    assert rc == 0, lib.arcq_last_error_string()
    rc = lib.arcq_dense_weight_gemm(xh.data_ptr(), w16.data_ptr(), bias.data_ptr() if bias is not None else None,
                                    M, N, K, y.data_ptr(), 1 if y.dtype == torch.float16 else 0, st)
    assert rc == 0, lib.arcq_last_error_string()


def test_static_scratch_linear_equals_the_caller_scratch_route_twice_in_a_row(pkg, cuda_device):
    lib = pkg._cabi.load()
    # two calls back to back with different weights and shapes: the second must not see the first one's weight
    cases = [(300, 1536, 384, 4, 1), (197, 384, 1152, 3, 2)]
    probs = [_problem(pkg, cuda_device, M, K, N, bits, seed) for M, K, N, bits, seed in cases]
    outs = []
    for (M, K, N, bits, _), pr in zip(cases, probs):
        y = torch.full((M, N), float("nan"), dtype=torch.float16, device=cuda_device)
        rc = _static(lib, *pr, bits, y)
        assert rc == 0, lib.arcq_last_error_string()
        outs.append(y)
    torch.cuda.synchronize()
    for (M, K, N, bits, _), pr, y in zip(cases, probs, outs):
        want = torch.empty_like(y)
        _caller_scratch(lib, *pr, bits, want)
        assert torch.equal(y, want)
        xh, pw, mu, sg, cs, cb, bias = pr
        ref = xh.double() @ pkg.ops.dequant(pw, mu, sg, cs, cb, bits, 64, torch.float32).double().t() + bias.double()
        assert float((y.double() - ref).abs().max() / ref.pow(2).mean().sqrt()) < 5e-3
    # fp32 output and no bias through the same entry
    M, K, N, bits, _ = cases[0]
    xh, pw, mu, sg, cs, cb, bias = probs[0]
    y32 = torch.empty((M, N), dtype=torch.float32, device=cuda_device)
    assert _static(lib, xh, pw, mu, sg, cs, cb, None, bits, y32) == 0
    want32 = torch.empty_like(y32)
    _caller_scratch(lib, xh, pw, mu, sg, cs, cb, None, bits, want32)
    assert torch.equal(y32, want32)
    assert pkg.ops.device_status() == 0


def test_static_scratch_linear_rejects_a_weight_beyond_its_capacity(pkg, cuda_device):
    lib = pkg._cabi.load()
    K, N = 3072, 832                                     # 832 * 3072 > 768 * 3072
    assert N * K > STATIC_ELEMS
    dummy = torch.zeros(16, dtype=torch.float32, device=cuda_device)
    x = torch.zeros(8, K, dtype=torch.float16, device=cuda_device)
    pw = torch.zeros(N, K // 2, dtype=torch.uint8, device=cuda_device)
    st = torch.zeros(N, K // 64, dtype=torch.float32, device=cuda_device)
    y = torch.zeros(8, N, dtype=torch.float16, device=cuda_device)
    rc = lib.arcq_packed_linear_static_scratch(x.data_ptr(), pw.data_ptr(), st.data_ptr(), st.data_ptr(), st.data_ptr(),
                                               dummy.data_ptr(), None, 4, 64, 8, N, K, y.data_ptr(), 1,
                                               torch.cuda.current_stream().cuda_stream)
    assert rc == E_TOO_LARGE
    assert b"exceeds the static scratch" in lib.arcq_last_error_string()
    # a null pointer is refused before anything else
    assert lib.arcq_packed_linear_static_scratch(None, pw.data_ptr(), st.data_ptr(), st.data_ptr(), st.data_ptr(),
                                                 dummy.data_ptr(), None, 4, 64, 8, N, K, y.data_ptr(), 1, None) == -1


def test_static_scratch_linear_rejects_bad_arguments_before_its_first_launch(pkg, cuda_device):
    """What either of its two launches would refuse (output type, N not a multiple of 16, a misaligned output) is
    refused up front, so a rejected call never gets as far as overwriting the shared weight scratch."""
    lib = pkg._cabi.load()
    M, K, N = 64, 384, 384
    dummy = torch.zeros(16, dtype=torch.float32, device=cuda_device)
    x = torch.zeros(M, K, dtype=torch.float16, device=cuda_device)
    pw = torch.zeros(N, K // 2, dtype=torch.uint8, device=cuda_device)
    st = torch.zeros(N, K // 64, dtype=torch.float32, device=cuda_device)
    y = torch.zeros(M * N + 8, dtype=torch.float16, device=cuda_device)
    stream = torch.cuda.current_stream().cuda_stream

    def call(n=N, k=K, ydt=1, yptr=None, bits=4):
        return lib.arcq_packed_linear_static_scratch(x.data_ptr(), pw.data_ptr(), st.data_ptr(), st.data_ptr(), st.data_ptr(),
                                                     dummy.data_ptr(), None, bits, 64, M, n, k,
                                                     y.data_ptr() if yptr is None else yptr, ydt, stream)
    assert call(ydt=2) == -1 and b"y_dtype" in lib.arcq_last_error_string()          # bf16 output is not built
    assert call(n=N - 8) == -3                                                        # N % 16 != 0
    assert call(yptr=y.data_ptr() + 2) == -4                                          # misaligned output
    assert call(bits=5) == -1
    assert call() == 0                                                                # and the plain call still runs
    torch.cuda.synchronize()
    assert pkg.ops.device_status() == 0
