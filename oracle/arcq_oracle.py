"""CPU oracle for the ARCQ packed inference path.  TEST INFRASTRUCTURE ONLY.

Python face of ``arcq_oracle.c`` (built by ``make -C oracle`` or by
``build()`` below) plus a numpy restatement of the reference's host-side
codebook fit.  Only tests, the smoke check and the CPU-baseline / reference leg
of the benchmark may import this module; the product package never does.

Parity status: pinned against the reference run on CPU through the committed
fixtures under ``tests/golden`` (made by ``tests/golden/make_golden.py``, which
imports the reference quantizer, packer and packed-linear constructor).

Reference paths are relative to the reference project; ``FQ`` stands for
``methods/fair_qat_framework``.
"""
from __future__ import annotations

import ctypes
import math
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_SO = _HERE / "libarcq_oracle.so"
_SRC = _HERE / "arcq_oracle.c"
_lib = None

_f32p = ctypes.POINTER(ctypes.c_float)
_u8p = ctypes.POINTER(ctypes.c_uint8)


def build(force: bool = False) -> Path:
    """Compile the C restatement with gcc (no fused multiply-add contraction)."""
    if force or not _SO.exists() or _SO.stat().st_mtime < _SRC.stat().st_mtime:
        cmd = ["gcc", "-O2", "-std=c11", "-fPIC", "-shared", "-fopenmp", "-ffp-contract=off",
               "-fvisibility=hidden", str(_SRC), "-o", str(_SO), "-lm"]
        subprocess.run(cmd, check=True)
    return _SO


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(str(_SO))
        i64, ci, cf = ctypes.c_int64, ctypes.c_int, ctypes.c_float
        L.arcq_oracle_row_sums.argtypes = [_f32p, i64, ci, _f32p]
        L.arcq_oracle_quantize.argtypes = [_f32p, i64, i64, ci, _f32p, _f32p, ci, cf, _u8p, _f32p, _f32p, _f32p]
        L.arcq_oracle_dequant.argtypes = [_u8p, i64, i64, ci, _f32p, _f32p, _f32p, _f32p]
        L.arcq_oracle_pack.argtypes = [_u8p, i64, i64, ci, _u8p]
        L.arcq_oracle_unpack.argtypes = [_u8p, i64, i64, ci, _u8p]
        L.arcq_oracle_linear_codesum.argtypes = [_u8p, _f32p, _f32p, _f32p, _u8p, _f32p, _f32p, _f32p,
                                                 _f32p, _f32p, _f32p, i64, i64, i64, ci, _f32p]
        L.arcq_oracle_linear_dense.argtypes = [_f32p, _f32p, _f32p, i64, i64, i64, _f32p]
        L.arcq_oracle_set_threads.argtypes = [ci]
        L.arcq_oracle_max_threads.restype = ci
        _lib = L
    return _lib


def set_threads(n: int) -> None:
    lib().arcq_oracle_set_threads(int(n))


def max_threads() -> int:
    return int(lib().arcq_oracle_max_threads())


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _u8(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.uint8)


def _p(a: np.ndarray, t):
    return a.ctypes.data_as(t)


def row_sums(x) -> np.ndarray:
    """Sum over the last axis in the reference's (torch CPU) fp32 order."""
    x = _f32(x)
    n = x.shape[-1]
    out = np.empty(x.shape[:-1], np.float32)
    lib().arcq_oracle_row_sums(_p(x, _f32p), x.size // n, n, _p(out, _f32p))
    return out


def quantize(x, thresholds, codebook, group_size: int = 64, eps: float = 1e-6):
    """Group-residual quantizer (FQ/quant/dcarcq.py:531-556).

    x: [rows, cols] (any float dtype; the arithmetic is fp32 on the values as
    given).  Returns (codes uint8 [rows, cols], mu, sigma, code_sum fp32
    [rows, cols/group_size]).
    """
    x = _f32(x)
    rows, cols = x.shape
    th, cb = _f32(thresholds), _f32(codebook)
    assert th.size == cb.size - 1
    G = cols // group_size
    codes = np.empty((rows, cols), np.uint8)
    mu = np.empty((rows, G), np.float32)
    sg = np.empty((rows, G), np.float32)
    cs = np.empty((rows, G), np.float32)
    rc = lib().arcq_oracle_quantize(_p(x, _f32p), rows, cols, group_size, _p(th, _f32p), _p(cb, _f32p),
                                    cb.size, eps, _p(codes, _u8p), _p(mu, _f32p), _p(sg, _f32p), _p(cs, _f32p))
    if rc != 0:
        raise ValueError("arcq_oracle_quantize: bad shape")
    return codes, mu, sg, cs


def dequant(codes, mu, sigma, codebook, group_size: int = 64) -> np.ndarray:
    """x_hat = mu + sigma * (cb[c] - mean_g cb[c])  (FQ/quant/dcarcq.py:556-563)."""
    codes = _u8(codes)
    rows, cols = codes.shape
    out = np.empty((rows, cols), np.float32)
    mu, sigma, cb = _f32(mu), _f32(sigma), _f32(codebook)
    rc = lib().arcq_oracle_dequant(_p(codes, _u8p), rows, cols, group_size, _p(cb, _f32p), _p(mu, _f32p),
                                   _p(sigma, _f32p), _p(out, _f32p))
    if rc != 0:
        raise ValueError("arcq_oracle_dequant: bad shape")
    return out


def fake_quant(x, thresholds, codebook, group_size: int = 64, eps: float = 1e-6) -> np.ndarray:
    """Forward value of the fake-quant module: x + (x_hat - x) in fp32, the straight-through
    form the reference returns (FQ/quant/dcarcq.py:565), which differs from x_hat by rounding."""
    x = _f32(x)
    codes, mu, sg, _ = quantize(x, thresholds, codebook, group_size, eps)
    x_hat = dequant(codes, mu, sg, codebook, group_size)
    return x + (x_hat - x)


def packed_cols(length: int, bits: int) -> int:
    return (length * bits + 7) // 8


def pack(codes, bits: int) -> np.ndarray:
    """Bit layout of FQ/fair_qat/arcq_packed_py.py:8-47."""
    codes = _u8(codes)
    rows, length = codes.shape
    out = np.empty((rows, packed_cols(length, bits)), np.uint8)
    lib().arcq_oracle_pack(_p(codes, _u8p), rows, length, bits, _p(out, _u8p))
    return out


def unpack(packed, bits: int, length: int) -> np.ndarray:
    """Inverse of pack (FQ/fair_qat/arcq_packed_py.py:50-78)."""
    packed = _u8(packed)
    rows = packed.shape[0]
    assert packed.shape[1] == packed_cols(length, bits)
    out = np.empty((rows, length), np.uint8)
    lib().arcq_oracle_unpack(_p(packed, _u8p), rows, length, bits, _p(out, _u8p))
    return out


def linear_codesum(ca, mu_a, sg_a, cs_a, cw, mu_w, sg_w, cs_w, cb_a, cb_w, bias, group_size: int = 64):
    """Packed linear in the code-sum form (arcq_infer_cuda/arcq_linear_kernel.cu:22-78), fp64 acc."""
    ca, cw = _u8(ca), _u8(cw)
    M, K = ca.shape
    N = cw.shape[0]
    y = np.empty((M, N), np.float32)
    b = _f32(bias) if bias is not None and np.size(bias) else None
    args = [_f32(a) for a in (mu_a, sg_a, cs_a, mu_w, sg_w, cs_w, cb_a, cb_w)]
    lib().arcq_oracle_linear_codesum(_p(ca, _u8p), _p(args[0], _f32p), _p(args[1], _f32p), _p(args[2], _f32p),
                                     _p(cw, _u8p), _p(args[3], _f32p), _p(args[4], _f32p), _p(args[5], _f32p),
                                     _p(args[6], _f32p), _p(args[7], _f32p),
                                     _p(b, _f32p) if b is not None else None, M, N, K, group_size, _p(y, _f32p))
    return y


def linear_dense(x_hat, w_hat, bias) -> np.ndarray:
    """Fake-quant contraction (FQ/fair_qat/quant_backends.py:320-322), fp64 acc, one rounding."""
    x_hat, w_hat = _f32(x_hat), _f32(w_hat)
    M, K = x_hat.shape
    N = w_hat.shape[0]
    y = np.empty((M, N), np.float32)
    b = _f32(bias) if bias is not None and np.size(bias) else None
    lib().arcq_oracle_linear_dense(_p(x_hat, _f32p), _p(w_hat, _f32p), _p(b, _f32p) if b is not None else None,
                                   M, N, K, _p(y, _f32p))
    return y


def fake_quant_linear(x, weight, bias, act_thresholds, act_codebook, w_thresholds, w_codebook,
                      group_size: int = 64, eps: float = 1e-6, fast_gemm: bool = False):
    """QuantLinearPCARCQ.forward with frozen codebooks (FQ/fair_qat/quant_backends.py:312-322).

    Returns (y fp32 [M,N], dict of intermediates).  ``fast_gemm`` contracts the
    two fake-quantised operands with the host BLAS in fp32 (what the reference
    does) instead of the fp64-accumulating loop; used for whole-model runs.
    """
    ca, mu_a, sg_a, cs_a = quantize(x, act_thresholds, act_codebook, group_size, eps)
    cw, mu_w, sg_w, cs_w = quantize(weight, w_thresholds, w_codebook, group_size, eps)
    xf, wf = _f32(x), _f32(weight)
    x_hat = dequant(ca, mu_a, sg_a, act_codebook, group_size)
    w_hat = dequant(cw, mu_w, sg_w, w_codebook, group_size)
    x_hat = xf + (x_hat - xf)          # straight-through forward value, FQ/quant/dcarcq.py:565
    w_hat = wf + (w_hat - wf)
    if fast_gemm:
        y = x_hat @ w_hat.T
        if bias is not None and np.size(bias):
            y = y + _f32(bias)[None, :]
        y = y.astype(np.float32, copy=False)
    else:
        y = linear_dense(x_hat, w_hat, bias)
    inter = dict(act_codes=ca, act_mu=mu_a, act_sigma=sg_a, act_code_sum=cs_a, w_codes=cw, w_mu=mu_w,
                 w_sigma=sg_w, w_code_sum=cs_w, x_hat=x_hat, w_hat=w_hat)
    return y, inter


# ---------------------------------------------------------------------------
# Codebook fit (host side, one-off; its outputs are inputs to the kernels)
# Restates ARCQQuantizer._build_codebook_from_flat and its moment tables,
# FQ/quant/dcarcq.py:24-105 and :155-290 (bits >= 3 and bits == 2 branches).
# ---------------------------------------------------------------------------
_N_BETA = 512
_TAU_N_U = 4096
_tables: dict = {}


def _moment_tables():
    if _tables:
        return _tables
    beta = np.linspace(0.75, 8.0, _N_BETA, dtype=np.float64).astype(np.float32)
    kappa = np.empty(_N_BETA, np.float32)
    for i in range(_N_BETA):
        b = float(beta[i])
        kappa[i] = math.exp(math.lgamma(5.0 / b) + math.lgamma(1.0 / b) - 2.0 * math.lgamma(3.0 / b))
    taus = {}
    for bits in (1, 2, 3, 4, 5, 6, 8):
        L = 2 ** bits
        target = 1.0 - 1.0 / (2.0 * L * L)
        tau = np.full(_N_BETA, 8.0, np.float32)
        for i in range(_N_BETA):
            b = float(beta[i])
            alpha = math.sqrt(math.exp(math.lgamma(1.0 / b) - math.lgamma(3.0 / b)))
            Z = math.exp(math.log(b) - math.log(alpha) - math.lgamma(1.0 / b))
            u_max = 8.0
            for _ in range(6):
                u = np.linspace(0.0, u_max, _TAU_N_U, dtype=np.float64).astype(np.float32)
                pdf = (np.float32(b / Z) * np.exp(-((u / np.float32(alpha)) ** np.float32(b)))).astype(np.float32)
                cdf = np.cumsum(pdf, dtype=np.float32)
                cdf = cdf / cdf[-1]
                if cdf[-1] >= target:
                    break
                u_max *= 2.0
            idx = np.nonzero(cdf >= np.float32(target))[0]
            if idx.size:
                tau[i] = u[idx[0]]
        taus[bits] = tau
    _tables.update(beta=beta, kappa=kappa, tau=taus)
    return _tables


def _lookup_beta(kurt: float) -> float:
    t = _moment_tables()
    k = max(float(t["kappa"].min()), min(float(t["kappa"].max()), float(kurt)))
    return float(t["beta"][int(np.abs(t["kappa"] - np.float32(k)).argmin())])


def _lookup_tau(beta: float, bits: int) -> float:
    t = _moment_tables()
    if bits not in t["tau"]:
        return 2.5
    idx = int(np.abs(t["beta"] - np.float32(beta)).argmin())
    return max(0.5, min(8.0, float(t["tau"][bits][idx])))


def _std(v: np.ndarray) -> float:
    return float(v.astype(np.float32).std(ddof=1, dtype=np.float32)) if v.size > 1 else float("nan")


def _tail_k(v: np.ndarray, tau: float) -> float:
    if v.size < 2:
        return tau
    return min(float(v.mean(dtype=np.float32)) + 3.0 * _std(v), tau * 1.2)


def fit_codebook(t_flat, bits: int, eps: float = 1e-6) -> np.ndarray:
    """Distribution fit -> sorted codebook of 2**bits fp32 levels."""
    t = _f32(t_flat).ravel()
    L = 2 ** bits
    t2 = t * t
    m2 = float(t2.mean(dtype=np.float32))
    m4 = float((t2 * t2).mean(dtype=np.float32))
    kurt = m4 / max(m2 * m2, eps)
    beta = _lookup_beta(kurt)
    tau = _lookup_tau(beta, bits)
    ts = np.clip(t, np.float32(-tau), np.float32(tau)) if bits >= 3 else t
    pos, neg = ts > np.float32(1e-8), ts < np.float32(-1e-8)
    p_pos, p_neg = float(pos.mean(dtype=np.float32)), float(neg.mean(dtype=np.float32))
    s_pos = _std(ts[pos]) if pos.any() else 1.0
    s_neg = _std(np.abs(ts[neg])) if neg.any() else 1.0
    mp = max(p_pos, 1e-8) ** (1.0 / 3.0) * s_pos ** (2.0 / 3.0)
    mn = max(p_neg, 1e-8) ** (1.0 / 3.0) * s_neg ** (2.0 / 3.0)
    total = mp + mn + 1e-8
    if bits == 1:
        n_neg, n_pos = 1, 1
    elif bits == 2:
        n_pos = max(1, round(L * mp / total))
        n_neg = L - n_pos
        if n_neg < 1:
            n_neg, n_pos = 1, L - 1
    else:
        n_pos = max(1, round(L * mp / total))
        n_neg = L - n_pos - 1
        if n_neg < 1:
            n_neg = 1
            n_pos = L - n_neg - 1
    k_pos = _tail_k(ts[pos], tau) if pos.any() else tau
    k_neg = _tail_k(-ts[neg], tau) if neg.any() else tau

    def lin(a, b, n):
        return np.linspace(a, b, n, dtype=np.float64).astype(np.float32)

    if bits == 1:
        cb = np.sort(np.array([-k_neg, k_pos], np.float32))
    elif bits == 2:
        cb = np.concatenate([-lin(0.05, k_neg, n_neg)[::-1], lin(0.05, k_pos, n_pos)])
        cb = np.sort(cb[:L])
    else:
        cb = np.concatenate([-lin(0.0, k_neg, n_neg + 1)[1:][::-1], np.zeros(1, np.float32),
                             lin(0.0, k_pos, n_pos + 1)[1:]])
        cb = np.sort(cb[:L])
    assert cb.size == L
    return cb.astype(np.float32)


def thresholds_of(codebook) -> np.ndarray:
    """Midpoints of adjacent levels (FQ/quant/dcarcq.py:483)."""
    cb = _f32(codebook)
    return ((cb[:-1] + cb[1:]) / np.float32(2.0)).astype(np.float32)


def normalized_groups(x, group_size: int = 64, eps: float = 1e-6) -> np.ndarray:
    """t = (x - mu) / sigma per group, as [n_groups, group_size] (FQ/quant/dcarcq.py:531-538)."""
    x = _f32(x)
    rows, cols = x.shape
    G = cols // group_size
    x3 = x.reshape(rows, G, group_size)
    mu = (row_sums(x3) / np.float32(group_size)).astype(np.float32)
    r = x3 - mu[..., None]
    var = (row_sums(r * r) / np.float32(group_size)).astype(np.float32)
    s = np.sqrt(var + np.float32(eps), dtype=np.float32)
    return (r / s[..., None]).reshape(-1, group_size)


def calibrate(x, bits: int, group_size: int = 64, eps: float = 1e-6, stats_sample_groups: int = 4096):
    """One codebook compile on x (FQ/quant/dcarcq.py:474-484): every step-th group when there
    are more than 4096 groups, then the fit; returns (codebook, thresholds)."""
    t = normalized_groups(x, group_size, eps)
    if t.shape[0] > stats_sample_groups:
        step = max(1, t.shape[0] // stats_sample_groups)
        t = t[::step]
    cb = fit_codebook(t.ravel(), bits, eps)
    return cb, thresholds_of(cb)
