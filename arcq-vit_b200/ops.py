"""Operator layer over the C ABI: torch tensors in, torch tensors out.

Mirrors the operator set of the reference's CUDA extension
(methods/fair_qat_framework/fair_qat/arcq_infer_cuda/arcq_infer_bind.cpp:57-66):
``quantize_activation``, ``quantize_activation_dequant``, ``arcq_linear_forward``,
``pack_codes``, ``unpack_codes`` / ``unpack_codes_u8``.  torch is used only for device
memory and the current stream; all arithmetic happens in ``libarcq_b200.so``.
Bad arguments raise ``RuntimeError`` like the reference's ``TORCH_CHECK``s.
"""
from __future__ import annotations

import os

import torch

from . import _cabi

_DT = {torch.float32: _cabi.DT_F32, torch.float16: _cabi.DT_F16, torch.bfloat16: _cabi.DT_BF16}


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed ({rc}): {_cabi.last_error()}")


def _dev(t: torch.Tensor, name: str, dtype=None) -> torch.Tensor:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if dtype is not None and t.dtype != dtype:
        raise RuntimeError(f"{name} must be {dtype}, got {t.dtype}")
    return t.contiguous()


def packed_cols(length: int, bits: int) -> int:
    return (length * bits + 7) // 8


def device_status() -> int:
    """0, or the code a kernel left when one of its bounded waits ran out (synchronises)."""
    return int(_cabi.load().arcq_device_status())


def quantize_activation(x: torch.Tensor, thresholds: torch.Tensor, codebook: torch.Tensor, bits: int,
                        group_size: int, want_code_sum: bool = True, pre_gelu: bool = False):
    """[M,K] float -> (packed uint8 [M, K*bits/8], center, scale, code_sum fp32 [M, K/group_size]).

    Same contract as the reference's ``quantize_activation`` (arcq_activation_kernel.cu:188-237),
    except that fp16 / bf16 inputs are read as they are instead of being copied to fp32 first.
    """
    lib = _cabi.load()
    if x.dim() != 2:
        raise RuntimeError(f"x must be 2-D, got shape {tuple(x.shape)}")
    if x.dtype not in _DT:
        raise RuntimeError(f"x must be float32, float16 or bfloat16, got {x.dtype}")
    x = _dev(x, "x")
    th = _dev(thresholds, "thresholds", torch.float32)
    cb = _dev(codebook, "codebook", torch.float32)
    if cb.numel() != 2 ** bits or th.numel() != 2 ** bits - 1:
        raise RuntimeError(f"codebook/thresholds must have {2 ** bits}/{2 ** bits - 1} entries")
    M, K = x.shape
    if group_size <= 0 or K % group_size != 0:
        raise RuntimeError(f"K={K} is not a multiple of group_size={group_size}")
    G = K // group_size
    packed = torch.empty((M, packed_cols(K, bits)), dtype=torch.uint8, device=x.device)
    mu = torch.empty((M, G), dtype=torch.float32, device=x.device)
    sg = torch.empty_like(mu)
    cs = torch.empty_like(mu) if want_code_sum else None
    if M == 0:
        return packed, mu, sg, cs
    fn = lib.arcq_gelu_act_quant if pre_gelu else lib.arcq_act_quant
    rc = fn(x.data_ptr(), _DT[x.dtype], M, K, th.data_ptr(), cb.data_ptr(), bits, group_size,
            packed.data_ptr(), mu.data_ptr(), sg.data_ptr(), cs.data_ptr() if cs is not None else None,
            None, 0, _stream())
    _check(rc, "arcq_act_quant")
    return packed, mu, sg, cs


def quantize_activation_dequant(x: torch.Tensor, thresholds: torch.Tensor, codebook: torch.Tensor, bits: int,
                                group_size: int, out_dtype: torch.dtype = torch.float32,
                                pre_gelu: bool = False) -> torch.Tensor:
    """[M,K] float -> reconstruction [M,K] (reference: arcq_activation_kernel.cu:286-326).
    ``pre_gelu``: the input is a pre-activation; GELU is applied (and rounded to fp16) on the fly."""
    lib = _cabi.load()
    if x.dim() != 2 or x.dtype not in _DT or out_dtype not in _DT:
        raise RuntimeError("x must be a 2-D float tensor and out_dtype a float dtype")
    x = _dev(x, "x")
    th = _dev(thresholds, "thresholds", torch.float32)
    cb = _dev(codebook, "codebook", torch.float32)
    M, K = x.shape
    out = torch.empty((M, K), dtype=out_dtype, device=x.device)
    if M == 0:
        return out
    fn = lib.arcq_gelu_act_quant if pre_gelu else lib.arcq_act_quant
    rc = fn(x.data_ptr(), _DT[x.dtype], M, K, th.data_ptr(), cb.data_ptr(), bits, group_size,
            None, None, None, None, out.data_ptr(), _DT[out_dtype], _stream())
    _check(rc, "arcq_act_quant")
    return out


# How ``arcq_linear_forward`` runs: "auto" takes two kernels (activation reconstruction, then the packed-weight
# GEMM) for every shape the packed-weight GEMM accepts, whatever the number of rows, so that a row's result does
# not depend on the batch it is computed in; "single" always runs the one kernel that rebuilds both operands.
LINEAR_FORWARD_ROUTE = os.environ.get("ARCQ_LINEAR_ROUTE", "auto")


def arcq_linear_forward(packed_x, x_center, x_scale, x_code_sum, packed_w, w_center, w_scale, w_code_sum,
                        act_codebook, w_codebook, bias, bits: int, group_size: int, in_features: int,
                        out_features: int, out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Packed linear (reference: arcq_linear_forward, arcq_linear_kernel.cu:206-278).

    The reference takes ``product_table = outer(act_codebook, w_codebook)``; the two codebooks
    are passed here instead.  Returns [M, out_features] in ``out_dtype`` (fp32 or fp16).
    """
    lib = _cabi.load()
    packed_x = _dev(packed_x, "packed_x", torch.uint8)
    packed_w = _dev(packed_w, "packed_w", torch.uint8)
    f = [_dev(t, n, torch.float32) for t, n in (
        (x_center, "x_center"), (x_scale, "x_scale"), (x_code_sum, "x_code_sum"), (w_center, "w_center"),
        (w_scale, "w_scale"), (w_code_sum, "w_code_sum"), (act_codebook, "act_codebook"), (w_codebook, "w_codebook"))]
    if out_dtype not in (torch.float32, torch.float16):
        raise RuntimeError("out_dtype must be float32 or float16")
    M = packed_x.shape[0]
    pc = packed_cols(in_features, bits)
    if packed_x.shape[1] != pc or tuple(packed_w.shape) != (out_features, pc):
        raise RuntimeError(f"packed shapes {tuple(packed_x.shape)}/{tuple(packed_w.shape)} do not match "
                           f"K={in_features} N={out_features} bits={bits}")
    b = None
    if bias is not None and bias.numel() > 0:
        b = _dev(bias, "bias", torch.float32)
        if b.numel() != out_features:
            raise RuntimeError("bias must have out_features entries")
    if (LINEAR_FORWARD_ROUTE != "single" and M > 0
            and packed_weight_gemm_supported(in_features, out_features, bits, group_size)):
        # Two kernels instead of one: reconstruct the activation once into an fp16 matrix (what the quantizer's
        # reconstruction output holds, bit for bit) and run the GEMM that rebuilds only the weight.  The single
        # kernel below rebuilds both operands inside every tile, which costs 4-6x more on large M.
        x_hat = dequant(packed_x, f[0], f[1], f[2], f[6], bits, group_size, torch.float16)
        return packed_weight_gemm(x_hat, packed_w, f[3], f[4], f[5], f[7], b, bits, group_size, out_dtype)
    y = torch.empty((M, out_features), dtype=out_dtype, device=packed_x.device)
    if M == 0:
        return y
    rc = lib.arcq_packed_gemm(packed_x.data_ptr(), f[0].data_ptr(), f[1].data_ptr(), f[2].data_ptr(),
                              packed_w.data_ptr(), f[3].data_ptr(), f[4].data_ptr(), f[5].data_ptr(),
                              f[6].data_ptr(), f[7].data_ptr(), b.data_ptr() if b is not None else None,
                              bits, group_size, M, out_features, in_features, y.data_ptr(), _DT[out_dtype], _stream())
    _check(rc, "arcq_packed_gemm")
    return y


def packed_weight_gemm_supported(in_features: int, out_features: int, bits: int, group_size: int) -> bool:
    """Shapes the persistent packed-weight kernel takes (the rest go through ``arcq_linear_forward``)."""
    return group_size == 64 and out_features % 16 == 0 and (in_features * bits // 8) % 16 == 0


def packed_weight_gemm(xhat: torch.Tensor, packed_w, w_center, w_scale, w_code_sum, w_codebook, bias, bits: int,
                       group_size: int, out_dtype: torch.dtype = torch.float16) -> torch.Tensor:
    """fp16 reconstructed activation [M,K] x packed weight -> [M,N].

    Steps 3-5 of the reference's on-the-fly forward (arcq_packed_on_the_fly.py:147-161: Triton weight
    unpack, bias cast, cuBLAS ``F.linear``) as one kernel; ``xhat`` is the output of
    ``quantize_activation_dequant(..., out_dtype=torch.float16)``.
    """
    lib = _cabi.load()
    xhat = _dev(xhat, "xhat", torch.float16)
    packed_w = _dev(packed_w, "packed_w", torch.uint8)
    f = [_dev(t, n, torch.float32) for t, n in ((w_center, "w_center"), (w_scale, "w_scale"),
                                                (w_code_sum, "w_code_sum"), (w_codebook, "w_codebook"))]
    if out_dtype not in (torch.float32, torch.float16):
        raise RuntimeError("out_dtype must be float32 or float16")
    M, K = xhat.shape
    N = packed_w.shape[0]
    if packed_w.shape[1] != packed_cols(K, bits) or tuple(f[0].shape) != (N, K // group_size):
        raise RuntimeError(f"packed weight {tuple(packed_w.shape)} / stats {tuple(f[0].shape)} do not match K={K}")
    b = None
    if bias is not None and bias.numel() > 0:
        b = _dev(bias, "bias", torch.float32)
        if b.numel() != N:
            raise RuntimeError("bias must have out_features entries")
    y = torch.empty((M, N), dtype=out_dtype, device=xhat.device)
    if M == 0:
        return y
    rc = lib.arcq_packed_weight_gemm(xhat.data_ptr(), packed_w.data_ptr(), f[0].data_ptr(), f[1].data_ptr(),
                                     f[2].data_ptr(), f[3].data_ptr(), b.data_ptr() if b is not None else None,
                                     bits, group_size, M, N, K, y.data_ptr(), _DT[out_dtype], _stream())
    _check(rc, "arcq_packed_weight_gemm")
    return y


def add_layernorm(x: torch.Tensor, y, norm: torch.nn.LayerNorm):
    """(x + y, LayerNorm(x + y)) for fp16 CUDA tensors in one kernel; with ``y is None``: (x, LayerNorm(x)).
    The sum is rounded to fp16 before it is normalised, as the separate add + LayerNorm would do."""
    lib = _cabi.load()
    shape = x.shape
    K = shape[-1]
    x2 = _dev(x.reshape(-1, K), "x", torch.float16)
    y2 = None if y is None else _dev(y.reshape(-1, K), "y", torch.float16)
    g32, b32 = _norm_params_f32(norm, x2.device)
    h = torch.empty_like(x2)
    s_out = torch.empty_like(x2) if y2 is not None else None
    if x2.shape[0] > 0:
        rc = lib.arcq_add_layernorm(x2.data_ptr(), y2.data_ptr() if y2 is not None else None, g32.data_ptr(),
                                    b32.data_ptr(), float(norm.eps), x2.shape[0], K,
                                    s_out.data_ptr() if s_out is not None else None, h.data_ptr(), _stream())
        _check(rc, "arcq_add_layernorm")
    return (x if s_out is None else s_out.reshape(shape)), h.reshape(shape)


def _norm_params_f32(norm: torch.nn.LayerNorm, device):
    """fp32 copies of the affine parameters, remade whenever the parameters were replaced, written to or moved."""
    key = (norm.weight.data_ptr(), norm.weight._version, norm.bias.data_ptr(), norm.bias._version, device)
    cached = getattr(norm, "_arcq_f32", None)
    if cached is None or cached[0] != key:
        cached = (key, norm.weight.detach().to(device=device, dtype=torch.float32).contiguous(),
                  norm.bias.detach().to(device=device, dtype=torch.float32).contiguous())
        norm._arcq_f32 = cached
    return cached[1], cached[2]


def add_layernorm_quant(x: torch.Tensor, y, norm: torch.nn.LayerNorm, thresholds: torch.Tensor, codebook: torch.Tensor,
                        bits: int, group_size: int = 64, want_h: bool = False):
    """``add_layernorm`` and the activation quantizer of the linear that consumes the LayerNorm output, in one
    kernel: returns (x + y, xhat) where xhat is what ``quantize_activation_dequant(LayerNorm(x + y), ...)`` gives
    in fp16; the LayerNorm output itself is not written.  ``want_h=True`` also returns it (third value), for
    checking."""
    lib = _cabi.load()
    shape = x.shape
    K = shape[-1]
    x2 = _dev(x.reshape(-1, K), "x", torch.float16)
    y2 = None if y is None else _dev(y.reshape(-1, K), "y", torch.float16)
    thresholds, codebook = _dev(thresholds, "thresholds", torch.float32), _dev(codebook, "codebook", torch.float32)
    if K not in (192, 384, 768):
        # widths the merged kernel is not built for: the two kernels it stands for (same results)
        s, h = add_layernorm(x, y, norm)
        xh = quantize_activation_dequant(h.reshape(-1, K), thresholds, codebook, bits, group_size, torch.float16)
        return (s, xh.reshape(shape), h) if want_h else (s, xh.reshape(shape))
    g32, b32 = _norm_params_f32(norm, x2.device)
    xhat = torch.empty_like(x2)
    s_out = torch.empty_like(x2) if y2 is not None else None
    h = torch.empty_like(x2) if want_h else None
    if x2.shape[0] > 0:
        rc = lib.arcq_add_layernorm_act_quant(x2.data_ptr(), y2.data_ptr() if y2 is not None else None, g32.data_ptr(),
                                              b32.data_ptr(), float(norm.eps), x2.shape[0], K, thresholds.data_ptr(),
                                              codebook.data_ptr(), bits, group_size,
                                              s_out.data_ptr() if s_out is not None else None,
                                              h.data_ptr() if h is not None else None, xhat.data_ptr(), _stream())
        _check(rc, "arcq_add_layernorm_act_quant")
    out = ((x if s_out is None else s_out.reshape(shape)), xhat.reshape(shape))
    return out + (h.reshape(shape),) if want_h else out


def attention(qkv: torch.Tensor, batch: int, tokens: int, heads: int, thresholds: torch.Tensor = None,
              codebook: torch.Tensor = None, bits: int = 4, group_size: int = 64) -> torch.Tensor:
    """softmax(q k^T / sqrt(64)) v for every (image, head) of ``qkv`` [batch*tokens, 3*heads*64] fp16 (the qkv linear's
    output); returns [batch*tokens, heads*64] fp16, heads side by side (timm ``Attention.forward`` between qkv and
    proj).  With ``thresholds`` / ``codebook`` (those of the proj linear) the result is quantised on the way out: the
    return value is the reconstruction ``quantize_activation_dequant`` would give, for ``proj(x, pre_quantized=True)``."""
    lib = _cabi.load()
    C = heads * 64
    q2 = _dev(qkv.reshape(-1, 3 * C), "qkv", torch.float16)
    if q2.shape[0] != batch * tokens:
        raise RuntimeError(f"qkv has {q2.shape[0]} rows, expected {batch} x {tokens}")
    out = torch.empty((batch * tokens, C), dtype=torch.float16, device=q2.device)
    if thresholds is None:
        rc = lib.arcq_attention(q2.data_ptr(), batch, tokens, heads, 64, out.data_ptr(), _stream())
        _check(rc, "arcq_attention")
    else:
        thresholds, codebook = _dev(thresholds, "thresholds", torch.float32), _dev(codebook, "codebook", torch.float32)
        rc = lib.arcq_attention_act_quant(q2.data_ptr(), batch, tokens, heads, 64, thresholds.data_ptr(),
                                          codebook.data_ptr(), bits, group_size, out.data_ptr(), _stream())
        _check(rc, "arcq_attention_act_quant")
    return out


def patchify(images: torch.Tensor, patch: int) -> torch.Tensor:
    """fp16 images [B, C, H, W] -> [B, (H/patch)*(W/patch), C*patch*patch]: row (gy, gx), column (c, py, px), i.e.
    ``images.reshape(B, C, gh, p, gw, p).permute(0, 2, 4, 1, 3, 5).reshape(B, gh*gw, C*p*p)`` in one kernel."""
    lib = _cabi.load()
    x = _dev(images, "images", torch.float16)
    B, C, H, W = x.shape
    out = torch.empty((B, (H // patch) * (W // patch), C * patch * patch), dtype=torch.float16, device=x.device)
    _check(lib.arcq_patchify(x.data_ptr(), B, C, H, W, patch, out.data_ptr(), _stream()), "arcq_patchify")
    return out


def assemble_tokens(patches: torch.Tensor, cls_token: torch.Tensor, pos_embed: torch.Tensor) -> torch.Tensor:
    """``torch.cat([cls_token.expand(B, 1, D), patches], dim=1) + pos_embed`` for fp16 tensors in one kernel;
    patches [B, T, D], cls_token [1, 1, D], pos_embed [1, 1+T, D]."""
    lib = _cabi.load()
    p = _dev(patches, "patches", torch.float16)
    B, T, D = p.shape
    c = _dev(cls_token.reshape(-1), "cls_token", torch.float16)
    e = _dev(pos_embed.reshape(-1, D), "pos_embed", torch.float16)
    if c.numel() != D or tuple(e.shape) != (T + 1, D):
        raise RuntimeError(f"cls_token {tuple(cls_token.shape)} / pos_embed {tuple(pos_embed.shape)} do not match patches {tuple(p.shape)}")
    out = torch.empty((B, T + 1, D), dtype=torch.float16, device=p.device)
    _check(lib.arcq_assemble_tokens(p.data_ptr(), c.data_ptr(), e.data_ptr(), B, T, D, out.data_ptr(), _stream()),
           "arcq_assemble_tokens")
    return out


def unpack_codes_u8(packed: torch.Tensor, bits: int, length: int) -> torch.Tensor:
    """uint8 [R, ceil(length*bits/8)] -> uint8 [R, length] (reference: arcq_pack_kernel.cu:136-157)."""
    lib = _cabi.load()
    packed = _dev(packed, "packed", torch.uint8)
    if packed.dim() != 2 or packed.shape[1] != packed_cols(length, bits):
        raise RuntimeError(f"packed shape {tuple(packed.shape)} does not match length={length} bits={bits}")
    out = torch.empty((packed.shape[0], length), dtype=torch.uint8, device=packed.device)
    _check(lib.arcq_unpack_codes(packed.data_ptr(), packed.shape[0], length, bits, out.data_ptr(), _stream()),
           "arcq_unpack_codes")
    return out


def unpack_codes(packed: torch.Tensor, bits: int, length: int) -> torch.Tensor:
    """As ``unpack_codes_u8`` but int64, the reference's ``unpack_codes`` (arcq_pack_kernel.cu:113-134)."""
    return unpack_codes_u8(packed, bits, length).to(torch.int64)


def pack_codes(codes: torch.Tensor, bits: int) -> torch.Tensor:
    """integer codes [R, length] -> uint8 [R, ceil(length*bits/8)] (reference: arcq_pack_kernel.cu:92-111)."""
    lib = _cabi.load()
    if not codes.is_cuda or codes.dim() != 2:
        raise RuntimeError("codes must be a 2-D CUDA tensor")
    c8 = codes.to(torch.uint8).contiguous()
    R, length = c8.shape
    out = torch.empty((R, packed_cols(length, bits)), dtype=torch.uint8, device=codes.device)
    _check(lib.arcq_pack_codes(c8.data_ptr(), R, length, bits, out.data_ptr(), _stream()), "arcq_pack_codes")
    return out


def dense_weight_gemm(xhat: torch.Tensor, w16: torch.Tensor, bias, out_dtype: torch.dtype = torch.float16,
                      prefetch=None) -> torch.Tensor:
    """fp16 reconstructed activation [M,K] x fp16 weight [N,K] (+ fp32 bias) -> [M,N]: the ``F.linear`` of the
    reference's on-the-fly forward (arcq_packed_on_the_fly.py:160) on the weight ``unpack_weight_f16`` wrote.

    ``prefetch = (packed, center, scale, code_sum, codebook, bits, group_size, out)``: also unpack that (the next
    layer's) weight into the fp16 buffer ``out`` with spare warps of the same kernel; ``out`` must be a different
    buffer from ``w16`` that no kernel still reads (see ``arcq_dense_weight_gemm_prefetch``)."""
    lib = _cabi.load()
    xhat = _dev(xhat, "xhat", torch.float16)
    w16 = _dev(w16, "w16", torch.float16)
    if out_dtype not in (torch.float32, torch.float16):
        raise RuntimeError("out_dtype must be float32 or float16")
    M, K = xhat.shape
    N = w16.shape[0]
    if w16.dim() != 2 or w16.shape[1] != K:
        raise RuntimeError(f"weight {tuple(w16.shape)} does not match K={K}")
    b = None
    if bias is not None and bias.numel() > 0:
        b = _dev(bias, "bias", torch.float32)
        if b.numel() != N:
            raise RuntimeError("bias must have out_features entries")
    y = torch.empty((M, N), dtype=out_dtype, device=xhat.device)
    if M == 0:
        if prefetch is not None:           # nothing to multiply, but the next layer still expects its weight
            unpack_weight_f16(*prefetch[:7], out=prefetch[7])
        return y
    if prefetch is not None:
        n_packed, n_mu, n_sg, n_cs, n_cb, n_bits, n_gs, n_out = prefetch
        n_packed = _dev(n_packed, "next packed", torch.uint8)
        n_mu, n_sg, n_cs, n_cb = (_dev(t, "next stats", torch.float32) for t in (n_mu, n_sg, n_cs, n_cb))
        R, G = n_mu.shape
        if (n_out.dtype != torch.float16 or not n_out.is_cuda or not n_out.is_contiguous() or n_out.numel() < R * G * n_gs
                or n_out.data_ptr() == w16.data_ptr()):
            raise RuntimeError("prefetch out must be a contiguous CUDA fp16 buffer of at least R*K elements, not w16 itself")
        rc = lib.arcq_dense_weight_gemm_prefetch(xhat.data_ptr(), w16.data_ptr(), b.data_ptr() if b is not None else None,
                                                 M, N, K, y.data_ptr(), _DT[out_dtype], n_packed.data_ptr(),
                                                 n_mu.data_ptr(), n_sg.data_ptr(), n_cs.data_ptr(), n_cb.data_ptr(),
                                                 n_bits, n_gs, R, G * n_gs, n_out.data_ptr(), _stream())
        _check(rc, "arcq_dense_weight_gemm_prefetch")
        return y
    rc = lib.arcq_dense_weight_gemm(xhat.data_ptr(), w16.data_ptr(), b.data_ptr() if b is not None else None,
                                    M, N, K, y.data_ptr(), _DT[out_dtype], _stream())
    _check(rc, "arcq_dense_weight_gemm")
    return y


def dequant(packed, center, scale, code_sum, codebook, bits: int, group_size: int,
            out_dtype: torch.dtype = torch.float16, out: torch.Tensor = None) -> torch.Tensor:
    """Packed codes + statistics -> [R, K] matrix; what the reference's ``unpack_weight_triton``
    (arcq_packed_triton.py:77-120) writes.  ``out``: write into this buffer (first R*K elements) instead
    of allocating, as the reference does with its ``_weight_buffer``."""
    lib = _cabi.load()
    packed = _dev(packed, "packed", torch.uint8)
    center, scale, code_sum, codebook = (_dev(t, "stats", torch.float32) for t in (center, scale, code_sum, codebook))
    R, G = center.shape
    K = G * group_size
    if out is not None:
        if out.dtype != out_dtype or not out.is_cuda or not out.is_contiguous() or out.numel() < R * K:
            raise RuntimeError("out must be a contiguous CUDA buffer of out_dtype with at least R*K elements")
        out = out.view(-1)[: R * K].view(R, K)
    else:
        out = torch.empty((R, K), dtype=out_dtype, device=packed.device)
    _check(lib.arcq_dequant(packed.data_ptr(), center.data_ptr(), scale.data_ptr(), code_sum.data_ptr(),
                            codebook.data_ptr(), bits, group_size, R, K, out.data_ptr(), _DT[out_dtype], _stream()),
           "arcq_dequant")
    return out


def unpack_weight_f16(packed, center, scale, code_sum, codebook, bits: int, group_size: int,
                      out: torch.Tensor = None, stream: torch.cuda.Stream = None) -> torch.Tensor:
    """Packed weight codes + statistics -> the fp16 matrix [N, K] the packed-weight GEMM kernels rebuild on chip
    (same bits), for ``dense_weight_gemm``.  ``out``: scratch buffer of at least N*K fp16 values;
    ``stream``: launch there instead of on the current stream."""
    lib = _cabi.load()
    packed = _dev(packed, "packed", torch.uint8)
    center, scale, code_sum, codebook = (_dev(t, "stats", torch.float32) for t in (center, scale, code_sum, codebook))
    R, G = center.shape
    K = G * group_size
    if out is not None:
        if out.dtype != torch.float16 or not out.is_cuda or not out.is_contiguous() or out.numel() < R * K:
            raise RuntimeError("out must be a contiguous CUDA fp16 buffer with at least R*K elements")
        out = out.view(-1)[: R * K].view(R, K)
    else:
        out = torch.empty((R, K), dtype=torch.float16, device=packed.device)
    handle = stream.cuda_stream if stream is not None else _stream()
    _check(lib.arcq_unpack_weight_f16(packed.data_ptr(), center.data_ptr(), scale.data_ptr(), code_sum.data_ptr(),
                                      codebook.data_ptr(), bits, group_size, R, K, out.data_ptr(), handle),
           "arcq_unpack_weight_f16")
    return out


# ---------------------------------------------------------------------------------------------------------
# The reference extension's exact operator signatures (arcq_infer_bind.cpp:57-66), for a shim that replaces
# `fair_qat/arcq_infer_cuda/__init__.py` without touching the reference's module classes.
_PRODUCT_TABLE_CACHE: dict = {}


def codebooks_from_product_table(product_table: torch.Tensor, packed_x: torch.Tensor, x_code_sum: torch.Tensor,
                                 bits: int, group_size: int):
    """(act_codebook, w_codebook) from ``product_table = outer(act_codebook, w_codebook)``.

    The reference operator is given only the table (arcq_packed_linear.py:114-117 builds it, :199-213 passes it);
    the kernels here rebuild each operand from its own codebook.  A rank-one table fixes the two factors up to one
    scale, and the activation code sums fix that scale: the sum of the (scaled) activation codebook over the codes
    of a group equals scale x that group's ``x_code_sum``.  Everything runs on the device without a
    synchronisation; the result is cached per table (the module's buffer), so a layer pays for it once.
    """
    key = (product_table.data_ptr(), product_table._version, str(product_table.device))
    hit = _PRODUCT_TABLE_CACHE.get(key)
    if hit is not None:
        return hit
    T = product_table.float()
    j0 = T.abs().amax(0).argmax().view(1)
    a1 = T.index_select(1, j0).squeeze(1)                                   # act_codebook * w_codebook[j0]
    i0 = a1.abs().argmax().view(1)
    w1 = T.index_select(0, i0).squeeze(0) / a1.index_select(0, i0)         # w_codebook / w_codebook[j0]
    G = x_code_sum.shape[1]
    flat = x_code_sum.abs().reshape(-1).argmax().view(1)                    # the group with the largest code sum
    row, grp = flat // G, flat % G
    codes = unpack_codes_u8(packed_x.index_select(0, row).contiguous(), bits, G * group_size)
    codes_g = codes.view(G, group_size).index_select(0, grp).long().view(-1)
    c = a1[codes_g].sum() / x_code_sum.reshape(-1).index_select(0, flat).squeeze(0)     # = w_codebook[j0]
    out = ((a1 / c).contiguous(), (w1 * c).contiguous())
    if len(_PRODUCT_TABLE_CACHE) > 4096:
        _PRODUCT_TABLE_CACHE.clear()
    _PRODUCT_TABLE_CACHE[key] = out
    return out


def arcq_linear_forward_product_table(packed_x, x_center, x_scale, x_code_sum, packed_w, w_center, w_scale, w_code_sum,
                                      product_table, bias, bits: int, group_size: int, in_features: int,
                                      out_features: int) -> torch.Tensor:
    """``arcq_linear_forward`` with the reference's argument list (product table instead of two codebooks)."""
    act_cb, w_cb = codebooks_from_product_table(product_table, packed_x, x_code_sum, bits, group_size)
    return arcq_linear_forward(packed_x, x_center, x_scale, x_code_sum, packed_w, w_center, w_scale, w_code_sum,
                               act_cb, w_cb, bias, bits, group_size, in_features, out_features)


def quantize_activation_u8(x: torch.Tensor, thresholds: torch.Tensor, codebook: torch.Tensor, bits: int, group_size: int):
    """[codes uint8 [M,K] (one byte per code), center, scale, code_sum]: the reference's ``quantize_activation_u8``
    (arcq_activation_kernel.cu:239-284).  Same quantizer kernel, codes unpacked afterwards."""
    packed, mu, sg, cs = quantize_activation(x, thresholds, codebook, bits, group_size)
    return unpack_codes_u8(packed, bits, x.shape[1]), mu, sg, cs


def arcq_linear_forward_u8(x_codes, x_center, x_scale, x_code_sum, w_codes, w_center, w_scale, w_code_sum,
                           product_table, bias, group_size: int) -> torch.Tensor:
    """The reference's ``arcq_linear_forward_u8`` (arcq_linear_kernel.cu:280-340): one-byte codes on both sides.
    The bit width is the table's: L x L entries <-> log2 L bits.  Codes are packed and the packed kernel runs."""
    L = int(product_table.shape[0])
    bits = L.bit_length() - 1
    if 2 ** bits != L or bits not in (2, 3, 4):
        raise RuntimeError(f"product_table of {L} levels: expected 4, 8 or 16")
    return arcq_linear_forward_product_table(pack_codes(x_codes, bits), x_center, x_scale, x_code_sum,
                                             pack_codes(w_codes, bits), w_center, w_scale, w_code_sum, product_table,
                                             bias, bits, group_size, x_codes.shape[1], w_codes.shape[0])
