"""The attention kernel between the qkv and proj linears (an opt-in replacement for the library attention) and its
form that also runs proj's activation quantizer: against an fp64 evaluation and the library kernel, and -- for the
quantizer form -- bit for bit against the quantizer kernel applied to the plain form's output."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _fp64(qkv, B, T, H):
    q = qkv.double().reshape(B, T, 3, H, 64).permute(2, 0, 3, 1, 4)
    s = (q[0] @ q[1].transpose(-1, -2)) / 8.0
    return (torch.softmax(s, -1) @ q[2]).transpose(1, 2).reshape(B * T, H * 64)


def _library(qkv, B, T, H):
    q = qkv.reshape(B, T, 3, H, 64).permute(2, 0, 3, 1, 4)
    return F.scaled_dot_product_attention(q[0], q[1], q[2]).transpose(1, 2).reshape(B * T, H * 64)


@pytest.mark.parametrize("B,T,H", [(1, 1, 1), (1, 16, 1), (2, 197, 3), (3, 64, 2), (2, 200, 6), (1, 256, 2), (4, 5, 12),
                                   (16, 197, 6)])
def test_attention_kernel(pkg, oracle, cuda_device, B, T, H):
    gen = torch.Generator().manual_seed(B * 1000 + T + H)
    qkv = (torch.randn(B * T, 3 * H * 64, generator=gen) * 1.5).half().to(cuda_device)
    out = pkg.ops.attention(qkv, B, T, H)
    assert out.dtype == torch.float16 and tuple(out.shape) == (B * T, H * 64)
    ref = _fp64(qkv, B, T, H)
    err = float((out.double() - ref).abs().max())
    err_lib = float((_library(qkv, B, T, H).double() - ref).abs().max())
    assert err <= max(2.5e-3, 1.5 * err_lib), (err, err_lib)          # fp16 outputs of magnitude ~1-4
    # images do not see each other: the first image alone gives the same rows
    alone = pkg.ops.attention(qkv[:T].contiguous(), 1, T, H)
    assert torch.equal(alone, out[:T])
    for bits in (4, 3, 2):
        cb = torch.sort(torch.randn(2 ** bits, generator=gen) * 1.1)[0].to(cuda_device)
        th = (cb[:-1] + cb[1:]) / 2
        xq = pkg.ops.attention(qkv, B, T, H, th, cb, bits)
        want = pkg.ops.quantize_activation_dequant(out, th, cb, bits, 64, torch.float16)
        assert torch.equal(xq, want), bits
    # the quantizer form against the CPU oracle on the plain form's output (first rows)
    rows = slice(0, min(B * T, 24))
    cb = np.sort(np.random.default_rng(T).normal(size=16).astype(np.float32) * 1.1)
    th = ((cb[:-1] + cb[1:]) / np.float32(2)).astype(np.float32)
    xq = pkg.ops.attention(qkv, B, T, H, torch.from_numpy(th).to(cuda_device), torch.from_numpy(cb).to(cuda_device), 4)
    codes, mu, sg, cs = oracle.quantize(out[rows].float().cpu().numpy(), th, cb, 64)
    want = oracle.dequant(codes, mu, sg, cb, 64).astype(np.float16)
    assert np.array_equal(xq[rows].cpu().numpy(), want)
    assert pkg.ops.device_status() == 0


def test_attention_kernel_rejects_what_it_does_not_take(pkg, cuda_device):
    qkv = torch.zeros(300 * 2, 3 * 64, dtype=torch.float16, device=cuda_device)
    with pytest.raises(RuntimeError):
        pkg.ops.attention(qkv, 2, 300, 1)                 # more than 256 tokens
    with pytest.raises(RuntimeError):
        pkg.ops.attention(qkv, 3, 197, 1)                 # row count does not match


def test_model_with_the_attention_kernel(pkg, cuda_device):
    """The ViT skeleton with ``Attention.implementation = "kernel"``: attention and proj's quantizer in one launch.
    The first block's attention output equals the library's to fp16 rounding; whole-model logits stay finite and
    close (they differ like any two fp16 attention implementations do, amplified by the quantizers downstream)."""
    dev = cuda_device
    gen = torch.Generator().manual_seed(13)
    model = pkg.create_vit("deit_tiny", seed=3).half().to(dev)
    x = torch.randn(4, 3, 224, 224, generator=gen).half().to(dev)
    from importlib import import_module
    attn_cls = type(model.blocks[0].attn)
    saved = attn_cls.implementation
    try:
        with torch.no_grad():
            model = pkg.quantise_model(model, x, 4)
            attn_cls.implementation = "sdpa"
            y0 = model(x).clone()
            attn_cls.implementation = "kernel"
            y1 = model(x).clone()
            g1 = pkg.GraphedModel(model, x)(x).clone()
        assert torch.equal(y1, g1)
        assert bool(torch.isfinite(y1).all()) and pkg.ops.device_status() == 0
        rms = float(y0.float().pow(2).mean().sqrt())
        assert float((y1.float() - y0.float()).pow(2).mean().sqrt()) < 0.5 * rms
    finally:
        attn_cls.implementation = saved
