"""The reference's data flow on two streams: the weight is unpacked into an fp16 scratch matrix
(``arcq_unpack_weight_f16``) and read by the dense-weight GEMM on CTA pairs, the unpack of the next layer
running beside the current layer.  Checked here: the unpacked matrix holds exactly the bits the packed-weight
kernels rebuild on chip, the pair form of the dense GEMM equals the one-CTA form, and a whole model gives the
same logits whichever way its weights reach the tensor cores, eagerly and from a CUDA graph."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _weight(pkg, dev, K, N, bits, seed):
    gen = torch.Generator().manual_seed(seed)
    cb = torch.sort(torch.randn(2 ** bits, generator=gen) * 1.2)[0].to(dev)
    th = (cb[:-1] + cb[1:]) / 2
    w = (torch.randn(N, K, generator=gen) * 0.02).to(dev)
    bias = (torch.randn(N, generator=gen) * 0.01).to(dev)
    pw, mw, sw, cw = pkg.ops.quantize_activation(w, th, cb, bits, 64)
    return pw, mw, sw, cw, cb, bias


@pytest.mark.parametrize("bits", [4, 3, 2])
@pytest.mark.parametrize("M,K,N", [(300, 384, 192), (64 * 197, 384, 1152), (2049, 1536, 384), (1500, 768, 2304)])
def test_unpacked_weight_and_dense_gemm_equal_the_packed_weight_gemm(pkg, oracle, cuda_device, M, K, N, bits):
    if not pkg.ops.packed_weight_gemm_supported(K, N, bits, 64):
        pytest.skip("shape is routed to the packed-codes kernel")
    pw, mw, sw, cw, cb, bias = _weight(pkg, cuda_device, K, N, bits, seed=K + N + bits)
    xh = torch.randn(M, K, generator=torch.Generator().manual_seed(M)).half().to(cuda_device)
    scratch = torch.full((N * K + 64,), float("nan"), dtype=torch.float16, device=cuda_device)
    w16 = pkg.ops.unpack_weight_f16(pw, mw, sw, cw, cb, bits, 64, out=scratch)
    assert w16.data_ptr() == scratch.data_ptr() and tuple(w16.shape) == (N, K)
    assert bool(torch.isnan(scratch[N * K:]).all()), "wrote past the matrix"
    # close to the fp32 reconstruction (it differs by the fp16 rounding of the folded statistics only)
    w32 = pkg.ops.dequant(pw, mw, sw, cw, cb, bits, 64, torch.float32)
    assert float((w16.float() - w32).abs().max()) < 4e-3 * float(w32.abs().max())
    for out_dtype in (torch.float16, torch.float32):
        with pkg._cabi.option("ARCQ_PAIR_MIN_M", 1):
            y_dense = pkg.ops.dense_weight_gemm(xh, w16, bias, out_dtype)
            y_packed = pkg.ops.packed_weight_gemm(xh, pw, mw, sw, cw, cb, bias, bits, 64, out_dtype)
        assert torch.equal(y_dense, y_packed)
    assert pkg.ops.device_status() == 0


@pytest.mark.parametrize("options", [dict(), dict(ARCQ_PAIR_BN=32), dict(ARCQ_PAIR_BN=64), dict(ARCQ_PAIR_BN=96),
                                     dict(ARCQ_PAIR_BN=128), dict(ARCQ_PAIR_BN=192), dict(ARCQ_PAIR_BN=256),
                                     dict(ARCQ_PAIR_KS=1), dict(ARCQ_PAIR_KS=3), dict(ARCQ_PAIR_SA=2),
                                     dict(ARCQ_PAIR_BN=192, ARCQ_PAIR_KS=1, ARCQ_PAIR_SA=5), dict(ARCQ_PAIR_PAIRS=7),
                                     dict(ARCQ_PAIR_STATIONARY=1), dict(ARCQ_PAIR_STATIONARY=0),
                                     dict(ARCQ_PAIR_STATIONARY=1, ARCQ_PAIR_BN=64), dict(ARCQ_PAIR_STATIONARY=1, ARCQ_PAIR_KS=1),
                                     dict(ARCQ_PAIR_STATIONARY=1, ARCQ_PAIR_BN=128, ARCQ_PAIR_PAIRS=5)])
@pytest.mark.parametrize("M,K,N", [(256, 64, 768), (2500, 384, 768), (64 * 197, 384, 1536), (5000, 1536, 768)])
def test_dense_pair_kernel_equals_the_one_cta_kernel(pkg, cuda_device, M, K, N, options):
    gen = torch.Generator().manual_seed(M + K + N)
    x = torch.randn(M, K, generator=gen).half().to(cuda_device)
    w = (torch.randn(N, K, generator=gen) * 0.05).half().to(cuda_device)
    b = torch.randn(N, generator=gen).to(cuda_device)
    for out_dtype in (torch.float16, torch.float32):
        with pkg._cabi.option("ARCQ_PAIR", 0):
            y_one = pkg.ops.dense_weight_gemm(x, w, b, out_dtype)
        saved = {k: pkg._cabi.get_option(k) for k in options}
        try:
            for k, v in options.items():
                pkg._cabi.set_option(k, v)
            with pkg._cabi.option("ARCQ_PAIR_MIN_M", 1):
                y_pair = pkg.ops.dense_weight_gemm(x, w, b, out_dtype)
        finally:
            for k, v in saved.items():
                pkg._cabi.set_option(k, v)
        assert pkg.ops.device_status() == 0, f"a bounded wait ran out with {options}"
        assert torch.equal(y_pair, y_one), options
    # rows do not depend on the batch they are computed in
    with pkg._cabi.option("ARCQ_PAIR_MIN_M", 1):
        y_all = pkg.ops.dense_weight_gemm(x, w, b, torch.float16)
        y_part = pkg.ops.dense_weight_gemm(x[: min(M, 131)].contiguous(), w, b, torch.float16)
    assert torch.equal(y_all[: y_part.shape[0]], y_part)


@pytest.mark.parametrize("bits", [4, 3])
def test_whole_model_logits_do_not_depend_on_the_weight_route(pkg, cuda_device, bits):
    """DeiT-T at batch 8: packed, dense on one stream, staged with the next layer's unpack inside the GEMM kernel, and
    staged with it on a second stream give the same logits, eagerly and replayed from a CUDA graph; the stager's
    scratch is two matrices of the largest layer."""
    dev = cuda_device
    gen = torch.Generator().manual_seed(5)
    model = pkg.create_vit("deit_tiny", seed=1).half().to(dev)
    x = torch.randn(8, 3, 224, 224, generator=gen).half().to(dev)
    x2 = torch.randn(8, 3, 224, 224, generator=gen).half().to(dev)
    cls = pkg.ARCQPackedLinearOnTheFly
    saved, saved_mode = cls.weight_form, pkg.WeightStager.mode
    try:
        with torch.no_grad():
            model = pkg.quantise_model(model, x, bits)
            stager = model._arcq_weight_stager
            assert len(stager.layers) == 48 and all(m._stager is stager for m in stager.layers)
            assert pkg.attach_weight_stager(model) is stager            # idempotent
            want = {}
            for form, mode in (("packed", "inline"), ("dense", "inline"), ("staged", "inline"), ("staged", "stream"),
                               ("auto", "inline")):
                cls.weight_form = form
                pkg.WeightStager.mode = mode
                y = model(x).clone()
                y2 = model(x2).clone()
                runner = pkg.GraphedModel(model, x)
                g = runner(x).clone()
                g2 = runner(x2).clone()
                torch.cuda.synchronize()
                assert pkg.ops.device_status() == 0
                assert torch.equal(y, g) and torch.equal(y2, g2), form
                if form == "packed":
                    want = {"y": y, "y2": y2}
                assert torch.equal(y, want["y"]) and torch.equal(y2, want["y2"]), (form, mode)
            assert stager.scratch_bytes() == 2 * 2 * 768 * 192
            # a layer called on its own, outside the model's forward, unpacks its weight when it is called
            cls.weight_form = "staged"
            layer = stager.layers[5]
            h = torch.randn(1500, layer.in_features, generator=gen).half().to(dev)
            y_alone = layer(h)
            cls.weight_form = "packed"
            assert torch.equal(y_alone, layer(h))
    finally:
        cls.weight_form = saved
        pkg.WeightStager.mode = saved_mode


@pytest.mark.parametrize("M,K,bits", [(5, 192, 4), (300, 384, 4), (64 * 197, 384, 4), (64 * 197, 384, 3), (1000, 768, 4),
                                      (777, 1024, 2), (2600, 192, 3)])
def test_layernorm_fused_with_the_quantizer(pkg, oracle, cuda_device, M, K, bits):
    """Residual add + LayerNorm + activation quantizer in one kernel: the residual sum, the LayerNorm output (returned
    on request) and the reconstruction equal, bit for bit, those of the separate LayerNorm and quantizer kernels,
    for both forms of the merged kernel; the LayerNorm output is within one fp16 step of torch's, and the
    reconstruction is what the CPU oracle makes of it."""
    dev = cuda_device
    gen = torch.Generator().manual_seed(M + K + bits)
    x = torch.randn(M, K, generator=gen).half().to(dev)
    y = (torch.randn(M, K, generator=gen) * 0.5).half().to(dev)
    norm = torch.nn.LayerNorm(K, eps=1e-6).to(dev)
    with torch.no_grad():
        norm.weight.copy_(1 + 0.1 * torch.randn(K, generator=gen))
        norm.bias.copy_(0.05 * torch.randn(K, generator=gen))
    cb = torch.sort(torch.randn(2 ** bits, generator=gen) * 1.1)[0].to(dev)
    th = (cb[:-1] + cb[1:]) / 2
    for yy in (y, None):
        s0, h0 = pkg.ops.add_layernorm(x, yy, norm)
        s1, xh1, h1 = pkg.ops.add_layernorm_quant(x, yy, norm, th, cb, bits, 64, want_h=True)
        s2, xh2 = pkg.ops.add_layernorm_quant(x, yy, norm, th, cb, bits, 64)
        assert torch.equal(s0, s1) and torch.equal(s1, s2) and torch.equal(xh1, xh2)
        with torch.no_grad():
            ref = torch.nn.functional.layer_norm(s0.float(), (K,), norm.weight.float(), norm.bias.float(), 1e-6)
        step = 2.0 ** -10 * float(ref.abs().max())                       # one fp16 step at the largest magnitude
        assert float((h1.float() - ref).abs().max()) <= step
        assert float((h1.float() - h0.float()).abs().max()) <= step and float((h1 == h0).float().mean()) > 0.999
        want = pkg.ops.quantize_activation_dequant(h1, th, cb, bits, 64, torch.float16)
        assert torch.equal(xh1, want)
        # both forms of the merged kernel (the small-input one and the tiled one) share the arithmetic of the two
        # separate kernels: same bits, so a model may switch forms by batch size
        assert torch.equal(h1, h0)
        assert torch.equal(xh1, pkg.ops.quantize_activation_dequant(h0, th, cb, bits, 64, torch.float16))
        with pkg._cabi.option("ARCQ_LNQ_SMALL", 0):            # the tiled (large-input) kernel on the same data
            s_big, xh_big, h_big = pkg.ops.add_layernorm_quant(x, yy, norm, th, cb, bits, 64, want_h=True)
        assert torch.equal(s_big, s0) and torch.equal(h_big, h0) and torch.equal(xh_big, xh1)
    # rows do not depend on the tile they fall in
    part = pkg.ops.add_layernorm_quant(x[: min(M, 37)].contiguous(), y[: min(M, 37)].contiguous(), norm, th, cb, bits, 64)[1]
    full = pkg.ops.add_layernorm_quant(x, y, norm, th, cb, bits, 64)[1]
    assert torch.equal(full[: part.shape[0]], part)
    # and against the CPU oracle on a few rows of the returned LayerNorm output
    rows = slice(0, min(M, 16))
    _, _, h = pkg.ops.add_layernorm_quant(x, y, norm, th, cb, bits, 64, want_h=True)
    hn = h[rows].float().cpu().numpy()
    codes, mu, sg, cs = oracle.quantize(hn, th.cpu().numpy(), cb.cpu().numpy(), 64)
    want_np = oracle.dequant(codes, mu, sg, cb.cpu().numpy(), 64).astype(np.float16)
    assert np.array_equal(full[rows].cpu().numpy(), want_np)
    assert pkg.ops.device_status() == 0


def test_model_with_the_fused_norm_quantizer(pkg, cuda_device):
    """The ViT skeleton with ``fuse_norm_quant``: same graph, one kernel fewer in front of qkv and fc1, same logits bit
    for bit with either form of the merged kernel."""
    dev = cuda_device
    gen = torch.Generator().manual_seed(11)
    model = pkg.create_vit("deit_tiny", seed=2).half().to(dev)
    x = torch.randn(8, 3, 224, 224, generator=gen).half().to(dev)
    saved = pkg.VisionTransformer.fuse_norm_quant
    try:
        with torch.no_grad():
            model = pkg.quantise_model(model, x, 4)
            pkg.VisionTransformer.fuse_norm_quant = False
            y0 = model(x).clone()
            pkg.VisionTransformer.fuse_norm_quant = True
            y1 = model(x).clone()
            g1 = pkg.GraphedModel(model, x)(x).clone()
        assert torch.equal(y1, g1)
        assert pkg.ops.device_status() == 0
        assert torch.equal(y1, y0)          # batch 8: the small-input kernel, bit-identical to the separate kernels
        with torch.no_grad(), pkg._cabi.option("ARCQ_LNQ_SMALL", 0):       # the tiled (large-input) kernel
            y2 = model(x).clone()
        assert torch.equal(y2, y0)
        lin = model.blocks[0].attn.qkv
        with pytest.raises(ValueError):
            lin(torch.zeros(4, lin.in_features, dtype=torch.float16, device=dev), pre_gelu=True, pre_quantized=True)
    finally:
        pkg.VisionTransformer.fuse_norm_quant = saved


@pytest.mark.parametrize("bits", [4, 3, 2])
def test_dense_gemm_that_unpacks_the_next_weight(pkg, cuda_device, bits):
    """``dense_weight_gemm(..., prefetch=...)``: the product is unchanged and the other scratch matrix holds the next
    layer's weight, bit for bit what ``unpack_weight_f16`` writes; also with no rows to multiply and on the one-CTA
    kernel."""
    dev = cuda_device
    gen = torch.Generator().manual_seed(70 + bits)
    M, K, N = 3000, 384, 768
    x = torch.randn(M, K, generator=gen).half().to(dev)
    w = (torch.randn(N, K, generator=gen) * 0.05).half().to(dev)
    b = torch.randn(N, generator=gen).to(dev)
    K2, N2 = 768, 384
    if not pkg.ops.packed_weight_gemm_supported(K2, N2, bits, 64):
        pytest.skip("shape not taken")
    pw, mw, sw, cw, cb, _ = _weight(pkg, dev, K2, N2, bits, seed=5 + bits)
    want_w = pkg.ops.unpack_weight_f16(pw, mw, sw, cw, cb, bits, 64)
    want_y = pkg.ops.dense_weight_gemm(x, w, b, torch.float16)
    for options in (dict(), dict(ARCQ_PAIR=0), dict(ARCQ_PAIR_PAIRS=3)):
        saved = {k: pkg._cabi.get_option(k) for k in options}
        try:
            for k, v in options.items():
                pkg._cabi.set_option(k, v)
            out = torch.full((N2 * K2 + 32,), float("nan"), dtype=torch.float16, device=dev)
            y = pkg.ops.dense_weight_gemm(x, w, b, torch.float16, prefetch=(pw, mw, sw, cw, cb, bits, 64, out))
        finally:
            for k, v in saved.items():
                pkg._cabi.set_option(k, v)
        assert torch.equal(y, want_y), options
        assert torch.equal(out[: N2 * K2].view(N2, K2), want_w), options
        assert bool(torch.isnan(out[N2 * K2:]).all())
    out = torch.zeros(N2 * K2, dtype=torch.float16, device=dev)
    y0 = pkg.ops.dense_weight_gemm(x[:0], w, b, torch.float16, prefetch=(pw, mw, sw, cw, cb, bits, 64, out))
    assert y0.shape[0] == 0 and torch.equal(out.view(N2, K2), want_w)
    with pytest.raises(RuntimeError):
        pkg.ops.dense_weight_gemm(x, w, b, torch.float16, prefetch=(pw, mw, sw, cw, cb, bits, 64, w.view(-1)))
    assert pkg.ops.device_status() == 0


@pytest.mark.parametrize("K,N", [(384, 1152), (384, 384), (384, 1536), (1536, 384), (768, 2304), (3072, 768)])
def test_benchmark_shapes_get_the_pair_kernels(pkg, cuda_device, K, N):
    """The entry points fall back to the one-CTA kernels when the device refuses a pair configuration (shared-memory
    ceiling, resident clusters); results would stay right and the benchmark would quietly lose a third.  Pin the form
    the DeiT layer shapes get at batch 64, for the dense, prefetching and packed entry points."""
    dev, cabi = cuda_device, pkg._cabi
    M, bits = 64 * 197, 4
    pw, mw, sw, cw, cb, bias = _weight(pkg, dev, K, N, bits, seed=K + N)
    x = torch.randn(M, K, generator=torch.Generator().manual_seed(1)).half().to(dev)
    w16 = pkg.ops.unpack_weight_f16(pw, mw, sw, cw, cb, bits, 64)
    pkg.ops.dense_weight_gemm(x, w16, bias, torch.float16)
    assert cabi.last_gemm_kernel() == cabi.GEMM_PAIR_DENSE
    other = torch.empty(N * K, dtype=torch.float16, device=dev)
    pkg.ops.dense_weight_gemm(x, w16, bias, torch.float16, prefetch=(pw, mw, sw, cw, cb, bits, 64, other))
    assert cabi.last_gemm_kernel() == cabi.GEMM_PAIR_DENSE_PREFETCH
    pkg.ops.packed_weight_gemm(x, pw, mw, sw, cw, cb, bias, bits, 64, torch.float16)
    assert cabi.last_gemm_kernel() == cabi.GEMM_PAIR_PACKED
    pkg.ops.dense_weight_gemm(x[:197].contiguous(), w16, bias, torch.float16)        # batch 1 too
    assert cabi.last_gemm_kernel() == cabi.GEMM_PAIR_DENSE
    with cabi.option("ARCQ_PAIR", 0):
        pkg.ops.dense_weight_gemm(x, w16, bias, torch.float16)
        assert cabi.last_gemm_kernel() == cabi.GEMM_ONE_CTA_DENSE
    assert pkg.ops.device_status() == 0
