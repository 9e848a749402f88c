"""Whole-model parity evidence for the hot path as the model runs it: every packed linear through
``ARCQPackedLinearOnTheFly.forward`` under teacher forcing, and the free-running top-1 agreement next to its
noise floor (how far the reference's own arithmetic moves under a rounding-only change)."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle.fakequant_vit import OracleViT

pytestmark = pytest.mark.gpu
TOL = 2e-2        # max-abs error over output RMS against the fp32 fake-quant forward


def _oracle_and_packed(pkg, name, bits, images, dev, fp16_operands=False):
    m = pkg.create_vit(name, seed=0)
    dim, heads, depth = pkg.DEIT_CONFIGS[name]
    o = OracleViT(m.state_dict(), dim, heads, depth, bits)
    o(images)                                                   # the calibrating forward; codebooks frozen after it
    packed = pkg.pack_model_with_codebooks(m, o.codebooks_as_torch(), bits).half().to(dev)
    return o, packed


@pytest.mark.parametrize("name,bits", [("deit_small", 4), ("deit_small", 3)])
def test_teacher_forced_parity_through_the_on_the_fly_module(pkg, oracle, cuda_device, report, name, bits):
    """All 48 packed linears of DeiT-S, each fed the tensor the oracle model feeds that layer (rounded to fp16,
    and the oracle layer is given the same rounded tensor): reconstruction bit-equal to the oracle's, output
    within 2e-2 of the output RMS.  fc2 is called with the pre-GELU tensor and ``pre_gelu=True``, as the model
    calls it."""
    from arcq_vit_b200.vit import _get
    dev = cuda_device
    imgs = torch.randn(4, 3, 224, 224, generator=torch.Generator().manual_seed(20260701))
    o, packed = _oracle_and_packed(pkg, name, bits, imgs, dev)
    cap = {}
    o(imgs, cap)
    worst, worst_layer, staged = 0.0, "", 0
    for lname in o.layer_names():
        layer = _get(packed, lname)
        assert isinstance(layer, pkg.ARCQPackedLinearOnTheFly)
        cbk = o.codebooks[lname]
        W, b = o.sd[lname + ".weight"].numpy(), o.sd[lname + ".bias"].numpy()
        if lname.endswith("mlp.fc2"):
            pre = torch.from_numpy(cap[lname.replace("fc2", "fc1")]["y"]).half()      # fc1's output, rounded as stored
            x16 = F.gelu(pre.float()).half()                                           # what a separate GELU would store
            y = layer(pre.to(dev), pre_gelu=True)
            xhat = pkg.ops.quantize_activation_dequant(pre.to(dev), layer.activation_thresholds,
                                                       layer.activation_codebook, bits, 64, torch.float16, True)
        else:
            x16 = torch.from_numpy(cap[lname]["x"]).half()
            y = layer(x16.to(dev))
            xhat = pkg.ops.quantize_activation_dequant(x16.to(dev), layer.activation_thresholds,
                                                       layer.activation_codebook, bits, 64, torch.float16)
        xf = x16.float().numpy()
        codes, mu, sg, _ = oracle.quantize(xf, cbk["act_th"], cbk["act_cb"], 64)
        want = torch.from_numpy(oracle.dequant(codes, mu, sg, cbk["act_cb"], 64)).half()
        if lname.endswith("mlp.fc2"):
            # the fused GELU rounds like a separate fp16 GELU kernel except for rare last-bit cases of erf near the
            # rounding boundary of the product; such an input may move one code
            same = float((xhat.cpu() == want).float().mean())
            assert same > 0.999, f"{lname}: {same:.5f} of the reconstruction equals the oracle's"
        else:
            assert torch.equal(xhat.cpu(), want), f"{lname}: reconstruction differs from the oracle's"
        y_ref, _ = oracle.fake_quant_linear(xf, W, b, cbk["act_th"], cbk["act_cb"], cbk["w_th"], cbk["w_cb"], 64)
        err = float(np.abs(y.float().cpu().numpy() - y_ref).max() / np.sqrt((y_ref.astype(np.float64) ** 2).mean()))
        if err > worst:
            worst, worst_layer = err, lname
        assert err < TOL, f"{lname}: max|dy|/rms = {err:.3e}"
        assert y.dtype == torch.float16 and tuple(y.shape) == (xf.shape[0], W.shape[0])
    report("teacher_forced_on_the_fly", model=name, bits=bits, layers=len(o.layer_names()), rows=int(xf.shape[0]),
           worst_max_abs_over_rms=worst, worst_layer=worst_layer)
    assert pkg.ops.device_status() == 0


def _agreement(a: torch.Tensor, ref: torch.Tensor) -> dict:
    """Top-1 agreement of logits ``a`` with ``ref``: raw, and over the images whose reference top-1 margin is
    large against the typical logit error (more than 3x the median |difference| of their own logits)."""
    same = a.argmax(-1) == ref.argmax(-1)
    top2 = ref.topk(2, dim=-1).values
    margin = top2[:, 0] - top2[:, 1]
    diff = (a - ref).abs()
    clear = margin > 3.0 * diff.median(dim=-1).values
    return dict(top1_agreement=float(same.float().mean()), images=int(a.shape[0]),
                clear_margin_images=int(clear.sum()),
                top1_agreement_clear_margin=float(same[clear].float().mean()) if int(clear.sum()) else None,
                max_abs_logit_diff=float(diff.max()), median_abs_logit_diff=float(diff.median()),
                ref_logit_std=float(ref.std()), ref_median_top1_margin=float(margin.median()))


@pytest.mark.parametrize("name", ["deit_tiny", "deit_small"])
def test_free_running_agreement_next_to_its_noise_floor(pkg, oracle, cuda_device, report, name):
    """64 noise images through the whole W4A4 model, free running.  Reported side by side, each against the fp32
    CPU oracle: this back end's fp16 chain; the oracle with nothing changed but both operands of every linear
    rounded to fp16 (a rounding-only change); and, where the reference's files are installed, the reference's
    own CPU layers (another fp32 summation order) and its own Triton path.  The quantizer is discontinuous and
    these random-weight models have top-1 margins of a fraction of the logit spread, so a rounding-only change
    already flips many arg-maxes: the >= 99.5 % agreement asked of trained models on real images is not reached
    by the reference against itself here, and the test asserts only that this back end sits at that floor."""
    dev = cuda_device
    bits, n = 4, 64
    imgs = torch.randn(n, 3, 224, 224, generator=torch.Generator().manual_seed(20260702))
    o, packed = _oracle_and_packed(pkg, name, bits, imgs, dev)
    ref = o(imgs)
    with torch.no_grad():
        got = packed(imgs.half().to(dev)).float().cpu()
    assert torch.isfinite(got).all() and got.shape == (n, 1000)
    rows = {"b200_fp16_chain": _agreement(got, ref)}
    # noise floor 1: same oracle, same codebooks, fp16-rounded operands, fp32 everything else
    m0 = pkg.create_vit(name, seed=0)
    dim, heads, depth = pkg.DEIT_CONFIGS[name]
    o16 = OracleViT(m0.state_dict(), dim, heads, depth, bits, fp16_operands=True)
    o16.codebooks = o.codebooks
    rows["oracle_with_fp16_rounded_operands"] = _agreement(o16(imgs), ref)
    # noise floors 2 and 3: the reference's own code, when its files are installed next to the repository
    import sys
    from conftest import ROOT
    sys.path.insert(0, str(ROOT / "baseline"))
    try:
        import ref_runner
        have_ref = ref_runner.available()
    except Exception:
        have_ref = False
    if have_ref:
        import contextlib
        import io
        with contextlib.redirect_stdout(io.StringIO()):
            cpu_ref = ref_runner.reference_cpu_model(pkg, name, bits, imgs)       # calibrated on the same batch
            with torch.no_grad():
                rows["reference_cpu_layers_fp32"] = _agreement(cpu_ref(imgs), ref)
            try:
                import copy
                tri = ref_runner.reference_triton_model(pkg, copy.deepcopy(packed))
                with torch.no_grad():
                    y_tri = tri(imgs.half().to(dev)).float().cpu()
                rows["reference_triton_path"] = _agreement(y_tri, ref)
                rows["b200_vs_reference_triton"] = _agreement(got, y_tri)
            except Exception as ex:                                                # Triton not usable on this box
                rows["reference_triton_path"] = {"unavailable": f"{type(ex).__name__}: {str(ex)[:200]}"}
    report("free_running", model=name, bits=bits, **rows)
    floor = rows["oracle_with_fp16_rounded_operands"]
    mine = rows["b200_fp16_chain"]
    # at the floor: no worse than the rounding-only emulation by more than the sampling noise of 64 images
    assert mine["top1_agreement"] >= floor["top1_agreement"] - 0.20
    assert mine["max_abs_logit_diff"] <= 3.0 * floor["max_abs_logit_diff"] + 0.05
    assert pkg.ops.device_status() == 0
