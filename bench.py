"""Benchmark of the ARCQ packed inference path: whole-model DeiT forward, images/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--model deit_small] [--bits 4] [--batch 64]

A step is one forward of a batch of synthetic 224x224 images through the packed model: per packed linear
(48 of them) one tcgen05 GEMM and one weight unpack on a side stream, an activation quantizer (merged with the
preceding residual add + LayerNorm in front of qkv and fc1, with the GELU in front of fc2), plus the floating-point
glue.  With N > 1 (one process per GPU under torchrun) every rank runs its own batch (weak scaling; `--global-batch`
divides one batch over the ranks instead) and the logits are all-gathered over NCCL each step, on a side stream.
Rank 0 prints one JSON line.

`value` is timed with the batch already in HBM (CUDA-graph replay); `e2e` copies each step's batch
from pinned host memory and reads the logits back inside the timed region.  `roofline` is the GEMM (the
dominant kernel) on the model's four layer shapes; `cpu_baseline` is the reference's own CPU layer code
(`baseline/_ref`, else the oracle port) on the host cores; `triton_baseline`, `bs1` and `memory` are the
reference's Triton path and benchmark columns measured in the same run.  `--impl reference` prints the
same line for the CPU path alone.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

import __graft_entry__ as entry  # noqa: E402

METRIC = "images_per_sec"
TOKENS = 197


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--model", default="deit_small", choices=["deit_tiny", "deit_small", "deit_base"])
    ap.add_argument("--bits", type=int, default=4, choices=[3, 4])
    ap.add_argument("--batch", type=int, default=64, help="images per GPU per step")
    ap.add_argument("--global-batch", type=int, default=0,
                    help="fixed global batch split over the GPUs (strong scaling) instead of --batch per GPU")
    ap.add_argument("--no-graph", action="store_true", help="eager launches instead of CUDA-graph replay")
    ap.add_argument("--cpu-sample", type=int, default=8, help="images in the CPU-baseline sample batch")
    ap.add_argument("--skip-cpu-baseline", action="store_true")
    ap.add_argument("--skip-side-records", action="store_true",
                    help="leave out the batch-1 record, the memory columns and the reference Triton baseline")
    ap.add_argument("--kernels-only", action="store_true",
                    help="time only the two kernels of the packed linear on the model's layer shapes (for profiling)")
    ap.add_argument("--layers", default="qkv,proj,fc1,fc2", help="layer shapes for --kernels-only")
    ap.add_argument("--reps", type=int, default=20, help="timed launches per shape in the kernel timing pass")
    return ap.parse_args()


def workload_name(a) -> str:
    return f"{a.model} W{a.bits}A{a.bits} packed forward, batch {a.batch}/GPU, 224x224 synthetic images"


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm_gbs=float(d["hbm_gbs"]), tflops=float(d["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, tflops=1590.0, source="fallback")


# ---------------------------------------------------------------------------------- clocks
class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.idx)], stdout=subprocess.PIPE, text=True)
            self.t = threading.Thread(target=lambda: [self.lines.append(l) for l in self.proc.stdout], daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()          # the exact process started above
        self.proc.wait(timeout=5)
        sm, smax, reasons = [], [], set()
        for l in self.lines:
            f = [x.strip() for x in l.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_max_mhz=max(smax) if smax else None,
                    reasons=sorted(reasons), samples=len(sm))


# ---------------------------------------------------------------------------------- CPU path
def _ref_runner():
    """baseline/ref_runner.py when the reference's files are installed under baseline/_ref, else None."""
    sys.path.insert(0, str(ROOT / "baseline"))
    try:
        import ref_runner
        return ref_runner if ref_runner.available() else None
    except Exception:
        return None
    finally:
        sys.path.pop(0)


def cpu_reference_run(a, steps: int, warmup: int, sample_images: int):
    """The reference's CPU fake-quant forward on all host cores: its own ``QuantLinearPCARCQ`` layers
    (quant_backends.py:282-322) when ``baseline/_ref`` is installed (kind "reference"), else the oracle's
    restatement of them (kind "port")."""
    import contextlib
    pkg = entry.import_package()
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    imgs = torch.randn(sample_images, 3, 224, 224, generator=torch.Generator().manual_seed(1))
    rr = _ref_runner()
    if rr is not None:
        kind = "reference"
        with contextlib.redirect_stdout(sys.stderr):          # the reference logs every codebook compile to stdout
            model = rr.reference_cpu_model(pkg, a.model, a.bits, imgs)   # includes the calibrating forward
        run = lambda: model(imgs)                                             # noqa: E731
    else:
        kind = "port"
        from oracle.fakequant_vit import OracleViT
        O = entry.import_oracle()
        O.set_threads(cores)
        m = pkg.create_vit(a.model, seed=0)
        dim, heads, depth = pkg.DEIT_CONFIGS[a.model]
        o = OracleViT(m.state_dict(), dim, heads, depth, a.bits, cache_weights=False)
        o(imgs)                                   # calibrating forward (codebook compile), not timed
        run = lambda: o(imgs)                                                 # noqa: E731
    with torch.no_grad():
        for _ in range(max(0, warmup - 1)):
            run()
        t0 = time.perf_counter()
        for _ in range(steps):
            run()
        dt = time.perf_counter() - t0
    return dict(value=sample_images * steps / dt, ms_per_step=1e3 * dt / steps, cores=cores, kind=kind,
                sample=f"{steps} forwards of a {sample_images}-image batch of the same model after one calibrating "
                       f"forward and {max(0, warmup - 1)} warm-up")


def run_reference_arm(a):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warmup = min(a.steps, 2), max(1, min(a.warmup, 2))
    r = cpu_reference_run(a, steps, warmup, a.cpu_sample)
    what = ("the reference's own QuantLinearPCARCQ layers (baseline/_ref)" if r["kind"] == "reference"
            else "oracle port of the reference's fake-quant layers")
    line = {
        "impl": "reference", "metric": METRIC, "value": r["value"], "unit": "images/s", "n_gpus": a.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(a), "note": f"CPU fake-quant path: {what}, "
                   f"{a.cpu_sample}-image batches on host cores"},
        "cpu_baseline": {"value": r["value"], "unit": "images/s", "cores": r["cores"], "kind": r["kind"],
                         "sample": r["sample"]},
        "e2e": {"value": r["value"], "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------- GPU path
def layer_shapes(pkg, model: str):
    dim = pkg.DEIT_CONFIGS[model][0]
    return [("qkv", dim, 3 * dim), ("proj", dim, dim), ("fc1", dim, 4 * dim), ("fc2", 4 * dim, dim)]


def kernel_rooflines(pkg, a, dev, pk):
    """Time the two kernels of the packed linear alone on the model's layer shapes (CUDA events on the
    launch stream; rotating buffers so operands and results come from / go to HBM rather than L2)."""
    M, bits = a.batch * TOKENS, a.bits
    # the shape of a fitted codebook: denser around zero, not symmetric, no threshold exactly at zero
    half = 2 ** (bits - 1)
    neg = -torch.linspace(0, 2.6, half + 1)[1:].flip(0) ** 1.15 / 2.6 ** 0.15
    pos = torch.linspace(0, 2.58, half + 1)[1:half] ** 1.15 / 2.58 ** 0.15
    cb = torch.cat([neg, torch.tensor([0.02]), pos]).to(dev)
    th = (cb[:-1] + cb[1:]) / 2
    gen = torch.Generator().manual_seed(7)
    reps, rot = a.reps, 4
    out = {}
    wanted = a.layers.split(",")
    tot_flop = tot_ms = tot_bytes = aq_bytes = aq_ms = aq_copy_ms = 0.0
    per_layer = []
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timed(fn):
        """Average device time of one call: `reps` calls captured into a CUDA graph and replayed, so host-side
        launch cost (argument checks, allocation, tensor-map encoding) is not in the measurement."""
        for i in range(3):
            fn(i)
        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                for i in range(reps):
                    fn(i)
        torch.cuda.current_stream().wait_stream(side)
        graph.replay()
        torch.cuda.synchronize()
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    for name, K, N in layer_shapes(pkg, a.model):
        if name not in wanted:
            continue
        xs = [torch.randn(M, K, generator=gen).half().to(dev) for _ in range(rot)]
        w = (torch.randn(N, K, generator=gen) * 0.02).to(dev)
        bias = torch.zeros(N, device=dev)
        pw, mw, sw, cw = pkg.ops.quantize_activation(w, th, cb, bits, 64)
        xh = [pkg.ops.quantize_activation_dequant(x, th, cb, bits, 64, torch.float16) for x in xs]
        G = K // 64
        staged = M >= pkg.WeightStager.min_rows          # the route the model takes at this batch size
        w16 = pkg.ops.unpack_weight_f16(pw, mw, sw, cw, cb, bits, 64)
        quant = lambda i: pkg.ops.quantize_activation_dequant(xs[i % rot], th, cb, bits, 64, torch.float16)  # noqa: E731
        packed_gemm = lambda a_op: pkg.ops.packed_weight_gemm(a_op, pw, mw, sw, cw, cb, bias, bits, 64, torch.float16)  # noqa: E731
        dense_gemm = lambda a_op: pkg.ops.dense_weight_gemm(a_op, w16, bias, torch.float16)  # noqa: E731
        gemm = dense_gemm if staged else packed_gemm
        # In the model the GEMM's activation operand was written by the quantizer just before, so it is read
        # from L2; time the pair and the quantizer alone, and take the GEMM as the difference.  The four
        # rotating inputs (and as many outputs) keep the working set of consecutive calls apart.  In the staged
        # route the weight was unpacked on the side stream during the previous layer: that kernel is timed alone.
        qms = timed(quant)
        pair_ms = timed(lambda i: gemm(quant(i)))
        cold_ms = timed(lambda i: gemm(xh[i % rot]))
        other_ms = timed(lambda i: (packed_gemm if staged else dense_gemm)(quant(i))) - qms
        unpack_ms = timed(lambda i: pkg.ops.unpack_weight_f16(pw, mw, sw, cw, cb, bits, 64, out=w16))
        # what a plain device copy of the quantizer's bytes (M*K fp16 in, as many out) takes in the same harness:
        # at 10-40 MB a copy is far from the large-copy peak, so this is the fairer yardstick for the quantizer
        copy_ms = timed(lambda i: xh[(i + 1) % rot].copy_(xs[i % rot]))
        aq_copy_ms += copy_ms
        ms = pair_ms - qms
        wbytes = N * K * 2 if staged else N * K * bits // 8 + N * G * 12 + (2 ** bits) * 4
        nbytes = M * K * 2 + wbytes + N * 4 + M * N * 2
        flop = 2.0 * M * N * K
        qbytes = M * K * 2 * 2
        per_layer.append(dict(layer=name, M=M, K=K, N=N, ms=ms, tflops=flop / ms / 1e9, gbs=nbytes / ms / 1e6,
                              act_quant_ms=qms, act_quant_gbs=qbytes / qms / 1e6, gemm_ms_operand_from_hbm=cold_ms,
                              weight_unpack_ms=unpack_ms, copy_of_act_quant_bytes_ms=copy_ms,
                              **{("packed_weight_gemm_ms" if staged else "dense_weight_gemm_ms"): other_ms}))
        tot_flop, tot_ms, tot_bytes = tot_flop + flop, tot_ms + ms, tot_bytes + nbytes
        aq_bytes, aq_ms = aq_bytes + qbytes, aq_ms + qms
    achieved = tot_flop / tot_ms / 1e9
    staged = M >= pkg.WeightStager.min_rows
    kernel = "dense_weight_gemm_pair_kernel" if staged else "packed_weight_gemm_ws_kernel"
    # DRAM bytes (read + write) per launch from ncu captures of this command's GEMM launches: a small table under
    # profiles/, keyed by model, batch, bits and kernel (null when no capture covers this workload)
    traffic = None
    try:
        with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "profiles", "ncu_dram_bytes.json")) as f:
            table = json.load(f)
        row = table.get(f"{a.model}/b{a.batch}/w{bits}/{kernel}")
        if row is not None and all(l["layer"] in row for l in per_layer):
            traffic = sum(row[l["layer"]] for l in per_layer) / len(per_layer)
    except (OSError, ValueError):
        pass
    out["roofline"] = {"kernel": kernel, "bound": "tensor", "achieved": achieved,
                       "peak": pk["tflops"], "unit": "TFLOP/s", "frac": achieved / pk["tflops"], "traffic": traffic,
                       "peak_source": pk["source"] + " cuBLAS bf16 burst",
                       "algorithmic_bytes_per_launch_avg": tot_bytes / len(per_layer),
                       "ms_per_launch_avg": tot_ms / len(per_layer),
                       "weight_route": "staged: unpacked on a side stream during the previous layer, read by TMA" if staged
                                       else "packed: rebuilt inside the GEMM kernel",
                       "per_layer": per_layer}
    aq = aq_bytes / aq_ms / 1e6
    # the form the model runs in front of qkv and fc1: residual add + LayerNorm + quantizer in one kernel (reads the
    # residual stream and the branch output, writes the new residual stream and the reconstruction), against the
    # two kernels it replaces, same harness
    merged = None
    dim = pkg.DEIT_CONFIGS[a.model][0]
    if dim in (192, 384, 768):
        norm = torch.nn.LayerNorm(dim, eps=1e-6).to(dev)
        xs = [torch.randn(M, dim, generator=gen).half().to(dev) for _ in range(rot)]
        ys = [torch.randn(M, dim, generator=gen).half().to(dev) for _ in range(rot)]
        t_merged = timed(lambda i: pkg.ops.add_layernorm_quant(xs[i % rot], ys[i % rot], norm, th, cb, bits, 64))
        t_apart = timed(lambda i: pkg.ops.quantize_activation_dequant(
            pkg.ops.add_layernorm(xs[i % rot], ys[i % rot], norm)[1], th, cb, bits, 64, torch.float16))
        mbytes = 4 * M * dim * 2
        merged = {"kernel": "add_layernorm_act_quant_kernel", "ms": t_merged, "separate_kernels_ms": t_apart,
                  "bytes": mbytes, "achieved": mbytes / t_merged / 1e6, "frac": mbytes / t_merged / 1e6 / pk["hbm_gbs"]}
    out["roofline_act_quant"] = {"kernel": "act_quant_v2_kernel (qkv / proj / fc1 inputs), act_quant_v4_kernel with GELU (fc2 input)", "bound": "hbm", "achieved": aq, "peak": pk["hbm_gbs"],
                                 "unit": "GB/s", "frac": aq / pk["hbm_gbs"], "traffic": None,
                                 "peak_source": pk["source"] + " copy",
                                 "frac_of_same_size_copy": aq_copy_ms / aq_ms,
                                 "merged_with_layernorm": merged}
    return out


def launches_per_forward(pkg, a, n_lin: int, batch: int) -> int:
    """This repository's kernel launches in one forward of the benchmark model (torch / cuDNN kernels not counted)."""
    dim, _, depth = pkg.DEIT_CONFIGS[a.model]
    staged = batch * TOKENS >= pkg.WeightStager.min_rows and pkg.ARCQPackedLinearOnTheFly.weight_form in ("auto", "staged")
    merged = str(pkg.VisionTransformer.fuse_norm_quant) in ("auto", "1", "True") and dim in (192, 384, 768)
    norms = 2 * depth + 1
    quantizers = n_lin - (2 * depth if merged else 0)
    return n_lin * (2 if staged else 1) + norms + quantizers + 2        # + patch gathering and token assembly


def _time_forward(runner, x, warm: int, iters: int) -> float:
    """Milliseconds per call of ``runner(x)`` (CUDA events on the current stream)."""
    with torch.no_grad():
        for _ in range(warm):
            runner(x)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            runner(x)
        e1.record()
        torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def _memory_columns(model) -> dict:
    """The memory columns of the reference's benchmark protocol (scripts/benchmark_arcq_on_the_fly.py:247-261)."""
    mb = 1024 * 1024
    params = sum(p.numel() * p.element_size() for p in model.parameters()) / mb
    bufs = sum(b.numel() * b.element_size() for b in model.buffers()) / mb
    return dict(param_mb=params, buffer_mb=bufs, persistent_mb=params + bufs)


def small_batch_record(pkg, a, dev, model, batch: int = 1):
    """Batch-1 forward (weight-bandwidth- and launch-bound): latency, images/s and the packed-weight bytes per
    second it streams; the reference's protocol at bs = 1 (CUDA-graph replay, 10 warm-up / 50 timed)."""
    x = torch.randn(batch, 3, 224, 224, generator=torch.Generator().manual_seed(5)).half().to(dev)
    torch.cuda.reset_peak_memory_stats()
    resident = torch.cuda.memory_allocated() / 1024 / 1024
    g = pkg.GraphedModel(model, x)
    ms = _time_forward(g, x, 10, 50)
    peak = torch.cuda.max_memory_allocated() / 1024 / 1024
    packed_bytes = sum(b.numel() * b.element_size() for n, b in model.named_buffers()
                       if any(k in n for k in ("packed_weight_codes", "weight_center", "weight_scale", "weight_code_sum",
                                               "bias_tensor")))
    rec = dict(batch=batch, ms=ms, images_per_s=batch * 1e3 / ms, packed_weight_mb=packed_bytes / 1e6,
               packed_weight_gbs=packed_bytes / ms / 1e6, resident_model_mb=resident, forward_peak_mb=peak,
               forward_delta_mb=peak - resident)
    del g
    return rec


def triton_baseline_run(pkg, a, dev, batches):
    """The reference's Triton on-the-fly path (its own ARCQPackedLinearOnTheFly, unmodified, from baseline/_ref)
    on the same packed buffers and the same inputs, CUDA-graph replay like the B200 arm, timed in this run."""
    rr = _ref_runner()
    if rr is None:
        return {"unavailable": "baseline/_ref is not installed (python baseline/install_ref.py --reference <checkout>)"}
    out = {"kind": "reference Triton path (fair_qat/arcq_packed_on_the_fly.py + arcq_packed_triton.py), CUDA graph",
           "protocol": "10 warm-up / 50 timed replays, CUDA events"}
    try:
        import contextlib
        gen = torch.Generator().manual_seed(100)
        calib = torch.randn(a.batch, 3, 224, 224, generator=gen).half().to(dev)
        model = pkg.create_vit(a.model, seed=0).half().to(dev)
        with torch.no_grad(), contextlib.redirect_stdout(sys.stderr):
            model = pkg.quantise_model(model, calib, a.bits)
            ref_model = rr.reference_triton_model(pkg, model)
        for b in batches:
            x = calib if b == a.batch else torch.randn(b, 3, 224, 224, generator=gen).half().to(dev)
            with contextlib.redirect_stdout(sys.stderr):
                try:
                    runner = pkg.GraphedModel(ref_model, x, warmup=5)
                    how = "graph"
                except Exception:                     # fall back to eager launches if capture is refused
                    torch.cuda.synchronize()
                    runner, how = ref_model, "eager"
                ms = _time_forward(runner, x, 10, 50)
            out[f"bs{b}"] = dict(ms=ms, images_per_s=b * 1e3 / ms, launch=how)
        out.update(_memory_columns(ref_model))
        del ref_model, model
        torch.cuda.empty_cache()
    except Exception as ex:                           # Triton missing, compile failure, ...
        return {"unavailable": f"unavailable on this box: {type(ex).__name__}: {str(ex)[:300]}"}
    return out


def run_gpu_arm(a):
    pkg = entry.import_package()
    pkg._cabi.load()                      # raises if the CUDA library is not built: there is no fallback
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (use --impl reference for the CPU path)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    import torch.distributed as dist
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    strong = a.global_batch > 0
    if strong:
        if a.global_batch % world != 0:
            raise SystemExit(f"--global-batch {a.global_batch} does not split over {world} GPUs")
        a.batch = a.global_batch // world
    B = a.batch
    n_rot = 4 if B <= 256 else 2

    def seeded_batches(r):
        g = torch.Generator().manual_seed(100 + r)
        return [torch.randn(B, 3, 224, 224, generator=g).half() for _ in range(n_rot)]

    host_batches = [h.pin_memory() for h in seeded_batches(rank)]
    dev_batches = [h.to(dev) for h in host_batches]

    model = pkg.create_vit(a.model, seed=0).half().to(dev)
    calib = torch.randn(min(B, 64), 3, 224, 224, generator=torch.Generator().manual_seed(99)).half().to(dev)
    with torch.no_grad():
        model = pkg.quantise_model(model, calib, a.bits)      # codebooks calibrated on one batch (the same on every rank)
    n_lin = pkg.count_packed_linear(model)
    runner = model if a.no_graph else pkg.GraphedModel(model, dev_batches[0])
    global_batch = B * world
    gatherer = pkg.sharding.LogitsGatherer(global_batch, 1000, torch.float16, dev) if world > 1 else None

    def step(x):
        with torch.no_grad():
            y = runner(x)
        if gatherer is not None:
            gatherer.submit(y)          # staged copy on this stream, the collective on a side stream
        return y

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    # ---- device-resident timing
    for i in range(max(3, a.warmup)):
        step(dev_batches[i % n_rot])
    sync_all()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.profiler.start()            # lets a profiler attach to the timed region only
    e0.record()
    for i in range(a.steps):
        step(dev_batches[i % n_rot])
    e1.record()
    sync_all()
    torch.cuda.profiler.stop()
    ms = e0.elapsed_time(e1)
    # ---- end to end through the package's host-facing runner: every step copies its pinned host batch in and
    # its logits out; the copy of batch i+1 overlaps the forward of batch i, the caller reads logits i-1 meanwhile
    pipe = pkg.HostPipeline(step, host_batches[0], (B, 1000), dev)
    seen = []
    pipe.run((host_batches[i % n_rot] for i in range(3)), on_result=lambda t: seen.append(float(t[0, 0])))
    sync_all()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    pipe.run((host_batches[i % n_rot] for i in range(a.steps)), on_result=lambda t: seen.append(float(t[0, 0])))
    f1.record()
    sync_all()
    ms_e2e = f0.elapsed_time(f1)
    host_logits = pipe.out_host[0]
    clocks = sampler.stop() if rank == 0 else None
    rank_ms = None
    if world > 1:
        # the same steps without the gather, so that the per-rank spread (one GPU slower than another) can be told
        # from what the collective costs
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sync_all()
        g0.record()
        with torch.no_grad():
            for i in range(a.steps):
                runner(dev_batches[i % n_rot])
        g1.record()
        sync_all()
        mine = torch.tensor([ms, g0.elapsed_time(g1)], device=dev, dtype=torch.float64) / a.steps
        every = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(every, mine)
        rank_ms = {"with_gather": [round(float(v[0]), 4) for v in every],
                   "forward_only": [round(float(v[1]), 4) for v in every]}
        t = torch.tensor([ms, ms_e2e], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_e2e = float(t[0]), float(t[1])
    status = pkg.ops.device_status()
    gather_check = None
    if world > 1:
        # outside the timed region: the slice of every rank in rank 0's gathered logits against rank 0 running
        # that rank's seeded batch itself (rows do not depend on the batch they are computed in)
        with torch.no_grad():
            y_loc = runner(dev_batches[0])
            gatherer.submit(y_loc)
            y_all = gatherer.result().clone()
        torch.cuda.synchronize()
        if rank == 0:
            ok_all = True
            for r in range(world):
                xr = seeded_batches(r)[0].to(dev)
                with torch.no_grad():
                    yr = runner(xr).clone()
                ok_all = ok_all and bool(torch.equal(yr, y_all[r * B:(r + 1) * B]))
            gather_check = "bit-identical" if ok_all else "MISMATCH"

    if rank == 0:
        pk = peaks()
        extra = kernel_rooflines(pkg, a, dev, pk)
        if world == 1 and not a.skip_side_records:
            extra["bs1"] = small_batch_record(pkg, a, dev, model, 1)
            extra["memory"] = _memory_columns(model)
            tb = triton_baseline_run(pkg, a, dev, sorted({a.batch, 1}, reverse=True))
            if f"bs{a.batch}" in tb:
                tb["b200_over_triton"] = {f"bs{a.batch}": tb[f"bs{a.batch}"]["ms"] / (ms / a.steps),
                                          "bs1": tb["bs1"]["ms"] / extra["bs1"]["ms"] if "bs1" in tb else None}
            extra["triton_baseline"] = tb
        cpu = None
        if world == 1 and not a.skip_cpu_baseline:
            r = cpu_reference_run(a, 1, 1, a.cpu_sample)
            cpu = {"value": r["value"], "unit": "images/s", "cores": r["cores"], "kind": r["kind"], "sample": r["sample"]}
        act_bytes = B * TOKENS * pkg.DEIT_CONFIGS[a.model][0] * 2
        line = {
            "metric": METRIC, "value": global_batch * a.steps / (ms / 1e3), "unit": "images/s", "n_gpus": world,
            "steps": a.steps, "warmup": max(3, a.warmup), "ms_per_step": ms / a.steps, "higher_is_better": True,
            "scaling": "strong" if strong else "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": workload_name(a), "global_batch": global_batch, "packed_linears": n_lin,
                       "cuda_graph": not a.no_graph,
                       "parallelism": f"batch-sharded x{world}, logits all-gather on a side stream",
                       "l2": f"{n_rot} rotating input batches; one forward streams > 1 GB of activations "
                             f"({act_bytes / 1e6:.0f} MB per [M,dim] tensor) through the 126 MB L2",
                       "weights": "random init, seed 0; codebooks fitted on the first batch, then frozen"},
            "e2e": {"value": global_batch * a.steps / (ms_e2e / 1e3), "unit": "images/s",
                    "h2d_bytes_per_step": host_batches[0].numel() * 2, "d2h_bytes_per_step": host_logits.numel() * 2,
                    "ms_per_step": ms_e2e / a.steps},
            # per forward: one GEMM and (staged weight route) one weight unpack per packed linear; one add+LayerNorm
            # kernel per norm, which also runs the quantizer of qkv / fc1 when the merged kernel is on; one
            # quantizer per remaining packed linear
            "gpu_launches": launches_per_forward(pkg, a, n_lin, B) * a.steps,
            "clocks": clocks, "device_status": status,
        }
        if gather_check is not None:
            line["gather_check"] = gather_check
            line["rank_ms_per_step"] = rank_ms
        line.update(extra)
        if cpu is not None:
            line["cpu_baseline"] = cpu
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_kernels_only(a):
    pkg = entry.import_package()
    pkg._cabi.load()
    torch.cuda.set_device(0)
    out = kernel_rooflines(pkg, a, torch.device("cuda", 0), peaks())
    out["device_status"] = pkg.ops.device_status()
    print(json.dumps(out), flush=True)


def main():
    a = parse_args()
    if a.kernels_only:
        run_kernels_only(a)
    elif a.impl == "reference":
        run_reference_arm(a)
    else:
        run_gpu_arm(a)


if __name__ == "__main__":
    main()
