"""Throughput of the DIMQ quantised-inference hot path on B200.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

One step = one forward of the synthetic DIMQ ViT-B/16 (12 layers, hidden 768, 197 tokens;
every qkv / proj / fc1 / fc2 / head Linear stored as 3-bit indices with one 8-entry codebook
per 128 output rows) over a batch of 128 images per GPU, bf16 activations.  All quantised
Linears run through ``libdimq_b200.so`` (weight-only LUT GEMM); attention, LayerNorm and the
patch embedding are dense bf16 PyTorch ops.  Rank 0 prints one JSON line.

``value``     — images/s with the images already in HBM (CUDA-graph replay, CUDA events).
``e2e``       — the same forward called with pinned HOST images: H2D copy + forward + D2H of the
                logits inside the timed region.
``roofline``  — the quantised layers: their algorithmic flops divided by the summed CUDA-event
                duration of exactly those calls (an instrumented eager pass).
``secondary`` — the same numbers for the other model of the metric (ResNet-18, batch 256 per GPU,
                4-bit per-layer codebooks, stem and classifier at 8 bits).
``strong``    — N > 1 only: the configurations' batches (128 / 256) split over the GPUs, and the
                gathered logits of one fixed batch compared with a single-GPU forward of it.
``w4a4``      — ResNet-18 in the reference's W4A4 contract: activations quantised to u4 per layer with
                calibrated parameters, on the tensor cores.
``micro``     — the index-streaming regime: M in {1, 4, 16} on the 1024 -> 4096 / 4096 -> 1024 shapes
                over a ring of distinct weights larger than the L2.
``cpu_baseline`` / ``--impl reference`` — the reference's CPU path (dequantise + fp32
                ``F.linear`` / ``F.conv2d``, PyTorch CPU, all host threads) on a bounded sample.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

# name -> (config.workload, images per GPU and step, weight description)
WORKLOADS = {
    "vit_b16": ("vit_b16_w3_g128_batch128_per_gpu", 128,
                "3-bit indices, 8-entry bf16 codebook per 128 output rows, random init"),
    "resnet18": ("resnet18_w4_stem_fc_w8_batch256_per_gpu", 256,
                 "BN folded; 4-bit per-layer bf16 codebooks, 8-bit for the stem conv and the classifier, random init"),
}
FALLBACK_TFLOPS = 1590.0
FALLBACK_HBM_GBS = 6650.0
CPU_SAMPLE_IMAGES = 8


def _peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return float(data.get("bf16_tflops_sustained", data.get("bf16_tflops", FALLBACK_TFLOPS))), "measured (sustained)"
    return FALLBACK_TFLOPS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while a timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int) -> None:
        self.index = index
        self.proc = None
        self.lines: list[str] = []
        self.thread = None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100", "-i",
                 str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self) -> None:
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, maxes, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                clocks.append(float(parts[0]))
                maxes.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        clocks.sort()
        return {"sm_mhz": clocks[len(clocks) // 2] if clocks else None, "sm_max_mhz": max(maxes) if maxes else None,
                "reasons": sorted(reasons), "samples": len(clocks)}


def run_reference(args) -> None:
    """The reference's CPU path (dequantised weights, fp32 PyTorch CPU ops), rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch

    from oracle import models_oracle as mo

    WORKLOAD, BATCH_PER_GPU, _ = WORKLOADS[args.workload]
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    if args.workload == "vit_b16":
        model = mo.ViTOracle(mo.build_vit_b16_checkpoint_cpu(seed=0))
    else:
        model = mo.ResNet18Oracle(mo.build_resnet18_checkpoint_cpu(seed=0))
    images = torch.randn(CPU_SAMPLE_IMAGES, 3, 224, 224, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16)
    for _ in range(max(1, min(args.warmup, 2))):
        model.forward(images)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        model.forward(images)
    dt = time.perf_counter() - t0
    value = CPU_SAMPLE_IMAGES * args.steps / dt
    sample = f"{CPU_SAMPLE_IMAGES} images per step (of the {BATCH_PER_GPU}-image batch), fp32, {cores} threads"
    print(json.dumps({
        "impl": "reference", "metric": f"{args.workload}_dimq_images_per_s", "value": value, "unit": "images/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": sample},
        "cpu_baseline": {"value": value, "unit": "images/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def cpu_baseline(ckpt, workload: str) -> dict:
    import torch

    from oracle.models_oracle import ResNet18Oracle, ViTOracle

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    cpu_ckpt = {"config": ckpt.get("config"),
                "layers": {k: {kk: (vv.cpu() if hasattr(vv, "cpu") else vv) for kk, vv in v.items()}
                           for k, v in ckpt["layers"].items()},
                "non_quantized_state_dict": {k: v.cpu() for k, v in ckpt["non_quantized_state_dict"].items()}}
    model = ViTOracle(cpu_ckpt) if workload == "vit_b16" else ResNet18Oracle(cpu_ckpt)
    images = torch.randn(CPU_SAMPLE_IMAGES, 3, 224, 224, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16)
    model.forward(images)
    passes, t0 = 0, time.perf_counter()
    while passes < 2 or time.perf_counter() - t0 < 10.0:
        model.forward(images)
        passes += 1
        if passes >= 40:
            break
    dt = time.perf_counter() - t0
    return {"value": CPU_SAMPLE_IMAGES * passes / dt, "unit": "images/s", "cores": cores, "kind": "port",
            "sample": f"{passes} passes of {CPU_SAMPLE_IMAGES} images (fp32 PyTorch CPU, dequantised weights)"}


def run_micro(args) -> None:
    """One LUT GEMM shape, timed with CUDA events over a CUDA graph of back-to-back calls.

    The single-kernel driver behind the per-kernel tables and the ncu captures under profiles/."""
    import torch

    from dimq_b200 import ops

    ops.require_extension()
    parts = args.micro.split(",")
    m, k, n, bits = (int(v) for v in parts[:4])
    algo = parts[4] if len(parts) > 4 and parts[4] not in ("", "auto") else None
    tiled = algo is not None and algo.endswith("_tiled")      # the small-M kernel over prepacked (tiled) indices
    if tiled:
        algo = algo[:-len("_tiled")]
    index_bytes = n * k * bits // 8
    copies = int(parts[5]) if len(parts) > 5 else max(1, min(64, (192 << 20) // max(index_bytes, 1) + 1))
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    x = torch.randn(m, k, device=dev, dtype=torch.bfloat16)
    packed = [torch.randint(0, 256, (index_bytes,), dtype=torch.uint8, device=dev) for _ in range(copies)]
    groups = n // 128 if bits == 3 and n % 128 == 0 else 1
    cb = (torch.randn(groups, 1 << bits, device=dev) * 0.02).sort(dim=1).values.to(torch.bfloat16)
    kw = dict(bits=bits, group_rows=128 if groups > 1 else None, out_dtype=torch.bfloat16, algo=algo)
    tiles = {id(pw): ops.linear_prepack(pw, n, k, bits) for pw in packed} if tiled else {}
    call = lambda pw: ops.dimq_linear_wq(x, pw, cb, None, n, k, packed_tiled=tiles.get(id(pw)), **kw)
    for pw in packed[:2]:
        call(pw)
    torch.cuda.synchronize()
    per_graph = max(copies, 8)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(per_graph):
            call(packed[i % copies])
    for _ in range(max(args.warmup, 3)):
        graph.replay()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        graph.replay()
    end.record()
    torch.cuda.synchronize()
    us = start.elapsed_time(end) * 1e3 / (args.steps * per_graph)
    tc_peak, peak_kind = _peaks()
    path = ROOT / "MEASURED_PEAKS.json"
    hbm_peak = float(json.loads(path.read_text()).get("hbm_gbs", FALLBACK_HBM_GBS)) if path.exists() else FALLBACK_HBM_GBS
    print(json.dumps({
        "metric": "linear_wq_us_per_call", "value": us, "unit": "us", "higher_is_better": False,
        "config": {"workload": f"lut_gemm_m{m}_k{k}_n{n}_w{bits}", "algo": (algo or "auto") + ("_tiled" if tiled else ""),
                   "weight_copies": copies,
                   "l2": "weights rotated over more than 126 MB" if copies * index_bytes > (126 << 20) else "weights fit L2"},
        "tflops": 2.0 * m * n * k / us / 1e6, "tflops_frac": 2.0 * m * n * k / us / 1e6 / tc_peak,
        "index_gbs": index_bytes / us / 1e3, "index_gbs_frac": index_bytes / us / 1e3 / hbm_peak,
        "peak_source": peak_kind, "dtype": "bf16", "data": "synthetic",
    }), flush=True)


def small_m_micro(dev) -> dict:
    """The index-streaming regime: M in {1, 4, 16} on the 1024 -> 4096, 4096 -> 1024 (2 MB of indices) and
    8192 -> 8192 (32 MB) shapes (4-bit, bf16 activations, fp16 codebook as the reference's packed export
    stores it), the weight of every call different and the ring of weights larger than the L2, one CUDA
    graph of back-to-back calls."""
    import torch

    from dimq_b200 import ops

    path = ROOT / "MEASURED_PEAKS.json"
    hbm_peak = float(json.loads(path.read_text()).get("hbm_gbs", FALLBACK_HBM_GBS)) if path.exists() else FALLBACK_HBM_GBS
    out = {"unit": "us per call", "index_gbs_peak": hbm_peak, "peak_source": "measured" if path.exists() else "fallback",
           "weights": "4-bit, one fp16 codebook per layer; rings of distinct index tensors larger than the L2 "
                      "(136 x 2 MB, 6 x 32 MB), L2-cold",
           "cases": []}
    bits = 4
    for (k, n) in ((1024, 4096), (4096, 1024), (8192, 8192)):
        index_bytes = n * k * bits // 8
        copies = 136 if index_bytes <= (2 << 20) else 6
        packed = [torch.randint(0, 256, (index_bytes,), dtype=torch.uint8, device=dev) for _ in range(copies)]
        cb = (torch.randn(1, 16, device=dev) * 0.02).sort(dim=1).values.to(torch.float16)
        # what a DIMQLinear module does on its own: a tiled copy of the indices where the small-M kernel takes
        # the weight (K a multiple of 128 and at least 2048, 2 MB of indices and more); the calls read that copy
        tiles = {}
        if k % 128 == 0 and k >= 2048 and index_bytes >= (2 << 20):
            tiles = {id(pw): ops.linear_prepack(pw, n, k, bits) for pw in packed}
        for m in (1, 4, 16):
            x = torch.randn(m, k, device=dev, dtype=torch.bfloat16)
            call = lambda pw: ops.dimq_linear_wq(x, pw, cb, None, n, k, bits=bits, out_dtype=torch.bfloat16,
                                                 packed_tiled=tiles.get(id(pw)))
            call(packed[0])
            torch.cuda.synchronize()
            reps = max(1, 24 // copies)      # a graph of at least 24 calls
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for _ in range(reps):
                    for pw in packed:
                        call(pw)
            for _ in range(3):
                graph.replay()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for _ in range(5):
                graph.replay()
            end.record()
            torch.cuda.synchronize()
            us = start.elapsed_time(end) * 1e3 / (5 * copies * reps)
            out["cases"].append({"m": m, "k": k, "n": n, "us": us, "index_gbs": index_bytes / us / 1e3,
                                 "index_gbs_frac": index_bytes / us / 1e3 / hbm_peak})
        del packed, tiles
    return out


class ModelBench:
    """One model on this rank: CUDA graphs over rotating inputs, timed resident and end to end."""

    def __init__(self, workload: str, batch: int, dev, rank: int, seed_images: int = 1234):
        import torch

        from dimq_b200 import _lib
        from dimq_b200.workloads import DIMQResNet18, DIMQViT, build_resnet18_checkpoint, build_vit_b16_checkpoint

        self.workload, self.batch, self.dev = workload, batch, dev
        if workload == "vit_b16":
            self.ckpt = build_vit_b16_checkpoint(seed=0, device=dev)
            self.model = DIMQViT(self.ckpt).to(dev).eval()
            self.flops_per_step = self.model.lut_gemm_flops(batch)
        else:
            self.ckpt = build_resnet18_checkpoint(seed=0, device=dev)
            self.model = DIMQResNet18(self.ckpt).to(dev).eval()
            self.flops_per_step = self.model.lut_flops(batch)
            if workload == "resnet18_w4a4":
                # the reference's actual contract: 4-bit weights AND 4-bit activations.  Per-layer u4
                # parameters from a calibration pass over 16 synthetic images, then every 4-bit
                # convolution runs in the W4A4 mode (stem and classifier stay 8-bit weight-only).
                gen_c = torch.Generator(device="cpu").manual_seed(99)
                calib = [torch.randn(8, 3, 224, 224, generator=gen_c).to(torch.bfloat16).to(dev) for _ in range(2)]
                self.model.set_activation_qparams(self.model.calibrate(calib))
        self.n_bufs = 4  # rotating image buffers: with the activations of a step, far more than the 126 MB L2
        gen = torch.Generator(device="cpu").manual_seed(seed_images + rank)
        self.host_images = [torch.randn(batch, 3, 224, 224, generator=gen).to(torch.bfloat16).pin_memory()
                            for _ in range(self.n_bufs)]
        self.dev_images = [h.to(dev, non_blocking=True) for h in self.host_images]
        torch.cuda.synchronize()
        self.stream = torch.cuda.Stream(device=dev)
        self.copy_stream = torch.cuda.Stream(device=dev)
        self.gather_stream = torch.cuda.Stream(device=dev)
        # two staging buffers: the host->device copy of step i + 1 runs on its own stream under step i
        self.staging = [torch.empty_like(self.dev_images[0]) for _ in range(2)]
        self.h2d_done = [torch.cuda.Event() for _ in range(2)]
        self.compute_done = [torch.cuda.Event() for _ in range(2)]
        self.host_logits = torch.empty(batch, 1000, dtype=torch.float32).pin_memory()
        self.graphs, self.outs = [], []
        self.gather_done = {}   # buffer index -> event of the last gather that read its logits
        with torch.cuda.stream(self.stream):
            for _ in range(2):
                self.model(self.dev_images[0])
            self.stream.synchronize()
            before = _lib.LAUNCH_COUNT[0]
            for src in self.dev_images + self.staging:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=self.stream):
                    out = self.model(src)
                self.graphs.append(g)
                self.outs.append(out)
            self.launches_per_forward = (_lib.LAUNCH_COUNT[0] - before) // len(self.graphs)

    def _replay(self, buf: int, world: int) -> None:
        """Replay the graph of buffer `buf`, then all-gather its logits on a side stream so that the
        collective overlaps the next step's forward.  A replay waits for the gather that last read the
        same logits buffer."""
        import torch

        from dimq_b200.dist import gather_logits

        if buf in self.gather_done:
            self.stream.wait_event(self.gather_done[buf])
        self.graphs[buf].replay()
        if world == 1:
            return
        done = torch.cuda.Event()
        done.record(self.stream)
        with torch.cuda.stream(self.gather_stream):
            self.gather_stream.wait_event(done)
            gather_logits(self.outs[buf])
            ev = torch.cuda.Event()
            ev.record(self.gather_stream)
            self.gather_done[buf] = ev

    def step_resident(self, i: int, world: int) -> None:
        self._replay(i % self.n_bufs, world)

    def step_e2e(self, i: int, world: int) -> None:
        import torch

        b = i % 2
        with torch.cuda.stream(self.copy_stream):
            self.copy_stream.wait_event(self.compute_done[b])  # the forward that last read this buffer
            self.staging[b].copy_(self.host_images[i % self.n_bufs], non_blocking=True)
            self.h2d_done[b].record(self.copy_stream)
        self.stream.wait_event(self.h2d_done[b])
        self._replay(self.n_bufs + b, world)
        self.host_logits.copy_(self.outs[self.n_bufs + b], non_blocking=True)
        self.compute_done[b].record(self.stream)

    def run_timed(self, step_fn, steps: int, warmup: int, world: int) -> float:
        """ms for `steps` steps: CUDA events on the launching stream, barrier + synchronize on both sides,
        the side-stream gathers joined before the end event, max over ranks."""
        import torch
        import torch.distributed as dist

        def barrier():
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        with torch.cuda.stream(self.stream):
            for i in range(warmup):
                step_fn(i, world)
            self.copy_stream.synchronize()
            self.gather_stream.synchronize()
            barrier()
            start = torch.cuda.Event(enable_timing=True)
            end = torch.cuda.Event(enable_timing=True)
            start.record(self.stream)
            self.copy_stream.wait_event(start)  # no copy of a timed step starts before the timed region
            for i in range(steps):
                step_fn(i, world)
            self.stream.wait_stream(self.gather_stream)
            end.record(self.stream)
            barrier()
            ms = torch.tensor([start.elapsed_time(end)], device=self.dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    def roofline(self, roof_steps: int = 3) -> dict:
        """The quantised layers alone: an eager pass with CUDA events around every LUT linear / conv call
        (launches queued behind a sleep kernel so that the events bracket execution, not launch gaps)."""
        import torch

        from dimq_b200 import modules as _modules
        from dimq_b200 import ops

        events = []          # one list per step
        orig, orig_conv = ops.dimq_linear_wq, ops.dimq_conv2d_wq

        def timed(fn):
            def wrapper(*a, **kw):
                s = torch.cuda.Event(enable_timing=True)
                e = torch.cuda.Event(enable_timing=True)
                s.record(torch.cuda.current_stream())
                y = fn(*a, **kw)
                e.record(torch.cuda.current_stream())
                events[-1].append((s, e))
                return y
            return wrapper

        _modules.ops.dimq_linear_wq = timed(orig)
        _modules.ops.dimq_conv2d_wq = timed(orig_conv)
        try:
            with torch.cuda.stream(self.stream):
                for i in range(roof_steps):
                    events.append([])
                    torch.cuda._sleep(int(60e6))
                    self.model(self.dev_images[i % self.n_bufs])
                    self.stream.synchronize()
        finally:
            _modules.ops.dimq_linear_wq = orig
            _modules.ops.dimq_conv2d_wq = orig_conv
        # the step whose launches ran furthest ahead of the GPU: a host stall inside a step only adds idle time
        # to that step's intervals (seen once: one step of three measured twice the others)
        per_step = [sum(s.elapsed_time(e) for s, e in step) for step in events]
        ms = min(per_step)
        n_calls = len(events[0])
        peak, peak_kind = _peaks()
        achieved = self.flops_per_step / (ms / 1e3) / 1e12
        return {"kernel": "lut_dense_tc_kernel (dense TMA + tcgen05 GEMM / implicit-GEMM conv over the weight "
                          "lut_expand_kernel writes once per call; both kernels are inside the timed calls)",
                "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "peak_source": peak_kind, "calls_timed": n_calls, "steps_timed": roof_steps,
                "avg_call_ms": ms / max(n_calls, 1),
                "flops_per_step": self.flops_per_step}

    def release(self) -> None:
        import torch

        self.graphs.clear()
        self.outs.clear()
        self.model = None
        torch.cuda.empty_cache()


def parity_vs_one_gpu(workload: str, global_batch: int, dev, world: int, rank: int):
    """Rank r runs its shard of one fixed global batch, the logits are all-gathered, and rank 0 compares
    them with its own forward of the whole batch."""
    import torch

    from dimq_b200.dist import gather_logits, shard_bounds
    from dimq_b200.workloads import DIMQResNet18, DIMQViT, build_resnet18_checkpoint, build_vit_b16_checkpoint

    if workload == "vit_b16":
        model = DIMQViT(build_vit_b16_checkpoint(seed=0, device=dev)).to(dev).eval()
    else:
        model = DIMQResNet18(build_resnet18_checkpoint(seed=0, device=dev)).to(dev).eval()
    images = torch.randn(global_batch, 3, 224, 224, generator=torch.Generator().manual_seed(77)).to(torch.bfloat16)
    lo, hi = shard_bounds(global_batch, rank, world)
    local = model(images[lo:hi].to(dev)).float()
    gathered = gather_logits(local, total=global_batch)
    result = None
    if rank == 0:
        whole = model(images.to(dev)).float()
        diff = (gathered - whole).double()
        result = {"max_abs": float(diff.abs().max()), "rel_l2": float(diff.norm() / whole.double().norm())}
    del model
    torch.cuda.empty_cache()
    return result


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--workload", default="vit_b16", choices=["vit_b16", "resnet18"],
                    help="the headline model of the line; the other one is reported under `secondary`")
    ap.add_argument("--only", action="store_true", help="skip the secondary model, the strong-scaling pass and the "
                                                         "small-M micro numbers (profiling runs)")
    ap.add_argument("--micro", default=None, metavar="M,K,N,BITS[,ALGO[,COPIES]]",
                    help="time one weight-only LUT GEMM instead of a model (bf16 activations, bf16 codebook per "
                         "128 rows at 3 bits, per layer otherwise); COPIES distinct weights are rotated so that "
                         "indices come from HBM")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.micro is not None:
        run_micro(args)
        return

    if args.impl == "reference":
        run_reference(args)
        return

    import torch
    import torch.distributed as dist

    from dimq_b200 import ops
    from dimq_b200.dist import shard_bounds

    ops.require_extension()  # no CPU fallback: fail loudly when the CUDA library is missing
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    other = "resnet18" if args.workload == "vit_b16" else "vit_b16"
    results = {}
    with torch.no_grad():
        # ---- weak scaling: the configuration's batch on every GPU (the headline and the secondary model) ----
        for name in ([args.workload] if args.only else [args.workload, other]):
            _, B, _ = WORKLOADS[name]
            mb = ModelBench(name, B, dev, rank)
            sampler = ClockSampler(local_rank)
            if rank == 0:
                sampler.start()
            ms_res = mb.run_timed(mb.step_resident, args.steps, args.warmup, world)
            clocks = sampler.stop() if rank == 0 else None
            ms_e2e = mb.run_timed(mb.step_e2e, args.steps, args.warmup, world)
            roof = mb.roofline()
            cpu = cpu_baseline(mb.ckpt, name) if (world == 1 and rank == 0 and not args.no_cpu_baseline
                                                  and name == args.workload) else None
            results[name] = {"B": B, "ms_res": ms_res, "ms_e2e": ms_e2e, "clocks": clocks, "roofline": roof,
                             "launches": mb.launches_per_forward, "cpu": cpu}
            mb.release()
            del mb
        w4a4 = None
        if not args.only:
            B = WORKLOADS["resnet18"][1]
            mb = ModelBench("resnet18_w4a4", B, dev, rank)
            ms_res = mb.run_timed(mb.step_resident, args.steps, args.warmup, world)
            ms_e2e = mb.run_timed(mb.step_e2e, args.steps, args.warmup, world)
            w4a4 = {"metric": "resnet18_dimq_w4a4_images_per_s", "value": world * B * args.steps / (ms_res / 1e3),
                    "unit": "images/s", "ms_per_step": ms_res / args.steps,
                    "e2e": {"value": world * B * args.steps / (ms_e2e / 1e3), "unit": "images/s",
                            "ms_per_step": ms_e2e / args.steps},
                    "gpu_launches": mb.launches_per_forward * args.steps,
                    "config": {"workload": "resnet18_w4a4_calibrated_batch256_per_gpu", "global_batch": world * B,
                               "activations": "per-tensor affine u4 per layer, parameters from a min/max calibration "
                                              "pass over 16 synthetic images; stem and classifier 8-bit weight-only"}}
            mb.release()
            del mb
        # ---- strong scaling: the configuration's batch split over the GPUs (BASELINE.json's wording) ----
        strong = None
        if world > 1 and not args.only:
            strong = {}
            for name in (args.workload, other):
                _, B, _ = WORKLOADS[name]
                lo, hi = shard_bounds(B, rank, world)
                mb = ModelBench(name, hi - lo, dev, rank)
                ms_res = mb.run_timed(mb.step_resident, args.steps, args.warmup, world)
                ms_e2e = mb.run_timed(mb.step_e2e, args.steps, args.warmup, world)
                mb.release()
                del mb
                par = parity_vs_one_gpu(name, B, dev, world, rank)
                strong[name] = {"global_batch": B, "images_per_gpu": hi - lo,
                                "value": B * args.steps / (ms_res / 1e3), "unit": "images/s",
                                "ms_per_step": ms_res / args.steps,
                                "e2e_value": B * args.steps / (ms_e2e / 1e3), "parity_vs_1gpu": par}
        micro = small_m_micro(dev) if (rank == 0 and not args.only) else None

    if world > 1:
        dist.barrier()
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    def model_line(name: str) -> dict:
        r = results[name]
        images_total = world * r["B"] * args.steps
        return {"metric": f"{name}_dimq_images_per_s", "value": images_total / (r["ms_res"] / 1e3), "unit": "images/s",
                "ms_per_step": r["ms_res"] / args.steps,
                "config": {"workload": WORKLOADS[name][0], "global_batch": world * r["B"], "weights": WORKLOADS[name][2],
                           "l2": "4 rotating image buffers and >126 MB of activations per step",
                           "parallelism": f"dp{world} (batch-sharded replicas, all-gather of logits on a side stream)"},
                "e2e": {"value": images_total / (r["ms_e2e"] / 1e3), "unit": "images/s",
                        "ms_per_step": r["ms_e2e"] / args.steps,
                        "h2d_bytes_per_step": world * r["B"] * 3 * 224 * 224 * 2,
                        "d2h_bytes_per_step": world * r["B"] * 1000 * 4},
                "gpu_launches": r["launches"] * args.steps, "clocks": r["clocks"], "roofline": r["roofline"]}

    main_line = model_line(args.workload)
    line = {"metric": main_line["metric"], "value": main_line["value"], "unit": "images/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": main_line["ms_per_step"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": main_line["config"], "e2e": main_line["e2e"], "gpu_launches": main_line["gpu_launches"],
            "clocks": main_line["clocks"], "roofline": main_line["roofline"]}
    if args.workload == "vit_b16":
        # DRAM bytes of one launch of the dominant kernel, from an ncu capture at the real launch shape
        # (profiles/lut_dense_tc_kernel_m25216_k768_n3072_w3.md): fc1, 43.6 MB read + 102.9 MB written
        line["roofline"]["traffic"] = 146.4e6
        line["roofline"]["traffic_source"] = ("ncu capture of the fc1 launch (M=25216, K=768, N=3072), one of the four "
                                              "shapes of the step; algorithmic bytes of that launch 198.3 MB")
    else:
        line["roofline"]["traffic"] = None
    if results[args.workload]["cpu"] is not None:
        line["cpu_baseline"] = results[args.workload]["cpu"]
    if other in results:
        sec = model_line(other)
        line["secondary"] = {k: sec[k] for k in ("metric", "value", "unit", "ms_per_step", "config", "e2e",
                                                  "gpu_launches", "roofline")}
    if w4a4 is not None:
        line["w4a4"] = w4a4
    if strong is not None:
        for name, s in strong.items():
            # one GPU's time for the whole batch = the weak pass's step (the same batch per GPU)
            one_gpu_ms = results[name]["ms_res"] / args.steps
            s["efficiency_vs_1gpu"] = one_gpu_ms / world / s["ms_per_step"]
            s["efficiency_basis"] = "ms per step of the weak pass (whole batch on one GPU) / N / ms per step here"
            s["note"] = ("fixed global batch split over the GPUs; per-GPU tiles shrink, so tile quantisation and "
                         "per-launch fixed cost bound it, not NCCL")
        line["strong"] = strong
    if micro is not None:
        line["micro"] = micro
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
