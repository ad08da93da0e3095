"""Throughput of the DIMQ quantised-inference hot path on B200.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

One step = one forward of the synthetic DIMQ ViT-B/16 (12 layers, hidden 768, 197 tokens;
every qkv / proj / fc1 / fc2 / head Linear stored as 3-bit indices with one 8-entry codebook
per 128 output rows) over a batch of 128 images per GPU, bf16 activations.  All quantised
Linears run through ``libdimq_b200.so`` (weight-only LUT GEMM); attention, LayerNorm and the
patch embedding are dense bf16 PyTorch ops.  Rank 0 prints one JSON line.

``value``  — images/s with the images already in HBM (CUDA-graph replay, CUDA events).
``e2e``    — the same forward called with pinned HOST images: H2D copy + forward + D2H of the
             logits inside the timed region.
``roofline`` — the LUT-GEMM kernel: algorithmic flops of the quantised Linears divided by the
             summed CUDA-event duration of exactly those launches (an instrumented eager pass).
``cpu_baseline`` / ``--impl reference`` — the reference's CPU path (dequantise + fp32
             ``F.linear``, PyTorch CPU, all host threads) on a bounded sample of the same workload.
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


NCU_DRAM_BYTES_PER_FLOP = 16.45e6 / 38.65e9


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
    index_bytes = n * k * bits // 8
    copies = int(parts[5]) if len(parts) > 5 else max(1, min(64, (192 << 20) // max(index_bytes, 1) + 1))
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    x = torch.randn(m, k, device=dev, dtype=torch.bfloat16)
    packed = [torch.randint(0, 256, (index_bytes,), dtype=torch.uint8, device=dev) for _ in range(copies)]
    groups = n // 128 if bits == 3 and n % 128 == 0 else 1
    cb = (torch.randn(groups, 1 << bits, device=dev) * 0.02).sort(dim=1).values.to(torch.bfloat16)
    kw = dict(bits=bits, group_rows=128 if groups > 1 else None, out_dtype=torch.bfloat16, algo=algo)
    call = lambda pw: ops.dimq_linear_wq(x, pw, cb, None, n, k, **kw)
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
        "config": {"workload": f"lut_gemm_m{m}_k{k}_n{n}_w{bits}", "algo": algo or "auto", "weight_copies": copies,
                   "l2": "weights rotated over more than 126 MB" if copies * index_bytes > (126 << 20) else "weights fit L2"},
        "tflops": 2.0 * m * n * k / us / 1e6, "tflops_frac": 2.0 * m * n * k / us / 1e6 / tc_peak,
        "index_gbs": index_bytes / us / 1e3, "index_gbs_frac": index_bytes / us / 1e3 / hbm_peak,
        "peak_source": peak_kind, "dtype": "bf16", "data": "synthetic",
    }), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--workload", default="vit_b16", choices=["vit_b16", "resnet18"],
                    help="vit_b16 is the headline line; resnet18 prints the same line for the ResNet-18 config")
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

    from dimq_b200 import _lib, ops
    from dimq_b200.dist import gather_logits
    from dimq_b200.workloads import DIMQResNet18, DIMQViT, build_resnet18_checkpoint, build_vit_b16_checkpoint

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

    WORKLOAD, B, weight_desc = WORKLOADS[args.workload]
    with torch.no_grad():
        if args.workload == "vit_b16":
            ckpt = build_vit_b16_checkpoint(seed=0, device=dev)
            model = DIMQViT(ckpt).to(dev).eval()
            flops_per_step = model.lut_gemm_flops(B)
        else:
            ckpt = build_resnet18_checkpoint(seed=0, device=dev)
            model = DIMQResNet18(ckpt).to(dev).eval()
            flops_per_step = model.lut_flops(B)
        n_bufs = 4  # rotating image buffers (4 x 38.5 MB or more): larger than the 126 MB L2
        gen = torch.Generator(device="cpu").manual_seed(1234 + rank)
        host_images = [torch.randn(B, 3, 224, 224, generator=gen).to(torch.bfloat16).pin_memory() for _ in range(n_bufs)]
        dev_images = [h.to(dev, non_blocking=True) for h in host_images]
        torch.cuda.synchronize()

        # ---- CUDA graphs: one per resident input buffer, plus one reading a staging buffer (e2e) ----
        stream = torch.cuda.Stream(device=dev)
        # two staging buffers: the host->device copy of step i + 1 runs on its own stream under step i
        staging = [torch.empty_like(dev_images[0]) for _ in range(2)]
        copy_stream = torch.cuda.Stream(device=dev)
        h2d_done = [torch.cuda.Event() for _ in range(2)]
        compute_done = [torch.cuda.Event() for _ in range(2)]
        host_logits = torch.empty(B, 1000, dtype=torch.float32).pin_memory()
        graphs, outs = [], []
        with torch.cuda.stream(stream):
            for _ in range(2):
                model(dev_images[0])
            stream.synchronize()
            launches_before = _lib.LAUNCH_COUNT[0]
            for src in dev_images + staging:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    out = model(src)
                graphs.append(g)
                outs.append(out)
            launches_per_forward = (_lib.LAUNCH_COUNT[0] - launches_before) // len(graphs)

        def barrier():
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        def step_resident(i: int) -> None:
            graphs[i % n_bufs].replay()
            if world > 1:
                gather_logits(outs[i % n_bufs])

        def step_e2e(i: int) -> None:
            b = i % 2
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(compute_done[b])  # the forward that last read this buffer
                staging[b].copy_(host_images[i % n_bufs], non_blocking=True)
                h2d_done[b].record(copy_stream)
            stream.wait_event(h2d_done[b])
            graphs[n_bufs + b].replay()
            if world > 1:
                gather_logits(outs[n_bufs + b])
            host_logits.copy_(outs[n_bufs + b], non_blocking=True)
            compute_done[b].record(stream)

        def run_timed(step_fn) -> float:
            with torch.cuda.stream(stream):
                for i in range(args.warmup):
                    step_fn(i)
                copy_stream.synchronize()
                barrier()
                start = torch.cuda.Event(enable_timing=True)
                end = torch.cuda.Event(enable_timing=True)
                start.record(stream)
                copy_stream.wait_event(start)  # no copy of a timed step starts before the timed region
                for i in range(args.steps):
                    step_fn(i)
                end.record(stream)
                barrier()
                ms = torch.tensor([start.elapsed_time(end)], device=dev)
            if world > 1:
                dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            return float(ms.item())

        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        ms_resident = run_timed(step_resident)
        clocks = sampler.stop() if rank == 0 else None
        ms_e2e = run_timed(step_e2e)

        # ---- roofline of the dominant kernel: eager pass with events around every LUT-GEMM launch ----
        events = []
        orig, orig_conv = ops.dimq_linear_wq, ops.dimq_conv2d_wq

        def timed(fn):
            def wrapper(*a, **kw):
                s = torch.cuda.Event(enable_timing=True)
                e = torch.cuda.Event(enable_timing=True)
                s.record(torch.cuda.current_stream())
                y = fn(*a, **kw)
                e.record(torch.cuda.current_stream())
                events.append((s, e))
                return y
            return wrapper

        roof_steps = 3
        from dimq_b200 import modules as _modules
        _modules.ops.dimq_linear_wq = timed(orig)
        _modules.ops.dimq_conv2d_wq = timed(orig_conv)
        try:
            with torch.cuda.stream(stream):
                for i in range(roof_steps):
                    # keep the GPU busy while the host queues the step, so that the event pairs
                    # bracket kernel execution and not launch gaps
                    torch.cuda._sleep(int(60e6))
                    model(dev_images[i % n_bufs])
                stream.synchronize()
        finally:
            _modules.ops.dimq_linear_wq = orig
            _modules.ops.dimq_conv2d_wq = orig_conv
        gemm_ms = sum(s.elapsed_time(e) for s, e in events)
        gemm_launches = len(events)

    if world > 1:
        dist.barrier()
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    images_total = world * B * args.steps
    value = images_total / (ms_resident / 1e3)
    e2e_value = images_total / (ms_e2e / 1e3)
    peak, peak_kind = _peaks()
    flops = flops_per_step * roof_steps
    achieved = flops / (gemm_ms / 1e3) / 1e12
    line = {
        "metric": f"{args.workload}_dimq_images_per_s", "value": value, "unit": "images/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_resident / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "global_batch": world * B, "weights": weight_desc,
                   "l2": f"{n_bufs} rotating image buffers and >126 MB of activations per step",
                   "parallelism": f"dp{world} (batch-sharded replicas, all-gather of logits)"},
        "e2e": {"value": e2e_value, "unit": "images/s", "ms_per_step": ms_e2e / args.steps,
                "h2d_bytes_per_step": world * B * 3 * 224 * 224 * 2, "d2h_bytes_per_step": world * B * 1000 * 4},
        "gpu_launches": launches_per_forward * args.steps,
        "clocks": clocks,
        "roofline": {"kernel": "linear_wq_tc_kernel (tcgen05 LUT GEMM / implicit-GEMM conv)", "bound": "tensor", "achieved": achieved,
                     "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak, "peak_source": peak_kind,
                     "launches_timed": gemm_launches, "avg_launch_ms": gemm_ms / max(gemm_launches, 1),
                     "flops_per_step": flops / roof_steps,
                     # DRAM bytes per launch: the ncu capture of the M = 8192 fc1 case (16.45 MB for 38.65 GFLOP,
                     # profiles/linear_wq_tc_kernel_m8192_k768_n3072_w3.md) scaled by the flops of an average launch
                     "traffic": NCU_DRAM_BYTES_PER_FLOP * flops / max(gemm_launches, 1),
                     "traffic_source": "ncu capture of a smaller launch, scaled by flops"},
    }
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(ckpt, args.workload)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
