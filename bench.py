"""Benchmark of the W8A8 Hadamard-linear path: the linears of one Z-Image-Turbo-shaped DiT block (M = 4608 tokens,
hidden 3840: QKV 3840->11520, out 3840->3840, w1|w3 3840->20480, w2 10240->3840 fed by value*silu(gate)), each
as rotate+quantise followed by the int8 product with bias. One "step" is one pass over the four linears
(8 kernel launches) on synthetic, seeded data.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config 1]

With N > 1 (one process per GPU under torch.distributed.run) every rank runs the block on its own M tokens
(token sharding: the path is row-independent, no collective is needed), and `value` is the total over ranks
divided by the slowest rank's time. Rank 0 prints ONE JSON line.

`--impl reference` times the reference's CPU (NumPy) arithmetic of the same path on the host cores, on a bounded
row sample of the same workload.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "dit_block_w8a8_linears_tokens_per_s"
UNIT = "tokens/s"
NOMINAL_INT8_TOPS = 4500.0  # B200 dense int8, datasheet


def measured_peaks():
    """HBM GB/s and int8 TOPS ceilings for the roofline: the pool's measured copy bandwidth and twice its measured
    dense bf16 rate (int8 runs on the same tensor pipe at twice the bf16 rate), else the documented fallback."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            p = json.load(fh)
        return {"hbm_gbs": float(p["hbm_gbs"]), "int8_tops": 2.0 * float(p["bf16_tflops_sustained"]),
                "source": "measured (MEASURED_PEAKS.json: hbm_gbs; 2 x bf16_tflops_sustained)"}
    except Exception:
        return {"hbm_gbs": 6650.0, "int8_tops": 2.0 * 1400.0, "source": "fallback (6.65 TB/s; 2 x 1.4 PFLOP/s sustained)"}


# DRAM traffic per launch of the dominant kernel (dram__bytes_read.sum + dram__bytes_write.sum from the ncu capture
# summarised under profiles/), keyed by workload; None until a capture exists for it.
NCU_TRAFFIC_BYTES = {
    # profiles/gemm_w8a8_config1_ncu.md: 538.8 MB over the step's four product launches
    "config 1": 134.7e6,
}


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None
        self.t_from = self.t_to = None  # host-time window whose samples count (the GPU is under load in it)

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "50"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def __exit__(self, *exc):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.thread.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], [], set()
        for stamp, r in self.rows:
            if len(r) < 7 or (self.t_from is not None and not (self.t_from <= stamp <= self.t_to)):
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons),
                "samples": len(sm)}


# ---- CPU arm: the reference's NumPy arithmetic of the path -------------------------------------------------------------
class CpuBlock:
    """Rotation as x.reshape(M, K/B, B) @ H in fp32, absmax int8 quantisation, product in float64 BLAS with the
    scales and bias applied as the reference's tests write it (tests/test_gemm.py:31, tests/test_ops.py:15-18),
    bf16 store. Weights are prepared (and widened to float64) once, outside the timed steps."""

    def __init__(self, cfg, rows: int, seed: int = 0):
        from oracle import quant_ref
        self.q = quant_ref
        self.cfg, self.rows = cfg, rows
        rng = np.random.default_rng(seed)
        self.layers = []
        for spec in cfg.layers:
            w = rng.integers(-127, 128, size=(spec.N, spec.K), dtype=np.int8)  # stands in for quantised weights
            sw = rng.uniform(1e-4, 2e-4, size=spec.N).astype(np.float32)
            bias = (rng.standard_normal(spec.N) * 0.01).astype(np.float32)
            x = None
            if not spec.swiglu_in:
                x = quant_ref.bf16_round_bits(rng.standard_normal((rows, spec.K)).astype(np.float32))
            self.layers.append((spec, np.ascontiguousarray(w.T.astype(np.float64)), sw, bias, x))

    def step(self):
        q = self.q
        prev = None
        for spec, wT, sw, bias, x in self.layers:
            if spec.swiglu_in:
                h = q.bf16_bits_to_f32(prev)
                g = h[:, spec.K:]
                xf = h[:, :spec.K] * (g / (1.0 + np.exp(-g)))
            else:
                xf = q.bf16_bits_to_f32(x)
            r = q.rotate_in(xf, None, self.cfg.block)
            amax = np.abs(r).max(axis=1)
            s = np.where(amax > 0, amax / np.float32(127), np.float32(1)).astype(np.float32)
            codes = np.rint(r * (np.float32(1) / s)[:, None])
            y = (codes.astype(np.float64) @ wT) * s[:, None] * sw[None, :] + bias[None, :]
            prev = q.bf16_round_bits(y.astype(np.float32))
        return prev


def use_all_host_threads() -> int:
    """BLAS on every host core (a launcher such as torch.distributed.run pins OMP_NUM_THREADS to 1)."""
    n = os.cpu_count() or 1
    try:
        from threadpoolctl import threadpool_limits
        threadpool_limits(limits=n)
    except Exception:
        pass
    return n


def time_cpu(cfg, rows: int, steps: int, warmup: int):
    use_all_host_threads()
    blk = CpuBlock(cfg, rows)
    for _ in range(warmup):
        blk.step()
    t0 = time.perf_counter()
    for _ in range(steps):
        blk.step()
    dt = (time.perf_counter() - t0) / max(steps, 1)
    return rows / dt, dt


def host_threads() -> int:
    try:
        from threadpoolctl import threadpool_info
        n = [p.get("num_threads", 0) for p in threadpool_info() if p.get("user_api") == "blas"]
        if n:
            return int(max(n))
    except Exception:
        pass
    return os.cpu_count() or 1


# ---- arms ---------------------------------------------------------------------------------------------------------
def run_reference(args, cfg, rank, world):
    if rank != 0:
        return None
    rows = args.cpu_rows or 512
    value, dt = time_cpu(cfg, rows, args.steps, args.warmup)
    cores = host_threads()
    sample = (f"{rows} of {cfg.M} rows of every linear of the block per step, NumPy fp32 rotation matmul + absmax int8 + "
              f"float64 BLAS product + bias + bf16 store, weights widened once outside the timed steps")
    return {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": workload_name(cfg), "block": cfg.block, "rows_per_step": rows},
        "tops": value * cfg.ops / cfg.M / 1e12,
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


def workload_name(cfg) -> str:
    from h3metal_b200 import workloads
    number = next(k for k, v in workloads.CONFIGS.items() if v is cfg)
    return f"config {number}: {cfg.name}, M={cfg.M}, " + ", ".join(f"{l.name} {l.K}->{l.N}" for l in cfg.layers)


def run_ours(args, cfg, rank, world):
    import torch
    import torch.distributed as dist
    from h3metal_b200.gpu import Gpu
    from h3metal_b200 import ops as ops_mod
    from h3metal_b200.linear import BlockLinears

    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    gpu = Gpu(device=local)
    if args.overlap:
        gpu.set_launch_overlap(True)
    dev = gpu.torch_device
    if args.parallel == "tp":
        return run_tensor_parallel(args, cfg, rank, world, gpu)
    blk = BlockLinears(gpu, cfg, seed=1234 + rank)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def timed(fn, steps):
        """K calls of fn between two events on the launching stream; returns milliseconds (max over ranks)."""
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        start.record(gpu.stream)
        for _ in range(steps):
            fn()
        end.record(gpu.stream)
        torch.cuda.synchronize(dev)
        ms = torch.tensor([start.elapsed_time(end)], device=dev, dtype=torch.float64)
        barrier()
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    # ---- device-resident throughput: inputs already in HBM --------------------------------------------------------
    for _ in range(max(args.warmup, 3)):
        blk.step()
    with ClockSampler(local) as clocks:
        launches0 = gpu.launch_count
        t_load = time.time()
        ms = timed(blk.step, args.steps)
        launches = gpu.launch_count - launches0
        # The timed region lasts milliseconds, shorter than one nvidia-smi sample. Keep the same steps running back
        # to back for about a second more so that the clock record is of this load; only samples taken from the
        # start of the timed region to the end of this window count.
        extra_steps = 0
        while time.time() - t_load < 1.2:
            for _ in range(args.steps):
                blk.step()
            extra_steps += args.steps
            torch.cuda.synchronize(dev)
        clocks.t_from, clocks.t_to = t_load, time.time()
        time.sleep(0.15)  # let the sampler's last line arrive
    gpu.wait()
    tokens = cfg.M * world * args.steps
    value = tokens / (ms * 1e-3)

    # ---- per-kernel durations for the roofline: the step's product launches alone, then its rotate+quantise launches
    # alone, each group K times back to back between one event pair (an event pair per launch would put the launch gaps
    # of 15-microsecond kernels into the figure). With a LoRA term the group also holds the narrow T products.
    peaks = measured_peaks()
    gemm_ops = rot_bytes = 0
    blk.step()
    gemm_s = timed(blk.gemm_only, args.steps) * 1e-3
    rot_s = timed(blk.rot_only, args.steps) * 1e-3
    for l in blk.layers:
        gemm_ops += 2 * l.m_pad * l.wt.K * l.wt.N * args.steps
        rot_bytes += blk.M * ((4 if l.swiglu_in else 2) * l.wt.K + l.wt.K + 4) * args.steps
    achieved_tops = gemm_ops / gemm_s / 1e12
    rot_gbs = rot_bytes / rot_s / 1e9
    wl = workload_name(cfg)
    roofline = {"bound": "tensor", "kernel": "gemm_w8a8_kernel (tcgen05 kind::i8)", "achieved": achieved_tops,
                "peak": peaks["int8_tops"], "unit": "TOP/s", "frac": achieved_tops / peaks["int8_tops"],
                "traffic": NCU_TRAFFIC_BYTES.get(wl.split(":")[0]),
                "algorithmic_bytes": sum(l.m_pad * l.wt.K + l.wt.N * l.wt.K + 2 * l.m_pad * l.wt.N for l in blk.layers) / len(blk.layers),
                "peak_source": peaks["source"],
                "frac_of_nominal_4500": achieved_tops / NOMINAL_INT8_TOPS,
                "time_share": gemm_s / (gemm_s + rot_s)}
    roofline_rot = {"bound": "hbm", "kernel": "rot_q8_tma_kernel (TMA-fed rotate + quantise)", "achieved": rot_gbs, "peak": peaks["hbm_gbs"],
                    "unit": "GB/s", "frac": rot_gbs / peaks["hbm_gbs"], "traffic": None,
                    "time_share": rot_s / (gemm_s + rot_s)}

    # ---- end to end through the public API with HOST buffers: H2D of every input, D2H of every output ---------------
    e2e = None
    if not args.no_e2e:
        host_in, host_out = blk.host_buffers()
        for h, x in zip(host_in, blk.inputs):
            if h is not None:
                h.copy_(x.torch().cpu())
        h2d = sum(h.numel() * 2 for h in host_in if h is not None)
        d2h = sum(h.numel() * 2 for h in host_out if h is not None)

        def e2e_step():
            blk.step_host(host_in, host_out)

        def timed_e2e(steps):
            """Like timed(), but the region ends when the LAST download has landed in host memory."""
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            blk.sync_host()
            barrier()
            start.record(gpu.stream)
            for _ in range(steps):
                e2e_step()
            blk._down.wait_stream(blk._up)
            gpu.stream.wait_stream(blk._down)
            end.record(gpu.stream)
            blk.sync_host()
            ms = torch.tensor([start.elapsed_time(end)], device=dev, dtype=torch.float64)
            barrier()
            if world > 1:
                dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            return float(ms.item())

        for _ in range(2):
            e2e_step()
        e2e_ms = timed_e2e(args.steps)
        e2e_value = tokens / (e2e_ms * 1e-3)
        e2e = {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "ms_per_step": e2e_ms / args.steps}

    # ---- the other producer of int8 activations, norm_mod_q8, at the block's hidden size (not part of the step) ----
    hidden = blk.layers[0].wt.K
    xres = torch.randn(blk.layers[0].m_pad, hidden, device=dev) * 3
    modt = torch.randn(3, 2, hidden, device=dev)
    rtt = torch.randint(0, 3, (blk.layers[0].m_pad,), device=dev, dtype=torch.uint8)
    X32, MODT, RTT = gpu.wrap(xres), gpu.wrap(modt), gpu.wrap(rtt)
    l0 = blk.layers[0]

    def norm_step():
        ops_mod.norm_mod_q8(gpu, X32, MODT, RTT, l0.a8, l0.sa, blk.M, hidden, eps=1e-5, block=cfg.block)

    for _ in range(3):
        norm_step()
    norm_ms = timed(norm_step, args.steps) / args.steps
    norm_bytes = blk.M * (4 * hidden + hidden + 4)
    norm_extra = {"kernel": "rot_q8_tma_kernel with the norm + modulation front end", "rows": blk.M, "channels": hidden, "us": norm_ms * 1e3,
                  "achieved_gbs": norm_bytes / (norm_ms * 1e-3) / 1e9, "frac_of_measured_hbm": norm_bytes / (norm_ms * 1e-3) / 1e9 / peaks["hbm_gbs"]}

    if world > 1:
        dist.barrier()
    if rank != 0:
        return None
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8", "data": "synthetic",
        "config": {"workload": wl, "block": cfg.block, "parallelism": f"token-sharded x{world} (no collective)",
                   "l2": f"per-step working set ({sum(l.wt.N * l.wt.K for l in blk.layers) / 1e6:.0f} MB of int8 weights plus "
                         f"{sum(2 * l.m_pad * (l.wt.K + l.wt.N) for l in blk.layers) / 1e9:.2f} GB of activations and outputs) "
                         f"exceeds the 126 MB L2"},
        "tops": value / cfg.M * cfg.ops / 1e12 ,
        "roofline": roofline, "roofline_rot_q8": roofline_rot, "norm_mod_q8": norm_extra,
        "e2e": e2e,
        "gpu_launches": int(launches),
        "clocks": dict(clocks.summary(), window=f"timed region + {extra_steps} identical steps run straight after it"),
    }
    if world == 1 and not args.no_cpu:
        rows = args.cpu_rows or 1024
        cpu_value, cpu_dt = time_cpu(cfg, rows, 2, 1)
        line["cpu_baseline"] = {
            "value": cpu_value, "unit": UNIT, "cores": host_threads(), "kind": "port",
            "sample": f"{rows} of {cfg.M} rows of every linear per step, 2 timed steps after 1 warm-up: the reference's NumPy "
                      f"arithmetic (fp32 rotation matmul, absmax int8, float64 BLAS product, bias, bf16 store)"}
    return line


def run_tensor_parallel(args, cfg, rank, world, gpu):
    """One block of cfg.M tokens over all ranks: QKV and w1|w3 column-parallel, out and w2 row-parallel with a MAX
    all-reduce of the row maxima and a SUM all-reduce of the partial products. Strong scaling; device-resident."""
    import torch
    import torch.distributed as dist
    from h3metal_b200.parallel import TensorParallelBlock
    if world == 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29531")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=gpu.torch_device)
    blk = TensorParallelBlock(gpu, None, cfg, seed=99, reduce=args.reduce, scatter=args.scatter)
    dev = gpu.torch_device
    for _ in range(max(args.warmup, 3)):
        blk.step()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dist.barrier()
    torch.cuda.synchronize(dev)
    start.record(gpu.stream)
    for _ in range(args.steps):
        blk.step()
    end.record(gpu.stream)
    torch.cuda.synchronize(dev)
    ms = torch.tensor([start.elapsed_time(end)], device=dev, dtype=torch.float64)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    # where the step's time goes: one event pair per layer (its rotate+quantise, product and communication), max over ranks
    n_layers = len(blk.layers)
    marks = [[torch.cuda.Event(enable_timing=True) for _ in range(n_layers + 1)] for _ in range(args.steps)]
    dist.barrier()
    torch.cuda.synchronize(dev)
    for s in range(args.steps):
        prev = None
        for i, (layer, x) in enumerate(zip(blk.layers, blk.inputs)):
            marks[s][i].record(gpu.stream)
            prev = layer(prev if x is None else x)
        marks[s][n_layers].record(gpu.stream)
    torch.cuda.synchronize(dev)
    per_layer = torch.tensor([sum(marks[s][i].elapsed_time(marks[s][i + 1]) for s in range(args.steps)) / args.steps
                              for i in range(n_layers)], device=dev, dtype=torch.float64)
    dist.all_reduce(per_layer, op=dist.ReduceOp.MAX)
    gpu.wait()
    if rank != 0:
        return None
    ms = float(ms.item())
    value = cfg.M * args.steps / (ms * 1e-3)
    return {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "int8", "data": "synthetic",
            "config": {"workload": workload_name(cfg), "block": cfg.block,
                       "parallelism": f"tp{world}: column-parallel qkv/w1w3, row-parallel out/w2 ({args.reduce} {'reduce-scatter' if args.scatter else 'all-reduce'})"},
            "tops": value / cfg.M * cfg.ops / 1e12,
            "layer_ms": {f"{spec.K}->{spec.N} ({spec.parallel})": round(float(t), 4)
                         for spec, t in zip(cfg.layers, per_layer.tolist())},
            "gpu_launches": None}


def library_int8_probe():
    """Yardstick, not part of the path: what the vendor library's int8 GEMM (cuBLASLt through torch._int_mm, int32
    output, no epilogue) and its bf16 GEMM reach on this GPU under the same power cap, for cubes of three sizes.
    Prints one JSON line."""
    import torch
    out = {"probe": "library int8 / bf16 GEMM", "results": []}
    for n in (4096, 8192, 16384):
        a = torch.randint(-127, 128, (n, n), device="cuda", dtype=torch.int8)
        b = torch.randint(-127, 128, (n, n), device="cuda", dtype=torch.int8).t()
        x = torch.randn(n, n, device="cuda", dtype=torch.bfloat16)
        y = torch.randn(n, n, device="cuda", dtype=torch.bfloat16)
        reps = 20 if n < 16384 else 8
        row = {"n": n}
        for name, fn in (("int8_tops", lambda: torch._int_mm(a, b)), ("bf16_tflops", lambda: x @ y)):
            for _ in range(3):
                fn()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            for _ in range(reps):
                fn()
            end.record()
            torch.cuda.synchronize()
            row[name] = 2 * n ** 3 / (start.elapsed_time(end) / reps * 1e-3) / 1e12
        out["results"].append(row)
    print(json.dumps(out), flush=True)


def whole_block(args):
    """Not the headline: one Z-Image-shaped block END TO END on one GPU (both quantising kernels with their norm
    front end, the four int8 products, the fused residual update, and attention + q/k norm + rotary from PyTorch),
    to show what share of a block the path is. Prints one JSON line."""
    import torch
    from h3metal_b200.gpu import Gpu
    from h3metal_b200.zimage_block import ZImageBlock
    gpu = Gpu(device=0)
    M = 4608
    blk = ZImageBlock(gpu, M, 3840, 30, 10240, block=128, seed=0)
    x = gpu.wrap(torch.randn(blk.m_pad, 3840, device=gpu.torch_device))
    pending = None
    for _ in range(3):
        pending = blk.forward(x, pending)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record(gpu.stream)
    for _ in range(args.steps):
        pending = blk.forward(x, pending)
    end.record(gpu.stream)
    torch.cuda.synchronize()
    ms = start.elapsed_time(end) / args.steps
    gpu.profile(True)
    blk.forward(x, pending)
    path_s = sum(s for _, s in gpu.profile_take())
    gpu.profile(False)
    print(json.dumps({"workload": "one Z-Image-Turbo-shaped block, M=4608, attention by PyTorch SDPA", "ms_per_block": ms,
                      "tokens_per_s": M / (ms * 1e-3), "path_kernels_ms": path_s * 1e3,
                      "path_share": path_s * 1e3 / ms}), flush=True)


def sweep(args):
    """Not the headline: the stress sweep of config 4 on one GPU. M = 66560 rows; for K in 3072 / 6144 / 16384 the
    rotate+quantise kernel at rotation blocks 64 / 128 / 256 (GB/s of algorithmic bytes, inputs of 0.4-2.2 GB, far
    larger than L2) and the K -> 6144 product (TOP/s). Device timing with CUDA events after warm-up; one JSON line."""
    import torch
    from h3metal_b200 import ops, workloads
    from h3metal_b200.gpu import Gpu
    gpu = Gpu(device=0)
    dev = gpu.torch_device
    peaks = measured_peaks()
    M, N = 66560, 6144

    def timed(fn, n):
        for _ in range(3):
            fn()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(dev)
        start.record(gpu.stream)
        for _ in range(n):
            fn()
        end.record(gpu.stream)
        torch.cuda.synchronize(dev)
        return start.elapsed_time(end) * 1e-3 / n

    gen = torch.Generator(device=dev)
    gen.manual_seed(4)
    rows = []
    for K in (3072, 6144, 16384):
        x = gpu.wrap(workloads.activations_torch(gen, M, K, round(0.002 * K), dev))
        a8, sa = gpu.empty((M, K), "i8"), gpu.empty((M,), "f32")
        for block in (64, 128, 256):
            t = timed(lambda: ops.rot_q8(gpu, x, a8, sa, M, K, block=block), 10)
            gbs = M * (3 * K + 4) / t / 1e9
            rows.append({"kernel": "rot_q8", "K": K, "block": block, "us": t * 1e6, "GB/s": gbs,
                         "frac_of_measured_hbm": gbs / peaks["hbm_gbs"]})
        codes, scales = workloads.weight_torch(gen, N, K, dev)
        wt = ops.QWeight("q8", gpu.wrap(codes), gpu.wrap(scales), N, K)
        out = gpu.empty((M, N), "bf16")
        t = timed(lambda: ops.gemm(gpu, a8, wt, out, M, sa=sa, tile=(128, 32, 4)), 5)
        tops = 2.0 * M * N * K / t / 1e12
        rows.append({"kernel": "gemm_w8a8", "K": K, "N": N, "us": t * 1e6, "TOP/s": tops,
                     "frac_of_measured_int8": tops / peaks["int8_tops"], "frac_of_nominal_4500": tops / NOMINAL_INT8_TOPS})
        del x, a8, out, wt, codes
        torch.cuda.empty_cache()
    gpu.wait()
    print(json.dumps({"workload": f"config 4 sweep: M={M}, K in 3072/6144/16384, N={N}, rotation blocks 64/128/256",
                      "peak_source": peaks["source"], "rows": rows}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", type=int, default=1)
    ap.add_argument("--cpu-rows", type=int, default=0, help="rows of the CPU sample (0 = default)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (it pins GBs of host memory on the largest configs)")
    ap.add_argument("--parallel", default="token", choices=["token", "tp"],
                    help="N > 1: token = every rank its own M tokens (default, weak scaling); tp = ONE block of M tokens "
                         "sharded column-/row-parallel over the ranks with NCCL all-reduces (strong scaling)")
    ap.add_argument("--reduce", default="int32", choices=["int32", "f32", "bf16", "push", "push_bf16"],
                    help="tp: what the row-parallel layers reduce (int32 = bit-exact, NCCL; push = bit-exact, partial "
                         "accumulators stored by the product kernel straight into the row owners' memory over NVLink; "
                         "push_bf16 = the same with bf16 partials)")
    ap.add_argument("--scatter", action="store_true",
                    help="tp: reduce-scatter instead of all-reduce (every rank finishes its M / N_gpus rows)")
    ap.add_argument("--overlap", action="store_true",
                    help="launch the kernels with programmatic dependent launch (off by default: slower on this block)")
    ap.add_argument("--library-int8-probe", action="store_true",
                    help="time the vendor library's int8 and bf16 GEMMs on this GPU (a yardstick; runs nothing of the path)")
    ap.add_argument("--sweep", action="store_true",
                    help="the K x rotation-block stress sweep of config 4 (M = 66560) instead of the block step")
    ap.add_argument("--whole-block", action="store_true",
                    help="time one whole Z-Image-shaped block with PyTorch attention (context for the path's share)")
    args = ap.parse_args()
    if args.library_int8_probe:
        library_int8_probe()
        return
    if args.whole_block:
        whole_block(args)
        return
    if args.sweep:
        sweep(args)
        return

    from h3metal_b200 import workloads
    cfg = workloads.CONFIGS[args.config]
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))

    if args.impl == "reference":
        line = run_reference(args, cfg, rank, world)
        if line is not None:
            print(json.dumps(line), flush=True)
        return

    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
        dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0))))
    try:
        line = run_ours(args, cfg, rank, world)
        if line is not None:
            print(json.dumps(line), flush=True)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
