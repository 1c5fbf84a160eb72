"""Benchmark of the W8A8 Hadamard-linear path on the linears of one DiT block: each linear is rotate+quantise followed
by the int8 product with its epilogue. One "step" is one pass over the block's four linears on synthetic, seeded data.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config 0..5] [--sweep]

Default workload: the 33B-class block (M = 17408 tokens, hidden 6144: QKV 6144->18432, out 6144->6144,
w1|w3 6144->32768, w2 16384->6144 fed by value*silu(gate)).
  N = 1   the block on one GPU.
  N > 1   (one process per GPU under torch.distributed.run) ONE block of the same M tokens over all ranks: QKV and
          w1|w3 column-parallel, out and w2 row-parallel with the exact int32 reduction pushed over NVLink by the
          product kernel itself (strong scaling). Before anything is timed every rank checks a small sharded chain
          against its own one-GPU result, bit for bit; a mismatch aborts the run.
A second object of the same line carries the largest configuration (M = 66560, rank-64 LoRA on every linear)
token-sharded at fixed M: every rank runs the whole block on M / N rows, no exchange.
The timed region is repeated: R windows of exactly K steps each, every window between a barrier + synchronize on both
sides and timed with CUDA events on the launching stream (max over ranks); `ms_per_step` is the median window.
Rank 0 prints ONE JSON line.

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
WINDOW_SECONDS = 1.0        # the repeated windows of the headline cover at least this much GPU time
PEER_COPY_GBS = 770.0       # measured peer copy on this pool, per direction and GPU (nominal NVLink 5: 900)

# DRAM traffic per launch of the dominant kernel: dram__bytes_read.sum + dram__bytes_write.sum of an ncu capture of this
# benchmark's own step (ncu --metrics dram__bytes_read.sum,dram__bytes_write.sum,gpu__time_duration.sum
# --clock-control none -k regex:gemm_w8a8 -s 12 -c 4 python bench.py --config C --no-cpu --no-e2e --no-probe
# --no-config4 --steps 2 --warmup 3), averaged over the step's four product launches, keyed by config number. Such a
# figure can only come from a profiler run, so it is recorded here; configs without a capture print null.
NCU_TRAFFIC_BYTES = {
    1: 139.9e6,   # 559.6 MB over the four launches (algorithmic 642.9 MB: part of the codes and outputs stays in L2)
    3: 1790.4e6,  # 7161.6 MB over the four launches (algorithmic 3269.5 MB: W is re-read once per 32 MB band of A rows)
}


def hbm_peak():
    """HBM GB/s ceiling: the pool's measured copy bandwidth, else the documented fallback."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
            p = json.load(fh)
        return float(p["hbm_gbs"]), "measured (MEASURED_PEAKS.json: hbm_gbs)", p
    except Exception:
        return 6650.0, "fallback (6.65 TB/s)", {}


class ClockSampler:
    """Samples SM clock, power and throttle reasons of one GPU with nvidia-smi while timed regions run."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

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

    def summary(self, t_from=None, t_to=None):
        """Median SM clock, largest power and the throttle reasons seen between two host times (all samples if None)."""
        sm, mx, power, reasons = [], [], [], set()
        for stamp, r in list(self.rows):
            if len(r) < 7 or (t_from is not None and not (t_from <= stamp <= t_to)):
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
                power.append(float(r[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "power_w": None, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "power_w": float(np.median(power)),
                "reasons": sorted(reasons), "samples": len(sm)}


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


def config_number(cfg) -> int:
    from h3metal_b200 import workloads
    return next(k for k, v in workloads.CONFIGS.items() if v is cfg)


def workload_name(cfg) -> str:
    return (f"config {config_number(cfg)}: {cfg.name}, M={cfg.M}, " + ", ".join(f"{l.name} {l.K}->{l.N}" for l in cfg.layers)
            + (f", rank-{cfg.lora_rank} LoRA on every linear" if cfg.lora_rank else ""))


def config_dict(cfg, world: int) -> dict:
    """The line's `config`: what is measured, identical for both arms at a given number of GPUs."""
    if world == 1:
        how = "one GPU"
    elif cfg.lora_rank:
        how = f"every linear N-sharded (column-parallel) x{world}, LoRA rows follow the weight's; no exchange"
    else:
        how = (f"tp{world}: ONE block of M tokens; qkv and w1|w3 column-parallel, out and w2 row-parallel with the exact int32 "
               f"reduction pushed over NVLink by the product kernel (reduce-scatter by peer stores, owner's sum + epilogue, "
               f"all-gather by peer stores); whole-row scales by a pushed MAX exchange")
    return {"workload": workload_name(cfg), "block": cfg.block, "parallelism": how,
            "timing": "windows of --steps steps covering at least 1 s of GPU time, median window of the per-window maximum "
                      "over ranks; barrier + synchronize around each window",
            "l2": "per-step working set per GPU (weights plus activations and outputs) is several times the 126 MB L2"}


def cpu_sample_text(cfg, rows: int) -> str:
    return (f"{rows} of {cfg.M} rows of every linear of the block per step (a row sample: the rate is per row and rows are "
            f"independent): the reference's NumPy arithmetic - fp32 rotation matmul, absmax int8, float64 BLAS product, "
            f"bias, bf16 store; weights widened to float64 once outside the timed steps")


# ---- arms ---------------------------------------------------------------------------------------------------------
def run_reference(args, cfg, rank, world):
    if rank != 0:
        return None
    rows = args.cpu_rows or (1024 if cfg.ops < 4e12 else 256)
    value, dt = time_cpu(cfg, rows, args.steps, args.warmup)
    cores = host_threads()
    return {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong" if args.gpus > 1 else "weak",
        "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": config_dict(cfg, world),
        "tops": value * cfg.ops / cfg.M / 1e12,
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": cpu_sample_text(cfg, rows)},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


class Timer:
    """Windows of K calls between CUDA events on the launching stream, a barrier + synchronize on both sides of every
    window, the maximum over ranks per window."""

    def __init__(self, gpu, world):
        import torch
        self.torch, self.gpu, self.world, self.dev = torch, gpu, world, gpu.torch_device

    def barrier(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        self.torch.cuda.synchronize(self.dev)

    def window(self, fn, steps, finish=None):
        """One window; returns (milliseconds on this rank, host time at its start, host time at its end)."""
        torch = self.torch
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.barrier()
        t0 = time.time()
        start.record(self.gpu.stream)
        for _ in range(steps):
            fn()
        if finish is not None:
            finish()
        end.record(self.gpu.stream)
        torch.cuda.synchronize(self.dev)
        t1 = time.time()
        ms = start.elapsed_time(end)
        self.barrier()
        return ms, t0, t1

    def windows(self, fn, steps, seconds=WINDOW_SECONDS, at_least=3, at_most=25, finish=None):
        """Repeats the window until `seconds` of GPU time are covered. Returns (median ms of a window - the maximum
        over ranks per window -, list of those maxima, [(t0, t1)] host spans of this rank's windows)."""
        torch = self.torch
        ms_list, spans = [], []
        first, t0, t1 = self.window(fn, steps, finish)
        ms_list.append(first)
        spans.append((t0, t1))
        # every rank must run the same number of windows: rank 0's first window decides
        n = int(min(at_most, max(at_least, np.ceil(seconds * 1e3 / max(first, 1e-3)))))
        if self.world > 1:
            import torch.distributed as dist
            t = torch.tensor([n], device=self.dev)
            dist.broadcast(t, 0)
            n = int(t.item())
        for _ in range(n - 1):
            ms, t0, t1 = self.window(fn, steps, finish)
            ms_list.append(ms)
            spans.append((t0, t1))
        if self.world > 1:
            import torch.distributed as dist
            t = torch.tensor(ms_list, device=self.dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms_list = t.tolist()
        return float(np.median(ms_list)), ms_list, spans


def int8_peak_probe(gpu, clocks):
    """The measured ceiling of the int8 tensor pipe: MMAs of the product's shape from operands resident in shared
    memory (no TMA, no epilogue), single CTAs and CTA pairs; one launch alone (burst) and launches back to back for
    about half a second under the power cap (sustained), with the clock and power sampled during the latter."""
    out = {"what": "tcgen05.mma kind::i8 issue rate, operands resident in shared memory, two TMEM accumulators, "
                   "one CTA per SM (128x256x32) or one CTA pair per two SMs (256x256x32, cta_group::2)"}
    for name, pair in (("single", False), ("pair", True)):
        gpu.mma_rate_probe(pair, 2000)  # warm-up (loads the kernel)
        time.sleep(0.3)                 # let the clocks recover: the burst figure is a launch from idle
        burst = gpu.mma_rate_probe(pair, 40000)
        t_from = time.time()
        runs = [gpu.mma_rate_probe(pair, 40000) for _ in range(40)]
        t_to = time.time()
        tail = runs[len(runs) // 2:]
        c = clocks.summary(t_from + 0.5 * (t_to - t_from), t_to)
        out[name] = {"burst_tops": burst["tops"], "sustained_tops": float(np.median([r["tops"] for r in tail])),
                     "ops_per_clk_per_sm": float(np.median([r["ops_per_clk_per_sm"] for r in tail])),
                     "ctas": burst["ctas"], "sm_mhz_sustained": c["sm_mhz"], "power_w_sustained": c["power_w"]}
        time.sleep(0.3)
    best = max(("single", "pair"), key=lambda k: out[k]["sustained_tops"])
    out["peak_tops"] = out[best]["sustained_tops"]
    out["peak_from"] = f"{best} CTAs, sustained (median of the second half of 40 launches of 11 ms back to back)"
    return out


def time_block(gpu, blk, cfg, M, args, timer, clocks, peak_tops=None, seconds=WINDOW_SECONDS):
    """Windows of the whole step, then of its product launches alone and of its rotate+quantise launches alone (an
    event pair per launch would put the launch gaps of short kernels into the figure). Returns a dict."""
    for _ in range(max(args.warmup, 3)):
        blk.step()
    launches0 = gpu.launch_count
    ms, ms_list, spans = timer.windows(blk.step, args.steps, seconds)
    launches = (gpu.launch_count - launches0) // len(ms_list)
    res = {"ms_per_step": ms / args.steps, "windows": len(ms_list), "window_ms": [round(x, 4) for x in ms_list],
           "launches_per_window": int(launches),
           "window_clocks": [clocks.summary(a, b)["sm_mhz"] for a, b in spans],
           "clocks": clocks.summary(spans[0][0], spans[-1][1])}
    if hasattr(blk, "gemm_only"):
        gemm_ms, _, gspans = timer.windows(blk.gemm_only, args.steps, seconds / 2)
        rot_ms, _, _ = timer.windows(blk.rot_only, args.steps, seconds / 4)
        gemm_s, rot_s = gemm_ms * 1e-3, rot_ms * 1e-3
        gemm_ops = sum(2 * l.m_pad * l.wt.K * l.wt.N for l in blk.layers) * args.steps
        rot_bytes = sum(M * ((4 if l.swiglu_in else 2) * l.wt.K + l.wt.K + 4) for l in blk.layers) * args.steps
        hbm, hbm_src, _ = hbm_peak()
        tops = gemm_ops / gemm_s / 1e12
        gc = clocks.summary(gspans[0][0], gspans[-1][1])
        res["roofline"] = {
            "bound": "tensor", "kernel": "gemm_w8a8_pair_kernel (tcgen05 kind::i8, cta_group::2; 256 x 256 tiles)", "achieved": tops,
            "peak": peak_tops, "unit": "TOP/s", "frac": tops / peak_tops if peak_tops else None,
            "traffic": NCU_TRAFFIC_BYTES.get(config_number(cfg)),
            "algorithmic_bytes": sum(l.m_pad * l.wt.K + l.wt.N * l.wt.K + 2 * l.m_pad * l.wt.N for l in blk.layers) / len(blk.layers),
            "peak_source": "measured in this run: tcgen05 kind::i8 issue-rate probe, sustained under the power cap (int8_probe)",
            "frac_of_nominal_4500": tops / NOMINAL_INT8_TOPS, "time_share": gemm_s / (gemm_s + rot_s),
            "sm_mhz": gc["sm_mhz"], "power_w": gc["power_w"],
            "ops_per_clk_per_sm": (tops * 1e12 / (gpu.sm_count * gc["sm_mhz"] * 1e6)) if gc["sm_mhz"] else None}
        gbs = rot_bytes / rot_s / 1e9
        res["roofline_rot_q8"] = {"bound": "hbm", "kernel": "rot_q8_tma_kernel (TMA-fed rotate + quantise)", "achieved": gbs,
                                  "peak": hbm, "unit": "GB/s", "frac": gbs / hbm, "traffic": None, "peak_source": hbm_src,
                                  "time_share": rot_s / (gemm_s + rot_s)}
    return res


def time_e2e(blk, timer, tokens_per_step, steps):
    """The same step through the public API with HOST buffers: H2D of every input and D2H of every output inside the
    timed region, which ends when the last download has landed."""
    host_in, host_out = blk.host_buffers()
    for h, x in zip(host_in, blk.inputs):
        if h is not None:
            h.copy_(x.torch().cpu())
    h2d = sum(h.numel() * 2 for h in host_in if h is not None)
    d2h = sum(h.numel() * 2 for h in host_out if h is not None)
    step = lambda: blk.step_host(host_in, host_out)  # noqa: E731
    for _ in range(2):
        step()
    blk.sync_host()
    ms, ms_list, _ = timer.windows(step, steps, seconds=0.5, at_least=3, at_most=5, finish=blk.finish_host)
    blk.sync_host()
    return {"value": tokens_per_step * steps / (ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d,
            "d2h_bytes_per_step": d2h, "ms_per_step": ms / steps, "windows": len(ms_list),
            "per_rank": "bytes are this rank's; every rank moves its own inputs and outputs"}, (host_in, host_out)


def time_without_low_rank(gpu, cfg, M, seed, steps, timer, ms_with, seconds=0.4):
    """The same block with the same weights and inputs but no low-rank term on any linear, timed the same way: what
    the term costs (its T product, the second accumulator's hand-over and the extra MMAs and loads)."""
    import dataclasses
    import torch
    from h3metal_b200.linear import BlockLinears
    blk = BlockLinears(gpu, dataclasses.replace(cfg, lora_rank=0), seed=seed, M=M)
    for _ in range(3):
        blk.step()
    ms, ms_list, _ = timer.windows(blk.step, steps, seconds, at_least=3, at_most=9)
    del blk
    torch.cuda.empty_cache()
    ms_without = ms / steps
    return {"rank": cfg.lora_rank, "ms_per_step_with": ms_with, "ms_per_step_without": ms_without,
            "overhead": ms_with / ms_without - 1.0, "windows": len(ms_list)}


def token_sharded_config4(gpu, args, timer, clocks, rank, world):
    """The largest configuration at FIXED M, token-sharded: every rank runs the whole block (rank-64 LoRA on every
    linear) on M / world rows with replicated weights; no exchange. Returns the line's second object."""
    import torch
    from h3metal_b200 import workloads
    from h3metal_b200.linear import BlockLinears
    cfg = workloads.CONFIGS[4]
    rows = cfg.M // world
    blk = BlockLinears(gpu, cfg, seed=4321 + rank, M=rows)
    steps = max(2, min(args.steps, 5))
    for _ in range(3):
        blk.step()
    launches0 = gpu.launch_count
    ms, ms_list, spans = timer.windows(blk.step, steps, seconds=0.4, at_least=3, at_most=9)
    launches = (gpu.launch_count - launches0) // len(ms_list)
    value = cfg.M * steps / (ms * 1e-3)
    out = {"workload": workload_name(cfg), "parallelism": f"token-sharded x{world} at fixed M: {rows} rows per rank, no exchange",
           "scaling": "strong", "value": value, "unit": UNIT, "ms_per_step": ms / steps, "steps": steps, "windows": len(ms_list),
           "tops_main_product": value / cfg.M * cfg.ops / 1e12, "gpu_launches": int(launches),
           "sm_mhz": clocks.summary(spans[0][0], spans[-1][1])["sm_mhz"]}
    del blk
    torch.cuda.empty_cache()
    out["low_rank_term"] = time_without_low_rank(gpu, cfg, rows, 4321 + rank, steps, timer, ms / steps)
    return out


def run_sweep(args):
    """Config 4's stress sweep: K in {3072, 6144, 16384} x rotation block in {64, 128, 256} at M = 66560, N = 6144 -
    rotate+quantise as achieved HBM GB/s, the product as TOP/s and int8 operations per clock and SM. One JSON line."""
    import torch
    from h3metal_b200 import ops
    from h3metal_b200.gpu import Gpu
    from h3metal_b200.linear import upload_weight
    gpu = Gpu(device=int(os.environ.get("LOCAL_RANK", 0)))
    dev = gpu.torch_device
    timer = Timer(gpu, 1)
    hbm, hbm_src, _ = hbm_peak()
    M, N = 66560, 6144
    out = {"workload": f"config 4 sweep: M={M}, N={N}", "hbm_peak_gbs": hbm, "hbm_peak_source": hbm_src, "rot_q8": {}, "gemm": {}}
    with ClockSampler(gpu.device_index) as clocks:
        probe = int8_peak_probe(gpu, clocks) if not args.no_probe else None
        for K in (3072, 6144, 16384):
            x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
            X, a8, sa = gpu.wrap(x), gpu.empty((M, K), "i8"), gpu.empty((M,), "f32")
            for block in (64, 128, 256):
                fn = lambda: ops.rot_q8(gpu, X, a8, sa, M, K, block=block)  # noqa: E731
                for _ in range(3):
                    fn()
                ms, _, _ = timer.windows(fn, args.steps, seconds=0.1)
                gbs = M * (3 * K + 4) * args.steps / (ms * 1e-3) / 1e9
                out["rot_q8"][f"K={K},block={block}"] = {"us": ms / args.steps * 1e3, "gbs": gbs, "frac_of_hbm_peak": gbs / hbm}
            w = torch.randint(-127, 128, (N, K), device=dev, dtype=torch.int8)
            wt = upload_weight(gpu, w, torch.rand(N, device=dev) * 1e-4 + 1e-4, torch.randn(N, device=dev) * 0.01)
            C = gpu.empty((M, N), "bf16")
            fn = lambda: ops.gemm(gpu, a8, wt, C, M, sa=sa, tile=(128, 32, 4))  # noqa: E731
            for _ in range(3):
                fn()
            ms, _, spans = timer.windows(fn, max(2, args.steps // 4), seconds=0.5)
            tops = 2.0 * M * N * K * max(2, args.steps // 4) / (ms * 1e-3) / 1e12
            c = clocks.summary(spans[0][0], spans[-1][1])
            out["gemm"][f"K={K}"] = {"us": ms / max(2, args.steps // 4) * 1e3, "tops": tops, "frac_of_nominal_4500": tops / NOMINAL_INT8_TOPS,
                                     "frac_of_probe": tops / probe["peak_tops"] if probe else None, "sm_mhz": c["sm_mhz"],
                                     "ops_per_clk_per_sm": tops * 1e12 / (gpu.sm_count * c["sm_mhz"] * 1e6) if c["sm_mhz"] else None}
            del x, X, a8, w, wt, C
            torch.cuda.empty_cache()
        out["int8_probe"] = probe
    return out


def run_ours(args, cfg, rank, world):
    import torch
    import torch.distributed as dist
    from h3metal_b200.gpu import Gpu
    from h3metal_b200 import ops as ops_mod
    from h3metal_b200.linear import BlockLinears

    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    gpu = Gpu(device=local)
    dev = gpu.torch_device
    timer = Timer(gpu, world)
    with ClockSampler(local) as clocks:
        probe = int8_peak_probe(gpu, clocks) if (rank == 0 and not args.no_probe) else None
        if world > 1:
            dist.barrier()
            return run_sharded(args, cfg, rank, world, gpu, timer, clocks, probe)

        blk = BlockLinears(gpu, cfg, seed=1234)
        res = time_block(gpu, blk, cfg, cfg.M, args, timer, clocks, probe["peak_tops"] if probe else None)
        value = cfg.M / (res["ms_per_step"] * 1e-3)
        e2e = None
        if not args.no_e2e:
            e2e, bufs = time_e2e(blk, timer, cfg.M, args.steps)
            del bufs

        # the other producer of int8 activations, norm_mod_q8, at the block's hidden size (not part of the step)
        hidden = blk.layers[0].wt.K
        xres = torch.randn(blk.layers[0].m_pad, hidden, device=dev) * 3
        modt = torch.randn(3, 2, hidden, device=dev)
        rtt = torch.randint(0, 3, (blk.layers[0].m_pad,), device=dev, dtype=torch.uint8)
        X32, MODT, RTT = gpu.wrap(xres), gpu.wrap(modt), gpu.wrap(rtt)
        l0 = blk.layers[0]
        norm_step = lambda: ops_mod.norm_mod_q8(gpu, X32, MODT, RTT, l0.a8, l0.sa, cfg.M, hidden, eps=1e-5, block=cfg.block)  # noqa: E731
        for _ in range(3):
            norm_step()
        norm_ms, _, _ = timer.windows(norm_step, args.steps, seconds=0.2)
        norm_ms /= args.steps
        norm_bytes = cfg.M * (4 * hidden + hidden + 4)
        hbm = hbm_peak()[0]
        norm_extra = {"kernel": "rot_q8_tma_kernel with the norm + modulation front end", "rows": cfg.M, "channels": hidden,
                      "us": norm_ms * 1e3, "achieved_gbs": norm_bytes / (norm_ms * 1e-3) / 1e9,
                      "frac_of_measured_hbm": norm_bytes / (norm_ms * 1e-3) / 1e9 / hbm}
        del blk, xres, X32
        torch.cuda.empty_cache()
        low_rank = time_without_low_rank(gpu, cfg, cfg.M, 1234, args.steps, timer, res["ms_per_step"]) if cfg.lora_rank else None
        second = None if args.no_config4 or config_number(cfg) == 4 else token_sharded_config4(gpu, args, timer, clocks, rank, world)
        gpu.wait()

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": res["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8", "data": "synthetic",
        "config": config_dict(cfg, 1),
        "tops": value / cfg.M * cfg.ops / 1e12, "windows": res["windows"],
        "window_ms": res["window_ms"], "window_sm_mhz": res["window_clocks"],
        "roofline": res["roofline"], "roofline_rot_q8": res["roofline_rot_q8"], "norm_mod_q8": norm_extra,
        "int8_probe": probe, "e2e": e2e, "gpu_launches": res["launches_per_window"], "clocks": res["clocks"],
        "config4_token_sharded": second,
    }
    if low_rank:
        line["low_rank_term"] = low_rank
    if not args.no_cpu:
        rows = args.cpu_rows or (1024 if cfg.ops < 4e12 else 256)
        cpu_value, _ = time_cpu(cfg, rows, 2, 1)
        line["cpu_baseline"] = {"value": cpu_value, "unit": UNIT, "cores": host_threads(), "kind": "port",
                                "sample": cpu_sample_text(cfg, rows) + "; 2 timed steps after 1 warm-up"}
    return line


def run_sharded(args, cfg, rank, world, gpu, timer, clocks, probe):
    """N > 1. Configs with a LoRA term on every linear and column/row-parallel roles (config 2): every linear
    N-sharded (column-parallel), no exchange. Otherwise ONE block over the ranks, column / row / column / row."""
    import torch
    import torch.distributed as dist
    from h3metal_b200 import parallel
    dev = gpu.torch_device

    # ---- parity first: a timed configuration that was not checked proves nothing --------------------------------
    check = parallel.check_sharded_chain(gpu, None, reduce="push")
    flags = [None] * world
    dist.all_gather_object(flags, check)
    exact = all(f["exact"] for f in flags)
    if not exact:
        if rank == 0:
            print(json.dumps({"parity": {"ranks": world, "exact": False, "failed": [f["failed"] for f in flags]}}), flush=True)
        raise SystemExit(3)

    all_column = bool(cfg.lora_rank)
    blk = parallel.TensorParallelBlock(gpu, None, cfg, seed=99, reduce="push", all_column=all_column)
    res = time_block(gpu, blk, cfg, cfg.M, args, timer, clocks)
    value = cfg.M / (res["ms_per_step"] * 1e-3)

    # where the step's time goes: one event pair per layer (its rotate+quantise, product and exchange), max over ranks
    n_layers = len(blk.layers)
    marks = [[torch.cuda.Event(enable_timing=True) for _ in range(n_layers + 1)] for _ in range(args.steps)]
    timer.barrier()
    for s in range(args.steps):
        prev = None
        for i, (layer, x) in enumerate(zip(blk.layers, blk.inputs)):
            marks[s][i].record(gpu.stream)
            prev = layer(prev if x is None else x)
        marks[s][n_layers].record(gpu.stream)
    torch.cuda.synchronize(dev)
    per_layer = torch.tensor([float(np.median([marks[s][i].elapsed_time(marks[s][i + 1]) for s in range(args.steps)]))
                              for i in range(n_layers)], device=dev, dtype=torch.float64)
    dist.all_reduce(per_layer, op=dist.ReduceOp.MAX)
    per_layer = per_layer.tolist()
    link = blk.link_bytes()
    layers = {}
    for spec, layer, t, b in zip(cfg.layers, blk.layers, per_layer, link):
        role = "column" if isinstance(layer, parallel.ColumnParallelLinear) else "row"
        layers[f"{spec.name} {spec.K}->{spec.N} ({role})"] = {
            "ms": round(t, 4), "nvlink_bytes_out_per_rank": int(b),
            "link_gbs": round(b / (t * 1e-3) / 1e9, 1) if b else 0.0,
            "frac_of_peer_copy_770": round(b / (t * 1e-3) / 1e9 / PEER_COPY_GBS, 3) if b else 0.0}

    e2e = None
    if not args.no_e2e:
        e2e, bufs = time_e2e(blk, timer, cfg.M, args.steps)
        e2e["h2d_bytes_per_step"] *= world   # whole job: every rank uploads its inputs and downloads its share
        e2e["d2h_bytes_per_step"] *= world
        e2e["per_rank"] = "bytes are the whole job's (all ranks); ms_per_step is the slowest rank's median window"
        del bufs
    blk.close()
    del blk
    torch.cuda.empty_cache()

    # the same block with NCCL's int32 all-reduce (also exact) beside the pushed reduction
    nccl = None
    if not all_column and not args.no_variants:
        alt = parallel.TensorParallelBlock(gpu, None, cfg, seed=99, reduce="int32")
        for _ in range(3):
            alt.step()
        ms, ms_list, _ = timer.windows(alt.step, args.steps, seconds=0.3, at_least=3, at_most=5)
        nccl = {"reduce": "NCCL all-reduce of int32 partial accumulators (exact)", "ms_per_step": ms / args.steps,
                "nvlink_bytes_out_per_rank_and_row_layer": alt.link_bytes()[1]}
        alt.close()
        del alt
        torch.cuda.empty_cache()

    second = None if args.no_config4 else token_sharded_config4(gpu, args, timer, clocks, rank, world)
    gpu.wait()
    dist.barrier()
    if rank != 0:
        return None
    return {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": res["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "int8", "data": "synthetic",
        "config": config_dict(cfg, world),
        "tops": value / cfg.M * cfg.ops / 1e12, "windows": res["windows"],
        "parity": {"ranks": world, "exact": True,
                   "what": "column-parallel -> swiglu quantiser -> row-parallel (push) chain equals each rank's own one-GPU result bit for bit"},
        "window_ms": res["window_ms"], "window_sm_mhz": res["window_clocks"],
        "layers": layers, "nccl_int32_allreduce": nccl, "int8_probe": probe,
        "e2e": e2e, "gpu_launches": res["launches_per_window"], "clocks": res["clocks"],
        "config4_token_sharded": second,
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", type=int, default=3)
    ap.add_argument("--cpu-rows", type=int, default=0, help="rows of the CPU sample (0 = default)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (it pins GBs of host memory)")
    ap.add_argument("--no-probe", action="store_true", help="skip the int8 issue-rate probe")
    ap.add_argument("--no-config4", action="store_true", help="skip the token-sharded second object (config 4)")
    ap.add_argument("--no-variants", action="store_true", help="N > 1: skip the NCCL all-reduce run beside the pushed one")
    ap.add_argument("--sweep", action="store_true", help="config 4's K x rotation-block stress sweep (one GPU) instead of a block")
    args = ap.parse_args()

    from h3metal_b200 import workloads
    cfg = workloads.CONFIGS[args.config]
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))

    if args.impl == "reference":
        line = run_reference(args, cfg, rank, world)
        if line is not None:
            print(json.dumps(line), flush=True)
        return
    if args.sweep:
        if rank == 0:
            print(json.dumps(run_sweep(args)), flush=True)
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
