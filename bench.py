"""Benchmark of the token-sampling hot path: sampled rows/s and logits-read HBM GB/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2] [--contexts M] [--impl ours|reference]

A step is one pass of the sampling path (row pass + survivor stage) over one batch of the
workload on every GPU: each rank owns its own batch (rows split across GPUs, no collective on
the data path), so per-GPU work is fixed and scaling is weak.  Inputs are synthetic, built on
the device with the workload's shapes and value distribution, and rotate through more batches
than fit in L2.  `value` is timed with CUDA events around exactly K steps with device-resident
inputs; `e2e` is the same metric through the host-buffer entry point, copies included;
`roofline` is the row pass alone (algorithmic bytes = 4 * rows * vocab per launch) against the
measured HBM peak; `cpu_baseline` is the reference's CPU sampler on this box's host cores.

Steps go round-robin to M sampler contexts (default 4), each with its own stream and scratch, the
way a server holds one context per batch in flight; the same loops with one context are timed too
and reported under `single_context`.  `--workload c5` is the vocabulary-sharded mode instead: the
batch is fixed, every rank holds rows x (vocab / N) logits, and a step is shard scan, one NCCL
all-gather of the per-row records, survivor stage (strong scaling, one context).

The driver's K (`--steps`) stays the unit: a region of exactly K steps is timed with CUDA events
between barriers, and the region is repeated until at least 50 ms of GPU time have been timed;
`ms_per_step` is the median over the repeats, with p10, p90 and the number of repeats beside it
(the reference's own benchmark schema reports the same three).  With more than one GPU the line
also carries a `sharded` record: workload C5 with its vocabulary split over the ranks, a few timed
steps and a check of the first 48 rows against the reference fixture.

`--impl reference` times the reference's own CPU sampler (compiled from its sources into
oracle/_ref, or the plain-C restatement when that is absent) on a bounded sample of the same
workload, rank 0 only.

`--top-k`, `--softmax`, `--lm-head` and `--attention` time the other kernels of the library instead
(one GPU, a JSON line of their own with the shapes, microseconds and GB/s against the measured HBM
peak, and the reference's CPU code on a bounded sample beside them).
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

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path[:0] = [str(ROOT), str(ROOT / "tests")]

from pulsatrix_b200.workloads import WORKLOADS  # noqa: E402

L2_BYTES = 126 * 1024 * 1024
# DRAM bytes (read + write) of one row-pass launch as ncu counted them, per workload that has been
# captured; workloads without a capture report no traffic figure.
ROW_PASS_TRAFFIC = {"c2": 39070464}
FALLBACK_HBM_GBS = 6650.0
MIN_TIMED_MS = 50.0   # a K-step region is repeated until this much GPU time has been timed
MAX_REPEATS = 400


# The one JSON line goes to the process's original standard output; everything else a library prints
# there while the benchmark runs (NCCL announces its version on it) is sent to standard error.
_RESULT_FD = None


def keep_stdout_for_the_result():
    global _RESULT_FD
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)


def emit(result):
    line = (json.dumps(result) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(line.decode())
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, line)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="vocabulary-sharded steps: records and results through peer memory, or through NCCL all-gathers")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--contexts", type=int, default=4,
                    help="sampler contexts in flight per GPU (one stream and one scratch each; steps go round-robin)")
    ap.add_argument("--cpu-seconds", type=float, default=15.0, help="CPU work of the cpu_baseline sample")
    ap.add_argument("--lm-head", action="store_true",
                    help="time the device head + sampling step on decode-sized batches instead (one GPU; prints its own JSON line)")
    ap.add_argument("--attention", action="store_true",
                    help="time the attention over the KV cache instead (one GPU; prints its own JSON line)")
    ap.add_argument("--softmax", action="store_true",
                    help="time psx_b200_softmax_rows / logsumexp_rows on a few shapes instead (one GPU; prints its own JSON line)")
    ap.add_argument("--top-k", action="store_true",
                    help="time psx_b200_top_k_rows on a few shapes instead (one GPU; prints its own JSON line)")
    return ap.parse_args()


def measured_hbm_peak():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU while a region runs: NVML from a thread
    every few milliseconds (the timed regions are short), nvidia-smi when NVML cannot be loaded.
    Reads only; changes no setting of the GPU."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []
        self.samples = []  # (sm_mhz, reasons bit mask)
        self.thread = None
        self.stopping = threading.Event()
        self.max_mhz = None
        self.nvml = None

    def _poll(self, handle):
        nvml = self.nvml
        while not self.stopping.is_set():
            try:
                self.samples.append((nvml.nvmlDeviceGetClockInfo(handle, nvml.NVML_CLOCK_SM),
                                     nvml.nvmlDeviceGetCurrentClocksEventReasons(handle)
                                     if hasattr(nvml, "nvmlDeviceGetCurrentClocksEventReasons")
                                     else nvml.nvmlDeviceGetCurrentClocksThrottleReasons(handle)))
            except Exception:  # noqa: BLE001 - a failed sample is just a missing sample
                pass
            time.sleep(0.0005)

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            physical = int(visible.split(",")[self.index]) if visible and visible.split(",")[self.index].isdigit() else self.index
            handle = pynvml.nvmlDeviceGetHandleByIndex(physical)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
            self.nvml = pynvml
            self.thread = threading.Thread(target=self._poll, args=(handle,), daemon=True)
            self.thread.start()
            return
        except Exception:  # noqa: BLE001 - fall back to the command-line tool
            self.nvml = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True).start()
        except OSError:
            self.proc = None

    def stop(self):
        if self.nvml is not None:
            self.stopping.set()
            self.thread.join(timeout=2)
            nvml = self.nvml
            bits = {"hw_slowdown": getattr(nvml, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
                    "hw_thermal_slowdown": getattr(nvml, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
                    "sw_thermal_slowdown": getattr(nvml, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
                    "sw_power_cap": getattr(nvml, "nvmlClocksThrottleReasonSwPowerCap", 0x4)}
            sm = [float(s[0]) for s in self.samples]
            seen = 0
            for _, mask in self.samples:
                seen |= int(mask)
            return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": self.max_mhz,
                    "reasons": sorted(name for name, bit in bits.items() if seen & bit), "samples": len(sm)}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def build_batches(w, device, count, seed):
    """`count` synthetic batches on the device: logits N(0,1)*sigma - zeta*log(rank+1) with a random
    rank per column and row, history ids uniform in [0, vocab)."""
    import torch
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    batches = []
    for _ in range(count):
        logits = torch.randn((w.rows, w.vocab), generator=gen, device=device, dtype=torch.float32) * w.sigma
        if w.zeta != 0.0:
            ranks = torch.rand((w.rows, w.vocab), generator=gen, device=device).argsort(dim=1)
            logits -= w.zeta * torch.log(ranks.to(torch.float32) + 1.0)
            del ranks
        if w.tie_row_fraction > 0:
            n = max(1, int(round(w.rows * w.tie_row_fraction)))
            rows = torch.randperm(w.rows, generator=gen, device=device)[:n]
            cols = torch.randint(0, w.vocab, (n, 2), generator=gen, device=device)
            logits[rows[:, None], cols] = logits[rows].max(dim=1, keepdim=True).values
        hist = torch.randint(0, w.vocab, (w.rows, w.history), generator=gen, device=device, dtype=torch.int64)
        batches.append((logits, hist.reshape(-1).contiguous()))
    offsets = torch.arange(w.rows + 1, device=device, dtype=torch.int64) * w.history
    return batches, offsets


def workload_text(w):
    """The same words in both arms' config.workload."""
    return (f"{w.name}: batch={w.rows} rows per GPU, vocab={w.vocab}, history={w.history}, penalty={w.repetition_penalty}, "
            f"T={w.temperature}, top_k={w.top_k}, top_p={w.top_p}, do_sample={w.do_sample}")


def spread(per_step_ms):
    """median, p10, p90 of a list of per-step times."""
    a = np.sort(np.asarray(per_step_ms, dtype=np.float64))
    pick = lambda q: float(a[min(len(a) - 1, max(0, int(round(q * (len(a) - 1)))))])  # noqa: E731
    return {"median": float(np.median(a)), "p10": pick(0.10), "p90": pick(0.90), "repeats": int(len(a))}


def workload_config(w):
    import pulsatrix_b200 as psx
    return psx.SamplingConfig.make(do_sample=w.do_sample, temperature=w.temperature, top_k=w.top_k, top_p=w.top_p,
                                   min_p=w.min_p, repetition_penalty=w.repetition_penalty)


def cpu_rows_per_second(w, logits, hist, offsets, seeds, cpu_seconds):
    """Times the reference's CPU sampler (oracle/_ref; the plain-C restatement when absent) on
    host rows with every host core.  Returns (rows/s, kind, cores, description of the sample)."""
    import oracle_lib as ol
    kind = "reference" if (ROOT / "oracle" / "_ref" / "libpsx_ref.so").exists() or ol.reference_available() else "port"
    which = "reference" if kind == "reference" else "oracle"
    cores = os.cpu_count() or 1
    cfg = ol.make_config(max_new_tokens=1, do_sample=w.do_sample, temperature=w.temperature, top_k=w.top_k,
                         top_p=w.top_p, min_p=w.min_p, repetition_penalty=w.repetition_penalty)
    t0 = time.perf_counter()
    ol.rows(which, logits, hist, offsets, cfg, seeds, threads=cores)  # also sizes the sample
    once = time.perf_counter() - t0
    repeats = max(1, min(50, int(cpu_seconds / max(once * cores, 1e-3))))
    t0 = time.perf_counter()
    for _ in range(repeats):
        ol.rows(which, logits, hist, offsets, cfg, seeds, threads=cores)
    elapsed = time.perf_counter() - t0
    n = logits.shape[0] * repeats
    return n / elapsed, kind, cores, f"{logits.shape[0]} rows of {w.name} x {repeats} repeats, {cores} threads"


def host_sample(w, batch, offsets, rows):
    logits, hist = batch
    rows = min(rows, w.rows)
    return (logits[:rows].cpu().numpy(), hist.view(w.rows, w.history)[:rows].cpu().numpy().reshape(-1),
            offsets[: rows + 1].cpu().numpy(), np.arange(rows, dtype=np.uint64))


def run_ours(args, rank, world):
    import torch
    import torch.distributed as dist
    import pulsatrix_b200 as psx

    w = WORKLOADS[args.workload]
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    # One context (stream + scratch) per batch in flight, the way a server that decodes several
    # batches at once would hold them: step i runs on context i % M, so the row pass of one batch
    # overlaps the survivor stage of another.  Every batch is complete in HBM before the first timed
    # call, which each context is told, so inside a context too the row pass of a step may start
    # reading while the survivor stage of the step before it is still running.
    m_ctx = max(1, args.contexts)
    ctxs = [psx.Context(local) for _ in range(m_ctx)]
    for c in ctxs:
        c.inputs_are_ready(True)
    ctx = ctxs[0]
    cfg = workload_config(w)
    n_batches = max(2, (2 * L2_BYTES) // w.logits_bytes + 2)
    batches, offsets = build_batches(w, device, n_batches, seed=1234 + rank)
    seeds = np.arange(w.rows, dtype=np.uint64)
    uniforms = torch.from_numpy(psx.uniforms_mt19937_64(seeds)).to(device)
    outs = [c.alloc_outputs(w.rows) for c in ctxs]
    stream = torch.cuda.current_stream(device)
    side = [torch.cuda.Stream(device) for _ in range(m_ctx)]

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def region(launch, m, steps):
        """Milliseconds for exactly `steps` calls of launch(i, context index, stream) spread round-robin
        over the first m contexts, each on its own stream, between two barriers: the begin event is
        recorded on the current stream and every side stream waits for it; the end event is recorded
        on the current stream after it has waited for the last work of every side stream."""
        barrier()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record(stream)
        for s in side[:m]:
            s.wait_event(begin)
        for i in range(steps):
            launch(i, i % m, side[i % m])
        for s in side[:m]:
            done = torch.cuda.Event()
            done.record(s)
            stream.wait_event(done)
        end.record(stream)
        barrier()
        return begin.elapsed_time(end)

    def timed(launch, m, steps, warmup):
        """Per-step milliseconds of every repeat of the K-step region (the max over the ranks of each
        repeat): warm-up calls first, then the region again and again until MIN_TIMED_MS of GPU time
        have been timed.  Every rank makes the same number of repeats (it follows from the first
        region's time, agreed on by all)."""
        for i in range(warmup):
            launch(i, i % m, side[i % m])
        if steps <= 0:
            barrier()
            return []
        first = torch.tensor([region(launch, m, steps)], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(first, op=dist.ReduceOp.MAX)
        repeats = int(min(MAX_REPEATS, max(3, np.ceil(MIN_TIMED_MS / max(float(first.item()), 1e-3)))))
        times = torch.tensor([region(launch, m, steps) for _ in range(repeats)], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(times, op=dist.ReduceOp.MAX)
        return (times / steps).tolist()

    # The loops run over fixed buffers: each (context, batch) pair's call is prepared once
    # (Context.bind_*), so a step costs the host one foreign call, not the conversion of 14 arguments.
    full_calls, scan_calls = {}, {}

    def full_step(i, c, s):
        b = i % n_batches
        call = full_calls.get((c, b))
        if call is None:
            logits, hist = batches[b]
            call = full_calls[(c, b)] = ctxs[c].bind_sample_rows(logits, hist, offsets, cfg, uniforms, out=outs[c],
                                                                 stream=s.cuda_stream)
        call()

    def row_pass(i, c, s):
        b = i % n_batches
        call = scan_calls.get((c, b))
        if call is None:
            logits, hist = batches[b]
            call = scan_calls[(c, b)] = ctxs[c].bind_row_pass_only(logits, hist, offsets, cfg, stream=s.cuda_stream)
        call()

    def read_only(i, c, s):
        psx.read_only_pass(batches[i % n_batches][0], sink, stream=s.cuda_stream)

    warm = max(args.warmup, 3)
    sink = torch.zeros(1, dtype=torch.float32, device=device)
    timed(full_step, m_ctx, 0, max(warm, n_batches) * m_ctx)
    failed = sum(int((o["status"].cpu().numpy() != 0).sum()) for o in outs)

    # Rank 0 samples its GPU's clocks; a polling thread in every rank would only take host time from
    # the launch loops of a box whose ranks already share its cores.
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    # ---- value: K steps, device-resident inputs, CUDA events, M contexts in flight ----
    launches0 = sum(c.launches for c in ctxs)
    step_ms = timed(full_step, m_ctx, args.steps, m_ctx)
    launches = (sum(c.launches for c in ctxs) - launches0 - 2 * m_ctx) // (len(step_ms) + 1)  # per K-step region
    # ---- roofline: the row pass alone, K launches over the rotating batches, same M streams ----
    scan_ms = timed(row_pass, m_ctx, args.steps, max(3, n_batches) * m_ctx)
    # ---- the same two with one context, every launch on one stream ----
    one_ms = timed(full_step, 1, args.steps, max(3, n_batches))
    one_scan_ms = timed(row_pass, 1, args.steps, max(3, n_batches))
    # ---- the practical ceiling: a kernel that only reads the same batches, same cadence ----
    read_ms = timed(read_only, m_ctx, args.steps, 3 * m_ctx)
    one_read_ms = timed(read_only, 1, args.steps, 3)
    # ---- what one Generate() sees: a single row per call, device-resident, one context ----
    single_row = None
    if w.name == "c1":
        row_calls = [ctx.bind_sample_rows(batches[0][0][r:r + 1], batches[0][1][r * w.history:(r + 1) * w.history],
                                          offsets[:2], cfg, uniforms[r:r + 1], out=ctx.alloc_outputs(1), stream=side[0].cuda_stream)
                     for r in range(64)]
        single_row = spread(timed(lambda i, c, s: row_calls[i % 64](), 1, min(args.steps, 200), 64))
    clocks = sampler.stop() if sampler else None

    # ---- e2e: the host-buffer entry point, pinned inputs, copies inside the timed region ----
    h_logits = batches[0][0].cpu().pin_memory()
    h_hist = batches[0][1].cpu().pin_memory()
    h_off = offsets.cpu().pin_memory()
    h_u = uniforms.cpu().pin_memory()
    e2e_steps = max(3, min(args.steps, 20))
    for _ in range(2):
        ctx.sample_rows_host(h_logits, h_hist, h_off, cfg, h_u, raise_on_row_failure=False)
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        ctx.sample_rows_host(h_logits, h_hist, h_off, cfg, h_u, raise_on_row_failure=False)
    e2e_s = time.perf_counter() - t0
    h2d = h_logits.numel() * 4 + h_hist.numel() * 8 + h_off.numel() * 8 + (h_u.numel() * 8 if w.do_sample else 0)
    d2h = w.rows * (8 + 4 + 4 + 24)

    e2e_ms = torch.tensor([e2e_s * 1e3], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
    e2e_ms = float(e2e_ms.item())
    sharded = sharded_record(args, rank, world, local) if world > 1 else None
    if rank != 0:
        return

    peak, peak_kind = measured_hbm_peak()
    step, scan, one, one_scan = spread(step_ms), spread(scan_ms), spread(one_ms), spread(one_scan_ms)
    read_med, one_read_med = spread(read_ms)["median"], spread(one_read_ms)["median"]
    achieved = w.logits_bytes / (scan["median"] * 1e-3) / 1e9
    result = {
        "metric": "sampled rows/sec and logits-read HBM GB/s vs B200 peak",
        "value": w.rows * world / (step["median"] * 1e-3),
        "unit": "rows/s",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": max(args.warmup, 3),
        "ms_per_step": step["median"],
        "p10_ms_per_step": step["p10"], "p90_ms_per_step": step["p90"], "repeats": step["repeats"],
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "f32 logits; f64 survivor stage",
        "data": "synthetic",
        "config": {"workload": workload_text(w),
                   "parallelism": f"rows split over {world} GPU(s), no data-path collective",
                   "contexts_in_flight": m_ctx,
                   "timing": f"a region of {args.steps} steps between barriers, repeated {step['repeats']} times; medians",
                   "l2": f"inputs rotate over {n_batches} batches = {n_batches * w.logits_bytes / 2**20:.0f} MiB > L2"},
        "e2e": {"value": w.rows * world * e2e_steps / (e2e_ms * 1e-3), "unit": "rows/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "steps": e2e_steps},
        "gpu_launches": int(launches) * world,
        "clocks": clocks,
        "roofline": {"bound": "hbm", "kernel": "scan_rows_kernel", "achieved": achieved, "peak": peak,
                     "unit": "GB/s", "frac": achieved / peak, "peak_kind": peak_kind,
                     "traffic": ROW_PASS_TRAFFIC.get(w.name),
                     "traffic_note": "dram read + write bytes of one launch from an ncu capture of this workload; null: not captured",
                     "algorithmic_bytes": w.logits_bytes,
                     "launch_ms": scan["median"], "launch_ms_p10": scan["p10"], "launch_ms_p90": scan["p90"],
                     "step_minus_row_pass_ms": max(step["median"] - scan["median"], 0.0),
                     "frac_of_nominal_8TBs": achieved / 8000.0,
                     "read_only_kernel_gbs": w.logits_bytes / (read_med * 1e-3) / 1e9,
                     "frac_of_read_only_kernel": read_med / scan["median"]},
        "single_context": {"value": w.rows * world / (one["median"] * 1e-3), "unit": "rows/s",
                           "ms_per_step": one["median"], "p10_ms_per_step": one["p10"], "p90_ms_per_step": one["p90"],
                           "row_pass_launch_ms": one_scan["median"],
                           "roofline_frac": w.logits_bytes / (one_scan["median"] * 1e-3) / 1e9 / peak,
                           "read_only_kernel_gbs": w.logits_bytes / (one_read_med * 1e-3) / 1e9},
        "failed_rows": failed,
    }
    if single_row is not None:
        result["single_row_call"] = {"us_per_call": single_row["median"] * 1e3, "p10_us": single_row["p10"] * 1e3,
                                     "p90_us": single_row["p90"] * 1e3,
                                     "note": "one row of the workload per call, device-resident, one context"}
    if sharded is not None:
        result["sharded"] = sharded
    if world == 1:
        sample = host_sample(w, batches[0], offsets, 64)
        value, kind, cores, text = cpu_rows_per_second(w, *sample, args.cpu_seconds)
        result["cpu_baseline"] = {"value": value, "unit": "rows/s", "cores": cores, "kind": kind, "sample": text}
    emit(result)


def sharded_setup(w, device, rank, world, n_batches_for, fixture_rows=48, exchange="peer"):
    """This rank's column shards of `w` (rotating batches), the shared histories, and a ShardedSampler.
    The first `fixture_rows` rows of batch 0 are the reference fixture's rows (built by the CPU
    checker's generator), so that a step over batch 0 can be compared with tests/golden."""
    import torch
    import pulsatrix_b200 as psx
    from pulsatrix_b200.sharded import ShardedSampler, shard_bounds
    import workload_rows

    ctx = psx.Context(device.index)
    ctx.inputs_are_ready(True)
    cfg = workload_config(w)
    begin_col, cols = shard_bounds(w.vocab, world, rank)
    shard_bytes = 4 * w.rows * cols
    n_batches = n_batches_for(shard_bytes)
    gen = torch.Generator(device=device)
    gen.manual_seed(4321 + rank)
    shards = []
    for _ in range(n_batches):  # the Zipf bias over this rank's share of the ranks of every row
        x = torch.randn((w.rows, cols), generator=gen, device=device, dtype=torch.float32) * w.sigma
        ranks = torch.rand((w.rows, cols), generator=gen, device=device).argsort(dim=1)
        x -= w.zeta * torch.log(ranks.to(torch.float32) * world + rank + 1.0)
        del ranks
        shards.append(x)
    same = torch.Generator(device=device)
    same.manual_seed(99)  # every rank holds the same histories
    hist = torch.randint(0, w.vocab, (w.rows * w.history,), generator=same, device=device, dtype=torch.int64)
    fixture_rows = min(fixture_rows, w.rows)
    f_logits, f_hist, _, _ = workload_rows.build(w.name, np.arange(fixture_rows))
    shards[0][:fixture_rows] = torch.from_numpy(np.ascontiguousarray(f_logits[:, begin_col: begin_col + cols])).to(device)
    hist[: fixture_rows * w.history] = torch.from_numpy(f_hist.reshape(-1).astype(np.int64)).to(device)
    offsets = torch.arange(w.rows + 1, device=device, dtype=torch.int64) * w.history
    uniforms = torch.from_numpy(psx.uniforms_mt19937_64(np.arange(w.rows, dtype=np.uint64))).to(device)
    sampler = ShardedSampler(ctx, w.rows, w.vocab, cfg, device, exchange=exchange, fall_back=True)
    return ctx, cfg, sampler, shards, hist, offsets, uniforms, shard_bytes, begin_col, fixture_rows


def fixture_rows_matched(w, sampler, fixture_rows):
    """Rows of the last step (over batch 0) whose token equals the reference fixture's, on this rank."""
    gold = np.load(ROOT / "tests" / "golden" / f"workload_{w.name}.npz")
    got = sampler.flat()
    tokens = got["tokens"][:fixture_rows].cpu().numpy()
    status = got["status"][:fixture_rows].cpu().numpy()
    return int(((tokens == gold["token"][:fixture_rows]) & (status == 0)).sum())


def sharded_record(args, rank, world, local):
    """Workload C5 with its vocabulary split over the ranks of this run: shard scan, one NCCL
    all-gather of the per-row records, the rows shared out for the draw, one small all-gather of
    the results.  A few timed steps and a check of the first 48 rows against the reference fixture."""
    import torch
    import torch.distributed as dist

    w = WORKLOADS["c5"]
    device = torch.device("cuda", local)
    stream = torch.cuda.current_stream(device)
    ctx, cfg, sampler, shards, hist, offsets, uniforms, shard_bytes, begin_col, n_fix = sharded_setup(
        w, device, rank, world, lambda nbytes: max(2, (2 * L2_BYTES) // nbytes + 2), exchange=args.exchange)

    def sync_all():
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup):
        for i in range(warmup):
            fn(i)
        sync_all()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record(stream)
        for i in range(steps):
            fn(i)
        end.record(stream)
        sync_all()
        return begin.elapsed_time(end) / steps

    steps = max(3, min(args.steps, 50))
    sampler.step(shards[0], hist, offsets, uniforms)
    sync_all()
    matched = fixture_rows_matched(w, sampler, n_fix)
    failed = int((sampler.flat()["status"].cpu().numpy() != 0).sum())
    step_ms = timed(lambda i: sampler.step(shards[i % len(shards)], hist, offsets, uniforms), steps, 3)
    scan_ms = timed(lambda i: ctx.shard_scan(shards[i % len(shards)], begin_col, w.vocab, hist, offsets, cfg, sampler.mine), steps, 3)
    stats = torch.tensor([step_ms, scan_ms, -float(matched), float(failed)], dtype=torch.float64, device=device)
    dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    step_ms, scan_ms, neg_matched, failed = stats.tolist()
    peak, _ = measured_hbm_peak()
    records_bytes, results_bytes = sampler.allgather_bytes
    sampler.close()
    return {"workload": f"c5: batch={w.rows} rows, vocab={w.vocab} in {world} column shard(s), history={w.history}, "
                        f"top_k={w.top_k}, top_p={w.top_p}",
            "exchange": sampler.exchange, "exchange_note": sampler.exchange_note, "step_us": step_ms * 1e3, "rows_per_s": w.rows / (step_ms * 1e-3), "steps": steps,
            "shard_scan_us": scan_ms * 1e3, "scan_frac": shard_bytes / (scan_ms * 1e-3) / 1e9 / peak,
            "allgather_bytes": records_bytes, "results_allgather_bytes": results_bytes,
            "fixture_rows": n_fix, "fixture_rows_matched": int(-neg_matched), "failed_rows": int(failed),
            "note": "max over ranks of the times; fixture_rows_matched is the fewest over the ranks"}


def run_sharded(args, rank, world):
    """Workloads whose vocabulary is split over the GPUs (C5): the batch is the same whatever N is, every
    rank holds rows x (vocab / N) logits, scans them, one NCCL all-gather of the per-row records brings
    the candidates together, the ranks share the rows out for the draw and a second, small all-gather
    spreads the results.  Strong scaling: the rows are fixed, the columns per GPU shrink with N."""
    import torch
    import torch.distributed as dist

    w = WORKLOADS[args.workload]
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world == 1:  # the all-gathers of one rank still go through torch.distributed
        dist.init_process_group("nccl", init_method="tcp://127.0.0.1:29591", rank=0, world_size=1,
                                device_id=device)
    ctx, cfg, sampler, shards, hist, offsets, uniforms, shard_bytes, begin_col, n_fix = sharded_setup(
        w, device, rank, world, lambda nbytes: max(2, (2 * L2_BYTES) // nbytes + 2), exchange=args.exchange)
    n_batches = len(shards)
    stream = torch.cuda.current_stream(device)

    def barrier():
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()

    issue_s = []  # host time to enqueue the steps of a region (a step that takes the GPU less is bound by it)

    def region(fn, steps):
        barrier()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record(stream)
        t0 = time.perf_counter()
        for i in range(steps):
            fn(i)
        issue_s.append((time.perf_counter() - t0) / steps)
        end.record(stream)
        barrier()
        return begin.elapsed_time(end)

    def timed(fn, steps, warmup):
        for i in range(warmup):
            fn(i)
        first = torch.tensor([region(fn, steps)], dtype=torch.float64, device=device)
        dist.all_reduce(first, op=dist.ReduceOp.MAX)
        repeats = int(min(MAX_REPEATS, max(3, np.ceil(MIN_TIMED_MS / max(float(first.item()), 1e-3)))))
        times = torch.tensor([region(fn, steps) for _ in range(repeats)], dtype=torch.float64, device=device)
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        return (times / steps).tolist()

    def full_step(i):
        sampler.step(shards[i % n_batches], hist, offsets, uniforms)

    def scan_only(i):
        ctx.shard_scan(shards[i % n_batches], begin_col, w.vocab, hist, offsets, cfg, sampler.mine)

    warm = max(args.warmup, 3)
    sampler.step(shards[0], hist, offsets, uniforms)
    barrier()
    matched = fixture_rows_matched(w, sampler, n_fix)
    failed = int((sampler.flat()["status"].cpu().numpy() != 0).sum())
    clock_sampler = ClockSampler(local) if rank == 0 else None
    if clock_sampler:
        clock_sampler.start()
    launches0 = ctx.launches
    step_ms = timed(full_step, args.steps, warm)
    host_issue_us = float(np.median(issue_s)) * 1e6
    launches = (ctx.launches - launches0) * args.steps // (warm + (len(step_ms) + 1) * args.steps)
    scan_ms = timed(scan_only, args.steps, 3)
    clocks = clock_sampler.stop() if clock_sampler else None
    other_ms = None
    if sampler.exchange == "peer":  # the same step with the two NCCL all-gathers instead, for comparison
        from pulsatrix_b200.sharded import ShardedSampler
        by_nccl = ShardedSampler(ctx, w.rows, w.vocab, cfg, device, exchange="nccl")
        other_ms = timed(lambda i: by_nccl.step(shards[i % n_batches], hist, offsets, uniforms), args.steps, warm)

    # ---- e2e: this rank's shard comes from pinned host memory every step, the tokens go back ----
    h_shard = shards[0].cpu().pin_memory()
    h_tokens = torch.empty((sampler.world, sampler.per), dtype=torch.int64).pin_memory()
    staged = torch.empty_like(shards[0])
    e2e_steps = max(3, min(args.steps, 20))

    def e2e_step(i):
        staged.copy_(h_shard, non_blocking=True)
        o = sampler.step(staged, hist, offsets, uniforms)
        h_tokens.copy_(o["tokens"], non_blocking=True)
        stream.synchronize()

    ctx.inputs_are_ready(False)  # the staged shard is being copied in by the transfer just enqueued
    for i in range(2):
        e2e_step(i)
    barrier()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        e2e_step(i)
    barrier()
    e2e_s = time.perf_counter() - t0

    stats = torch.tensor([e2e_s * 1e3, -float(matched), float(failed)], dtype=torch.float64, device=device)
    dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    e2e_ms, neg_matched, failed = stats.tolist()
    sampler.close()
    if rank != 0:
        return
    peak, peak_kind = measured_hbm_peak()
    step, scan = spread(step_ms), spread(scan_ms)
    achieved = shard_bytes / (scan["median"] * 1e-3) / 1e9
    records_bytes, results_bytes = sampler.allgather_bytes
    result = {
        "metric": "sampled rows/sec and logits-read HBM GB/s vs B200 peak",
        "value": w.rows / (step["median"] * 1e-3), "unit": "rows/s", "n_gpus": world, "steps": args.steps,
        "warmup": warm, "ms_per_step": step["median"], "p10_ms_per_step": step["p10"], "p90_ms_per_step": step["p90"],
        "repeats": step["repeats"], "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32 logits; f64 survivor stage", "data": "synthetic",
        "config": {"workload": f"{w.name}: batch={w.rows} rows, vocab={w.vocab} in {world} column shard(s), "
                               f"history={w.history}, penalty={w.repetition_penalty}, T={w.temperature}, "
                               f"top_k={w.top_k}, top_p={w.top_p}",
                   "parallelism": (f"vocabulary split over {world} GPU(s); per step {records_bytes} bytes of records per rank "
                                   f"written straight into the memory of the ranks that decide the rows and {results_bytes} "
                                   f"bytes of results into every rank's (peer stores over NVLink, counters in peer memory, "
                                   f"no library collective)" if sampler.exchange == "peer" else
                                   f"vocabulary split over {world} GPU(s); per step one NCCL all-gather of "
                                   f"{records_bytes} bytes per rank (records) and one of {results_bytes} (results)"),
                   "exchange": sampler.exchange, "exchange_note": sampler.exchange_note,
                   "contexts_in_flight": 1,
                   "l2": f"shards rotate over {n_batches} batches = {n_batches * shard_bytes / 2**20:.0f} MiB > L2"},
        "e2e": {"value": w.rows * e2e_steps / (e2e_ms * 1e-3), "unit": "rows/s", "h2d_bytes_per_step": shard_bytes,
                "d2h_bytes_per_step": w.rows * 8, "steps": e2e_steps},
        "gpu_launches": int(launches) * world,
        "clocks": clocks,
        "roofline": {"bound": "hbm", "kernel": "scan_rows_kernel (+ pack_records_kernel)", "achieved": achieved,
                     "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_kind": peak_kind,
                     "traffic": None, "traffic_note": "not captured for this workload",
                     "algorithmic_bytes": shard_bytes, "launch_ms": scan["median"]},
        "failed_rows": int(failed), "fixture_rows": n_fix, "fixture_rows_matched": int(-neg_matched),
    }
    result["host_issue_us_per_step"] = host_issue_us  # rank 0's
    if other_ms is not None:
        result["nccl_all_gather_ms_per_step"] = spread(other_ms)["median"]
    emit(result)


def run_reference(args, rank, world):
    if rank != 0:
        return
    import oracle_lib as ol
    w = WORKLOADS[args.workload]
    import workload_rows
    rows = min(w.rows, 64)
    logits, hist, offsets, seeds = workload_rows.build(w.name, np.arange(rows))
    kind = "reference" if ol.reference_available() else "port"
    which = "reference" if kind == "reference" else "oracle"
    cores = os.cpu_count() or 1
    cfg = workload_rows.config_of(w)
    hist = hist.reshape(-1)
    for _ in range(max(args.warmup, 1)):
        ol.rows(which, logits, hist, offsets, cfg, seeds, threads=cores)
    steps = max(1, min(args.steps, 40))
    t0 = time.perf_counter()
    for _ in range(steps):
        ol.rows(which, logits, hist, offsets, cfg, seeds, threads=cores)
    elapsed = time.perf_counter() - t0
    value = rows * steps / elapsed
    text = f"{rows} rows of {w.name} per step, {cores} threads"
    emit({
        "impl": "reference", "metric": "sampled rows/sec and logits-read HBM GB/s vs B200 peak", "value": value,
        "unit": "rows/s", "n_gpus": world, "steps": steps, "warmup": max(args.warmup, 1),
        "ms_per_step": elapsed / steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32 logits; f64 softmax", "data": "synthetic",
        "config": {"workload": workload_text(w), "parallelism": "host threads, one row each",
                   "sample": text},
        "cpu_baseline": {"value": value, "unit": "rows/s", "cores": cores, "kind": kind, "sample": text},
        "e2e": {"value": value, "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    })


TOP_K_SHAPES = [(4096, 16384, 64), (1024, 65536, 32), (64, 151936, 20), (8192, 4096, 16), (256, 128256, 1024)]


def run_top_k(args):
    """The selection primitive alone (DeviceBackend::top_k_rows): rows/s and input GB/s per shape,
    inputs rotating over more than L2, CUDA events on the launching stream."""
    import torch
    import pulsatrix_b200 as psx

    import ctypes as C
    ctx = psx.Context(0)
    results = []
    harness = ROOT / "oracle" / "_ref" / "libpsx_refcuda.so"  # the reference's own CUDA backend, compiled in place
    reference = None
    if harness.exists():
        reference = C.CDLL(str(harness))
        reference.psxrefcuda_time_top_k_rows.restype = C.c_double
    for rows, cols, k in TOP_K_SHAPES:
        count = max(2, (2 * L2_BYTES) // (rows * cols * 4) + 1)
        xs = [torch.randn(rows, cols, device="cuda") for _ in range(count)]
        for i in range(max(args.warmup, 3)):
            ctx.top_k_rows(xs[i % count], k)
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        steps = max(3, min(args.steps, 50))
        begin.record()
        for i in range(steps):
            ctx.top_k_rows(xs[i % count], k)
        end.record()
        torch.cuda.synchronize()
        ms = begin.elapsed_time(end) / steps
        entry = {"rows": rows, "cols": cols, "k": k, "us": ms * 1e3, "rows_per_s": rows / (ms * 1e-3),
                 "input_gbs": rows * cols * 4 / (ms * 1e-3) / 1e9}
        if reference is not None and rows <= 4096:
            # the reference's unmodified CUDABackend::top_k_rows on this GPU (one thread per row), each
            # call synchronised as its backend does; beside it the same call through the override
            entry["reference_cuda_us"] = reference.psxrefcuda_time_top_k_rows(None, C.c_int64(rows), C.c_int64(cols), C.c_int64(k), C.c_int(2))
            entry["through_override_us"] = reference.psxrefcuda_time_top_k_rows(str(psx.library_path()).encode(), C.c_int64(rows),
                                                                               C.c_int64(cols), C.c_int64(k), C.c_int(5))
        results.append(entry)
        del xs
    peak, peak_kind = measured_hbm_peak()
    emit({"metric": "top_k_rows rows/s", "unit": "rows/s", "n_gpus": 1, "dtype": "f32", "data": "synthetic",
          "hbm_peak_gbs": peak, "peak_kind": peak_kind, "results": results})


SOFTMAX_SHAPES = [(65536, 128), (8192, 4096), (1024, 49152), (256, 128256), (64, 151936), (512, 262144)]


def run_softmax(args):
    """The row primitives beside the path (DeviceBackend::softmax_rows / logsumexp_rows): GB/s against
    8 bytes per element (read + write) for softmax and 4 (read) for logsumexp, inputs rotating over more
    than L2, CUDA events on the launching stream."""
    import torch
    import pulsatrix_b200 as psx

    ctx = psx.Context(0)
    results = []
    for rows, cols in SOFTMAX_SHAPES:
        count = max(2, (2 * L2_BYTES) // (rows * cols * 4) + 1)
        xs = [torch.randn(rows, cols, device="cuda") * 3 for _ in range(count)]
        out = torch.empty_like(xs[0])
        entry = {"rows": rows, "cols": cols}
        for name, fn, bytes_per in (("softmax", lambda x: ctx.softmax_rows(x, out=out), 8),
                                    ("logsumexp", lambda x: ctx.logsumexp_rows(x), 4)):
            for i in range(max(args.warmup, 3)):
                fn(xs[i % count])
            torch.cuda.synchronize()
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            steps = max(3, min(args.steps, 50))
            begin.record()
            for i in range(steps):
                fn(xs[i % count])
            end.record()
            torch.cuda.synchronize()
            ms = begin.elapsed_time(end) / steps
            entry[name + "_us"] = ms * 1e3
            entry[name + "_gbs"] = rows * cols * bytes_per / (ms * 1e-3) / 1e9
        results.append(entry)
        del xs, out
    peak, peak_kind = measured_hbm_peak()
    # The reference's CPU backend beside it on a bounded sample (src/cpu_backend.cpp:292-338, single-threaded).
    import oracle_lib as ol
    which = "reference" if ol.reference_available() else "oracle"
    sample = (np.random.RandomState(0).randn(64, 4096) * 3).astype(np.float32)
    t0 = time.perf_counter()
    ol.row_primitive(which, "softmax_rows", sample)
    cpu_gbs = sample.size * 8 / (time.perf_counter() - t0) / 1e9
    emit({"metric": "softmax_rows / logsumexp_rows GB/s", "unit": "GB/s", "n_gpus": 1, "dtype": "f32", "data": "synthetic",
          "hbm_peak_gbs": peak, "peak_kind": peak_kind, "results": results,
          "cpu_baseline": {"value": cpu_gbs, "unit": "GB/s (softmax_rows, read + write)", "cores": 1,
                           "kind": "reference" if which == "reference" else "port", "sample": "64 rows of 4096"}})


LM_HEAD_SHAPES = [(1, 2048, 151936), (8, 2048, 151936), (64, 2048, 151936), (1, 576, 49152), (8, 4096, 128256)]


def run_lm_head(args):
    """Head and sampling in one call (psx_b200_lm_head_sample_rows) on decode-sized batches: the weight
    matrix (vocab x d, fp32) is the traffic, 4 * vocab * d bytes per call; beside it the same step with
    the logits coming from the host as the reference's adapter hands them over (src/generation.cpp:248-256)."""
    import torch
    import pulsatrix_b200 as psx

    ctx = psx.Context(0)
    results = []
    peak, peak_kind = measured_hbm_peak()
    for rows, d, vocab in LM_HEAD_SHAPES:
        weight = torch.randn((vocab, d), device="cuda") * 0.05
        hidden = torch.randn((rows, d), device="cuda")
        hist = torch.randint(0, vocab, (rows * 64,), device="cuda", dtype=torch.int64)
        offsets = torch.arange(rows + 1, device="cuda", dtype=torch.int64) * 64
        cfg = psx.SamplingConfig.make(do_sample=True, temperature=0.8, top_k=50, top_p=0.9, repetition_penalty=1.1)
        u = torch.from_numpy(psx.uniforms_mt19937_64(np.arange(rows, dtype=np.uint64))).cuda()
        out = ctx.alloc_outputs(rows)
        for _ in range(max(args.warmup, 3)):
            ctx.lm_head_sample_rows(hidden, weight, hist, offsets, cfg, u, out=out)
        torch.cuda.synchronize()
        steps = max(3, min(args.steps, 30))
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for _ in range(steps):
            ctx.lm_head_sample_rows(hidden, weight, hist, offsets, cfg, u, out=out)
        end.record()
        torch.cuda.synchronize()
        ms = begin.elapsed_time(end) / steps
        # the reference's hand-over: logits on the host, every step
        logits = ctx.lm_head_logits(hidden, weight).cpu().pin_memory()
        h_hist, h_off, h_u = hist.cpu().pin_memory(), offsets.cpu().pin_memory(), u.cpu().pin_memory()
        ctx.sample_rows_host(logits, h_hist, h_off, cfg, h_u)
        t0 = time.perf_counter()
        for _ in range(steps):
            ctx.sample_rows_host(logits, h_hist, h_off, cfg, h_u)
        host_ms = (time.perf_counter() - t0) * 1e3 / steps
        results.append({"rows": rows, "d_model": d, "vocab": vocab, "us": ms * 1e3, "rows_per_s": rows / (ms * 1e-3),
                        "weight_gbs": 4 * vocab * d / (ms * 1e-3) / 1e9, "frac_of_hbm_peak": 4 * vocab * d / (ms * 1e-3) / 1e9 / peak,
                        "sampling_from_host_logits_us": host_ms * 1e3})
        del weight
    # The reference's loop beside it, on a bounded sample: one row against a 4096-entry slice of the first shape's
    # head (src/cpu_backend.cpp:188-196: one accumulator per logit, products in order; numpy does the same
    # arithmetic feature by feature), scaled to the whole vocabulary.
    _, d, vocab = LM_HEAD_SHAPES[0]
    rng = np.random.RandomState(0)
    h = rng.randn(d).astype(np.float32)
    wslice = (rng.randn(4096, d) * 0.05).astype(np.float32)
    t0 = time.perf_counter()
    acc = np.zeros(4096, dtype=np.float32)
    for p_ in range(d):
        acc = (acc + (h[p_] * wslice[:, p_]).astype(np.float32)).astype(np.float32)
    cpu_us = (time.perf_counter() - t0) * 1e6 * vocab / 4096
    emit({"metric": "lm head + sampling step", "unit": "us per call", "n_gpus": 1, "dtype": "f32", "data": "synthetic",
          "hbm_peak_gbs": peak, "peak_kind": peak_kind, "results": results,
          "cpu_baseline": {"value": cpu_us, "unit": "us per row (head alone)", "cores": 1, "kind": "port",
                           "sample": f"one row against 4096 of {vocab} vocabulary entries, d = {d}, scaled to the vocabulary"}})


ATTENTION_SHAPES = [  # (batch, heads, kv_heads, head_dim, cached positions)
    (64, 32, 8, 128, 4096), (8, 32, 8, 128, 16384), (1, 32, 8, 128, 32768), (256, 16, 16, 64, 1024), (64, 32, 32, 128, 2048),
    (64, 8, 4, 256, 4096),
]


def run_attention(args):
    """One new position per sequence over the KV cache (psx_b200_decode_attention): the cache is the traffic,
    8 * (cached + 1) * head_dim bytes per (batch, kv head).  Caches rotate so that a launch never finds its
    cache in L2."""
    import torch
    import pulsatrix_b200 as psx

    ctx = psx.Context(0)
    peak, peak_kind = measured_hbm_peak()
    results = []
    for batch, heads, kv_heads, d, cached in ATTENTION_SHAPES:
        max_len = cached + 1
        cache_bytes = 2 * batch * kv_heads * max_len * d * 4
        copies = max(2, int(np.ceil(2 * L2_BYTES / cache_bytes)) + 1)
        caches = [(torch.randn((batch, kv_heads, max_len, d), device="cuda"), torch.randn((batch, kv_heads, max_len, d), device="cuda"))
                  for _ in range(copies)]
        q = torch.randn((batch, heads, 1, d), device="cuda")
        for i in range(max(args.warmup, 3)):
            ctx.decode_attention(q, caches[i % copies][0], caches[i % copies][1], cached)
        torch.cuda.synchronize()
        steps = max(3, min(args.steps, 30))
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for i in range(steps):
            ctx.decode_attention(q, caches[i % copies][0], caches[i % copies][1], cached)
        end.record()
        torch.cuda.synchronize()
        ms = begin.elapsed_time(end) / steps
        gbs = cache_bytes / (ms * 1e-3) / 1e9
        results.append({"batch": batch, "heads": heads, "kv_heads": kv_heads, "head_dim": d, "cached": cached, "us": ms * 1e3,
                        "cache_mb": cache_bytes / 1e6, "cache_gbs": gbs, "frac_of_hbm_peak": gbs / peak})
        del caches
    # The reference's CPU backend beside it, on a bounded sample: one sequence of the first shape (the loops of
    # src/multihead_attention_module.cpp:562-586, single-threaded as there; the compiled reference when present).
    import oracle_lib as ol
    which = "reference" if ol.reference_available() else "oracle"
    _, heads, kv_heads, d, cached = ATTENTION_SHAPES[0]
    rng = np.random.RandomState(0)
    q = rng.randn(1, heads, 1, d).astype(np.float32)
    k = rng.randn(1, kv_heads, cached + 1, d).astype(np.float32)
    v = rng.randn(1, kv_heads, cached + 1, d).astype(np.float32)
    t0 = time.perf_counter()
    ol.decode_attention(which, q, k, v, cached, float(1.0 / np.sqrt(d)))
    cpu_us = (time.perf_counter() - t0) * 1e6
    emit({"metric": "attention of one new position over the KV cache", "unit": "us per call", "n_gpus": 1, "dtype": "f32",
          "data": "synthetic", "hbm_peak_gbs": peak, "peak_kind": peak_kind, "results": results,
          "cpu_baseline": {"value": cpu_us, "unit": "us per sequence", "cores": 1, "kind": "reference" if which == "reference" else "port",
                           "sample": f"one sequence of {heads} heads over {kv_heads} kv heads, head_dim {d}, {cached} cached positions"}})


def main():
    args = parse_args()
    keep_stdout_for_the_result()
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if args.top_k or args.softmax or args.lm_head or args.attention:
        if rank == 0:
            (run_top_k if args.top_k else run_softmax if args.softmax else run_lm_head if args.lm_head else run_attention)(args)
        return
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if world > 1:
        import torch
        import torch.distributed as dist
        local = int(os.environ.get("LOCAL_RANK", 0))
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    sharded = WORKLOADS[args.workload].shards > 1
    try:
        (run_sharded if sharded else run_ours)(args, rank, world)
    finally:
        if world > 1 or sharded:
            import torch.distributed as dist
            if dist.is_initialized():
                dist.destroy_process_group()


if __name__ == "__main__":
    main()
