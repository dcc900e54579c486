#!/usr/bin/env python
"""Benchmark of the per-step token sampler.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A step is one pass of the sampler over one batch of the large-vocabulary stress
configuration (256 rows x 248,320 bf16 logits, repetition / presence / frequency
penalties over 32,768-token histories held in device-resident histograms, top-k / top-p /
min-p, seeded Philox draw), each rank working on its own 256 rows (weak scaling, no
inter-GPU traffic).  Prints one JSON line on rank 0.

value   rows/s with the logits already in HBM (CUDA events around K back-to-back steps
        over rotating input sets, max over ranks)
e2e     rows/s through the Python drop-in ``sample_logits`` with the logits in pinned host
        memory: host-to-device copy of the step's logits, histogram delta and parameters,
        and device-to-host copy of the result records, all inside the timed region
roofline  HBM: algorithmic bytes of one launch / average launch time, against the measured
        copy bandwidth in MEASURED_PEAKS.json
cpu_baseline  the reference's CPU operator sequence (oracle/reference_port.py) timed on a
        bounded sample of the same rows on this box's host cores
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

METRIC = "sampled rows/sec"
UNIT = "rows/s"
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of the two kernels of one step, from the ncu
# capture summarised in profiles/ (same workload, one step)
NCU_DRAM_BYTES_PER_STEP = 152.8e6
ROTATING_SETS = 8


def workload_config(batch, vocab, history_len, n_gpus, extra=None):
    cfg = {
        "workload": "config3: large-vocab stress, 256 x 248,320 bf16, all penalties over 32,768-token "
                    "histories, half near-flat rows (top_p 0.99), half peaked rows with ties at the top-k "
                    "boundary (top_k 50, top_p 0.9, min_p 0.02), seeded Philox",
        "batch_per_gpu": batch, "vocab": vocab, "history_len": history_len,
        "sharding": f"rows x{n_gpus}, no inter-GPU traffic",
        "cache": f"{ROTATING_SETS} rotating input sets of {batch * vocab * 2 / 1e6:.0f} MB each (> 126 MB L2)",
    }
    if extra:
        cfg.update(extra)
    return cfg


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, uuid):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", uuid], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            pass

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# --------------------------------------------------------------------------- CPU arms
_CPU_ROWS = None


def _cpu_rows_worker(index_range):
    import torch

    from oracle import reference_port

    torch.set_num_threads(1)
    logits, histories, params, steps = _CPU_ROWS
    lo, hi = index_range
    if hi <= lo:
        return 0
    reference_port.sample_batch(logits[lo:hi], histories[lo:hi], params[lo:hi], steps[lo:hi])
    return hi - lo


def cpu_sample_of(w, n_rows):
    """A bounded sample of the workload's rows covering both row classes evenly."""
    import torch

    half = w.batch // 2
    take = list(range(n_rows // 2)) + list(range(half, half + n_rows - n_rows // 2))
    sub = w.rows(take)
    logits = torch.from_numpy(sub.logits.view(np.int16)).view(torch.bfloat16)
    return logits, [h.tolist() for h in sub.histories], sub.params, sub.steps


def time_cpu_single(w, n_rows):
    """The reference's deployment shape: one process, its per-row Python loop, default
    torch intra-op threads."""
    import torch

    from oracle import reference_port

    logits, histories, params, steps = cpu_sample_of(w, n_rows)
    reference_port.sample_batch(logits[:2], histories[:2], params[:2], steps[:2])
    t0 = time.perf_counter()
    reference_port.sample_batch(logits, histories, params, steps)
    dt = time.perf_counter() - t0
    return n_rows / dt, torch.get_num_threads(), dt


def run_reference_arm(args, world, rank):
    """bench.py --impl reference: the reference's CPU path on all host cores, rows split
    over one single-threaded process per core (the shape most favourable to the CPU)."""
    global _CPU_ROWS
    if rank != 0:
        return
    import multiprocessing as mp

    from hydraserve_b200 import workloads

    cores = os.cpu_count() or 1
    procs = max(1, min(cores, 64))
    rows_per_step = max(16, 2 * procs)
    w = workloads.config3(batch=max(rows_per_step, 2))
    _CPU_ROWS = cpu_sample_of(w, rows_per_step)
    bounds = np.linspace(0, rows_per_step, procs + 1).astype(int)
    ranges = [(int(bounds[i]), int(bounds[i + 1])) for i in range(procs)]
    ctx = mp.get_context("fork")
    with ctx.Pool(procs) as pool:
        for _ in range(max(args.warmup, 1)):
            pool.map(_cpu_rows_worker, ranges)
        t0 = time.perf_counter()
        for _ in range(args.steps):
            pool.map(_cpu_rows_worker, ranges)
        dt = time.perf_counter() - t0
    value = rows_per_step * args.steps / dt
    sample = (f"{rows_per_step} rows per step (half near-flat, half peaked) of the 256 x 248,320 workload, "
              f"split over {procs} single-threaded processes")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3 * 256 / rows_per_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(256, 248_320, 32_768, args.gpus, {"cache": "host memory"}),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": procs, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "the reference is Python and does not travel to this box; its CPU operator sequence is timed "
                "through oracle/reference_port.py (checked against the reference's outputs in tests/test_oracle.py); "
                "ms_per_step is scaled to the full 256-row step",
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- GPU arm
def run_ours(args, world, rank, local_rank):
    import torch

    from hydraserve_b200 import _lib, workloads
    from hydraserve_b200.engine import _device, sample_logits

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA GPU (there is no CPU sampling path)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        dist.init_process_group("nccl", device_id=device)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    w = workloads.config3(seed=3 + 1000 * rank, batch=args.batch, vocab=args.vocab, history_len=args.history)
    batch, vocab = w.batch, w.vocab
    sampler = _device.DeviceSampler(device, vocab_max=vocab, batch_max=batch, resident_slots=batch)
    lib, handle = sampler.lib, sampler.handle

    # device-resident histograms, one slot per row (request); built once, outside the timed region
    slots = list(range(batch))
    sampler.reset_slots(slots)
    sampler.append_tokens(slots, w.histories, vocab)
    uniques = [int(np.unique(h[(h >= 0) & (h < vocab)]).size) for h in w.histories]

    host_logits = torch.from_numpy(w.logits.view(np.int16)).view(torch.bfloat16).pin_memory()
    sets = [host_logits.to(device, non_blocking=True).clone() for _ in range(ROTATING_SETS)]
    total_steps = args.steps + args.warmup
    # one parameter set per step: the step number advances the seeded stream, as in serving.
    # (Replaying a few sets round robin while the sampled tokens are appended makes every
    # replayed draw land on the token it already moved out of its class.)
    n_param_sets = min(total_steps, 2048)
    param_sets = []
    for i in range(n_param_sets):
        rec = _device.pack_params(w.params, [s + i for s in w.steps], slots)
        param_sets.append(sampler._to_device(rec.view(np.uint8).reshape(batch, -1)))
    d_out = torch.empty((batch, _lib.ROW_OUT.itemsize), dtype=torch.uint8, device=device)
    stream = C.c_void_p(torch.cuda.current_stream(device).cuda_stream)
    torch.cuda.synchronize()

    def step(i):
        st = lib.hs_sample(handle, sets[i % ROTATING_SETS].data_ptr(), _lib.HS_DTYPE_BF16, vocab, batch, vocab,
                           param_sets[i % n_param_sets].data_ptr(), d_out.data_ptr(), None, None,
                           _lib.HS_SAMPLE_APPEND_TOKEN, stream)
        if st != 0:
            raise RuntimeError(lib.hs_last_error(handle).decode())

    for i in range(args.warmup):
        step(i)
    launches0 = sampler.query(3, vocab)
    uuid = str(torch.cuda.get_device_properties(device).uuid)
    clocks = ClockSampler(uuid if uuid.startswith("GPU-") else "GPU-" + uuid) if rank == 0 else None
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.warmup, total_steps):
        step(i)
    e1.record()
    barrier()
    elapsed_ms = e0.elapsed_time(e1)
    launches = sampler.query(3, vocab) - launches0
    clock_info = clocks.stop() if clocks else None
    records = d_out.cpu().numpy().view(_lib.ROW_OUT).reshape(batch)
    if int((records["status"] != 0).sum()):
        raise RuntimeError("a row reported a non-zero status")
    if dist is not None:
        t = torch.tensor([elapsed_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    ms_per_step = elapsed_ms / args.steps
    value = world * batch * args.steps / (elapsed_ms * 1e-3)

    # ---- end to end through the drop-in Python API, logits in pinned host memory -------
    e2e_steps = 0 if args.kernel_only else max(1, min(args.steps, args.e2e_steps))
    histories = [h.tolist() for h in w.histories]
    request_ids = [f"bench-{rank}-{i}" for i in range(batch)]
    e2e_sampler = _device.sampler_for(device, vocab, batch) if e2e_steps else None
    steps_now = list(w.steps)
    h2d = host_logits.numel() * 2 + batch * _lib.ROW_PARAMS.itemsize + batch * 4 * 3
    d2h = batch * _lib.ROW_OUT.itemsize

    def e2e_step():
        out = sample_logits(host_logits, histories, w.params, steps=steps_now, request_ids=request_ids)
        for i, s in enumerate(out):
            histories[i].append(s.token_id)
            steps_now[i] += 1

    e2e_s = float("inf")
    if e2e_steps:
        for _ in range(2):
            e2e_step()  # the first call uploads the full histories; later calls only the new token
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        torch.cuda.synchronize()
        e2e_s = time.perf_counter() - t0
    if dist is not None:
        t = torch.tensor([e2e_s], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e_value = world * batch * e2e_steps / e2e_s
    del e2e_sampler

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    peaks_file = ROOT / "MEASURED_PEAKS.json"
    if peaks_file.exists():
        peak, peak_src = float(json.loads(peaks_file.read_text())["hbm_gbs"]), "measured copy bandwidth (MEASURED_PEAKS.json)"
    else:
        peak, peak_src = FALLBACK_HBM_GBS, "fallback"
    logits_bytes = batch * vocab * 2
    algo_bytes = logits_bytes + 8 * sum(uniques) + batch * (_lib.ROW_PARAMS.itemsize + _lib.ROW_OUT.itemsize)
    achieved = algo_bytes / (ms_per_step * 1e-3) / 1e9
    roofline = {
        "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
        "traffic": NCU_DRAM_BYTES_PER_STEP if (batch, vocab, args.history) == (256, 248_320, 32_768) else None,
        "kernel": "hs::row_kernel_v3 (counting rows) and hs::row_kernel_topk (small top_k rows), side by side on "
                  "two streams; one step = both",
        "peak_source": peak_src,
        "algorithmic_bytes_per_launch": algo_bytes, "logits_bytes_per_launch": logits_bytes,
        "logits_only_gbs": logits_bytes / (ms_per_step * 1e-3) / 1e9,
    }
    cpu = None
    if world == 1 and not args.no_cpu and not args.kernel_only:
        rows = args.cpu_rows
        v, threads, dt = time_cpu_single(w, rows)
        cpu = {"value": v, "unit": UNIT, "cores": threads, "kind": "port",
               "sample": f"{rows} of the {batch} rows (half near-flat, half peaked), one process, the reference's "
                         f"per-row loop, {dt:.1f} s", "host_cores": os.cpu_count()}
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(batch, vocab, args.history, world, {"cluster_ctas_per_row": sampler.query(0, vocab),
                                             "row_staged_in_shared_memory": bool(sampler.query(1, vocab))}),
        "roofline": roofline,
        "cpu_baseline": cpu,
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "steps": e2e_steps, "path": "hydraserve_b200.engine.sample_logits(pinned host logits, request_ids=...)"},
        "gpu_launches": launches,
        "clocks": clock_info,
    }
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=500)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--vocab", type=int, default=248_320)
    ap.add_argument("--history", type=int, default=32_768)
    ap.add_argument("--e2e-steps", type=int, default=20)
    ap.add_argument("--cpu-rows", type=int, default=64)
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--kernel-only", action="store_true",
                    help="time only the device-resident steps (for profiler runs): no e2e, no CPU baseline")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference_arm(args, world, rank)
    else:
        if args.warmup < 3:
            args.warmup = 3
        run_ours(args, world, rank, local_rank)


if __name__ == "__main__":
    main()
