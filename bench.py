#!/usr/bin/env python
"""Benchmark of the per-step token sampler.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config 1|2|3|4|5]

A step is one pass of the sampler over one batch of synthetic logits.  The default workload
(``--config 3``) is the large-vocabulary stress configuration: 256 rows x 248,320 bf16 logits,
repetition / presence / frequency penalties over 32,768-token histories held in
device-resident histograms, top-k / top-p / min-p, seeded Philox draw; under ``--gpus N``
each rank works on its own 256 rows (weak scaling, no inter-GPU traffic).  The other
configurations of the same path:

  --config 1   the reference's CPU-runnable check, 4 x 151,936 fp32 (top_k 50 rows; --batch B for more rows)
  --config 2   decode step, 64 x 151,936 bf16, mixed parameters, 20 logprobs per row
               (small and launch-bound: the single-step latency is reported too)
  --config 4   1,024 x 151,936 bf16 with per-row random parameters, the rows split evenly
               over the N GPUs (fixed total work: strong scaling), no inter-GPU traffic
  --config 5   128 x 248,320 bf16 split by VOCABULARY over the N GPUs: per-slice candidate
               records, an NCCL all-gather of 536 bytes per row and rank, and a merge kernel;
               the three parts are timed separately and NVLink bytes reported apart from HBM

Prints one JSON line on rank 0.

value   rows/s with the logits already in HBM (CUDA events around K back-to-back steps
        over rotating input sets larger than L2, max over ranks)
e2e     rows/s through the Python drop-in ``sample_logits`` with the logits in pinned host
        memory: host-to-device copy of the step's logits, histogram delta and parameters,
        and device-to-host copy of the result records, all inside the timed region
        (``e2e_device_logits``: the same call with the logits already on the device, which
        is where a serving worker's LM head leaves them)
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
# dram__bytes_read.sum + dram__bytes_write.sum of one step's kernel on config 3, from the ncu
# capture summarised in profiles/bf16_row_kernel_config3.md
NCU_DRAM_BYTES_PER_STEP = {3: 162_255_616}

WORKLOADS = {
    1: dict(batch=4, vocab=151_936, history=256, sets=8, scaling="weak",
            text="config1: the reference's CPU-runnable check, 4 x 151,936 fp32 N(0,2.5^2) with 8 tokens per row "
                 "raised by 12; row 0 greedy, the others T 0.7, top_k 50, top_p 0.9, repetition penalty 1.1 over "
                 "256-token histories (--batch B repeats that parameter mix over B rows)"),
    2: dict(batch=64, vocab=151_936, history=4096, sets=8, scaling="weak",
            text="config2: decode step, 64 x 151,936 bf16 N(0,3^2) + Zipf bias, rows cycle through greedy / "
                 "top_p 0.95 / top_k 20 + min_p 0.05 / top_k 40 + top_p 0.8 + T 1.2, presence 0.5 and frequency 0.3 "
                 "over histories of 1-4,096 tokens, 20 logprobs per row"),
    3: dict(batch=256, vocab=248_320, history=32_768, sets=8, scaling="weak",
            text="config3: large-vocab stress, 256 x 248,320 bf16, all penalties over 32,768-token "
                 "histories, half near-flat rows (top_p 0.99), half peaked rows with ties at the top-k "
                 "boundary (top_k 50, top_p 0.9, min_p 0.02), seeded Philox"),
    4: dict(batch=1024, vocab=151_936, history=8192, sets=2, scaling="strong",
            text="config4: row-sharded decode, 1,024 x 151,936 bf16 N(0,3^2) in total, per-row parameters drawn "
                 "from a seed (T 0.3-1.5, top_k in {0,20,50,200}, top_p 0.7-1, min_p in {0,0.05}, penalties 0-0.6), "
                 "histories of 512-8,192 tokens, rows split evenly over the GPUs"),
    5: dict(batch=128, vocab=248_320, history=0, sets=8, scaling="strong",
            text="config5: vocabulary-sharded sampling, 128 x 248,320 bf16 N(0,3^2) cut into one contiguous slice "
                 "per GPU, top_k 50, top_p 0.9, T 0.8, 20 logprobs; per-slice records merged after an NCCL all-gather"),
}


def workload_config(cfg: int, n_gpus: int, batch=None, vocab=None, history=None, sets=None):
    """The `config` object of the JSON line; the same for both arms of one configuration."""
    w = WORKLOADS[cfg]
    batch = w["batch"] if batch is None else batch
    vocab = w["vocab"] if vocab is None else vocab
    history = w["history"] if history is None else history
    sets = w["sets"] if sets is None else sets
    if cfg == 4:
        sharding = f"{batch} rows in total, {batch // n_gpus} per GPU, no inter-GPU traffic"
    elif cfg == 5:
        sharding = f"vocabulary x{n_gpus} ({(vocab + n_gpus - 1) // n_gpus} tokens per GPU), NCCL all-gather of the records"
    else:
        sharding = f"rows x{n_gpus} ({batch} per GPU), no inter-GPU traffic"
    return {"workload": w["text"], "batch": batch, "vocab": vocab, "history_len": history, "sharding": sharding,
            "cache": f"GPU arm: {sets} rotating input sets, together larger than the 126 MB L2; reference arm: host memory"}


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
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": ["nvidia-smi unavailable"]}
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
        # "under load": the samples in the upper half of the observed clock range (the sampler
        # also runs while the host prepares inputs and the GPU idles at a low clock)
        busy = [v for v in sm if v >= 0.5 * max(sm)] if sm else []
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons),
                "window": "from before the warm-up to after the end-to-end leg"}


# --------------------------------------------------------------------------- workloads
def host_tensor(w):
    """A workload's logits as a host tensor of its dtype (bf16 bit patterns or fp32)."""
    import torch

    if w.dtype == "bf16":
        return torch.from_numpy(w.logits.view(np.int16)).view(torch.bfloat16)
    return torch.from_numpy(w.logits)


def make_workload(cfg: int, rank: int, world: int, args):
    from hydraserve_b200 import workloads

    w = WORKLOADS[cfg]
    batch = args.batch or w["batch"]
    vocab = args.vocab or w["vocab"]
    if cfg == 1:
        return workloads.config1(seed=1 + 1000 * rank, batch=batch, vocab=vocab)
    if cfg == 2:
        return workloads.config2(seed=2 + 1000 * rank, batch=batch, vocab=vocab)
    if cfg == 3:
        return workloads.config3(seed=3 + 1000 * rank, batch=batch, vocab=vocab,
                                 history_len=args.history if args.history is not None else w["history"])
    if cfg == 4:
        return workloads.config4(seed=4 + 1000 * rank, batch=max(1, batch // world), vocab=vocab)
    return workloads.config5(seed=5, batch=batch, vocab=vocab)  # the same rows on every rank


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
    """A bounded sample of the workload's rows, evenly spread over the batch (config 3's two
    halves, near-flat and peaked, are covered evenly)."""
    import torch

    take = sorted({int(i) for i in np.linspace(0, w.batch - 1, min(n_rows, w.batch))})
    if w.name == "config3" and w.batch >= 2:
        half = w.batch // 2
        n = min(n_rows, w.batch)
        take = list(range(n // 2)) + list(range(half, half + n - n // 2))
    sub = w.rows(take)
    logits = host_tensor(sub)
    return logits, [h.tolist() for h in sub.histories], sub.params, sub.steps


def time_cpu_single(w, n_rows):
    """The reference's deployment shape: one process, its per-row Python loop, default
    torch intra-op threads."""
    import torch

    from oracle import reference_port

    logits, histories, params, steps = cpu_sample_of(w, n_rows)
    n_rows = logits.shape[0]
    reference_port.sample_batch(logits[:2], histories[:2], params[:2], steps[:2])
    t0 = time.perf_counter()
    reference_port.sample_batch(logits, histories, params, steps)
    dt = time.perf_counter() - t0
    return n_rows / dt, torch.get_num_threads(), dt, n_rows


def run_reference_arm(args, world, rank):
    """bench.py --impl reference: the reference's CPU path on all host cores, rows split
    over one single-threaded process per core (the shape most favourable to the CPU)."""
    global _CPU_ROWS
    if rank != 0:
        return
    import multiprocessing as mp

    cores = os.cpu_count() or 1
    procs = max(1, min(cores, 64))
    rows_per_step = max(16, 2 * procs)
    cfg = args.config
    spec = dict(WORKLOADS[cfg])
    # only the sampled rows are generated: the reference arm never needs the whole batch
    ns = argparse.Namespace(batch=max(rows_per_step, 2), vocab=args.vocab, history=args.history)
    w = make_workload(cfg, 0, 1, ns)
    _CPU_ROWS = cpu_sample_of(w, rows_per_step)
    rows_per_step = int(_CPU_ROWS[0].shape[0])
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
    full = args.batch or spec["batch"]
    sample = (f"{rows_per_step} rows per step, evenly spread over the {full} x {args.vocab or spec['vocab']} workload, "
              f"split over {procs} single-threaded processes")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "rows_per_step": rows_per_step, "ms_per_full_batch": dt / args.steps * 1e3 * full / rows_per_step,
        "higher_is_better": True, "scaling": spec["scaling"], "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(cfg, args.gpus, args.batch, args.vocab, args.history, args.sets),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": procs, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "the reference is Python and does not travel to this box; its CPU operator sequence is timed "
                "through oracle/reference_port.py (checked against the reference's outputs in tests/test_oracle.py); "
                "a step is the bounded sample named in cpu_baseline.sample, ms_per_step is that step's own time",
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- GPU arm
def _peak():
    peaks_file = ROOT / "MEASURED_PEAKS.json"
    if peaks_file.exists():
        return float(json.loads(peaks_file.read_text())["hbm_gbs"]), "measured copy bandwidth (MEASURED_PEAKS.json)"
    return FALLBACK_HBM_GBS, "fallback"


def _setup_dist(world, device):
    import torch

    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        dist.init_process_group("nccl", device_id=device)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if dist is None:
            return x
        t = torch.tensor([x], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    return dist, barrier, max_over_ranks


def run_ours(args, world, rank, local_rank):
    import torch

    from hydraserve_b200 import _lib
    from hydraserve_b200.engine import _device, sample_logits

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA GPU (there is no CPU sampling path)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist, barrier, max_over_ranks = _setup_dist(world, device)
    if args.config == 5:
        run_vocab_sharded(args, world, rank, device, dist, barrier, max_over_ranks)
        return
    cfg = args.config
    spec = WORKLOADS[cfg]
    n_sets = args.sets or spec["sets"]

    uuid = str(torch.cuda.get_device_properties(device).uuid)
    clocks = ClockSampler(uuid if uuid.startswith("GPU-") else "GPU-" + uuid) if rank == 0 else None

    w = make_workload(cfg, rank, world, args)
    batch, vocab = w.batch, w.vocab
    history_len = max((int(h.size) for h in w.histories), default=0)
    sampler = _device.DeviceSampler(device, vocab_max=vocab, batch_max=batch, resident_slots=batch,
                                    hist_cap=min(vocab, max(history_len, 4096) + args.steps + args.warmup + 64))
    lib, handle = sampler.lib, sampler.handle

    # device-resident histograms, one slot per row (request); built once, outside the timed region
    slots = [i if _device._has_penalties(p) and w.histories[i].size else -1 for i, p in enumerate(w.params)]
    live = [s for s in slots if s >= 0]
    sampler.reset_slots(live)
    sampler.append_tokens(live, [w.histories[s] for s in live], vocab)
    uniques = [int(np.unique(h[(h >= 0) & (h < vocab)]).size) if slots[i] >= 0 else 0
               for i, h in enumerate(w.histories)]

    host_logits = host_tensor(w).pin_memory()
    elem = host_logits.element_size()
    dtype_code = _lib.HS_DTYPE_BF16 if w.dtype == "bf16" else _lib.HS_DTYPE_F32
    sets = [host_logits.to(device, non_blocking=True).clone() for _ in range(n_sets)]
    total_steps = args.steps + args.warmup
    # one parameter set per step: the step number advances the seeded stream, as in serving.
    # (Replaying a few sets round robin while the sampled tokens are appended makes every
    # replayed draw land on the token it already moved out of its class.)
    n_param_sets = min(total_steps, 2048)
    param_sets = []
    for i in range(n_param_sets):
        rec = _device.pack_params(w.params, [s + i for s in w.steps], slots)
        param_sets.append(torch.from_numpy(rec.view(np.uint8).copy()).to(device))
    d_out = torch.empty((batch, _lib.ROW_OUT.itemsize), dtype=torch.uint8, device=device)
    stream = C.c_void_p(torch.cuda.current_stream(device).cuda_stream)
    torch.cuda.synchronize()

    def step(i):
        st = lib.hs_sample(handle, sets[i % n_sets].data_ptr(), dtype_code, vocab, batch, vocab,
                           param_sets[i % n_param_sets].data_ptr(), d_out.data_ptr(), None, None,
                           _lib.HS_SAMPLE_APPEND_TOKEN, stream)
        if st != 0:
            raise RuntimeError(lib.hs_last_error(handle).decode())

    for i in range(args.warmup):
        step(i)
    launches0 = sampler.query(3, vocab)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.warmup, total_steps):
        step(i)
    e1.record()
    barrier()
    elapsed_ms = e0.elapsed_time(e1)
    launches = sampler.query(3, vocab) - launches0
    records = d_out.cpu().numpy().view(_lib.ROW_OUT).reshape(batch)
    if int((records["status"] != 0).sum()):
        raise RuntimeError("a row reported a non-zero status")
    elapsed_ms = max_over_ranks(elapsed_ms)
    ms_per_step = elapsed_ms / args.steps
    value = world * batch * args.steps / (elapsed_ms * 1e-3)

    # single steps with the GPU idle before each: the kernel's own duration; what a back-to-back
    # step takes beyond it is time the GPU waited for the host between launches
    single = []
    for i in range(16):
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        step(total_steps + i)
        b.record()
        torch.cuda.synchronize()
        single.append(a.elapsed_time(b))
    single_ms = statistics.median(single)

    # ---- end to end through the drop-in Python API ------------------------------------
    e2e_steps = 0 if args.kernel_only else max(1, min(args.steps, args.e2e_steps))
    h2d = host_logits.numel() * elem + batch * _lib.ROW_PARAMS.itemsize + batch * 4 * 3
    d2h = batch * _lib.ROW_OUT.itemsize

    def e2e_leg(logits, tag):
        histories = [h.tolist() for h in w.histories]
        request_ids = [f"bench-{tag}-{rank}-{i}" for i in range(batch)]
        steps_now = list(w.steps)

        def one():
            out = sample_logits(logits, histories, w.params, steps=steps_now, request_ids=request_ids)
            for i, s in enumerate(out):
                histories[i].append(s.token_id)
                steps_now[i] += 1

        for _ in range(2):
            one()  # the first call uploads the full histories; later calls only the new token
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            one()
        torch.cuda.synchronize()
        dt = max_over_ranks(time.perf_counter() - t0)
        for rid in request_ids:
            _device.release_request(rid)
        return world * batch * e2e_steps / dt, dt / e2e_steps * 1e3

    e2e_value = e2e_ms = dev_value = dev_ms = None
    if e2e_steps:
        e2e_value, e2e_ms = e2e_leg(host_logits, "host")
        dev_value, dev_ms = e2e_leg(sets[0], "device")
    clock_info = clocks.stop() if clocks else None

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    peak, peak_src = _peak()
    logits_bytes = batch * vocab * elem
    algo_bytes = logits_bytes + 8 * sum(uniques) + batch * (_lib.ROW_PARAMS.itemsize + _lib.ROW_OUT.itemsize)
    achieved = algo_bytes / (ms_per_step * 1e-3) / 1e9
    default_shape = (batch, vocab) == (spec["batch"] // (world if cfg == 4 else 1), spec["vocab"])
    roofline = {
        "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
        "traffic": NCU_DRAM_BYTES_PER_STEP.get(cfg) if default_shape else None,
        "kernel": ("hs::row_kernel_bf16 (one launch per step: counting rows and candidate-row parts, two CTAs per SM)"
                   if w.dtype == "bf16" else
                   "hs::row_kernel_f32_topk (rows with 0 < top_k <= 256) + hs::row_kernel (the other rows)"),
        "peak_source": peak_src,
        "algorithmic_bytes_per_launch": algo_bytes, "logits_bytes_per_launch": logits_bytes,
        "logits_only_gbs": logits_bytes / (ms_per_step * 1e-3) / 1e9,
    }
    cpu = None
    if world == 1 and not args.no_cpu and not args.kernel_only:
        v, threads, dt, rows = time_cpu_single(w, args.cpu_rows)
        cpu = {"value": v, "unit": UNIT, "cores": threads, "kind": "port",
               "sample": f"{rows} of the {batch} rows, evenly spread, one process, the reference's per-row loop, "
                         f"{dt:.1f} s", "host_cores": os.cpu_count()}
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": spec["scaling"],
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(cfg, world, args.batch, args.vocab, args.history, n_sets),
        "roofline": roofline,
        "cpu_baseline": cpu,
        "e2e": None if e2e_value is None else {
            "value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "steps": e2e_steps, "ms_per_step": e2e_ms,
            "path": "hydraserve_b200.engine.sample_logits(pinned host logits, request_ids=...)"},
        "e2e_device_logits": None if dev_value is None else {
            "value": dev_value, "unit": UNIT, "ms_per_step": dev_ms, "steps": e2e_steps,
            "h2d_bytes_per_step": h2d - host_logits.numel() * elem, "d2h_bytes_per_step": d2h,
            "path": "the same call with the logits already on the device (where the LM head leaves them)"},
        "gpu_launches": launches,
        "single_step": {"ms": single_ms, "what": "one launch with the GPU idle before it (median of 16)",
                        "gpu_wait_for_host_us_per_step": max(0.0, (ms_per_step - single_ms) * 1e3)},
        "rows_per_gpu": batch,
        "hbm_held_mb": sampler.device_bytes() / 1e6,
        "clocks": clock_info,
    }
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def run_vocab_sharded(args, world, rank, device, dist, barrier, max_over_ranks):
    """Config 5: every rank holds a contiguous slice of the vocabulary of all 128 rows."""
    import torch

    from hydraserve_b200 import _lib
    from hydraserve_b200.engine import _device, sharded

    spec = WORKLOADS[5]
    n_sets = args.sets or spec["sets"]
    uuid = str(torch.cuda.get_device_properties(device).uuid)
    clocks = ClockSampler(uuid if uuid.startswith("GPU-") else "GPU-" + uuid) if rank == 0 else None
    w = make_workload(5, rank, world, args)
    batch, vocab = w.batch, w.vocab
    lo, hi = sharded.shard_bounds(vocab, world)[rank]
    width = hi - lo
    sampler = _device.DeviceSampler(device, vocab_max=width, batch_max=batch, resident_slots=4, hist_cap=4096)
    lib, handle = sampler.lib, sampler.handle
    local = np.ascontiguousarray(w.logits[:, lo:hi])
    host = torch.from_numpy(local.view(np.int16)).view(torch.bfloat16).pin_memory()
    # a slice is 8 MB at 8 GPUs: enough rotating sets to exceed L2 would be 16+; the sets rotate
    # all the same, and the slice size is stated in the line
    sets = [host.to(device, non_blocking=True).clone() for _ in range(n_sets)]
    total_steps = args.steps + args.warmup
    n_param_sets = min(total_steps, 512)
    param_sets = []
    for i in range(n_param_sets):
        rec = _device.pack_params(w.params, [s + i for s in w.steps], [-1] * batch)
        param_sets.append(torch.from_numpy(rec.view(np.uint8).copy()).to(device))
    recs = torch.empty((batch, _lib.SHARD_REC.itemsize), dtype=torch.uint8, device=device)
    gathered = torch.empty((world, batch, _lib.SHARD_REC.itemsize), dtype=torch.uint8, device=device)
    d_out = torch.empty((batch, _lib.ROW_OUT.itemsize), dtype=torch.uint8, device=device)
    stream = C.c_void_p(torch.cuda.current_stream(device).cuda_stream)

    def ev():
        return torch.cuda.Event(enable_timing=True)

    marks = []

    def step(i, timed):
        p = param_sets[i % n_param_sets]
        m = [ev() for _ in range(4)] if timed else None
        if timed:
            m[0].record()
        st = lib.hs_sharded_partial(handle, sets[i % n_sets].data_ptr(), _lib.HS_DTYPE_BF16, width, batch, width, lo,
                                    p.data_ptr(), recs.data_ptr(), stream)
        if st != 0:
            raise RuntimeError(lib.hs_last_error(handle).decode())
        if timed:
            m[1].record()
        if dist is not None:
            dist.all_gather_into_tensor(gathered, recs)
        else:
            gathered[0].copy_(recs)
        if timed:
            m[2].record()
        st = lib.hs_sharded_merge(handle, gathered.data_ptr(), world, batch, vocab, p.data_ptr(), d_out.data_ptr(),
                                  None, None, stream)
        if st != 0:
            raise RuntimeError(lib.hs_last_error(handle).decode())
        if timed:
            m[3].record()
            marks.append(m)

    for i in range(args.warmup):
        step(i, False)
    launches0 = sampler.query(3)
    barrier()
    e0, e1 = ev(), ev()
    e0.record()
    for i in range(args.warmup, total_steps):
        step(i, False)
    e1.record()
    barrier()
    elapsed_ms = max_over_ranks(e0.elapsed_time(e1))
    launches = sampler.query(3) - launches0
    ms_per_step = elapsed_ms / args.steps
    # the three parts, timed apart on a second, shorter pass (events between them cost a little)
    n_parts = min(args.steps, 100)
    for i in range(n_parts):
        step(total_steps + i, True)
    torch.cuda.synchronize()
    part_ms = [statistics.median(m[k].elapsed_time(m[k + 1]) for m in marks) for k in range(3)]
    part_ms = [max_over_ranks(v) for v in part_ms]
    records = d_out.cpu().numpy().view(_lib.ROW_OUT).reshape(batch)
    sharded.check_records(records)
    tokens = torch.from_numpy(records["token"].astype(np.int64)).to(device)
    if dist is not None:
        everyone = [torch.empty_like(tokens) for _ in range(world)]
        dist.all_gather(everyone, tokens)
        if not all(bool((t == everyone[0]).all()) for t in everyone):
            raise RuntimeError("ranks disagree on the sampled tokens")
    clock_info = clocks.stop() if clocks else None
    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return
    peak, peak_src = _peak()
    rec_b = _lib.SHARD_REC.itemsize
    hbm_bytes = batch * width * 2 + batch * rec_b + batch * world * rec_b + batch * (_lib.ROW_PARAMS.itemsize * 2 + _lib.ROW_OUT.itemsize)
    achieved = hbm_bytes / (ms_per_step * 1e-3) / 1e9
    line = {
        "metric": METRIC, "value": batch * args.steps / (elapsed_ms * 1e-3), "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(5, world, args.batch, args.vocab, 0, n_sets),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": None, "peak_source": peak_src, "kernel": "hs::shard_partial_kernel + hs::shard_merge_kernel",
                     "algorithmic_bytes_per_launch": hbm_bytes, "logits_bytes_per_launch": batch * width * 2,
                     "note": "per GPU; the step is latency-bound (three dependent operations on one stream)"},
        "parts_ms": {"partial_kernel": part_ms[0], "all_gather": part_ms[1], "merge_kernel": part_ms[2],
                     "what": "median per step, max over ranks, CUDA events between the parts"},
        "nvlink_bytes_per_step_per_gpu": {"sent": batch * rec_b, "received": batch * rec_b * (world - 1)},
        "cpu_baseline": None, "e2e": None,
        "gpu_launches": launches, "clocks": clock_info,
        "slice_tokens_per_gpu": width, "all_ranks_agree": True,
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
    ap.add_argument("--config", type=int, choices=[1, 2, 3, 4, 5], default=3)
    ap.add_argument("--batch", type=int, default=None, help="rows (config 4: in total over all GPUs)")
    ap.add_argument("--vocab", type=int, default=None)
    ap.add_argument("--history", type=int, default=None, help="history length (config 3)")
    ap.add_argument("--sets", type=int, default=None,
                    help="rotating input sets held on the device (profiler runs: 2)")
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
