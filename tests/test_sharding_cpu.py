"""The multi-GPU paths on CPU, over a real process group (gloo, world size 2).

* Row sharding: ranks take disjoint row ranges and need no exchange; the union of their
  results is the single-process result (checked with the CPU checker standing in for the
  kernel, which needs a GPU).
* Vocabulary sharding: per-slice candidates, all-gather, merge == the full-row result."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from hydraserve_b200 import workloads
from hydraserve_b200.engine import sharded
from oracle import sampler_oracle as O
from oracle import sharded_oracle as S


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, queue):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # --- vocabulary sharding -------------------------------------------------------
        w = workloads.config5(batch=4, vocab=8192)
        x = w.logits_f32()
        lo, hi = sharded.shard_bounds(w.vocab, world)[rank]
        mine = [S.partial(x[r, lo:hi], sharded.local_history(w.histories[r], lo, hi), w.params[r], lo)
                for r in range(w.batch)]
        gathered = [None] * world
        dist.all_gather_object(gathered, mine)
        tokens = []
        for r in range(w.batch):
            draws = O.exponential_draws(O.mixed_seed(w.params[r].seed, w.steps[r]), w.vocab)
            merged = S.merge(w.vocab, [gathered[k][r] for k in range(world)], w.params[r], w.steps[r], draws)
            full = O.sample_row(x[r], w.histories[r], w.params[r], w.steps[r], draws=draws)
            assert merged.token == full.token
            assert np.array_equal(merged.kept, full.kept)
            assert merged.top_logprobs == full.top_logprobs
            lse = S.full_logsumexp([gathered[k][r] for k in range(world)])
            _, sc = O.scaled_scores(x[r], w.histories[r], w.params[r])
            want = float(np.log(np.exp(sc.astype(np.float64) - sc.max()).sum()) + sc.max())
            assert abs(lse - want) < 1e-9 * max(1.0, abs(want))
            tokens.append(merged.token)
        # every rank must hold the same answer
        everyone = [None] * world
        dist.all_gather_object(everyone, tokens)
        assert all(t == everyone[0] for t in everyone)
        # --- row sharding: disjoint rows, no exchange needed for the data path -------------
        w4 = workloads.config4(batch=8, vocab=4096)
        rows = list(range(rank, w4.batch, world))
        x4 = w4.logits_f32()
        part = {r: O.sample_row(x4[r], w4.histories[r], w4.params[r], w4.steps[r]).token for r in rows}
        parts = [None] * world
        dist.all_gather_object(parts, part)
        if rank == 0:
            union = {k: v for d in parts for k, v in d.items()}
            single = {r: O.sample_row(x4[r], w4.histories[r], w4.params[r], w4.steps[r]).token
                      for r in range(w4.batch)}
            assert union == single
        queue.put((rank, "ok"))
    except Exception as exc:  # pragma: no cover - reported to the parent
        queue.put((rank, repr(exc)))
    finally:
        dist.destroy_process_group()


def test_sharded_paths_over_gloo_world_size_2():
    world = 2
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, queue)) for r in range(world)]
    for p in procs:
        p.start()
    results = [queue.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(results) == [(0, "ok"), (1, "ok")], results


def test_shard_bounds_and_history_mapping():
    assert sharded.shard_bounds(248_320, 8) == [(i * 31_040, (i + 1) * 31_040) for i in range(8)]
    assert sharded.shard_bounds(10, 3) == [(0, 4), (4, 8), (8, 10)]
    assert sharded.local_history([0, 5, 9, 4, 12, -1], 4, 8).tolist() == [1, 0]
    from hydraserve_b200.engine import SamplingParams

    with pytest.raises(ValueError, match="top_k"):
        sharded.check_params([SamplingParams(temperature=1.0)])
    with pytest.raises(ValueError, match="top_k"):
        sharded.check_params([SamplingParams(temperature=1.0, top_k=57)])
