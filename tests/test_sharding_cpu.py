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


def _seed_worker(rank, world, port, queue):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from hydraserve_b200.engine import SamplingParams, _device

        torch.manual_seed(1000 + 17 * rank)  # the ranks' global generators differ
        for _ in range(rank * 3):
            torch.rand(())
        params = [SamplingParams(temperature=1.0, top_k=5), SamplingParams(temperature=0.8, top_k=9, seed=4),
                  SamplingParams(temperature=1.2, top_k=2)]
        keys = sharded.agree_on_unseeded_keys(params)
        rec = _device.pack_params(params, [3, 4, 5], None, keys)
        mine = [int(v) for v in rec["seed"]]
        everyone = [None] * world
        dist.all_gather_object(everyone, mine)
        assert all(e == everyone[0] for e in everyone), everyone
        assert keys[1] is None and keys[0] is not None and keys[0] != keys[2]
        # every row seeded: nothing to agree on, no collective is issued
        assert sharded.agree_on_unseeded_keys([SamplingParams(temperature=1.0, top_k=5, seed=1)]) is None
        queue.put((rank, "ok"))
    except Exception as exc:  # pragma: no cover - reported to the parent
        queue.put((rank, repr(exc)))
    finally:
        dist.destroy_process_group()


def test_unseeded_rows_get_the_same_stream_key_on_every_rank():
    """Rows with seed=None take their stream key from torch's global generator, whose state
    differs between ranks: rank 0's keys are broadcast so that tensor-parallel replicas draw
    the same token."""
    world = 2
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_seed_worker, args=(r, world, port, queue)) for r in range(world)]
    for p in procs:
        p.start()
    results = [queue.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(results) == [(0, "ok"), (1, "ok")], results
