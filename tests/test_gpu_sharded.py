"""Vocabulary-sharded sampling on the GPU: the slices of every row go through
hs_sharded_partial one after the other (one process stands in for the ranks; the exchange
is a concatenation), hs_sharded_merge finishes the rows, and the result must equal the CPU
checker on the concatenated row."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

from hydraserve_b200 import workloads  # noqa: E402
from hydraserve_b200.engine import _device, sharded  # noqa: E402
from hydraserve_b200.engine.sampling import SamplingParams  # noqa: E402
from oracle import sampler_oracle as O  # noqa: E402
from tests import parity  # noqa: E402


def run_sharded(w, ranks):
    bits = torch.from_numpy(w.logits.view(np.int16)).view(torch.bfloat16).cuda()
    bounds = sharded.shard_bounds(w.vocab, ranks)
    width = bounds[0][1] - bounds[0][0]
    sampler = _device.DeviceSampler("cuda:0", vocab_max=width, batch_max=w.batch, resident_slots=4)
    noise = np.ones((w.batch, w.vocab), np.float32)
    rows = []
    for r in range(w.batch):
        q = O.exponential_draws(O.mixed_seed(w.params[r].seed, w.steps[r]), w.vocab)
        noise[r] = q
        rows.append(O.sample_row(w.logits_f32()[r], w.histories[r], w.params[r], w.steps[r], draws=q,
                                 want_probabilities=False))
    recs, d_params = [], None
    for lo, hi in bounds:
        rec, d_params = sharded.partial_records(sampler, bits[:, lo:hi].contiguous(), w.histories, w.params,
                                                w.steps, lo)
        recs.append(rec)
    gathered = torch.stack(recs)
    records, lse = sharded.merge_records(sampler, gathered, ranks, d_params, w.batch, w.vocab,
                                         noise=torch.from_numpy(noise))
    host_recs = gathered.cpu().numpy().view(np.uint8).reshape(ranks, w.batch, -1)
    sampler.close()
    return rows, records, lse.cpu().numpy(), host_recs


@pytest.mark.parametrize("ranks", [2, 4, 8])
def test_sharded_rows_match_full_row_checker(built_library, ranks):
    """Config 5 at its full size: all 128 rows, the vocabulary cut into 2, 4 and 8 slices."""
    w = workloads.config5()
    assert w.batch == 128
    rows, records, lse, _ = run_sharded(w, ranks)
    report = parity.Report()
    x = w.logits_f32()
    for r, o in enumerate(rows):
        rec = records[r]
        assert rec["status"] == 0, (r, rec["status"])
        n_top = int(rec["n_top"])
        top = list(zip(rec["top_ids"][:n_top].tolist(), rec["top_logprobs"][:n_top].tolist()))
        taken, i = {t for t, _ in top}, 0
        while len(top) < min(w.params[r].logprobs, w.vocab):  # fewer kept than asked for: -inf filler
            if i not in taken:
                top.append((i, float("-inf")))
            i += 1
        parity.compare_with_oracle(report, r, o, token=int(rec["token"]), logprob=float(rec["logprob"]), top=top,
                                   kept_n=int(rec["n_kept"]), eps=2e-7, exact_ties=True)
        assert int(rec["n_after_topk"]) == o.n_after_topk
        _, sc = O.scaled_scores(x[r], w.histories[r], w.params[r])
        want = float(np.log(np.exp(sc.astype(np.float64) - sc.max()).sum()) + sc.max())
        assert abs(lse[r] - want) <= 1e-5 * max(1.0, abs(want))
    report.assert_ok(max_sensitive_fraction=0.1, name=f"config5 full (128 rows, {ranks} slices)")


def test_sharded_with_penalties_ties_and_min_p(built_library):
    rng = np.random.default_rng(77)
    vocab, batch = 31_040 * 2, 6
    x = np.round(rng.standard_normal((batch, vocab)) * 3 * 4) / 4  # quarter steps: ties at the k-th
    bits = workloads.f32_to_bf16_bits(x.astype(np.float32))
    params = [SamplingParams(temperature=0.9, top_k=k, top_p=p, min_p=mp, seed=100 + i, logprobs=lp,
                             repetition_penalty=1.2, presence_penalty=0.3, frequency_penalty=0.1)
              for i, (k, p, mp, lp) in enumerate([(5, 0.9, 0.0, 20), (40, 1.0, 0.05, 5), (56, 0.5, 0.0, None),
                                                  (1, 0.9, 0.0, 3), (20, 0.8, 0.1, 0), (50, 0.95, 0.01, 20)])]
    hist = [rng.integers(0, vocab, 2000).astype(np.int32) for _ in range(batch)]
    w = workloads.Workload("sharded-ties", bits, "bf16", hist, params, list(range(batch)))
    rows, records, _, host_recs = run_sharded(w, 2)
    report = parity.Report()
    for r, o in enumerate(rows):
        rec = records[r]
        if rec["status"] & 32:
            # more ties at a slice's k-th value than a record holds: the row is reported as
            # failed, and the Python entry raises for it
            with pytest.raises(Exception, match="cut short"):
                sharded.check_records(records[r:r + 1])
            continue
        assert rec["status"] == 0
        n_top = int(rec["n_top"])
        top = list(zip(rec["top_ids"][:n_top].tolist(), rec["top_logprobs"][:n_top].tolist()))
        if w.params[r].logprobs is not None:
            want = min(w.params[r].logprobs, w.vocab)
            taken, i = {t for t, _ in top}, 0
            while len(top) < want:
                if i not in taken:
                    top.append((i, float("-inf")))
                i += 1
        parity.compare_with_oracle(report, r, o, token=int(rec["token"]),
                                   logprob=float(rec["logprob"]) if w.params[r].logprobs is not None else None,
                                   top=top, kept_n=int(rec["n_kept"]), eps=2e-7, exact_ties=True)
    report.assert_ok(name="sharded: penalties, ties, min-p (2 slices)")
    assert report.rows >= 3


def _nccl_worker(rank, world, port, queue):
    import os

    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        w = workloads.config5(batch=32)
        lo, hi = sharded.shard_bounds(w.vocab, world)[rank]
        bits = torch.from_numpy(np.ascontiguousarray(w.logits[:, lo:hi]).view(np.int16)).view(torch.bfloat16).cuda()
        samples = sharded.sample_logits_sharded(bits, w.histories, w.params, steps=w.steps, vocab_offset=lo,
                                                vocab_total=w.vocab)
        again = sharded.sample_logits_sharded(bits, w.histories, w.params, steps=w.steps, vocab_offset=lo,
                                              vocab_total=w.vocab)
        assert samples == again
        x = w.logits_f32()
        for r, s in enumerate(samples):
            o = O.sample_row(x[r], w.histories[r], w.params[r], w.steps[r], draws=np.ones(w.vocab, np.float32),
                             want_probabilities=False)
            assert s.token_id in set(o.kept.tolist())
            assert len(s.top_logprobs) == 20
            want = [v for _, v in o.top_logprobs]
            got = [v for _, v in s.top_logprobs]
            assert np.allclose(got, want, rtol=1e-5, atol=2e-6), (r, got[:3], want[:3])
        gathered = [None] * world
        dist.all_gather_object(gathered, [s.token_id for s in samples])
        assert all(g == gathered[0] for g in gathered)
        queue.put((rank, "ok"))
    except Exception as exc:  # pragma: no cover
        import traceback

        queue.put((rank, traceback.format_exc()))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_sampling_over_nccl(built_library):
    """One process per GPU, records exchanged with an NCCL all-gather."""
    import socket

    import torch.multiprocessing as mp

    world = min(torch.cuda.device_count(), 8)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    procs = [ctx.Process(target=_nccl_worker, args=(r, world, port, queue)) for r in range(world)]
    for p in procs:
        p.start()
    results = [queue.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(results) == [(r, "ok") for r in range(world)], results
