"""The sampler as a serving process uses it: from several threads and streams at once, with
request ids and release, with the sampled ids left on the device for the next step, and
with the result as one packed array."""
import ctypes as C
import threading

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

from hydraserve_b200 import _lib, workloads  # noqa: E402
from hydraserve_b200.engine import (SamplingParams, TokenSample, release_request, sample_logits,  # noqa: E402
                                    sample_logits_packed)
from hydraserve_b200.engine import _device  # noqa: E402
from oracle import sampler_oracle as O  # noqa: E402


@pytest.fixture(autouse=True)
def _library(built_library):
    return built_library


def bf16_cuda(bits):
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).view(torch.bfloat16).cuda()


def test_decode_loop_and_replay_thread_do_not_disturb_each_other():
    """Two threads on two streams, as the reference's decode loop and its first-token replay
    (pd_service.py:916-967, pd_worker.py:305-308, 475-480): batch-64 plain greedy on one,
    a batch-1 seeded row with penalties and logprobs on the other, 300 times each; every
    result equals the single-threaded answer."""
    rng = np.random.default_rng(71)
    vocab = 151_936
    big = bf16_cuda(workloads.f32_to_bf16_bits((rng.standard_normal((64, vocab)) * 3).astype(np.float32)))
    one = bf16_cuda(workloads.f32_to_bf16_bits((rng.standard_normal((1, vocab)) * 3).astype(np.float32)))
    greedy_params = tuple(SamplingParams() for _ in range(64))
    replay_params = (SamplingParams(temperature=0.8, top_k=40, top_p=0.9, seed=11, presence_penalty=0.4,
                                    logprobs=5),)
    history = tuple(int(t) for t in rng.integers(0, vocab, 300))
    want_greedy = sample_logits(big, [()] * 64, greedy_params, steps=[0] * 64)
    assert [s.token_id for s in want_greedy] == big.float().argmax(dim=1).tolist()
    want_replay = sample_logits(one, (history,), replay_params, steps=(3,))
    errors = []

    def decode_loop():
        try:
            with torch.cuda.stream(torch.cuda.Stream()):
                for _ in range(300):
                    if sample_logits(big, [()] * 64, greedy_params, steps=[0] * 64) != want_greedy:
                        errors.append("greedy batch differs")
                        return
        except Exception as exc:  # pragma: no cover
            errors.append(repr(exc))

    def replay():
        try:
            with torch.cuda.stream(torch.cuda.Stream()):
                for _ in range(300):
                    if sample_logits(one, (history,), replay_params, steps=(3,)) != want_replay:
                        errors.append("replayed row differs")
                        return
        except Exception as exc:  # pragma: no cover
            errors.append(repr(exc))

    threads = [threading.Thread(target=decode_loop), threading.Thread(target=replay)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=600)
    assert not any(t.is_alive() for t in threads)
    assert not errors, errors


def test_growing_the_shared_sampler_does_not_pull_it_from_under_a_caller():
    """A call that outgrows the process-wide sampler replaces it; a sampler that another call
    still holds is closed only when that call leaves."""
    device = torch.device("cuda", 0)
    with _device.lease_sampler(device, 1000, 4) as held:
        handle_before = held.handle
        with _device.lease_sampler(device, 600_000, 4) as bigger:  # larger vocabulary: a new sampler
            assert bigger is not held and bigger.vocab_max >= 600_000
            assert held.retired and held.handle is not None and held.handle is handle_before
            x = torch.randn(2, 1000, device=device)
            assert held.greedy(x).tolist() == x.argmax(dim=1).tolist()  # still usable
    assert held.handle is None  # closed once its last user left


def test_slot_outside_the_pool_is_reported_not_followed():
    """params.slot comes from device memory, so the host cannot check it: a slot number the
    sampler does not have gets no penalties and status bit 64 on every path (counting,
    candidate, general, vocabulary shard); nothing is read or written through it."""
    lib = _lib.load()
    handle = C.c_void_p()
    vocab, batch = 40_000, 4
    assert lib.hs_create(0, vocab, 2, 4096, batch, C.byref(handle)) == 0  # slots 0..5 exist
    try:
        rng = np.random.default_rng(3)
        bits = workloads.f32_to_bf16_bits((rng.standard_normal((batch, vocab)) * 2).astype(np.float32))
        params = [SamplingParams(temperature=1.0, top_p=0.9, seed=1, presence_penalty=0.5),           # counting path
                  SamplingParams(temperature=1.0, top_k=20, seed=2, frequency_penalty=0.5),          # candidate path
                  SamplingParams(temperature=0.0, repetition_penalty=1.3, logprobs=2),               # penalised greedy
                  SamplingParams(temperature=0.9, top_k=10, seed=4)]                                # no penalties
        for bad_slot in (6, 2**31 - 1):
            rec = _device.pack_params(params, [0] * batch, [bad_slot, bad_slot, bad_slot, -1])
            d_params = torch.from_numpy(rec.view(np.uint8).copy()).cuda()
            clean = _device.pack_params([SamplingParams(**{**{f: getattr(p, f) for f in p.__slots__},
                                                           "repetition_penalty": 1.0, "presence_penalty": 0.0,
                                                           "frequency_penalty": 0.0}) for p in params],
                                        [0] * batch, [-1] * batch)
            d_clean = torch.from_numpy(clean.view(np.uint8).copy()).cuda()
            for dtype, logits in ((_lib.HS_DTYPE_BF16, bf16_cuda(bits)),
                                  (_lib.HS_DTYPE_F32, torch.from_numpy(workloads.bf16_bits_to_f32(bits)).cuda())):
                outs = []
                for p in (d_params, d_clean):
                    d_out = torch.zeros((batch, _lib.ROW_OUT.itemsize), dtype=torch.uint8, device="cuda")
                    st = lib.hs_sample(handle, logits.data_ptr(), dtype, vocab, batch, vocab, p.data_ptr(),
                                       d_out.data_ptr(), None, None, _lib.HS_SAMPLE_APPEND_TOKEN, None)
                    assert st == 0, lib.hs_last_error(handle)
                    torch.cuda.synchronize()
                    outs.append(d_out.cpu().numpy().view(_lib.ROW_OUT).reshape(batch))
                got, want = outs
                assert got["status"].tolist() == [64, 64, 64, 0]
                assert want["status"].tolist() == [0, 0, 0, 0]
                np.testing.assert_array_equal(got["token"], want["token"])  # sampled as if unpenalised
                np.testing.assert_array_equal(got["n_kept"], want["n_kept"])
            recs = torch.zeros((batch, _lib.SHARD_REC.itemsize), dtype=torch.uint8, device="cuda")
            sh = _device.pack_params([params[1]] * batch, [0] * batch, [bad_slot] * batch)
            d_sh = torch.from_numpy(sh.view(np.uint8).copy()).cuda()
            st = lib.hs_sharded_partial(handle, bf16_cuda(bits).data_ptr(), _lib.HS_DTYPE_BF16, vocab, batch, vocab, 0,
                                        d_sh.data_ptr(), recs.data_ptr(), None)
            assert st == 0
            torch.cuda.synchronize()
            assert recs.cpu().numpy().view(_lib.SHARD_REC).reshape(batch)["status"].tolist() == [64] * batch
    finally:
        lib.hs_destroy(handle)


def test_memory_queries_match_the_arithmetic():
    vocab, hist_cap, slots, batch = 248_320, 32_768, 16, 8
    s = _device.DeviceSampler("cuda:0", vocab_max=vocab, batch_max=batch, resident_slots=slots, hist_cap=hist_cap)
    try:
        per_slot = s.query(6)
        assert per_slot == _device.slot_bytes(vocab, hist_cap) and per_slot <= 1.5 * 2**20
        held = s.device_bytes()
        assert held >= (slots + batch) * per_slot
        # the scratch of the bf16 kernel is sized by the CTAs that can be resident, not by the batch
        resident = s.query(7)
        assert resident >= s.query(2)
        assert held <= (slots + batch) * per_slot + resident * (18_432 * 16 + 16_384 * 8) + 64 * 2**20
    finally:
        s.close()


def test_packed_results_equal_the_tuple():
    w = workloads.config2(batch=16, vocab=32_768)
    logits = bf16_cuda(w.logits)
    as_tuple = sample_logits(logits, w.histories, w.params, steps=w.steps)
    packed = sample_logits_packed(logits, w.histories, w.params, steps=w.steps)
    assert isinstance(packed, _device.PackedSamples) and len(packed) == w.batch
    assert packed.to_samples() == as_tuple
    import pickle

    assert pickle.loads(pickle.dumps(packed)) == as_tuple
    greedy = sample_logits_packed(logits, [()] * w.batch, [SamplingParams()] * w.batch, steps=[0] * w.batch)
    assert greedy.to_samples() == tuple(TokenSample(int(t)) for t in logits.float().argmax(dim=1).tolist())


def _fake_lm_head(table, prev_tokens, step):
    """Next-step logits as a function of the previous token ids, computed on the device."""
    rows = (prev_tokens.long() * 7 + step) % table.shape[0]
    return table.index_select(0, rows)


def test_device_chained_decode_steps():
    """16 decode steps whose sampled ids never leave the device (hs_sample_ex writes them into
    the next step's input-id buffer and counts them into the histograms in its epilogue; no
    host synchronisation inside the loop) equal 16 steps that read every result back, token
    for token; first and last step are also checked against the CPU checker."""
    rng = np.random.default_rng(91)
    vocab, batch, n_steps, n_table = 50_000, 6, 16, 64
    table_bits = workloads.f32_to_bf16_bits((rng.standard_normal((n_table, vocab)) * 2.5).astype(np.float32))
    table = bf16_cuda(table_bits)
    table_f32 = workloads.bf16_bits_to_f32(table_bits)
    params = [SamplingParams(temperature=0.9, top_k=30, top_p=0.95, seed=100 + i, presence_penalty=0.3,
                             frequency_penalty=0.2, repetition_penalty=1.1) if i % 2 == 0 else
              SamplingParams(temperature=1.0, top_p=0.9, seed=100 + i, frequency_penalty=0.4, logprobs=3)
              for i in range(batch)]
    prompts = [rng.integers(0, vocab, 40).astype(np.int32) for _ in range(batch)]
    first = torch.from_numpy(np.array([int(p[-1]) for p in prompts], dtype=np.int32)).cuda()

    def run(chained: bool):
        s = _device.DeviceSampler("cuda:0", vocab_max=vocab, batch_max=batch, resident_slots=batch, hist_cap=4096)
        try:
            slots = list(range(batch))
            s.reset_slots(slots)
            s.append_tokens(slots, prompts, vocab)
            d_params = [s._to_device(_device.pack_params(params, [t] * batch, slots).view(np.uint8))
                        for t in range(n_steps)]
            d_out = [torch.zeros((batch, _lib.ROW_OUT.itemsize), dtype=torch.uint8, device="cuda")
                     for _ in range(n_steps)]
            input_ids = first.clone()
            tokens = []
            for t in range(n_steps):
                logits = _fake_lm_head(table, input_ids, t)
                nxt = torch.empty(batch, dtype=torch.int32, device="cuda")
                s.launch(logits, d_params[t], d_out[t], tokens_out=nxt, append_token=True)
                if chained:
                    input_ids = nxt  # stays on the device; nothing is read back in the loop
                else:
                    host = d_out[t].cpu().numpy().view(_lib.ROW_OUT).reshape(batch)["token"].copy()
                    tokens.append(host)
                    input_ids = torch.from_numpy(host).cuda()
            torch.cuda.synchronize()
            records = [o.cpu().numpy().view(_lib.ROW_OUT).reshape(batch).copy() for o in d_out]
            if chained:
                tokens = [r["token"].copy() for r in records]
            return np.stack(tokens), records, [s.unique_count(i) for i in slots]
        finally:
            s.close()

    chained_tokens, chained_records, uniq_a = run(True)
    host_tokens, _, uniq_b = run(False)
    np.testing.assert_array_equal(chained_tokens, host_tokens)
    assert uniq_a == uniq_b
    assert all(int((r["status"] != 0).sum()) == 0 for r in chained_records)
    # the checker on the first and the last step, with the histories the chain implies
    for t in (0, n_steps - 1):
        prev = first.cpu().numpy() if t == 0 else chained_tokens[t - 1]
        for b in range(batch):
            history = np.concatenate([prompts[b], chained_tokens[:t, b]]).astype(np.int32)
            x = table_f32[(int(prev[b]) * 7 + t) % n_table]
            o = O.sample_row(x, history, params[b], t, draws=np.ones(vocab, np.float32), want_probabilities=False)
            rec = chained_records[t][b]
            assert int(rec["n_kept"]) == o.kept.size, (t, b)
            assert int(rec["token"]) in set(o.kept.tolist())
            assert np.float32(rec["row_max"]) == o.scores[o.kept].max()


class _FakeRuntime:
    """Stands in for the model runtime of the reference's backends: decode_batch returns
    [batch, 1, vocab] logits on the device (runtime.py:631-690), here a seeded function of
    (request, position)."""

    def __init__(self, vocab, seed):
        self.vocab = vocab
        self.gen = torch.Generator(device="cuda").manual_seed(seed)
        self.table = (torch.randn((97, vocab), generator=self.gen, device="cuda") * 3).bfloat16()

    def decode_batch(self, requests):
        rows = torch.tensor([(r.request_id * 31 + len(r.generated)) % 97 for r in requests], device="cuda")
        return self.table.index_select(0, rows).unsqueeze(1)


class _Request:
    def __init__(self, request_id, prompt, params):
        self.request_id, self.prompt, self.params, self.generated = request_id, list(prompt), params, []


class _FakeBackend:
    """The sampling part of the reference's RuntimeGenerationBackend.decode / release
    (serving_loop.py:1402-1437, 1481-1488) with the two changes the integration asks for:
    request ids are passed along, and release frees the request's histogram."""

    def __init__(self, runtime, resident: bool):
        self.runtime, self.resident = runtime, resident

    def decode(self, requests):
        logits = self.runtime.decode_batch(requests)
        samples = sample_logits(
            logits[:, -1],
            histories=[r.prompt + r.generated for r in requests],
            params=[r.params for r in requests],
            steps=[len(r.generated) for r in requests],
            request_ids=[("fake", r.request_id) for r in requests] if self.resident else None)
        for r, s in zip(requests, samples):
            r.generated.append(s.token_id)
        return samples

    def release(self, request):
        if self.resident:
            release_request(("fake", request.request_id))


def test_backend_decode_loop_with_request_ids_and_release():
    """A decode loop shaped like the reference's backend: requests join and leave between
    steps, batches are re-ordered, one request is replayed after a preemption (its history
    shrinks).  With request ids (resident histograms, only new tokens uploaded) the samples
    equal those of the stateless call, and a released request gives its slot back."""
    rng = np.random.default_rng(17)
    vocab = 60_000
    mk = lambda i: _Request(i, rng.integers(0, vocab, int(rng.integers(5, 400))).tolist(),  # noqa: E731
                            SamplingParams(temperature=0.9, top_k=[0, 40][i % 2], top_p=0.92, seed=500 + i,
                                           presence_penalty=0.4, frequency_penalty=0.25, repetition_penalty=1.05,
                                           logprobs=[None, 4][i % 3 == 0]))
    histories = {}

    def drive(resident):
        nonlocal rng
        rng = np.random.default_rng(17)
        backend = _FakeBackend(_FakeRuntime(vocab, 5), resident)
        live = [mk(i) for i in range(6)]
        out = []
        for step in range(12):
            order = np.random.default_rng(step).permutation(len(live))
            batch = [live[i] for i in order]
            out.append([(r.request_id, s) for r, s in zip(batch, backend.decode(batch))])
            if step == 3:       # a request finishes
                backend.release(live.pop(1))
            if step == 5:       # a new one joins
                live.append(mk(10))
            if step == 7:       # preempt + replay: the last two tokens are generated again
                del live[0].generated[-2:]
        for r in live:
            backend.release(r)
        histories[resident] = {r.request_id: list(r.generated) for r in live}
        return out

    with_ids = drive(True)
    stateless = drive(False)
    assert with_ids == stateless
    assert histories[True] == histories[False]
    sampler = _device.sampler_for(torch.device("cuda", 0), vocab, 1)
    assert not any(isinstance(k, tuple) and k and k[0] == "fake" for k in sampler.book.entries)
