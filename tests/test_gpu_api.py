"""The reference's own sampler tests (tests/test_sampling.py of the reference), run
against the drop-in module on the GPU, plus the host-buffer C-ABI call."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

from hydraserve_b200.engine import SamplingParams, sample_logits  # noqa: E402


@pytest.fixture(autouse=True)
def _lib(built_library):
    return built_library


def test_greedy_penalties_and_logprobs():
    # reference tests/test_sampling.py:17-30 (CPU tensor in, sampled on the GPU)
    logits = torch.tensor([[0.0, 5.0, 4.0]])
    samples = sample_logits(logits, histories=((1, 1),),
                            params=(SamplingParams(frequency_penalty=2.0, logprobs=2),), steps=(0,))
    assert samples[0].token_id == 2
    assert samples[0].logprob is not None
    assert len(samples[0].top_logprobs) == 2
    assert samples[0].top_logprobs[0][0] == 2


def test_plain_greedy_sampling_uses_batched_fast_path(monkeypatch):
    # reference tests/test_sampling.py:33-48
    import hydraserve_b200.engine.sampling as sampling

    def fail_per_row(*_args, **_kwargs):
        raise AssertionError("plain greedy sampling should not use the per-row path")

    monkeypatch.setattr(sampling, "_sample_row", fail_per_row)
    logits = torch.tensor([[0.0, 5.0, 4.0], [9.0, 2.0, 3.0]])
    samples = sampling.sample_logits(logits, histories=((1, 1), (2,)),
                                     params=(SamplingParams(), SamplingParams()), steps=(0, 4))
    assert tuple(s.token_id for s in samples) == (1, 0)


def test_batched_greedy_fast_path_can_be_disabled(monkeypatch):
    # reference tests/test_sampling.py:51-73
    import hydraserve_b200.engine.sampling as sampling

    calls = 0
    original = sampling._sample_row

    def count_per_row(*args, **kwargs):
        nonlocal calls
        calls += 1
        return original(*args, **kwargs)

    monkeypatch.setenv("HYDRASERVE_BATCHED_GREEDY", "0")
    monkeypatch.setattr(sampling, "_sample_row", count_per_row)
    logits = torch.tensor([[0.0, 5.0], [9.0, 2.0]])
    samples = sampling.sample_logits(logits, histories=((), ()),
                                     params=(SamplingParams(), SamplingParams()), steps=(0, 0))
    assert tuple(s.token_id for s in samples) == (1, 0)
    assert calls == 2


def test_sampling_without_logprobs_skips_log_softmax(monkeypatch):
    # reference tests/test_sampling.py:76-90
    import hydraserve_b200.engine.sampling as sampling

    def fail_log_softmax(*_args, **_kwargs):
        raise AssertionError("log_softmax should only run when logprobs are requested")

    monkeypatch.setattr(torch, "log_softmax", fail_log_softmax)
    sample = sampling._sample_row(torch.tensor([0.0, 5.0, 4.0]), history=(1,),
                                  params=SamplingParams(frequency_penalty=1.0), step=0)
    assert sample.token_id == 1


def test_seeded_sampling_is_independent_of_batch_order():
    # reference tests/test_sampling.py:93-111
    logits = torch.tensor([[1.0, 2.0, 3.0], [3.0, 1.0, 2.0]])
    configs = (SamplingParams(temperature=1.0, top_p=0.9, seed=123),
               SamplingParams(temperature=0.8, top_k=2, seed=456))
    together = sample_logits(logits, histories=((), ()), params=configs, steps=(3, 7))
    reversed_samples = sample_logits(logits.flip(0), histories=((), ()), params=configs[::-1], steps=(7, 3))
    assert together == reversed_samples[::-1]


def test_shape_errors_match_reference():
    with pytest.raises(ValueError, match="shape"):
        sample_logits(torch.zeros(3), histories=((),), params=(SamplingParams(),), steps=(0,))
    with pytest.raises(ValueError, match="metadata"):
        sample_logits(torch.zeros(2, 3), histories=((),), params=(SamplingParams(),), steps=(0,))


def test_cuda_tensors_bf16_and_logprob_padding():
    logits = torch.tensor([[0.5, 2.0, -1.0, 2.0]], device="cuda", dtype=torch.bfloat16)
    (s,) = sample_logits(logits, histories=((),), params=(SamplingParams(temperature=1.0, top_k=1, seed=9, logprobs=4),),
                         steps=(0,))
    assert s.token_id in (1, 3)
    assert len(s.top_logprobs) == 4
    kept = [i for i, v in s.top_logprobs if v != float("-inf")]
    assert sorted(kept) == [1, 3]
    assert abs(s.top_logprobs[0][1] - np.log(0.5)) < 1e-6


def test_host_buffer_entry_point_matches_device_entry_point():
    """hs_sample_host: host pointers in, host records out, histories rebuilt per call."""
    from hydraserve_b200 import _lib
    from hydraserve_b200.engine import _device
    from tests import cases

    w = cases.build("config2_8rows")
    lib = _lib.load()
    handle = C.c_void_p()
    assert lib.hs_create(0, w.vocab, 8, 0, w.batch, C.byref(handle)) == 0
    try:
        rec = _device.pack_params(w.params, w.steps, [-1] * w.batch)
        lens = [h.size for h in w.histories]
        offsets = np.zeros(w.batch + 1, np.int32)
        np.cumsum(lens, out=offsets[1:])
        tokens = np.concatenate(w.histories).astype(np.int32)
        for i, p in enumerate(w.params):
            if _device._has_penalties(p) and lens[i]:
                rec["slot"][i] = -2
        out = np.zeros(w.batch, dtype=_lib.ROW_OUT)
        logits = np.ascontiguousarray(w.logits)
        st = lib.hs_sample_host(handle, logits.ctypes.data, _lib.HS_DTYPE_BF16, w.vocab, w.batch, w.vocab,
                                rec.ctypes.data, out.ctypes.data, tokens.ctypes.data, offsets.ctypes.data, 0, None)
        assert st == 0, lib.hs_last_error(handle)
        sampler = _device.sampler_for(torch.device("cuda", 0), w.vocab, w.batch)
        t = torch.from_numpy(w.logits.view(np.int16)).view(torch.bfloat16).cuda()
        records, _ = sampler.sample(t, w.histories, w.params, w.steps, None)
        np.testing.assert_array_equal(out["token"], records["token"])
        np.testing.assert_array_equal(out["n_kept"], records["n_kept"])
        np.testing.assert_array_equal(out["top_ids"], records["top_ids"])
        # argument errors come back as status codes, not crashes
        assert lib.hs_sample_host(handle, logits.ctypes.data, 7, w.vocab, w.batch, w.vocab, rec.ctypes.data,
                                  out.ctypes.data, None, None, 0, None) == -1
        assert lib.hs_sample_host(handle, logits.ctypes.data, 1, w.vocab, w.batch + 1, w.vocab, rec.ctypes.data,
                                  out.ctypes.data, None, None, 0, None) == -2
    finally:
        lib.hs_destroy(handle)
