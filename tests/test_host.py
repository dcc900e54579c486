"""Host-side logic and the C-ABI surface; no GPU needed."""
import ctypes as C
import pickle
import re
from pathlib import Path

import numpy as np
import pytest

from hydraserve_b200.engine import SamplingParams, TokenSample
from hydraserve_b200.engine import sampling

ROOT = Path(__file__).resolve().parent.parent


def test_sampling_params_validate_production_bounds():
    # reference tests/test_sampling.py:6-14
    with pytest.raises(ValueError, match="temperature"):
        SamplingParams(temperature=-0.1)
    with pytest.raises(ValueError, match="top_p"):
        SamplingParams(top_p=0)
    with pytest.raises(ValueError, match="logprobs"):
        SamplingParams(logprobs=21)
    with pytest.raises(ValueError, match="stop"):
        SamplingParams(stop_token_sequences=((),))


@pytest.mark.parametrize("kwargs,word", [
    (dict(temperature=2.1), "temperature"), (dict(top_p=1.01), "top_p"), (dict(top_k=-1), "top_k"),
    (dict(min_p=-0.1), "min_p"), (dict(min_p=1.1), "min_p"), (dict(repetition_penalty=0.0), "repetition_penalty"),
    (dict(repetition_penalty=2.5), "repetition_penalty"), (dict(presence_penalty=-2.1), "presence_penalty"),
    (dict(frequency_penalty=2.1), "frequency_penalty"), (dict(seed=-1), "seed"), (dict(seed=2**63), "seed"),
    (dict(logprobs=-1), "logprobs"),
])
def test_sampling_params_reject_out_of_range(kwargs, word):
    with pytest.raises(ValueError, match=word):
        SamplingParams(**kwargs)


def test_sampling_params_are_frozen_slotted_picklable():
    p = SamplingParams(temperature=0.7, top_k=5, seed=3, logprobs=2, stop_token_sequences=((1, 2),))
    with pytest.raises(Exception):
        p.temperature = 1.0
    assert not hasattr(p, "__dict__")
    assert pickle.loads(pickle.dumps(p)) == p
    assert p.with_seed(9).seed == 9 and p.with_seed(9).top_k == 5
    s = TokenSample(4, -0.5, ((4, -0.5),))
    assert pickle.loads(pickle.dumps(s)) == s
    assert TokenSample(1) == TokenSample(1, None, ())


def test_greedy_and_penalty_predicates():
    assert sampling._is_plain_greedy(SamplingParams())
    assert not sampling._is_plain_greedy(SamplingParams(logprobs=0))
    assert not sampling._is_plain_greedy(SamplingParams(temperature=0.1))
    assert not sampling._is_plain_greedy(SamplingParams(presence_penalty=0.1))
    assert sampling._has_penalties(SamplingParams(repetition_penalty=1.1))
    assert sampling._has_penalties(SamplingParams(frequency_penalty=-0.1))
    assert not sampling._has_penalties(SamplingParams(temperature=1.0, top_k=4))


def test_metadata_mismatch_raises_before_touching_the_gpu():
    class FakeLogits:
        ndim = 2
        shape = (2, 3)

    with pytest.raises(ValueError, match="metadata"):
        sampling.sample_logits(FakeLogits(), ((),), (SamplingParams(),), steps=(0,))
    FakeLogits.ndim = 3
    with pytest.raises(ValueError, match="shape"):
        sampling.sample_logits(FakeLogits(), ((),), (SamplingParams(),), steps=(0,))


def test_param_packing_matches_the_c_struct():
    from hydraserve_b200 import _lib
    from hydraserve_b200.engine import _device

    ps = [SamplingParams(), SamplingParams(temperature=0.7, top_k=50, top_p=0.9, min_p=0.05, repetition_penalty=1.1,
                                           presence_penalty=0.5, frequency_penalty=0.3, seed=123, logprobs=20)]
    rec = _device.pack_params(ps, [0, 3], [-1, 4])
    assert rec.dtype.itemsize == 48 and rec.nbytes == 96
    assert rec["flags"].tolist() == [_lib.HS_ROW_PLAIN_GREEDY, 0]
    assert rec["n_logprobs"].tolist() == [-1, 20]
    assert rec["slot"].tolist() == [-1, 4]
    assert int(rec["seed"][1]) == 8709371129873690831  # (123, step 3): reference sampling.py:148
    assert rec["temperature"][1] == np.float32(0.7)
    raw = rec.view(np.uint8).reshape(2, 48)
    assert raw[1, 24:28].view(np.int32)[0] == 50 and raw[1, 32:40].view(np.uint64)[0] == 8709371129873690831


def test_history_array_drops_out_of_range_ids():
    from hydraserve_b200.engine import _device

    h = _device.history_array((-1, 3, 99, 2, 2), 3)
    assert h.dtype == np.int32 and h.tolist() == [2, 2]
    assert _device.history_array((), 5).size == 0
    assert _device.history_array(iter([1, 2, 3]), 5).tolist() == [1, 2, 3]
    assert _device.history_array(np.array([4, 5, 0]), 5).tolist() == [4, 0]


def test_library_builds_and_exports_every_declared_symbol(built_library):
    """Every function include/hs_sampler.h declares is exported by the built library and
    bound in hydraserve_b200._lib (no compute call: that needs a GPU)."""
    from hydraserve_b200 import _lib

    header = (ROOT / "include" / "hs_sampler.h").read_text()
    declared = set(re.findall(r"^\s*(?:int|const char\*)\s+(hs_[a-z_]+)\s*\(", header, flags=re.M))
    assert declared, "no declarations parsed"
    assert declared == set(_lib.EXPORTS), declared ^ set(_lib.EXPORTS)
    lib = C.CDLL(str(built_library))
    for name in declared:
        assert hasattr(lib, name), f"{name} not exported"
    lib.hs_abi_version.restype = C.c_int
    assert lib.hs_abi_version() == 1
    lib.hs_status_string.restype = C.c_char_p
    assert lib.hs_status_string(-2) == b"capacity exceeded"


def test_missing_gpu_fails_loudly():
    torch = pytest.importorskip("torch")
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(RuntimeError, match="no CPU sampling path"):
        sampling.sample_logits(torch.zeros(1, 3), ((),), (SamplingParams(temperature=1.0, seed=1),), steps=(0,))


def test_slot_book_evicts_least_recently_used_and_never_a_row_of_the_batch():
    """More live requests than resident slots: the least recently used request outside the
    current batch loses its slot; when every slot belongs to the batch, the caller is told to
    use a per-call slot (no two rows of a call may share one)."""
    from hydraserve_b200.engine._device import SlotBook

    book = SlotBook(3)
    batch = {"a", "b", "c"}
    slots = {}
    for rid in ("a", "b", "c"):
        entry, new = book.lookup(rid, batch)
        assert new and entry[1] == 0
        entry[1] = 10
        slots[rid] = entry[0]
    assert sorted(slots.values()) == [0, 1, 2]
    # a fourth request in the same batch finds every slot held by the batch: no eviction
    entry, new = book.lookup("d", batch | {"d"})
    assert entry is None and not new
    assert {rid: book.entries[rid][0] for rid in "abc"} == slots
    # touching "a" makes "b" the least recently used; a later batch without "b" evicts it
    assert book.lookup("a", {"a"})[0][0] == slots["a"]
    entry, new = book.lookup("d", {"a", "d"})
    assert new and entry[0] == slots["b"] and entry[1] == 0 and "b" not in book.entries
    # the evicted request comes back as new (its histogram is rebuilt), evicting "c"
    entry, new = book.lookup("b", {"b"})
    assert new and entry[0] == slots["c"] and "c" not in book.entries
    assert book.release("a") and not book.release("a")
    assert book.lookup("e", {"e"})[0][0] == slots["a"]
    # slots held never repeat
    held = [e[0] for e in book.entries.values()]
    assert len(held) == len(set(held)) == 3


def test_unseeded_rows_take_the_keys_they_are_given():
    from hydraserve_b200.engine import _device

    ps = [SamplingParams(temperature=1.0), SamplingParams(temperature=1.0, seed=7), SamplingParams()]
    rec = _device.pack_params(ps, [0, 1, 2], None, [11, None, None])
    assert int(rec["seed"][0]) == _device.mixed_seed(11, 0)
    assert int(rec["seed"][1]) == _device.mixed_seed(7, 1)
    assert int(rec["seed"][2]) == _device.mixed_seed(0, 2)
    again = _device.pack_params(ps, [0, 1, 2], None, [11, None, None])
    assert rec.tobytes() == again.tobytes()


def test_packed_samples_behave_like_the_tuple_and_pickle_small():
    """The array-form result: same TokenSample objects on demand, and what crosses a process
    boundary is the raw records (the reference pickles tuple[TokenSample] per step,
    pd_service.py:1097-1104).  64 rows x 20 logprobs."""
    import pickle
    import time

    from hydraserve_b200 import _lib
    from hydraserve_b200.engine import TokenSample, _device

    rng = np.random.default_rng(5)
    n = 64
    records = np.zeros(n, dtype=_lib.ROW_OUT)
    records["token"] = rng.integers(0, 151_936, n)
    records["logprob"] = -rng.random(n).astype(np.float32)
    records["n_top"] = 20
    records["top_ids"] = rng.integers(0, 151_936, (n, 20))
    records["top_logprobs"] = -np.sort(rng.random((n, 20)).astype(np.float32), axis=1)
    records["n_top"][3] = 2  # fewer candidates than requested: -inf filler, as in the reference
    params = [SamplingParams(temperature=1.0, seed=i, logprobs=20) for i in range(n)]
    params[5] = SamplingParams(temperature=1.0, seed=5)
    packed = _device.PackedSamples(records, [-1 if p.logprobs is None else p.logprobs for p in params], 151_936)
    as_tuple = _device.records_to_samples(records, params, 151_936)
    assert len(packed) == n and packed.to_samples() == as_tuple and packed == as_tuple
    assert packed[5] == TokenSample(int(records["token"][5]))
    assert len(packed[3].top_logprobs) == 20 and packed[3].top_logprobs[-1][1] == float("-inf")
    assert packed.token_ids.tolist() == [s.token_id for s in as_tuple]
    t0 = time.perf_counter()
    wire_packed = pickle.dumps(packed, protocol=pickle.HIGHEST_PROTOCOL)
    back = pickle.loads(wire_packed)
    t_packed = time.perf_counter() - t0
    t0 = time.perf_counter()
    wire_tuple = pickle.dumps(as_tuple, protocol=pickle.HIGHEST_PROTOCOL)
    pickle.loads(wire_tuple)
    t_tuple = time.perf_counter() - t0
    assert back == as_tuple and back.records.tobytes() == records.tobytes()
    assert len(wire_packed) < 64 * 208 + 512
    assert len(wire_packed) < len(wire_tuple)
    print(f"packed: {len(wire_packed)} bytes, {t_packed * 1e6:.0f} us; tuple[TokenSample]: "
          f"{len(wire_tuple)} bytes, {t_tuple * 1e6:.0f} us")


def test_slot_bytes_arithmetic():
    """Device memory per histogram slot: 8 B (id, count) + 4 B (heavy list) per distinct id the
    slot can hold, a 4-byte position and 2 bits of class per vocabulary entry."""
    from hydraserve_b200.engine import _device

    assert _device.slot_bytes(248_320, 32_768) == 12 * 32_768 + 4 * 248_320 + 4 * ((248_320 + 15) // 16 + 4) + 8
    assert _device.slot_bytes(248_320, 32_768) <= 1.5 * 2**20
    assert _device.slot_bytes(151_936, 0) == _device.slot_bytes(151_936, 151_936)


def test_token_only_builds_the_same_object_as_the_dataclass():
    import pickle

    from hydraserve_b200.engine.sampling import TokenSample, _token_only

    a, b = _token_only(7), TokenSample(7)
    assert a == b and hash(a) == hash(b) and repr(a) == repr(b)
    assert pickle.loads(pickle.dumps(a)) == b
    with pytest.raises(Exception):
        a.token_id = 8  # still frozen


def test_packed_parameters_are_cached_per_batch_of_objects_and_follow_steps_and_slots():
    from hydraserve_b200.engine import _device
    from hydraserve_b200.engine.sampling import SamplingParams

    params = [SamplingParams(temperature=0.8, top_k=5, seed=11, presence_penalty=0.5),
              SamplingParams(temperature=0.0),
              SamplingParams(temperature=1.0, top_p=0.9, seed=3)]
    first = _device.pack_params(params, [0, 1, 2], [4, -1, 6])
    again = _device.pack_params(params, [0, 1, 2], [4, -1, 6])
    np.testing.assert_array_equal(first, again)
    assert _device.batch_static(params) is _device.batch_static(list(params))  # same objects: one entry
    later = _device.pack_params(params, [5, 1, 2], [9, -1, 6])
    assert later["seed"][0] == _device.mixed_seed(11, 5) and later["seed"][2] == first["seed"][2]
    assert later["slot"].tolist() == [9, -1, 6] and first["slot"].tolist() == [4, -1, 6]
    assert _device.batch_static(params)[4] == (True, False, False)
    # equal but different objects get their own entry, with the same packed bytes
    twins = [SamplingParams(temperature=0.8, top_k=5, seed=11, presence_penalty=0.5),
             SamplingParams(temperature=0.0),
             SamplingParams(temperature=1.0, top_p=0.9, seed=3)]
    np.testing.assert_array_equal(_device.pack_params(twins, [0, 1, 2], [4, -1, 6]), first)


def test_a_row_without_history_goes_without_a_slot_with_and_without_request_ids():
    """The slot plan on the host alone (a stand-in for the device calls): a penalised row whose
    history is still empty takes no slot in a stateless call, and none with a request id
    either — the kernels pick a row's path by whether it has a slot, and the path decides where
    a seeded draw lands, so both calls must present the row the same way.  The request keeps
    the (reset) slot it was given and uses it from its first token on."""
    from types import SimpleNamespace

    from hydraserve_b200.engine import _device
    from hydraserve_b200.engine.sampling import SamplingParams

    calls = []
    fake = SimpleNamespace(book=_device.SlotBook(4), scratch_base=100,
                           reset_slots=lambda slots: calls.append(("reset", list(slots))),
                           append_tokens=lambda slots, tokens, vocab: calls.append(
                               ("append", list(slots), [list(t) for t in tokens])))
    fake._slot_for_request = lambda *a: _device.DeviceSampler._slot_for_request(fake, *a)
    plan = lambda *a, **k: _device.DeviceSampler.plan_slots(fake, *a, **k)  # noqa: E731
    params = [SamplingParams(temperature=1.0, top_k=40, seed=1, presence_penalty=-1.5),
              SamplingParams(temperature=1.0, top_k=40, seed=2, presence_penalty=0.5),
              SamplingParams(temperature=1.0, seed=3)]
    assert plan([[], [7, 7, 9], [1, 2]], params, 1000) == [-1, 101, -1]
    assert calls == [("reset", [101]), ("append", [101], [[7, 7, 9]])]
    calls.clear()
    slots = plan([[], [7, 7, 9], [1, 2]], params, 1000, request_ids=["a", "b", "c"])
    held = {rid: e[0] for rid, e in fake.book.entries.items()}
    assert slots == [-1, held["b"], -1] and set(held) == {"a", "b"}
    assert calls == [("reset", [held["a"], held["b"]]), ("append", [held["b"]], [[7, 7, 9]])]
    calls.clear()
    # next step: both histories grew by one token; "a" now uses the slot that was reset for it
    assert plan([[5], [7, 7, 9, 4], [1, 2, 3]], params, 1000, request_ids=["a", "b", "c"]) == [held["a"], held["b"], -1]
    assert calls == [("reset", []), ("append", [held["a"], held["b"]], [[5], [4]])]
