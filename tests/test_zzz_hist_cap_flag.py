"""hs_query(what = 8): the flag the histogram kernels raise when a slot is asked to hold more
distinct ids than hist_cap.  The Python host sizes hist_cap by the longest history, so only a
caller of the C ABI can get there; the ids beyond the capacity are left out (no penalty), never
written anywhere.

Collected after the rest of the suite on purpose (file name): this case had not run on a GPU
when it was written."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def test_more_distinct_ids_than_hist_cap_raise_the_flag_and_are_left_out(built_library):
    from hydraserve_b200.engine import _device

    vocab = 1000
    s = _device.DeviceSampler("cuda:0", vocab_max=vocab, batch_max=2, resident_slots=2, hist_cap=8)
    try:
        assert s.query(8) == 0
        s.reset_slots([0, 1])
        s.append_tokens([0, 1], [np.arange(8, dtype=np.int32), np.full(30, 5, np.int32)], vocab)
        assert s.query(8) == 0 and s.unique_count(0) == 8 and s.unique_count(1) == 1
        # twenty more distinct ids for slot 0, which is full; slot 1 takes two more
        s.append_tokens([0, 1], [np.arange(100, 120, dtype=np.int32), np.array([5, 6, 7], np.int32)], vocab)
        assert s.query(8) == 1
        assert s.unique_count(0) == 8 and s.unique_count(1) == 3
        # the flag stays up, and the sampler still works: the full slot penalises its eight ids
        from hydraserve_b200.engine.sampling import SamplingParams

        logits = torch.full((1, vocab), -1.0, dtype=torch.bfloat16, device="cuda")
        logits[0, :8] = 4.0          # the eight counted ids lead ...
        logits[0, 100] = 3.0         # ... ahead of an id that was left out
        rec = _device.pack_params([SamplingParams(temperature=0.0, presence_penalty=2.0)], [0], [0])
        records, _ = s.run(logits, rec)
        assert int(records["status"][0]) == 0 and int(records["token"][0]) == 100  # 4 - 2 < 3, and 100 unpenalised
        assert s.query(8) == 1
    finally:
        s.close()
