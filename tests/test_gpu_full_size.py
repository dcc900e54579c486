"""The benchmark configurations at their FULL size against the CPU checker, through the C
ABI: every row of configs 2 and 3, a seeded quarter of config 4's 1,024 rows (launched as
one 1,024-row call, so the kernel runs with that batch's launch geometry), plus the
properties that need no checker (reproducibility, independence of the batch order, the two
independent CUDA implementations agreeing).  Config 5 is in test_gpu_sharded.py."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

from hydraserve_b200 import _lib, workloads  # noqa: E402
from hydraserve_b200.engine import _device  # noqa: E402
from tests.test_gpu_parity import compare_case, device_logits  # noqa: E402

# Measured shares of rounding-sensitive rows (a cut closer than 2e-7 relative to its
# threshold) plus a margin; see the "parity row counts" table the run prints.
MAX_SENSITIVE = {"config2": 0.10, "config3": 0.15, "config4": 0.10}


def test_config2_every_row(built_library):
    w = workloads.config2()
    s = _device.DeviceSampler("cuda:0", vocab_max=w.vocab, batch_max=w.batch, resident_slots=4, hist_cap=8192)
    try:
        assert s.query(4, w.vocab) == 1
        compare_case(s, w).assert_ok(max_sensitive_fraction=MAX_SENSITIVE["config2"], name="config2 full (64 rows)")
    finally:
        s.close()


def test_config3_every_row(built_library):
    w = workloads.config3()
    B, V = w.batch, w.vocab
    fast = _device.DeviceSampler("cuda:0", vocab_max=V, batch_max=B, resident_slots=4, hist_cap=32_768)
    try:
        assert fast.query(4, V) == 1
        compare_case(fast, w).assert_ok(max_sensitive_fraction=MAX_SENSITIVE["config3"], name="config3 full (256 rows)")
        logits = device_logits(w)
        # reproducible, and independent of where a row sits in the batch (seeded Philox draws)
        p1, _ = fast.sample(logits, w.histories, w.params, w.steps, None)
        p2, _ = fast.sample(logits, w.histories, w.params, w.steps, None)
        np.testing.assert_array_equal(p1["token"], p2["token"])
        perm = np.random.default_rng(0).permutation(B)
        wp = w.rows(perm.tolist())
        p3, _ = fast.sample(device_logits(wp), wp.histories, wp.params, wp.steps, None)
        np.testing.assert_array_equal(p3["token"], p1["token"][perm])
        np.testing.assert_array_equal(p3["n_kept"], p1["n_kept"][perm])
        # a Philox-drawn token lies in its candidate set: its score is at or above the cut
        scored, scores = fast.sample(logits, w.histories, w.params, w.steps, None, want_scores=True)
        picked = scores[torch.arange(B, device=scores.device),
                        torch.from_numpy(scored["token"].astype(np.int64)).to(scores.device)]
        assert bool(torch.isfinite(picked).all()), "a drawn token is outside its candidate set"
        np.testing.assert_array_equal(torch.isfinite(scores).sum(dim=1).cpu().numpy(), scored["n_kept"])
        del scores
        assert int(p1["n_kept"][: B // 2].min()) > 10_000  # the near-flat half keeps more than 10,000 tokens
        # the general (fp32-resident) kernel, an independent implementation, agrees on every exact field
        general = _device.DeviceSampler("cuda:0", vocab_max=V, batch_max=B, resident_slots=4, hist_cap=32_768,
                                        flags=_lib.HS_CREATE_FORCE_GENERAL)
        try:
            assert general.query(4, V) == 0
            gen = torch.Generator(device="cuda").manual_seed(1234)
            noise = torch.empty((B, V), dtype=torch.float32, device="cuda").exponential_(1.0, generator=gen)
            a, _ = fast.sample(logits, w.histories, w.params, w.steps, None, noise=noise)
            b, _ = general.sample(logits, w.histories, w.params, w.steps, None, noise=noise)
            for field in ("token", "n_kept", "n_after_topk", "n_after_minp", "n_after_topp", "cut_bits", "n_cut_ties"):
                np.testing.assert_array_equal(a[field], b[field], err_msg=field)
            np.testing.assert_array_equal(a["row_max"].view(np.uint32), b["row_max"].view(np.uint32))
        finally:
            general.close()
    finally:
        fast.close()


@pytest.mark.parametrize("split", [0, 2])
def test_config4_full_batch_geometry(built_library, split):
    """1,024 rows in one call (one CTA per candidate row at that size; also with two, the
    geometry of a smaller batch); a seeded quarter of the rows against the checker."""
    w = workloads.config4()
    assert w.batch == 1024
    s = _device.DeviceSampler("cuda:0", vocab_max=w.vocab, batch_max=w.batch, resident_slots=4, hist_cap=8192)
    try:
        s.set_split(split)
        pick = np.sort(np.random.default_rng(44 + split).choice(w.batch, 256 if split == 0 else 64, replace=False))
        compare_case(s, w, only=pick.tolist()).assert_ok(
            max_sensitive_fraction=MAX_SENSITIVE["config4"],
            name=f"config4 at batch 1,024 ({pick.size} rows checked, split {split or 'auto'})")
    finally:
        s.close()
