"""The kernels' seeded stream, bit for bit: which token a seeded draw lands on when the
candidate set is 256 equally likely tokens must be the one the published Philox4x32-10 words
name.  (The chi-square tests show that draws follow the distribution; this shows that the stream
is the generator it claims to be: counter 0, key = the row's 63-bit stream key.)

With n equal masses q the inverse-CDF draw is index = floor(mulhi(r64, n q) / q), and for
n = 256 that is the top byte of the first Philox word; candidates are laid out by ascending id
on the candidate paths (equal scores sort by id) and in the general kernel (id order).

Collected after the rest of the suite on purpose (file name): this case had not run on a GPU
when it was written."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

from oracle.philox import first_draw_words  # noqa: E402


@pytest.mark.parametrize("kind", ["bf16 candidate kernel", "fp32 candidate kernel", "general kernel (fp32, min-p)"])
def test_seeded_draws_land_where_the_published_generator_says(built_library, kind):
    from hydraserve_b200.engine import _device
    from hydraserve_b200.engine.sampling import SamplingParams

    rng = np.random.default_rng(2027)
    vocab, batch = 32_000, 64
    s = _device.DeviceSampler("cuda:0", vocab_max=vocab, batch_max=batch, resident_slots=batch)
    try:
        for launch in range(3):
            # the other tokens are spread out below the leaders (a row tied at one value below
            # them would overflow a candidate list and be served by another path)
            logits = np.minimum(rng.standard_normal((batch, vocab)) - 5.0, 2.0).astype(np.float32)
            leaders = [np.sort(rng.choice(vocab, 256, replace=False)) for _ in range(batch)]
            for r in range(batch):
                logits[r, leaders[r]] = 5.0
            seeds = [int(v) for v in rng.integers(0, 2**63 - 1, batch)]
            steps = [int(v) for v in rng.integers(0, 100_000, batch)]
            if kind == "general kernel (fp32, min-p)":
                params = [SamplingParams(temperature=1.0, min_p=0.5, seed=sd) for sd in seeds]
            else:
                params = [SamplingParams(temperature=1.0, top_k=256, seed=sd) for sd in seeds]
            x = torch.from_numpy(logits).cuda()
            if kind == "bf16 candidate kernel":
                x = x.bfloat16()  # (5 is a bf16 value; the others may round as they like)
            records, _ = s.sample(x, [[] for _ in range(batch)], params, steps, None)
            assert int((records["status"] != 0).sum()) == 0
            assert (records["n_kept"] == 256).all()
            for r in range(batch):
                word0 = first_draw_words(_device.mixed_seed(seeds[r], steps[r]))[0]
                want = int(leaders[r][word0 >> 24])
                assert int(records["token"][r]) == want, (kind, launch, r, int(records["token"][r]), want)
    finally:
        s.close()
