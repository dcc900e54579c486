"""Generates tests/golden/*.npz by running the UNMODIFIED reference sampler.

Run where the reference checkout is available (it is not on the GPU box):

    python tests/golden/make_golden.py /path/to/reference [case-name prefix ...]

Inputs are never stored: each fixture names a seeded generator of
``hydraserve_b200.workloads`` (or ``tests/cases.py``) and its arguments, and holds only what
the reference produced on those inputs: the sampled token, the log-probabilities, and
the final candidate set (captured by observing the tensor the reference hands to its
last ``torch.softmax`` / ``torch.log_softmax`` call, without editing its code).
"""
from __future__ import annotations

import json
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))
if len(sys.argv) < 2:
    raise SystemExit("usage: python tests/golden/make_golden.py /path/to/reference")
REFERENCE = Path(sys.argv[1])
sys.path.insert(0, str(REFERENCE))

import hydraserve.engine.sampling as ref  # noqa: E402  (the reference)

from tests import cases  # noqa: E402


def ref_params(p):
    return ref.SamplingParams(
        temperature=p.temperature, top_p=p.top_p, top_k=p.top_k, min_p=p.min_p,
        repetition_penalty=p.repetition_penalty, presence_penalty=p.presence_penalty,
        frequency_penalty=p.frequency_penalty, seed=p.seed, logprobs=p.logprobs)


def run_reference_row(row_f32: np.ndarray, history, p, step):
    """Reference result for one row plus its final `scores` tensor."""
    seen = {}
    real_softmax, real_log_softmax = torch.softmax, torch.log_softmax

    def spy_softmax(x, *a, **k):
        seen["scores"] = x.detach().clone()
        return real_softmax(x, *a, **k)

    def spy_log_softmax(x, *a, **k):
        seen["scores"] = x.detach().clone()
        return real_log_softmax(x, *a, **k)

    torch.softmax, torch.log_softmax = spy_softmax, spy_log_softmax
    try:
        sample = ref._sample_row(torch.from_numpy(row_f32.copy()),
                                 tuple(int(t) for t in history), ref_params(p), int(step))
    finally:
        torch.softmax, torch.log_softmax = real_softmax, real_log_softmax
    scores = seen.get("scores")
    return sample, None if scores is None else scores.numpy()


def make_fixture(case_name: str, out: Path, keep_ids_below: int = 20000) -> dict:
    w = cases.build(case_name)
    x = w.logits_f32()
    tokens, logprobs, has_lp = [], [], []
    top_ids, top_vals, top_off = [], [], [0]
    kept_ids, kept_off, kept_n, kept_sum, kept_min = [], [0], [], [], []
    for r in range(w.batch):
        sample, scores = run_reference_row(x[r], w.histories[r], w.params[r], w.steps[r])
        tokens.append(sample.token_id)
        has_lp.append(sample.logprob is not None)
        logprobs.append(np.nan if sample.logprob is None else sample.logprob)
        for i, v in sample.top_logprobs:
            top_ids.append(i)
            top_vals.append(v)
        top_off.append(len(top_ids))
        if scores is None:  # greedy row without logprobs: nothing but the token is defined
            kept_n.append(-1); kept_sum.append(0); kept_min.append(np.nan)
            kept_off.append(len(kept_ids))
            continue
        ids = np.nonzero(np.isfinite(scores))[0]
        kept_n.append(ids.size)
        kept_sum.append(int(ids.astype(np.int64).sum()))
        kept_min.append(float(scores[ids].min()))
        if ids.size <= keep_ids_below:
            kept_ids.extend(ids.tolist())
        kept_off.append(len(kept_ids))
    np.savez_compressed(
        out,
        case=np.array(case_name),
        tokens=np.asarray(tokens, np.int64),
        has_logprob=np.asarray(has_lp, bool),
        logprobs=np.asarray(logprobs, np.float64),
        top_ids=np.asarray(top_ids, np.int64), top_vals=np.asarray(top_vals, np.float64),
        top_off=np.asarray(top_off, np.int64),
        kept_ids=np.asarray(kept_ids, np.int32), kept_off=np.asarray(kept_off, np.int64),
        kept_n=np.asarray(kept_n, np.int64), kept_sum=np.asarray(kept_sum, np.int64),
        kept_min=np.asarray(kept_min, np.float64),
    )
    return {"case": case_name, "rows": w.batch, "vocab": w.vocab, "bytes": out.stat().st_size}


def main() -> None:
    torch.set_num_threads(1)
    # further arguments: prefixes of the cases to (re)generate; the others keep their files
    # and their manifest entries
    prefixes = tuple(sys.argv[2:])
    manifest = HERE / "MANIFEST.json"
    old = {f["case"]: f for f in json.loads(manifest.read_text())["fixtures"]} if prefixes and manifest.exists() else {}
    meta = {"torch": torch.__version__, "numpy": np.__version__, "fixtures": []}
    for name in cases.GOLDEN_CASES:
        if prefixes and not name.startswith(prefixes) and name in old:
            meta["fixtures"].append(old[name])
            continue
        info = make_fixture(name, HERE / f"{name}.npz")
        print(info)
        meta["fixtures"].append(info)
    manifest.write_text(json.dumps(meta, indent=1) + "\n")


if __name__ == "__main__":
    main()
