"""Vocabulary-sharded sampling: each rank holds a contiguous slice of the logits' vocabulary
dimension (a tensor-parallel LM head) and every rank returns the same samples.

The reference has no sharded head; the result is defined as ``sample_logits`` on the
concatenated ``[batch, vocab_total]`` logits (reference sampling.py:54-163).  Per rank one
CUDA kernel reduces each row's slice to its top-k candidates, maximum and soft-max
denominator (``hs_sharded_partial``), the 536-byte records are all-gathered with
``torch.distributed`` (NCCL over NVLink), and a second kernel finishes every row from the
union of the candidates (``hs_sharded_merge``).  Every row needs ``0 < top_k <= 56``.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from .. import _lib
from . import _device
from .sampling import SamplingParams, TokenSample, _has_penalties

MAX_TOP_K = _lib.HS_SHARD_CAND - 8


def shard_bounds(vocab: int, ranks: int):
    width = (vocab + ranks - 1) // ranks
    return [(r * width, min(vocab, (r + 1) * width)) for r in range(ranks)]


def local_history(history, lo: int, hi: int) -> np.ndarray:
    h = np.asarray(history, dtype=np.int64).reshape(-1)
    return (h[(h >= lo) & (h < hi)] - lo).astype(np.int32)


def check_params(params) -> None:
    for p in params:
        if not 0 < p.top_k <= MAX_TOP_K:
            raise ValueError(f"vocabulary-sharded sampling needs 0 < top_k <= {MAX_TOP_K} on every row")
        if p.temperature == 0.0:
            raise ValueError("vocabulary-sharded sampling is for sampled rows (temperature > 0)")


def agree_on_unseeded_keys(params, group=None):
    """Stream keys for rows that sample without a seed, the SAME on every rank: rank 0 of the
    group draws them (from torch's global generator, where the reference gets its unseeded
    draws, sampling.py:145) and broadcasts them.  None when every sampled row has a seed."""
    import torch
    import torch.distributed as dist

    if not any(p.seed is None and p.temperature != 0.0 for p in params):
        return None
    keys = _device.draw_unseeded_keys(params)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        packed = torch.tensor([-1 if k is None else k for k in keys], dtype=torch.int64)
        backend = dist.get_backend(group)
        if backend == "nccl":
            packed = packed.cuda()
        dist.broadcast(packed, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        keys = [None if k < 0 else int(k) for k in packed.cpu().tolist()]
    return keys


def partial_records(sampler, local_logits, histories, params, steps, vocab_offset: int, unseeded_keys=None):
    """This rank's [batch] records (a uint8 CUDA tensor of 536-byte rows) and the packed
    parameters (device tensor) that the merge needs."""
    torch = sampler.torch
    check_params(params)
    logits, dtype, stride = sampler.prepare_logits(local_logits)
    batch, width = logits.shape
    lo, hi = vocab_offset, vocab_offset + width
    with sampler.lock:
        slots = [-1] * batch
        resets, appends = [], []
        for i, p in enumerate(params):
            if not _has_penalties(p):
                continue
            tokens = local_history(histories[i], lo, hi)
            if tokens.size == 0:
                continue
            slots[i] = sampler.scratch_base + i
            resets.append(slots[i])
            appends.append((slots[i], tokens))
        sampler.reset_slots(resets)
        sampler.append_tokens([s for s, _ in appends], [t for _, t in appends], width)
        rec = _device.pack_params(params, steps, slots, unseeded_keys)
        d_params = sampler._to_device(rec.view(np.uint8).reshape(batch, -1))
        recs = torch.empty((batch, _lib.SHARD_REC.itemsize), dtype=torch.uint8, device=sampler.device)
        st = sampler.lib.hs_sharded_partial(sampler.handle, logits.data_ptr(), dtype, stride, batch, width,
                                            vocab_offset, d_params.data_ptr(), recs.data_ptr(), sampler._stream())
        _lib.check(sampler.lib, sampler.handle, st, "hs_sharded_partial")
    return recs, d_params


def merge_records(sampler, all_recs, ranks: int, d_params, batch: int, vocab_total: int, *, noise=None):
    """all_recs: [ranks, batch, 536] uint8 CUDA tensor.  Returns (records, full log-sum-exp)."""
    torch = sampler.torch
    d_out = torch.empty((batch, _lib.ROW_OUT.itemsize), dtype=torch.uint8, device=sampler.device)
    lse = torch.empty(batch, dtype=torch.float32, device=sampler.device)
    d_noise = noise.to(sampler.device, dtype=torch.float32).contiguous() if noise is not None else None
    st = sampler.lib.hs_sharded_merge(sampler.handle, all_recs.data_ptr(), ranks, batch, vocab_total,
                                      d_params.data_ptr(), d_out.data_ptr(),
                                      d_noise.data_ptr() if d_noise is not None else None, lse.data_ptr(),
                                      sampler._stream())
    _lib.check(sampler.lib, sampler.handle, st, "hs_sharded_merge")
    host = sampler._pinned_records(batch)
    host.copy_(d_out, non_blocking=True)
    torch.cuda.current_stream(sampler.device).synchronize()
    return host.numpy().view(_lib.ROW_OUT).reshape(batch).copy(), lse


def check_records(records) -> None:
    """A record whose candidates were cut short (a slice's list overflowed, or more ties at
    the k-th value than a record holds) cannot be finished exactly: raise instead of
    returning a token drawn from a wrong candidate set."""
    bad = records["status"] & (_device.STATUS_SHARD_CUT | _device.STATUS_APPEND_FAILED | _device.STATUS_BAD_SLOT)
    if bad.any():
        row = int(np.argmax(bad != 0))
        raise _lib.SamplerError(
            f"vocabulary-sharded sampling: row {row} reported status {int(records['status'][row])} "
            "(a shard's candidate record was cut short); sample this batch from the gathered full rows instead")


def sample_logits_sharded(local_logits, histories, params, *, steps, vocab_offset: int, vocab_total: int,
                          group=None) -> tuple[TokenSample, ...]:
    """Every rank of ``group`` calls this with its own slice ``[batch, width]`` (bf16, CUDA)
    and the SAME histories / params / steps; every rank gets the same samples."""
    import torch
    import torch.distributed as dist

    if local_logits.ndim != 2:
        raise ValueError("sampling logits must have shape [batch, vocabulary]")
    histories, params = tuple(histories), tuple(params)
    steps = tuple(int(s) for s in steps)
    if not (len(histories) == len(params) == len(steps) == local_logits.shape[0]):
        raise ValueError("sampling metadata must match the logits batch")
    batch, width = int(local_logits.shape[0]), int(local_logits.shape[1])
    keys = agree_on_unseeded_keys(params, group)
    hist_need = max((len(h) for h, p in zip(histories, params) if _has_penalties(p)), default=0)
    with _device.lease_sampler(local_logits.device, width, batch, hist_need) as sampler:
        recs, d_params = partial_records(sampler, local_logits, histories, params, steps, vocab_offset, keys)
        ranks = dist.get_world_size(group) if dist.is_initialized() else 1
        if ranks > 1:
            gathered = torch.empty((ranks,) + tuple(recs.shape), dtype=torch.uint8, device=recs.device)
            dist.all_gather_into_tensor(gathered, recs, group=group)
        else:
            gathered = recs.unsqueeze(0)
        records, _ = merge_records(sampler, gathered, ranks, d_params, batch, vocab_total)
    check_records(records)
    return _device.records_to_samples(records, params, vocab_total)
