"""Host side of the CUDA sampler: packs per-row parameters and histories, owns one C-ABI
sampler handle per GPU, and turns result records into ``TokenSample`` objects.

PyTorch is used here only for device memory, pinned host buffers and the current stream;
all arithmetic happens in the CUDA library.  There is no CPU path: host tensors are
copied to the GPU, and a machine without a GPU or without the built library raises.
"""
from __future__ import annotations

import ctypes as C
import threading

import numpy as np

from .. import _lib
from .sampling import SamplingParams, TokenSample, _has_penalties, _is_plain_greedy

SEED_STRIDE = 0x1E3779B97F4A7C15  # reference sampling.py:148
_NEG_INF = float("-inf")


def mixed_seed(seed: int, step: int) -> int:
    return (int(seed) + (int(step) + 1) * SEED_STRIDE) % (2**63)


def pack_params(params, steps, slots=None) -> np.ndarray:
    """SamplingParams -> the C struct array ``hs_row_params[batch]`` (host, numpy)."""
    import torch

    n = len(params)
    rec = np.zeros(n, dtype=_lib.ROW_PARAMS)
    for i, (p, step) in enumerate(zip(params, steps)):
        rec["temperature"][i] = p.temperature
        rec["top_p"][i] = p.top_p
        rec["min_p"][i] = p.min_p
        rec["repetition_penalty"][i] = p.repetition_penalty
        rec["presence_penalty"][i] = p.presence_penalty
        rec["frequency_penalty"][i] = p.frequency_penalty
        rec["top_k"][i] = min(int(p.top_k), 2**31 - 1)
        rec["n_logprobs"][i] = -1 if p.logprobs is None else int(p.logprobs)
        seed = p.seed
        if seed is None and p.temperature != 0.0:
            # The reference falls back to torch's global generator (sampling.py:145);
            # draw this row's stream key from the same place.
            seed = int(torch.randint(0, 2**62, (), dtype=torch.int64))
        rec["seed"][i] = mixed_seed(seed or 0, step)
        rec["flags"][i] = _lib.HS_ROW_PLAIN_GREEDY if _is_plain_greedy(p) else 0
        rec["slot"][i] = -1 if slots is None else slots[i]
    return rec


def history_array(history, vocab: int) -> np.ndarray:
    """A row's history as int32; ids outside [0, vocab) are dropped here already
    (the reference ignores them, sampling.py:108)."""
    if isinstance(history, np.ndarray):
        h = history.reshape(-1).astype(np.int64, copy=False)
    else:
        h = np.fromiter(history, dtype=np.int64) if not isinstance(history, (list, tuple)) \
            else np.asarray(history, dtype=np.int64).reshape(-1)
    if h.size and (h.min() < 0 or h.max() >= vocab):
        h = h[(h >= 0) & (h < vocab)]
    return h.astype(np.int32)


class DeviceSampler:
    """One C-ABI sampler handle on one GPU plus the torch buffers around it."""

    def __init__(self, device, vocab_max: int, batch_max: int = 256, resident_slots: int = 256):
        import torch

        if not torch.cuda.is_available():
            raise RuntimeError("hydraserve_b200 needs a CUDA GPU: there is no CPU sampling path")
        self.torch = torch
        self.lib = _lib.load()
        self.device = torch.device(device)
        self.vocab_max = int(vocab_max)
        self.batch_max = int(batch_max)
        self.resident_slots = int(resident_slots)
        # user slot space = resident request slots, then one scratch slot per batch row
        self.scratch_base = self.resident_slots
        handle = C.c_void_p()
        st = self.lib.hs_create(self.device.index or 0, self.vocab_max,
                                self.resident_slots + self.batch_max, 0, self.batch_max,
                                C.byref(handle))
        _lib.check(self.lib, None, st, "hs_create")
        self.handle = handle
        self.lock = threading.RLock()
        self._pinned = threading.local()
        self.requests: dict = {}  # request id -> [slot, tokens already counted]
        self.free_slots = list(range(self.resident_slots - 1, -1, -1))

    def close(self) -> None:
        if getattr(self, "handle", None):
            self.lib.hs_destroy(self.handle)
            self.handle = None

    def __del__(self):  # best effort
        try:
            self.close()
        except Exception:
            pass

    # -- small helpers -------------------------------------------------------------
    def _stream(self):
        return C.c_void_p(self.torch.cuda.current_stream(self.device).cuda_stream)

    def _to_device(self, array: np.ndarray):
        t = self.torch.from_numpy(array)
        return t.pin_memory().to(self.device, non_blocking=True)

    def query(self, what: int, vocab: int, dtype: int = 1) -> int:
        return int(self.lib.hs_query(self.handle, what, vocab, dtype))

    def prepare_logits(self, logits):
        torch = self.torch
        if logits.device != self.device:
            logits = logits.to(self.device, non_blocking=True)
        if logits.dtype not in (torch.bfloat16, torch.float32):
            logits = logits.float()
        if logits.stride(-1) != 1 or (logits.shape[0] > 1 and logits.stride(0) < logits.shape[1]):
            logits = logits.contiguous()
        dtype = _lib.HS_DTYPE_BF16 if logits.dtype == torch.bfloat16 else _lib.HS_DTYPE_F32
        stride = logits.stride(0) if logits.shape[0] > 1 else logits.shape[1]
        return logits, dtype, int(stride)

    # -- histograms ----------------------------------------------------------------
    def reset_slots(self, slots) -> None:
        if len(slots) == 0:
            return
        d = self._to_device(np.asarray(slots, dtype=np.int32))
        st = self.lib.hs_slots_reset(self.handle, d.data_ptr(), len(slots), self._stream())
        _lib.check(self.lib, self.handle, st, "hs_slots_reset")

    def append_tokens(self, slots, token_arrays, vocab: int) -> None:
        """Count token_arrays[i] into slot slots[i]."""
        if len(slots) == 0:
            return
        lens = [int(a.size) for a in token_arrays]
        if max(lens) == 0:
            return
        offsets = np.zeros(len(slots) + 1, dtype=np.int32)
        np.cumsum(lens, out=offsets[1:])
        flat = np.concatenate(token_arrays).astype(np.int32, copy=False)
        d_tok = self._to_device(flat)
        d_off = self._to_device(offsets)
        d_slots = self._to_device(np.asarray(slots, dtype=np.int32))
        st = self.lib.hs_slots_append(self.handle, d_tok.data_ptr(), d_off.data_ptr(),
                                      d_slots.data_ptr(), len(slots), vocab, max(lens),
                                      self._stream())
        _lib.check(self.lib, self.handle, st, "hs_slots_append")

    def unique_count(self, slot: int) -> int:
        out = C.c_int(0)
        st = self.lib.hs_slot_unique_count(self.handle, slot, self._stream(), C.byref(out))
        _lib.check(self.lib, self.handle, st, "hs_slot_unique_count")
        return out.value

    def release_request(self, request_id) -> None:
        with self.lock:
            entry = self.requests.pop(request_id, None)
            if entry is not None:
                self.free_slots.append(entry[0])

    def _slot_for_request(self, request_id, history, vocab, resets, appends):
        """Resident slot of a request, scheduling only the not-yet-counted tail of its
        history for upload; falls back to a rebuild when the history shrank."""
        entry = self.requests.get(request_id)
        n = len(history)
        if entry is None:
            if not self.free_slots:  # evict the oldest request
                oldest = next(iter(self.requests))
                self.free_slots.append(self.requests.pop(oldest)[0])
            entry = [self.free_slots.pop(), 0]
            self.requests[request_id] = entry
            resets.append(entry[0])
        elif n < entry[1]:
            resets.append(entry[0])
            entry[1] = 0
        if n > entry[1]:
            tail = history[entry[1]:] if hasattr(history, "__getitem__") else tuple(history)[entry[1]:]
            appends.append((entry[0], history_array(tail, vocab)))
            entry[1] = n
        return entry[0]

    # -- the calls -------------------------------------------------------------------
    def greedy(self, logits):
        torch = self.torch
        logits, dtype, stride = self.prepare_logits(logits)
        batch, vocab = logits.shape
        tokens = torch.empty(batch, dtype=torch.int32, device=self.device)
        st = self.lib.hs_greedy(self.handle, logits.data_ptr(), dtype, stride, batch, vocab,
                                tokens.data_ptr(), self._stream())
        _lib.check(self.lib, self.handle, st, "hs_greedy")
        return tokens

    def run(self, logits, rec: np.ndarray, *, noise=None, want_scores: bool = False,
            append_token: bool = False):
        """Launch hs_sample for packed parameters ``rec``; returns (records, scores)."""
        torch = self.torch
        logits, dtype, stride = self.prepare_logits(logits)
        batch, vocab = logits.shape
        d_params = self._to_device(rec.view(np.uint8).reshape(batch, -1))
        d_out = torch.empty((batch, _lib.ROW_OUT.itemsize), dtype=torch.uint8, device=self.device)
        d_noise = None
        if noise is not None:
            d_noise = noise.to(self.device, dtype=torch.float32).contiguous()
        scores = torch.empty((batch, vocab), dtype=torch.float32, device=self.device) if want_scores else None
        st = self.lib.hs_sample(
            self.handle, logits.data_ptr(), dtype, stride, batch, vocab, d_params.data_ptr(),
            d_out.data_ptr(), d_noise.data_ptr() if d_noise is not None else None,
            scores.data_ptr() if scores is not None else None,
            _lib.HS_SAMPLE_APPEND_TOKEN if append_token else 0, self._stream())
        _lib.check(self.lib, self.handle, st, "hs_sample")
        host = self._pinned_records(batch)
        host.copy_(d_out, non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        records = host.numpy().view(_lib.ROW_OUT).reshape(batch).copy()  # the pinned buffer is reused
        return records, scores

    def _pinned_records(self, batch: int):
        """A pinned host buffer for the result records (pinning per call costs more than the copy);
        one per thread, since calls on different streams may overlap."""
        cache = self._pinned.__dict__.setdefault("buffers", {})
        buf = cache.get(batch)
        if buf is None:
            buf = self.torch.empty((batch, _lib.ROW_OUT.itemsize), dtype=self.torch.uint8).pin_memory()
            cache[batch] = buf
        return buf

    def sample(self, logits, histories, params, steps, request_ids=None, *, noise=None,
               want_scores: bool = False):
        """Stateless (histories rebuilt on the device for this call) or, with
        ``request_ids``, incremental sampling.  Returns (records, scores)."""
        batch, vocab = logits.shape
        # start the host-to-device copy of the logits (if they are on the host) first: the
        # bookkeeping below then runs while they travel
        logits, _, _ = self.prepare_logits(logits)
        with self.lock:
            slots = [-1] * batch
            resets, appends = [], []
            for i, p in enumerate(params):
                if not _has_penalties(p):
                    continue
                history = histories[i]
                if request_ids is not None and request_ids[i] is not None:
                    slots[i] = self._slot_for_request(request_ids[i], history, vocab, resets, appends)
                else:
                    tokens = history_array(history, vocab)
                    if tokens.size == 0:
                        continue
                    slots[i] = self.scratch_base + i
                    resets.append(slots[i])
                    appends.append((slots[i], tokens))
            self.reset_slots(resets)
            self.append_tokens([s for s, _ in appends], [t for _, t in appends], vocab)
            rec = pack_params(params, steps, slots)
            return self.run(logits, rec, noise=noise, want_scores=want_scores)


_samplers: dict = {}
_samplers_lock = threading.Lock()


def sampler_for(device, vocab: int, batch: int) -> DeviceSampler:
    """The process-wide sampler of a GPU, re-created larger when a call outgrows it."""
    key = str(device)
    with _samplers_lock:
        s = _samplers.get(key)
        if s is None or vocab > s.vocab_max or batch > s.batch_max:
            vocab_max = max(vocab, s.vocab_max if s else 0)
            batch_max = max(batch, s.batch_max if s else 64)
            if s is not None:
                s.close()
            s = DeviceSampler(device, vocab_max, batch_max)
            _samplers[key] = s
        return s


def _target_device(logits):
    import torch

    if not torch.cuda.is_available():
        raise RuntimeError("hydraserve_b200 needs a CUDA GPU: there is no CPU sampling path")
    if logits.is_cuda:
        return logits.device
    return torch.device("cuda", torch.cuda.current_device())


def records_to_samples(records, params, vocab: int):
    samples = []
    for rec, p in zip(records, params):
        if p.logprobs is None:
            samples.append(TokenSample(int(rec["token"])))
            continue
        want = min(int(p.logprobs), vocab)
        n = int(rec["n_top"])
        ids = rec["top_ids"][:n].tolist()
        vals = rec["top_logprobs"][:n].tolist()
        top = list(zip(ids, vals))
        if n < want:  # fewer candidates than requested: the reference lists filtered ids at -inf
            taken = set(ids)
            i = 0
            while len(top) < want:
                if i not in taken:
                    top.append((i, _NEG_INF))
                i += 1
        samples.append(TokenSample(int(rec["token"]), float(rec["logprob"]), tuple(top)))
    return tuple(samples)


def sample_batch(logits, histories, params, steps, request_ids, all_plain_greedy: bool = False):
    device = _target_device(logits)
    batch, vocab = int(logits.shape[0]), int(logits.shape[1])
    if batch == 0:
        return ()
    sampler = sampler_for(device, vocab, batch)
    if all_plain_greedy:
        tokens = sampler.greedy(logits).tolist()
        return tuple(TokenSample(int(t)) for t in tokens)
    records, _ = sampler.sample(logits, histories, params, steps, request_ids)
    return records_to_samples(records, params, vocab)


def release_request(request_id, device=None) -> None:
    """Forget a request's resident histogram (call when the request finishes)."""
    with _samplers_lock:
        targets = list(_samplers.values()) if device is None else [_samplers.get(str(device))]
    for s in targets:
        if s is not None:
            s.release_request(request_id)
