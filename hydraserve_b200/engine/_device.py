"""Host side of the CUDA sampler: packs per-row parameters and histories, owns one C-ABI
sampler handle per GPU, and turns result records into ``TokenSample`` objects.

PyTorch is used here only for device memory, pinned host buffers and the current stream;
all arithmetic happens in the CUDA library.  There is no CPU path: host tensors are
copied to the GPU, and a machine without a GPU or without the built library raises.

Threads: the reference calls its sampler from the serving loop and, concurrently, from
threads that replay a request's first token on a side stream (pd_service.py:916-967,
pd_worker.py:305-308, 475-480).  Every public method here may be called from several
threads; calls on one sampler are serialised (the C library orders their GPU work too),
and the process-wide sampler of a GPU is never destroyed while a call is inside it.
"""
from __future__ import annotations

import ctypes as C
import itertools
import os
import threading
from collections import OrderedDict

import numpy as np

from .. import _lib
from .sampling import SamplingParams, TokenSample, _has_penalties, _is_plain_greedy, _token_only

SEED_STRIDE = 0x1E3779B97F4A7C15  # reference sampling.py:148
_NEG_INF = float("-inf")
_MASK63 = np.uint64(2**63 - 1)

# status bits of hs_row_out.status (include/hs_sampler.h)
STATUS_FELL_BACK, STATUS_APPEND_FAILED, STATUS_NEEDS_GENERAL = 1, 2, 4
STATUS_SHARD_CUT = 16 | 32
STATUS_BAD_SLOT = 64
STATUS_NO_SCRATCH = 128


def mixed_seed(seed: int, step: int) -> int:
    return (int(seed) + (int(step) + 1) * SEED_STRIDE) % (2**63)


def _static_row(p: SamplingParams) -> bytes:
    """The 48 bytes of hs_row_params that depend on the SamplingParams alone (seed and slot
    are filled in per call)."""
    rec = np.zeros(1, dtype=_lib.ROW_PARAMS)
    rec["temperature"] = p.temperature
    rec["top_p"] = p.top_p
    rec["min_p"] = p.min_p
    rec["repetition_penalty"] = p.repetition_penalty
    rec["presence_penalty"] = p.presence_penalty
    rec["frequency_penalty"] = p.frequency_penalty
    rec["top_k"] = min(int(p.top_k), 2**31 - 1)
    rec["n_logprobs"] = -1 if p.logprobs is None else int(p.logprobs)
    rec["flags"] = _lib.HS_ROW_PLAIN_GREEDY if _is_plain_greedy(p) else 0
    rec["slot"] = -1
    return rec.tobytes()


_static_rows: dict = {}  # id(params) -> (params, packed bytes); the object is kept so the id stays its own
_STATIC_ROWS_MAX = 8192
_static_batches: dict = {}  # ids of a batch's params -> (the params, packed static part, any unseeded, seeds)
_STATIC_BATCHES_MAX = 64


def _static_row_cached(p: SamplingParams) -> bytes:
    hit = _static_rows.get(id(p))
    if hit is not None and hit[0] is p:
        return hit[1]
    row = _static_row(p)
    if len(_static_rows) >= _STATIC_ROWS_MAX:
        _static_rows.clear()
    _static_rows[id(p)] = (p, row)
    return row


def draw_unseeded_keys(params):
    """Stream keys for the rows that sample without a seed.  The reference falls back to
    torch's global generator there (sampling.py:145); the keys come from the same place."""
    import torch

    return [int(torch.randint(0, 2**62, (), dtype=torch.int64))
            if (p.seed is None and p.temperature != 0.0) else None for p in params]


def batch_static(params):
    """What depends on a batch's SamplingParams alone: (the params, packed static part, any
    unseeded row, seeds, which rows have penalties).  A serving loop passes the same objects
    step after step, so this is kept per batch (the entry holds the objects: their ids stay
    theirs while it lives)."""
    n = len(params)
    key = tuple(map(id, params))
    hit = _static_batches.get(key)
    if hit is None:
        static = np.frombuffer(b"".join(_static_row_cached(p) for p in params), dtype=_lib.ROW_PARAMS).copy() \
            if n else np.zeros(0, dtype=_lib.ROW_PARAMS)
        unseeded = any(p.seed is None and p.temperature != 0.0 for p in params)
        fixed_seeds = None if unseeded else np.fromiter((p.seed if p.seed is not None else 0 for p in params),
                                                        dtype=np.uint64, count=n)
        if len(_static_batches) >= _STATIC_BATCHES_MAX:
            _static_batches.clear()
        hit = _static_batches[key] = (tuple(params), static, unseeded, fixed_seeds,
                                      tuple(_has_penalties(p) for p in params))
    return hit


def pack_params(params, steps, slots=None, unseeded_keys=None) -> np.ndarray:
    """SamplingParams -> the C struct array ``hs_row_params[batch]`` (host, numpy).

    unseeded_keys: per row, the stream key of a row whose ``seed`` is None (or None); drawn
    from torch's global generator when not given."""
    n = len(params)
    hit = batch_static(params)
    _, static, unseeded, fixed_seeds, _ = hit
    rec = static.copy()
    if unseeded:
        if unseeded_keys is None:
            unseeded_keys = draw_unseeded_keys(params)
        seeds = np.fromiter(
            ((p.seed if p.seed is not None else ((unseeded_keys[i] if unseeded_keys else None) or 0))
             for i, p in enumerate(params)), dtype=np.uint64, count=n)
    else:
        seeds = fixed_seeds
    step_arr = (np.asarray(steps, dtype=np.int64) + 1).astype(np.uint64)
    with np.errstate(over="ignore"):
        rec["seed"] = (seeds + step_arr * np.uint64(SEED_STRIDE)) & _MASK63  # == mixed_seed, vectorised
    if slots is not None:
        rec["slot"] = np.asarray(slots, dtype=np.int32)
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


def slot_bytes(vocab_max: int, hist_cap: int = 0) -> int:
    """Device bytes one histogram slot takes (what hs_query(6) reports): (id, count) pairs and
    the list of often-repeated ids per distinct id the slot can hold, a position and a 2-bit
    count class per vocabulary entry, two counters."""
    cap = min(int(hist_cap), int(vocab_max)) if hist_cap else int(vocab_max)
    return 12 * cap + 4 * int(vocab_max) + 4 * ((int(vocab_max) + 15) // 16 + 4) + 8


class SlotBook:
    """Which request holds which resident histogram slot, and how much of its history the
    device has already counted.  Pure host bookkeeping (no GPU): least recently used
    requests are evicted first, never one that belongs to the batch being packed."""

    def __init__(self, n_slots: int):
        self.n_slots = int(n_slots)
        self.entries: OrderedDict = OrderedDict()  # request id -> [slot, tokens counted]
        self.free = list(range(self.n_slots - 1, -1, -1))

    def release(self, request_id) -> bool:
        entry = self.entries.pop(request_id, None)
        if entry is None:
            return False
        self.free.append(entry[0])
        return True

    def lookup(self, request_id, in_batch):
        """(entry, is_new) for the request, or (None, False) when every slot is held by a
        request of the current batch (the caller then rebuilds that row's histogram in a
        per-call slot).  ``in_batch``: the ids of all requests of the call."""
        entry = self.entries.get(request_id)
        if entry is not None:
            self.entries.move_to_end(request_id)
            return entry, False
        if not self.free:
            victim = next((rid for rid in self.entries if rid not in in_batch), None)
            if victim is None:
                return None, False
            self.free.append(self.entries.pop(victim)[0])
        entry = [self.free.pop(), 0]
        self.entries[request_id] = entry
        return entry, True


class DeviceSampler:
    """One C-ABI sampler handle on one GPU plus the torch buffers around it."""

    def __init__(self, device, vocab_max: int, batch_max: int = 256, resident_slots: int = 256,
                 hist_cap: int = 0, flags: int = 0):
        import torch

        if not torch.cuda.is_available():
            raise RuntimeError("hydraserve_b200 needs a CUDA GPU: there is no CPU sampling path")
        self.torch = torch
        self.lib = _lib.load()
        self.device = torch.device(device)
        self.vocab_max = int(vocab_max)
        self.batch_max = int(batch_max)
        self.resident_slots = int(resident_slots)
        self.hist_cap = int(hist_cap) if hist_cap else self.vocab_max
        # slot space: the resident request slots, then one per-call slot per batch row (the
        # library adds those batch_max slots itself)
        self.scratch_base = self.resident_slots
        handle = C.c_void_p()
        st = self.lib.hs_create_ex(self.device.index or 0, self.vocab_max, self.resident_slots,
                                   int(hist_cap), self.batch_max, int(flags), C.byref(handle))
        _lib.check(self.lib, None, st, "hs_create_ex")
        self.handle = handle
        self.lock = threading.RLock()
        self._pinned = threading.local()
        self.book = SlotBook(self.resident_slots)
        self.users = 0        # calls inside this sampler (guarded by _samplers_lock)
        self.retired = False  # replaced by a larger one: closed when the last user leaves

    def close(self) -> None:
        with self.lock:
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
        """Host array -> device tensor through this thread's pinned arena (no cudaHostAlloc per
        call).  A ring of buffers, each with the event of its last copy, so that a buffer is
        not rewritten while a copy from it may still be in flight."""
        torch = self.torch
        flat = np.ascontiguousarray(array).view(np.uint8).reshape(-1)
        out = torch.empty(flat.size, dtype=torch.uint8, device=self.device)
        if flat.size == 0:
            return out
        state = self._pinned.__dict__
        ring = state.setdefault("ring", [])
        if not ring:
            ring.extend([None, None, 0] for _ in range(16))  # [pinned tensor, event of its last copy, size]
            state["at"] = 0
        state["at"] = at = (state["at"] + 1) % len(ring)
        slot = ring[at]
        if slot[0] is None or slot[2] < flat.size:
            slot[0] = torch.empty(max(4096, 2 * flat.size), dtype=torch.uint8).pin_memory()
            slot[2] = slot[0].numel()
            slot[1] = torch.cuda.Event()
        else:
            slot[1].synchronize()
        staged = slot[0][: flat.size]
        staged.numpy()[:] = flat
        out.copy_(staged, non_blocking=True)
        slot[1].record(torch.cuda.current_stream(self.device))
        return out  # bytes on the device; callers pass its address to the C library

    def query(self, what: int, vocab: int = 0, dtype: int = 1) -> int:
        return int(self.lib.hs_query(self.handle, what, vocab, dtype))

    def device_bytes(self) -> int:
        return self.query(5) * 1024

    def set_split(self, split: int) -> None:
        """CTAs per candidate row (tests and tuning); 0 = chosen per call."""
        _lib.check(self.lib, self.handle, self.lib.hs_debug_set(self.handle, 0, int(split)), "hs_debug_set")

    def set_count_split(self, split: int) -> None:
        """CTAs per counting row (tests and tuning); 0 = chosen per call."""
        _lib.check(self.lib, self.handle, self.lib.hs_debug_set(self.handle, 1, int(split)), "hs_debug_set")

    def set_token_draw(self, on: bool) -> None:
        """Near-flat counting rows draw by rejection on tokens (default) or always class by
        class (tests and tuning)."""
        _lib.check(self.lib, self.handle, self.lib.hs_debug_set(self.handle, 3, 1 if on else 0), "hs_debug_set")

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
        """Count token_arrays[i] (a numpy array or any sequence of ints) into slot slots[i].
        Ids outside [0, vocab) are ignored, as in the reference (sampling.py:108)."""
        if len(slots) == 0:
            return
        lens = [len(a) for a in token_arrays]
        total = sum(lens)
        if total == 0:
            return
        if all(not isinstance(a, np.ndarray) for a in token_arrays):
            # short Python sequences (the one token a request gained since its last step): one pass
            flat = np.fromiter(itertools.chain.from_iterable(token_arrays), dtype=np.int64, count=total)
        else:
            flat = np.concatenate([np.asarray(a, dtype=np.int64).reshape(-1) for a in token_arrays])
        # the device ignores ids outside [0, vocab); -1 stands for everything that is
        flat = np.where((flat < 0) | (flat >= vocab), -1, flat).astype(np.int32)
        offsets = np.zeros(len(slots) + 1, dtype=np.int32)
        np.cumsum(lens, out=offsets[1:])
        # one staged copy for tokens, offsets and slot numbers
        packed = np.concatenate([flat, offsets, np.asarray(slots, dtype=np.int32)])
        d = self._to_device(packed)
        base = d.data_ptr()
        st = self.lib.hs_slots_append(self.handle, base, base + 4 * flat.size,
                                      base + 4 * (flat.size + offsets.size), len(slots), vocab, max(lens),
                                      self._stream())
        _lib.check(self.lib, self.handle, st, "hs_slots_append")

    def unique_count(self, slot: int) -> int:
        out = C.c_int(0)
        st = self.lib.hs_slot_unique_count(self.handle, slot, self._stream(), C.byref(out))
        _lib.check(self.lib, self.handle, st, "hs_slot_unique_count")
        return out.value

    def release_request(self, request_id) -> None:
        with self.lock:
            self.book.release(request_id)

    def _slot_for_request(self, request_id, history, vocab, resets, appends, in_batch):
        """Resident slot of a request, scheduling only the not-yet-counted tail of its
        history for upload; falls back to a rebuild when the history shrank.  Returns -1
        when no resident slot can be had (the caller uses a per-call slot)."""
        entry, is_new = self.book.lookup(request_id, in_batch)
        if entry is None:
            return -1
        n = len(history)
        if is_new:
            resets.append(entry[0])
        elif n < entry[1]:
            resets.append(entry[0])
            entry[1] = 0
        if n > entry[1]:
            tail = history[entry[1]:] if hasattr(history, "__getitem__") else tuple(history)[entry[1]:]
            appends.append((entry[0], tail))
            entry[1] = n
        return entry[0]

    # -- the calls -------------------------------------------------------------------
    def greedy(self, logits):
        torch = self.torch
        logits, dtype, stride = self.prepare_logits(logits)
        batch, vocab = logits.shape
        tokens = torch.empty(batch, dtype=torch.int32, device=self.device)
        with self.lock:
            st = self.lib.hs_greedy(self.handle, logits.data_ptr(), dtype, stride, batch, vocab,
                                    tokens.data_ptr(), self._stream())
            _lib.check(self.lib, self.handle, st, "hs_greedy")
        return tokens

    def launch(self, logits, d_params, d_out, *, noise=None, scores=None, tokens_out=None,
               append_token: bool = False, general: bool = False) -> None:
        """hs_sample_ex on the current stream with everything already on the device; nothing
        is copied back and nothing synchronises (the device-chained decode step)."""
        logits, dtype, stride = self.prepare_logits(logits)
        batch, vocab = logits.shape
        flags = (_lib.HS_SAMPLE_APPEND_TOKEN if append_token else 0) | (_lib.HS_SAMPLE_GENERAL_KERNEL if general else 0)
        st = self.lib.hs_sample_ex(
            self.handle, logits.data_ptr(), dtype, stride, batch, vocab, d_params.data_ptr(),
            d_out.data_ptr(), noise.data_ptr() if noise is not None else None,
            scores.data_ptr() if scores is not None else None,
            tokens_out.data_ptr() if tokens_out is not None else None, flags, self._stream())
        _lib.check(self.lib, self.handle, st, "hs_sample_ex")

    def run(self, logits, rec: np.ndarray, *, noise=None, want_scores: bool = False,
            append_token: bool = False, general: bool = False):
        """Launch hs_sample for packed parameters ``rec``; returns (records, scores).  Rows
        the bf16 kernel reports as beyond its side-list capacity are sampled again by the
        general kernel."""
        torch = self.torch
        logits, dtype, stride = self.prepare_logits(logits)
        batch, vocab = logits.shape
        d_params = self._to_device(rec.view(np.uint8).reshape(batch, -1))
        d_out = torch.empty((batch, _lib.ROW_OUT.itemsize), dtype=torch.uint8, device=self.device)
        d_noise = None
        if noise is not None:
            d_noise = noise.to(self.device, dtype=torch.float32).contiguous()
        scores = torch.empty((batch, vocab), dtype=torch.float32, device=self.device) if want_scores else None
        with self.lock:
            self.launch(logits, d_params, d_out, noise=d_noise, scores=scores, append_token=append_token,
                        general=general)
            host = self._pinned_records(batch)
            host.copy_(d_out, non_blocking=True)
            torch.cuda.current_stream(self.device).synchronize()
            records = host.numpy().view(_lib.ROW_OUT).reshape(batch).copy()  # the pinned buffer is reused
        again = np.nonzero(records["status"] & STATUS_NEEDS_GENERAL)[0]
        if again.size and not general:
            idx = torch.from_numpy(again.astype(np.int64)).to(self.device)
            sub, sub_scores = self.run(
                logits.index_select(0, idx), rec[again], noise=None if d_noise is None else d_noise.index_select(0, idx),
                want_scores=want_scores, append_token=append_token, general=True)
            records[again] = sub
            if scores is not None:
                scores[idx] = sub_scores
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

    def plan_slots(self, histories, params, vocab: int, request_ids=None):
        """Slot per row plus the histogram resets / appends that bring the device up to date
        (issued here, on the current stream).  Call with the sampler lock held."""
        batch = len(params)
        slots = [-1] * batch
        resets, appends = [], []
        in_batch = None
        entries = self.book.entries if request_ids is not None else None
        for i, penalised in enumerate(batch_static(params)[4]):
            if not penalised:
                continue
            history = histories[i]
            slot = -1
            if entries is not None and request_ids[i] is not None:
                # the common step in line: a known request whose history grew by one token
                entry = entries.get(request_ids[i])
                if entry is not None and len(history) == entry[1] + 1 and type(history) in (list, tuple):
                    entries.move_to_end(request_ids[i])
                    appends.append((entry[0], history[-1:]))
                    entry[1] += 1
                    slots[i] = entry[0]
                    continue
                if in_batch is None:
                    in_batch = {r for r in request_ids if r is not None}
                slot = self._slot_for_request(request_ids[i], history, vocab, resets, appends, in_batch)
                if slot >= 0 and len(history) == 0:
                    # nothing to penalise yet: the row goes without a slot, as it does in a
                    # stateless call, so that the same kernel path serves it either way (the
                    # path decides which token a seeded draw lands on); the slot stays the
                    # request's and is filled from the next step on
                    continue
            if slot < 0:
                if len(history) == 0:
                    continue
                slot = self.scratch_base + i
                resets.append(slot)
                appends.append((slot, history if isinstance(history, (np.ndarray, list, tuple)) else tuple(history)))
            slots[i] = slot
        self.reset_slots(resets)
        self.append_tokens([s for s, _ in appends], [t for _, t in appends], vocab)
        return slots

    def sample(self, logits, histories, params, steps, request_ids=None, *, noise=None,
               want_scores: bool = False):
        """Stateless (histories rebuilt on the device for this call) or, with
        ``request_ids``, incremental sampling.  Returns (records, scores)."""
        batch, vocab = logits.shape
        # start the host-to-device copy of the logits (if they are on the host) first: the
        # bookkeeping below then runs while they travel
        logits, _, _ = self.prepare_logits(logits)
        with self.lock:
            slots = self.plan_slots(histories, params, vocab, request_ids)
            rec = pack_params(params, steps, slots)
            return self.run(logits, rec, noise=noise, want_scores=want_scores)


_samplers: dict = {}
_samplers_lock = threading.Lock()
DEFAULT_HIST_CAP = int(os.environ.get("HYDRASERVE_SAMPLER_HIST_CAP", "65536"))


class _Lease:
    """The process-wide sampler of a GPU for the time of one call."""

    def __init__(self, sampler):
        self.sampler = sampler

    def __enter__(self):
        return self.sampler

    def __exit__(self, *exc):
        s = self.sampler
        with _samplers_lock:
            s.users -= 1
            close = s.retired and s.users == 0
        if close:
            s.close()
        return False


def lease_sampler(device, vocab: int, batch: int, hist_need: int = 0) -> _Lease:
    """The process-wide sampler of a GPU, replaced by a larger one when a call outgrows it.
    The old one is closed only after the last call inside it has returned."""
    key = str(device)
    hist_need = min(int(vocab), max(int(hist_need), min(DEFAULT_HIST_CAP, int(vocab))))
    with _samplers_lock:
        s = _samplers.get(key)
        if s is None or vocab > s.vocab_max or batch > s.batch_max or hist_need > s.hist_cap:
            vocab_max = max(vocab, s.vocab_max if s else 0)
            batch_max = max(batch, s.batch_max if s else 64)
            hist_cap = min(vocab_max, max(hist_need, s.hist_cap if s else 0))
            fresh = DeviceSampler(device, vocab_max, batch_max, resident_slots=max(256, batch_max),
                                  hist_cap=hist_cap)
            if s is not None:
                s.retired = True
                if s.users == 0:
                    s.close()
            _samplers[key] = s = fresh
        s.users += 1
        return _Lease(s)


def sampler_for(device, vocab: int, batch: int, hist_need: int = 0) -> DeviceSampler:
    """The process-wide sampler of a GPU (not leased: for single-threaded tools and tests)."""
    lease = lease_sampler(device, vocab, batch, hist_need)
    with lease as s:
        return s


def _target_device(logits):
    import torch

    if not torch.cuda.is_available():
        raise RuntimeError("hydraserve_b200 needs a CUDA GPU: there is no CPU sampling path")
    if logits.is_cuda:
        return logits.device
    return torch.device("cuda", torch.cuda.current_device())


def record_to_sample(rec, logprobs, vocab: int) -> TokenSample:
    if logprobs is None:
        return TokenSample(int(rec["token"]))
    want = min(int(logprobs), vocab)
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
    return TokenSample(int(rec["token"]), float(rec["logprob"]), tuple(top))


def records_to_samples(records, params, vocab: int):
    tokens = records["token"].tolist()
    out = list(map(_token_only, tokens))
    for i, p in enumerate(params):
        if p.logprobs is not None:
            out[i] = record_to_sample(records[i], p.logprobs, vocab)
    return tuple(out)


class PackedSamples:
    """One step's results as ONE array of 208-byte records instead of a tuple of per-row
    Python objects: what a worker process sends back (the reference pickles
    ``tuple[TokenSample]`` per step, pd_service.py:1097-1104) and what an API layer can
    format from without touching rows it does not need (api/server.py:491-530).

    Behaves like the tuple the reference returns: ``len``, indexing and iteration give
    ``TokenSample`` objects, built on demand and equal to those of ``sample_logits``."""

    __slots__ = ("records", "logprobs", "vocab")

    def __init__(self, records: np.ndarray, logprobs, vocab: int):
        self.records = records            # numpy structured array, dtype _lib.ROW_OUT
        self.logprobs = np.asarray(logprobs, dtype=np.int8)  # per row: -1 = none requested, else 0..20
        self.vocab = int(vocab)

    @property
    def token_ids(self) -> np.ndarray:
        return self.records["token"]

    def __len__(self) -> int:
        return int(self.records.shape[0])

    def __getitem__(self, i) -> TokenSample:
        if isinstance(i, slice):
            return tuple(self[j] for j in range(*i.indices(len(self))))
        lp = int(self.logprobs[i])
        return record_to_sample(self.records[i], None if lp < 0 else lp, self.vocab)

    def __iter__(self):
        return (self[i] for i in range(len(self)))

    def to_samples(self) -> tuple:
        return tuple(self)

    def __eq__(self, other):
        if isinstance(other, PackedSamples):
            return self.to_samples() == other.to_samples()
        if isinstance(other, tuple):
            return self.to_samples() == other
        return NotImplemented

    def __reduce__(self):
        return (_unpack_samples, (self.records.tobytes(), self.logprobs.tobytes(), self.vocab))


def _unpack_samples(record_bytes: bytes, logprob_bytes: bytes, vocab: int) -> PackedSamples:
    return PackedSamples(np.frombuffer(record_bytes, dtype=_lib.ROW_OUT),
                         np.frombuffer(logprob_bytes, dtype=np.int8), vocab)


def _logprob_codes(params):
    return [-1 if p.logprobs is None else int(p.logprobs) for p in params]


def sample_batch(logits, histories, params, steps, request_ids, all_plain_greedy: bool = False,
                 packed: bool = False):
    device = _target_device(logits)
    batch, vocab = int(logits.shape[0]), int(logits.shape[1])
    if batch == 0:
        return PackedSamples(np.zeros(0, _lib.ROW_OUT), [], vocab) if packed else ()
    hist_need = 0
    if not all_plain_greedy:
        pen = batch_static(params)[4]
        hist_need = max((len(h) for h, on in zip(histories, pen) if on), default=0)
    with lease_sampler(device, vocab, batch, hist_need) as sampler:
        if all_plain_greedy:
            tokens = sampler.greedy(logits).cpu().numpy()
            if packed:
                records = np.zeros(batch, _lib.ROW_OUT)
                records["token"] = tokens
                return PackedSamples(records, [-1] * batch, vocab)
            return tuple(TokenSample(int(t)) for t in tokens.tolist())
        records, _ = sampler.sample(logits, histories, params, steps, request_ids)
    bad = records["status"] & (STATUS_APPEND_FAILED | STATUS_NEEDS_GENERAL | STATUS_BAD_SLOT | STATUS_NO_SCRATCH)
    if bad.any():
        raise _lib.SamplerError(f"sampler reported status {int(bad.max())} for row {int(np.argmax(bad != 0))}")
    if packed:
        return PackedSamples(records, _logprob_codes(params), vocab)
    return records_to_samples(records, params, vocab)


def release_request(request_id, device=None) -> None:
    """Forget a request's resident histogram (call when the request finishes)."""
    with _samplers_lock:
        targets = list(_samplers.values()) if device is None else [_samplers.get(str(device))]
    for s in targets:
        if s is not None:
            s.release_request(request_id)
