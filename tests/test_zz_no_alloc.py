"""hs_greedy_noalloc: the arg-max entry point for callers that cannot allocate device memory
(their framework's allocator owns the GPU, or they sit on a path where cudaMalloc's
device-wide synchronisation is not acceptable).  It must give exactly what hs_greedy gives,
call after call, with its scratch in the library's fixed device array.

Collected last on purpose (file name), and self-contained: it passes alone in a fresh
process and after the rest of the suite."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def _bf16(x):
    return torch.from_numpy(x).cuda().bfloat16()


def test_no_alloc_greedy_matches_hs_greedy_on_two_calls_in_a_row(built_library):
    from hydraserve_b200 import _lib

    lib = _lib.load()
    torch.cuda.set_device(0)
    handle = C.c_void_p()
    assert lib.hs_create(0, 151_936, 4, 0, 64, C.byref(handle)) == 0
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    rng = np.random.default_rng(2024)
    try:
        for call, (batch, vocab, dtype) in enumerate(((37, 151_936, "bf16"), (64, 50_257, "f32"))):
            x = (rng.standard_normal((batch, vocab)) * 3).astype(np.float32)
            logits = _bf16(x) if dtype == "bf16" else torch.from_numpy(x).cuda()
            # exact ties at the maximum, at a higher id, so the lowest-id rule is exercised
            top = logits.argmax(dim=1)
            logits[torch.arange(0, batch, 3), vocab - 1] = logits[torch.arange(0, batch, 3), top[::3]]
            code = _lib.HS_DTYPE_BF16 if dtype == "bf16" else _lib.HS_DTYPE_F32
            want = torch.empty(batch, dtype=torch.int32, device="cuda")
            got = torch.full((batch,), -7, dtype=torch.int32, device="cuda")
            assert lib.hs_greedy(handle, logits.data_ptr(), code, vocab, batch, vocab, want.data_ptr(), stream) == 0
            st = lib.hs_greedy_noalloc(logits.data_ptr(), code, vocab, batch, vocab, got.data_ptr(), stream)
            assert st == 0, lib.hs_greedy_noalloc_error()
            torch.cuda.synchronize()
            assert torch.equal(got, want), f"call {call}: {int((got != want).sum())} rows differ"
            assert torch.equal(got.long(), logits.float().argmax(dim=1))
        # a batch beyond the fixed array is refused with a message, and nothing is launched
        too_many = _lib.HS_NOALLOC_MAX_BATCH + 1
        st = lib.hs_greedy_noalloc(logits.data_ptr(), code, vocab, too_many, vocab, got.data_ptr(), stream)
        assert st == -2
        assert b"HS_NOALLOC_MAX_BATCH" in lib.hs_greedy_noalloc_error()
        assert lib.hs_greedy_noalloc(logits.data_ptr(), 9, vocab, 1, vocab, got.data_ptr(), stream) == -1
    finally:
        lib.hs_destroy(handle)
