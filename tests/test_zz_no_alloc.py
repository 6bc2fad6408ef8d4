"""liger_attention_decode_noalloc: the decode-attention entry point for callers that may not allocate
device memory (frozen memory pools, plugins living inside another allocator).  Its split-KV partials
live in a buffer built into the library instead of caller scratch, so the result must be the same
as liger_attention_decode's: both run the same two kernels in the same order, hence bit-identical
fp16 output (checked with the 1e-2 relative bound the other decode tests use, and exactly).

Collected last on purpose: the file name sorts after every other test file, so a run that stops at
the first failure has already been through the rest.  It needs nothing from the other tests and
passes alone in a fresh process as well."""
import ctypes as C

import numpy as np
import pytest

from helpers import assert_close, dev_fill, ptr, stream_ptr, to_np

pytestmark = pytest.mark.gpu


def _decode_inputs(liger, B, h, L, D, seed):
    Lmax = L + 3
    q = dev_fill(liger, B * h, D, seed, 410).reshape(B, h, D)
    kc = dev_fill(liger, B * h * Lmax, D, seed, 0x10001).reshape(B, h, Lmax, D)
    vc = dev_fill(liger, B * h * Lmax, D, seed, 0x10002).reshape(B, h, Lmax, D)
    return q, kc, vc, Lmax


def test_noalloc_decode_matches_scratch_decode_twice_in_a_row(gpu, liger):
    import torch
    # two calls back to back with different shapes: the second one finds the first one's partials in
    # the shared buffer and must not be affected by them
    for call, (B, h, L, D) in enumerate([(4, 6, 1000, 128), (3, 5, 300, 64)]):
        q, kc, vc, Lmax = _decode_inputs(liger, B, h, L, D, seed=call)
        scale = 1.0 / np.sqrt(D)
        nbytes = gpu.liger_attention_decode_scratch_bytes(B, h, D, L)
        assert nbytes <= gpu.liger_attention_decode_noalloc_max_bytes()
        scratch = torch.empty(nbytes // 4, dtype=torch.float32, device="cuda")
        want = torch.zeros((B, h * D), dtype=torch.float16, device="cuda")
        liger.check(gpu.liger_attention_decode(ptr(q), ptr(kc), ptr(vc), ptr(want), ptr(scratch), B, h, L, Lmax, D, h * D,
                                               scale, stream_ptr()))
        got = torch.full((B, h * D), float("nan"), dtype=torch.float16, device="cuda")
        # free device memory as the driver reports it (this sees a cudaMalloc made anywhere in the process, which
        # torch's own allocator statistics would not)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        liger.check(gpu.liger_attention_decode_noalloc(ptr(q), ptr(kc), ptr(vc), ptr(got), B, h, L, Lmax, D, h * D, scale,
                                                       stream_ptr()))
        torch.cuda.synchronize()
        if call > 0:   # the very first call on a device may make the runtime load the library's device code
            assert torch.cuda.mem_get_info()[0] == free_before, "the no-alloc entry point changed the device's free memory"
        assert_close(to_np(got), to_np(want), rel=1e-2, what=f"no-alloc decode, call {call}")
        assert torch.equal(got, want)


def test_noalloc_decode_rejects_requests_beyond_the_builtin_buffer(gpu, liger):
    import torch
    t = torch.zeros(16, dtype=torch.float16, device="cuda")   # never touched: the call must fail before launching
    limit = gpu.liger_attention_decode_noalloc_max_bytes()
    assert limit == 16 << 20
    B, h, L, D = 64, 96, 8192, 128
    assert gpu.liger_attention_decode_scratch_bytes(B, h, D, L) > limit
    rc = gpu.liger_attention_decode_noalloc(ptr(t), ptr(t), ptr(t), ptr(t), B, h, L, L, D, h * D, 1.0, stream_ptr())
    assert rc == -5
    msg = gpu.liger_last_error().decode()
    assert "built-in" in msg and "liger_attention_decode" in msg
