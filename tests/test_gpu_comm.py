"""Two-rank parity of the fused all-reduce (one process per GPU, handles exchanged over
torch.distributed) against the CPU oracle.  Needs >= 2 GPUs; bit-exactness is not expected because
the fp32 summation order differs from the oracle's rank order, so the tolerance is 1e-2 relative
(results are fp16)."""
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


def _worker(rank, world, port, results):
    import ctypes as C
    import torch
    import torch.distributed as dist
    sys.path.insert(0, HERE)
    sys.path.insert(0, os.path.dirname(HERE))
    from conftest import load_package
    from helpers import dev_fill, ptr, stream_ptr, to_np
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    liger = load_package()
    from liger_b200.dist import Comm
    lib = liger.lib()
    out = {}
    for (m, n, mode) in [(64, 1024, "ln_res"), (256, 12288, "ln"), (33, 512, "plain"), (32, 1024, "one_shot")]:
        bytes_t = m * n * 2
        out_off = (bytes_t + 255) // 256 * 256
        comm = Comm(rank, world, out_off + bytes_t, channels=2)
        part = comm.tensor(0, (m, n))
        dst = comm.tensor(out_off, (m, n))
        dev_fill(liger, m, n, 0, 500 + rank, out=part)
        dst.zero_()
        hidden = dev_fill(liger, m, n, 0, 510)
        bias = dev_fill(liger, 1, n, 0, 511, std=0.02).reshape(-1)
        g = dev_fill(liger, 1, n, 0, 512, mean=1.0, std=0.02).reshape(-1)
        b = dev_fill(liger, 1, n, 0, 513, std=0.02).reshape(-1)
        torch.cuda.synchronize()
        dist.barrier()
        use_h = mode in ("ln_res", "one_shot")
        use_ln = mode in ("ln_res", "ln", "one_shot")
        for rep in range(2):   # second call re-uses the flags with new epochs
            if use_h:
                dev_fill(liger, m, n, 0, 510, out=hidden)
            liger.check(lib.liger_allreduce_fused(comm.handle, rep % 2, 0, out_off, None, ptr(hidden) if use_h else None,
                                                  ptr(bias) if use_h else None, ptr(g) if use_ln else None,
                                                  ptr(b) if use_ln else None, m, n, 0, m, 1 if mode == "one_shot" else 0,
                                                  stream_ptr()))
            torch.cuda.synchronize()
        st = (C.c_uint * 4)()
        assert lib.liger_device_status(C.byref(st)) == 0, list(st)
        out[(m, n, mode)] = (to_np(dst), to_np(hidden))
        dist.barrier()
        comm.close()
    results[rank] = out
    dist.destroy_process_group()


def test_allreduce_fused_two_ranks(oracle):
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    world = 2
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, 29533, results), nprocs=world, join=True)
    from helpers import assert_close
    for key in results[0].keys():
        m, n, mode = key
        parts = np.stack([oracle.fill_normal(m * n, 0, 500 + r).reshape(m, n) for r in range(world)])
        red = oracle.allreduce_sum(parts)
        hidden = oracle.fill_normal(m * n, 0, 510).reshape(m, n)
        bias = oracle.fill_normal(n, 0, 511, std=0.02)
        g = oracle.fill_normal(n, 0, 512, mean=1.0, std=0.02)
        b = oracle.fill_normal(n, 0, 513, std=0.02)
        if mode in ("ln_res", "one_shot"):
            want_h, want = oracle.add_bias_input_layernorm_2(red, g, b, bias, hidden)
        elif mode == "ln":
            want_h, want = None, oracle.layernorm(oracle.round_fp16(red), g, b)
        else:
            want_h, want = None, red
        rpr = (m + world - 1) // world
        for r in range(world):
            got, got_h = results[r][key]
            assert_close(got, want, rel=1e-2, what=f"rank {r} {key} out")
            if want_h is not None:
                rows = slice(0, m) if mode == "one_shot" else slice(r * rpr, min(m, (r + 1) * rpr))
                assert_close(got_h[rows], want_h[rows], rel=1e-2, what=f"rank {r} {key} hidden")
        # every rank ends with the same bits
        assert np.array_equal(results[0][key][0], results[1][key][0]) or mode == "one_shot"


def _two_ranks_in_one_process(liger, lib, data_bytes, channels=1):
    """Both ends of a 2-rank communicator on this one GPU (handles exchanged in memory, peers mapped directly)."""
    import ctypes as C
    handles = [C.c_void_p(), C.c_void_p()]
    blobs = b""
    for r in range(2):
        liger.check(lib.liger_comm_create(C.byref(handles[r]), r, 2, data_bytes, channels))
        blob = (C.c_uint8 * liger.capi.COMM_HANDLE_BYTES)()
        liger.check(lib.liger_comm_export(handles[r], blob))
        blobs += bytes(blob)
    for r in range(2):
        liger.check(lib.liger_comm_connect(handles[r], blobs))
    return handles


def test_bounded_wait_gives_up_and_the_context_stays_usable(gpu, liger):
    """Failure detection without a fault: rank 1 of a 2-rank communicator never launches its side of the collective,
    so rank 0's barrier waits on a flag that nothing sets.  With the wait budget at 50 ms the kernels give up,
    record LIGER_DEV_TIMEOUT with the entry barrier's location id, and return; after clearing the status the next
    launch works as if nothing had happened."""
    import ctypes as C
    import time
    import torch
    from helpers import dev_fill, ptr, stream_ptr
    lib = gpu
    m, n = 16, 1024
    bytes_t = m * n * 2
    handles = _two_ranks_in_one_process(liger, lib, 2 * bytes_t)
    st = (C.c_uint * 4)()
    assert lib.liger_device_status(C.byref(st)) == 0
    liger.check(lib.liger_set_wait_budget_ms(50))
    try:
        torch.cuda.synchronize()
        t0 = time.time()
        liger.check(lib.liger_allreduce_fused(handles[0], 0, 0, bytes_t, None, None, None, None, None, m, n, 0, m, 0, stream_ptr()))
        torch.cuda.synchronize()
        elapsed = time.time() - t0
        assert lib.liger_device_status(C.byref(st)) == liger.capi.DEV_TIMEOUT
        assert st[0] == liger.capi.DEV_TIMEOUT and st[1] == 0x200 and st[2] == 1, list(st)   # entry barrier, waiting for rank 1
        assert 0.04 < elapsed < 2.0, elapsed   # two waits of 50 ms (entry and exit barrier), not the default 2 s each
    finally:
        liger.check(lib.liger_set_wait_budget_ms(2000))
    liger.check(lib.liger_device_status_clear())
    assert lib.liger_device_status(C.byref(st)) == 0
    # the context is intact: an ordinary launch runs and is correct
    x = dev_fill(liger, 8, 1024, 0, 900)
    g = torch.ones(1024, dtype=torch.float16, device="cuda")
    b = torch.zeros(1024, dtype=torch.float16, device="cuda")
    y = torch.empty_like(x)
    liger.check(lib.liger_layernorm(ptr(x), ptr(g), ptr(b), ptr(y), 8, 1024, stream_ptr()))
    torch.cuda.synchronize()
    want = torch.nn.functional.layer_norm(x.float(), (1024,), eps=1e-6)
    assert (y.float() - want).abs().max().item() < 2e-2
    assert lib.liger_device_status(C.byref(st)) == 0
    for h in handles:
        lib.liger_comm_destroy(h)
    assert lib.liger_set_wait_budget_ms(0) == -1


def test_copy_engine_collective_rejects_misaligned_pointers(gpu, liger):
    import ctypes as C
    lib = gpu
    h = C.c_void_p()
    liger.check(lib.liger_comm_create(C.byref(h), 0, 1, 1 << 20, 1))
    ok, odd = 0x7f0000001000, 0x7f0000001008
    assert lib.liger_allreduce_ce(h, 0, 0, 65536, 131072, None, odd, None, None, None, 8, 64, 0, 8, None) == -1
    assert b"aligned" in lib.liger_last_error()
    assert lib.liger_allreduce_ce(h, 0, 0, 65536, 131072, None, ok, odd, None, None, 8, 64, 0, 8, None) == -1
    assert lib.liger_allgather_ce(h, 3, 0, 8, 64, 0, 8, None) == -1    # channel out of range
    lib.liger_comm_destroy(h)
