"""Whole-stack parity: the function-assembled layer stack (liger_model_forward) against the fp32 CPU
oracle on the same seeded weights and inputs.  Bound: max |got - want| / max |want| <= 1e-2 against
the pure-fp32 oracle (the GPU path stores fp16 between kernels and accumulates in fp32; with
world_size > 1 the partial sums are rounded to fp16 before the fp32 reduction, whose order starts
at rank (row mod world_size) instead of rank 0)."""
import ctypes as C
import os
import sys

import numpy as np
import pytest

from helpers import assert_close, dev_fill, max_rel_err, ptr, stream_ptr, to_np

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))

CASES = {
    # the reference graph: post-LayerNorm, no residual, GELU 4H, mask tensor of ones (src/layer/bert.h:59-79)
    "ref_gelu": dict(head_num=4, size_per_head=64, layer_num=2, graph=0, act=0, ffn_inner=0, causal=0, B=2, S=64),
    # BASELINE config 1: 2 layers, hidden 1024, 16 x 64, FFN 4096 GELU, pre-LN, causal, batch 4 x seq 128
    "tiny_preln": dict(head_num=16, size_per_head=64, layer_num=2, graph=1, act=0, ffn_inner=4096, causal=1, B=4, S=128),
    # gated FFN, head_dim 128, ragged sequence length
    "preln_geglu": dict(head_num=4, size_per_head=128, layer_num=3, graph=1, act=1, ffn_inner=1024, causal=1, B=3, S=72),
    # large enough (2 MiB of activations) for the bandwidth path: GEMM epilogues scatter their partial sums to
    # the owning ranks and the all-reduce finishes from local slots; M not divisible by 128
    "preln_two_shot": dict(head_num=16, size_per_head=64, layer_num=2, graph=1, act=0, ffn_inner=2048, causal=1, B=4, S=264),
    "ref_two_shot": dict(head_num=16, size_per_head=64, layer_num=1, graph=0, act=1, ffn_inner=2048, causal=0, B=2, S=520),
    "ref_geglu_causal": dict(head_num=8, size_per_head=64, layer_num=1, graph=0, act=1, ffn_inner=2048, causal=1, B=1, S=200),
    # big enough for the CTA-pair GEMM kernels (256x256 and, in the FFN-down GEMM with K >= 8192, 256x512 tiles) with
    # every epilogue kind including the scatter to the owning rank at TP = 2, and for the tcgen05 attention kernel
    "preln_pair_kernels": dict(head_num=32, size_per_head=128, layer_num=1, graph=1, act=0, ffn_inner=16384, causal=1, B=8,
                               S=512),
}


def make_cfg(liger, case, slots=2):
    c = CASES[case]
    return liger.default_config(max_batch_size=c["B"], max_seq_len=c["S"], head_num=c["head_num"],
                                size_per_head=c["size_per_head"], layer_num=c["layer_num"], graph=c["graph"], act=c["act"],
                                ffn_inner=c["ffn_inner"], causal=c["causal"], seed=0, workspace_slots=slots,
                                schedule_deep=1)


def oracle_out(oracle, case, tp, round16):
    c = CASES[case]
    H = c["head_num"] * c["size_per_head"]
    cfg = oracle.Config(hidden=H, heads=c["head_num"], head_dim=c["size_per_head"], ffn_inner=c["ffn_inner"] or 4 * H,
                        layers=c["layer_num"], tp=tp, graph=c["graph"], act=c["act"], causal=c["causal"], round16=round16,
                        seed=0)
    M = c["B"] * c["S"]
    x = oracle.fill_normal(M * H, 0, oracle.INPUT).reshape(M, H)
    return oracle.stack_forward(cfg, x, c["B"], c["S"])


@pytest.mark.parametrize("case", list(CASES))
def test_stack_forward_single_gpu(gpu, liger, oracle, case):
    import torch
    c = CASES[case]
    H = c["head_num"] * c["size_per_head"]
    M = c["B"] * c["S"]
    cfg = make_cfg(liger, case)
    model = C.c_void_p()
    liger.check(gpu.liger_model_create(C.byref(model), C.byref(cfg), 0, 1, None))
    x = dev_fill(liger, M, H, 0, oracle.INPUT)
    out = torch.zeros((M, H), dtype=torch.float16, device="cuda")
    n = liger.check(gpu.liger_model_forward(model, ptr(x), ptr(out), c["B"], c["S"], 0, stream_ptr()))
    torch.cuda.synchronize()
    st = (C.c_uint * 4)()
    assert gpu.liger_device_status(C.byref(st)) == 0, list(st)
    assert n == 7 * c["layer_num"]   # pre-LN: one LayerNorm in front, none after the last layer
    want = oracle_out(oracle, case, 1, 0)
    assert_close(to_np(out), want, rel=1e-2, what=case)
    # the oracle with fp16 rounding at the same places agrees more closely
    assert max_rel_err(to_np(out), oracle_out(oracle, case, 1, 1)) < 5e-3
    # host-buffer entry point gives the same bits; a second slot too
    hin = x.cpu().pin_memory()
    hout = torch.zeros((M, H), dtype=torch.float16).pin_memory()
    liger.check(gpu.liger_model_forward_host(model, C.c_void_p(hin.data_ptr()), C.c_void_p(hout.data_ptr()), c["B"],
                                             c["S"], 1, stream_ptr()))
    torch.cuda.synchronize()
    assert torch.equal(hout, out.cpu())
    gpu.liger_model_destroy(model)


def test_shorter_request_than_maximum(gpu, liger, oracle):
    """A request smaller than (max_batch, max_seq) uses the same model (ragged serving lengths)."""
    import torch
    case = "tiny_preln"
    c = dict(CASES[case])
    cfg = make_cfg(liger, case)
    model = C.c_void_p()
    liger.check(gpu.liger_model_create(C.byref(model), C.byref(cfg), 0, 1, None))
    B, S, H = 2, 36, 1024
    x = dev_fill(liger, B * S, H, 0, oracle.INPUT)
    out = torch.zeros((B * S, H), dtype=torch.float16, device="cuda")
    liger.check(gpu.liger_model_forward(model, ptr(x), ptr(out), B, S, -1, stream_ptr()))
    ocfg = oracle.Config(hidden=H, heads=16, head_dim=64, ffn_inner=4096, layers=2, tp=1, graph=1, act=0, causal=1,
                         round16=0, seed=0)
    want = oracle.stack_forward(ocfg, to_np(x), B, S)
    assert_close(to_np(out), want, rel=1e-2, what="short request")
    assert gpu.liger_model_forward(model, ptr(x), ptr(out), 5, 128, 0, stream_ptr()) == -1   # batch > max
    gpu.liger_model_destroy(model)


def _tp_worker(rank, world, port, case, results):
    import torch
    import torch.distributed as dist
    sys.path.insert(0, HERE)
    sys.path.insert(0, os.path.dirname(HERE))
    from conftest import load_package
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    liger = load_package()
    from liger_b200.dist import Comm
    lib = liger.lib()
    c = CASES[case]
    H = c["head_num"] * c["size_per_head"]
    M = c["B"] * c["S"]
    cfg = make_cfg(liger, case, slots=4)
    # two flag sets per workspace slot: the pipelined schedule keeps a slot's copy-engine all-gather (communication
    # stream) and its next reduction (compute stream) in flight at the same time
    # (three with the gathered schedule, whose all-gather also announces row blocks to the next GEMM)
    comm = Comm(rank, world, lib.liger_model_comm_bytes(C.byref(cfg), world), channels=3 * cfg.workspace_slots)
    model = C.c_void_p()
    liger.check(lib.liger_model_create(C.byref(model), C.byref(cfg), rank, world, comm.handle))
    x = dev_fill(liger, M, H, 0, 0x10000)
    out = torch.zeros((M, H), dtype=torch.float16, device="cuda")
    dist.barrier()
    for rep in range(2):
        liger.check(lib.liger_model_forward(model, ptr(x), ptr(out), c["B"], c["S"], rep % 2, stream_ptr()))
        torch.cuda.synchronize()
    # the gathered schedule (whole batch; the all-gather runs beside the GEMM that consumes it, which waits tile by
    # tile for its rows) gives the same bits, pass after pass, with and without per-kernel timing
    liger.check(lib.liger_model_set_overlap(model, 2))
    outg = torch.zeros_like(out)
    for rep in range(3):
        if rep == 2:
            liger.check(lib.liger_model_set_kernel_timing(model, 1))
        outg.zero_()
        liger.check(lib.liger_model_forward(model, ptr(x), ptr(outg), c["B"], c["S"], rep % 2, stream_ptr()))
        torch.cuda.synchronize()
        assert torch.equal(outg, out), f"gathered schedule differs from the in-line pass (rep {rep})"
    kms0, kcnt0 = (C.c_double * 9)(), (C.c_longlong * 9)()
    liger.check(lib.liger_model_kernel_times(model, C.byref(kms0), C.byref(kcnt0)))
    liger.check(lib.liger_model_set_kernel_timing(model, 0))
    assert kcnt0[0] == c["layer_num"] and kcnt0[4] == c["layer_num"]
    liger.check(lib.liger_model_set_overlap(model, 1))
    # host-buffer entry point: every rank uploads its rows, rank 0 receives the result
    hin = x.cpu().pin_memory()
    hout = torch.zeros((M, H), dtype=torch.float16).pin_memory()
    liger.check(lib.liger_model_forward_host(model, C.c_void_p(hin.data_ptr()), C.c_void_p(hout.data_ptr()), c["B"], c["S"],
                                             1, stream_ptr()))
    torch.cuda.synchronize()
    if rank == 0:
        assert torch.equal(hout, out.cpu())
    # sharded download: every rank receives exactly the rows it uploaded, nothing else is written
    liger.check(lib.liger_model_set_output_sharding(model, 1))
    hpart = torch.zeros((M, H), dtype=torch.float16).pin_memory()
    liger.check(lib.liger_model_forward_host(model, C.c_void_p(hin.data_ptr()), C.c_void_p(hpart.data_ptr()), c["B"], c["S"],
                                             1, stream_ptr()))
    torch.cuda.synchronize()
    rpr = (M + world - 1) // world
    lo, hi = min(rank * rpr, M), min((rank + 1) * rpr, M)
    assert torch.equal(hpart[lo:hi], out.cpu()[lo:hi])
    assert not hpart[:lo].any() and not hpart[hi:].any()
    liger.check(lib.liger_model_set_output_sharding(model, 0))
    # the batch split into two micro-requests gives the same bits, with either way of sharing the GPU: 1 = one
    # compute stream + copy-engine all-gathers underneath (the default), 0 = one stream per micro-request
    if c["B"] % 2 == 0:
        liger.check(lib.liger_model_set_micro_batches(model, 2))
        for overlap in (1, 0):
            liger.check(lib.liger_model_set_overlap(model, overlap))
            out2 = torch.zeros_like(out)
            for rep in range(2):
                liger.check(lib.liger_model_forward(model, ptr(x), ptr(out2), c["B"], c["S"], 0, stream_ptr()))
                torch.cuda.synchronize()
            assert torch.equal(out2, out), f"micro-batches (overlap mode {overlap}) differ from the un-split pass"
        liger.check(lib.liger_model_set_overlap(model, 1))
        # per-kernel timing inside the pipelined pass does not change the result
        liger.check(lib.liger_model_set_kernel_timing(model, 1))
        out3 = torch.zeros_like(out)
        liger.check(lib.liger_model_forward(model, ptr(x), ptr(out3), c["B"], c["S"], 2, stream_ptr()))
        kms, kcnt, ov = (C.c_double * 9)(), (C.c_longlong * 9)(), (C.c_double * 4)()
        liger.check(lib.liger_model_kernel_times(model, C.byref(kms), C.byref(kcnt)))
        liger.check(lib.liger_model_overlap_times(model, C.byref(ov)))
        liger.check(lib.liger_model_set_kernel_timing(model, 0))
        assert torch.equal(out3, out)
        assert kcnt[0] == 2 * c["layer_num"] and kcnt[3] == 2 * c["layer_num"]   # both micro-requests, every layer
        # round-robin slots (-1) with two micro-batches on four slots: pairs (0,1), (2,3), (0,1), ... never overlap
        # and never run past the last slot, however often the host-buffer entry point is called
        hrr = torch.zeros((M, H), dtype=torch.float16).pin_memory()
        for rep in range(5):
            liger.check(lib.liger_model_forward_host(model, C.c_void_p(hin.data_ptr()), C.c_void_p(hrr.data_ptr()), c["B"],
                                                     c["S"], -1, stream_ptr()))
            torch.cuda.synchronize()
        if rank == 0:
            assert torch.equal(hrr, out.cpu())
        assert lib.liger_model_set_micro_batches(model, 5) == -1   # more micro-batches than workspace slots
        liger.check(lib.liger_model_set_micro_batches(model, 1))
    st = (C.c_uint * 4)()
    assert lib.liger_device_status(C.byref(st)) == 0, list(st)
    results[rank] = to_np(out)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("case", ["tiny_preln", "ref_gelu", "preln_geglu", "preln_two_shot", "ref_two_shot",
                                  "preln_pair_kernels"])
def test_stack_forward_tensor_parallel_2(oracle, case):
    """BASELINE config 1 is the tiny pre-LN stack at TP = 2."""
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_tp_worker, args=(2, 29541, case, results), nprocs=2, join=True)
    want = oracle_out(oracle, case, 2, 0)
    for r in range(2):
        assert_close(results[r], want, rel=1e-2, what=f"{case} rank {r}")
    assert np.array_equal(results[0], results[1])
    # tensor parallelism does not change the result beyond rounding: TP=2 vs the TP=1 oracle
    assert max_rel_err(results[0], oracle_out(oracle, case, 1, 0)) < 1e-2


@pytest.mark.parametrize("B,kv_len,cap,heads,D,F,act", [(4, 300, 512, 8, 128, 2048, 1), (3, 17, 64, 4, 64, 1024, 0)])
def test_decode_step_single_gpu(gpu, liger, oracle, B, kv_len, cap, heads, D, F, act):
    """BASELINE config 3 in miniature: one new token per sequence against a seeded N(0,1) KV cache."""
    import torch
    H = heads * D
    cfg = liger.default_config(max_batch_size=B, max_seq_len=8, head_num=heads, size_per_head=D, layer_num=2, graph=1,
                               act=act, ffn_inner=F, causal=1, seed=0, workspace_slots=2, schedule_deep=1, kv_capacity=cap)
    model = C.c_void_p()
    liger.check(gpu.liger_model_create(C.byref(model), C.byref(cfg), 0, 1, None))
    liger.check(gpu.liger_model_fill_kv_cache(model))
    x = dev_fill(liger, B, H, 0, oracle.INPUT)
    out = torch.zeros((B, H), dtype=torch.float16, device="cuda")
    n = liger.check(gpu.liger_model_decode(model, ptr(x), ptr(out), B, kv_len, 0, stream_ptr()))
    torch.cuda.synchronize()
    assert n == 7 * 2
    ocfg = oracle.Config(hidden=H, heads=heads, head_dim=D, ffn_inner=F, layers=2, tp=1, graph=1, act=act, causal=1,
                         round16=0, seed=0)
    want = oracle.stack_decode(ocfg, to_np(x), B, kv_len, cap)
    assert_close(to_np(out), want, rel=1e-2, what="decode step")
    # the step appended the token's K/V: a second step at kv_len + 1 must see them (result changes, stays finite)
    out2 = torch.zeros_like(out)
    liger.check(gpu.liger_model_decode(model, ptr(x), ptr(out2), B, kv_len + 1, 0, stream_ptr()))
    assert torch.isfinite(out2.float()).all() and not torch.equal(out2, out)
    assert gpu.liger_model_decode(model, ptr(x), ptr(out), B, cap, 0, stream_ptr()) == -1   # cache full
    gpu.liger_model_destroy(model)


def _decode_tp_worker(rank, world, port, results):
    import torch
    import torch.distributed as dist
    sys.path.insert(0, HERE)
    sys.path.insert(0, os.path.dirname(HERE))
    from conftest import load_package
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    liger = load_package()
    from liger_b200.dist import Comm
    lib = liger.lib()
    B, kv_len, cap, heads, D, F = DECODE_TP["B"], DECODE_TP["kv_len"], DECODE_TP["cap"], DECODE_TP["heads"], DECODE_TP["D"], DECODE_TP["F"]
    H = heads * D
    cfg = liger.default_config(max_batch_size=B, max_seq_len=8, head_num=heads, size_per_head=D, layer_num=2, graph=1, act=1,
                               ffn_inner=F, causal=1, seed=0, workspace_slots=2, schedule_deep=1, kv_capacity=cap)
    comm = Comm(rank, world, lib.liger_model_comm_bytes(C.byref(cfg), world), channels=4)
    model = C.c_void_p()
    liger.check(lib.liger_model_create(C.byref(model), C.byref(cfg), rank, world, comm.handle))
    liger.check(lib.liger_model_fill_kv_cache(model))
    x = dev_fill(liger, B, H, 0, 0x10000)
    out = torch.zeros((B, H), dtype=torch.float16, device="cuda")
    dist.barrier()
    liger.check(lib.liger_model_decode(model, ptr(x), ptr(out), B, kv_len, 0, stream_ptr()))
    torch.cuda.synchronize()
    # the same step again, eight times back to back without host synchronisation: it appends the same K / V at the
    # same position, so every repetition must give the same bits (the one-shot all-reduces of consecutive steps reuse
    # their two partial buffers in turn and have no exit barrier)
    outs = [torch.zeros_like(out) for _ in range(8)]
    for o in outs:
        liger.check(lib.liger_model_decode(model, ptr(x), ptr(o), B, kv_len, 0, stream_ptr()))
    torch.cuda.synchronize()
    for o in outs:
        assert torch.equal(o, out)
    st = (C.c_uint * 4)()
    assert lib.liger_device_status(C.byref(st)) == 0, list(st)
    results[rank] = to_np(out)
    dist.barrier()
    lib.liger_model_destroy(model)
    comm.close()
    dist.destroy_process_group()


DECODE_TP = dict(B=4, kv_len=300, cap=512, heads=8, D=128, F=2048)


def test_decode_step_tensor_parallel_2(oracle):
    """BASELINE config 3 in miniature at TP = 2: KV cache sharded by head, one-shot all-reduce of the [B, H] partials."""
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_decode_tp_worker, args=(2, 29547, results), nprocs=2, join=True)
    d = DECODE_TP
    H = d["heads"] * d["D"]
    x = oracle.fill_normal(d["B"] * H, 0, oracle.INPUT).reshape(d["B"], H)
    for tp in (2, 1):
        ocfg = oracle.Config(hidden=H, heads=d["heads"], head_dim=d["D"], ffn_inner=d["F"], layers=2, tp=tp, graph=1, act=1,
                             causal=1, round16=0, seed=0)
        want = oracle.stack_decode(ocfg, x, d["B"], d["kv_len"], d["cap"])
        for r in range(2):
            assert_close(results[r], want, rel=1e-2, what=f"decode TP=2 rank {r} vs oracle tp={tp}")
    assert np.array_equal(results[0], results[1])


def test_model_destroy_returns_device_memory(gpu, liger):
    """liger_model_destroy frees weights, workspaces, caches and staging buffers (the reference never frees)."""
    import torch
    cfg = liger.default_config(max_batch_size=4, max_seq_len=256, head_num=16, size_per_head=64, layer_num=4, graph=1, act=0,
                               ffn_inner=4096, causal=1, seed=0, workspace_slots=2, schedule_deep=1, kv_capacity=128)
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info()[0]
    held = []
    for rep in range(3):
        model = C.c_void_p()
        liger.check(gpu.liger_model_create(C.byref(model), C.byref(cfg), 0, 1, None))
        held.append(free0 - torch.cuda.mem_get_info()[0])
        liger.check(gpu.liger_model_destroy(model))
    torch.cuda.synchronize()
    assert min(held) > 100 << 20                       # the model did hold its ~130 MB of weights and buffers
    assert free0 - torch.cuda.mem_get_info()[0] < 8 << 20   # and gave all of it back (allocator granularity aside)
