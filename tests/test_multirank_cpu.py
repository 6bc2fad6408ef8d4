"""world_size-2 tests on CPU (gloo): the scheduler's cross-rank logic.  Two ranks whose clocks and
devices differ must still issue the same launches in the same order, because rank 0 decides every
admission and broadcasts it (the reference leaves admissions to per-rank thread timing although all
ranks must issue their collectives in the same order)."""
import ctypes as C
import os
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
COMM, COMP, GEMM = 0, 1, 2
LAYER = [(GEMM, 1.0), (COMP, 0.2), (GEMM, 0.4), (COMM, 0.5), (GEMM, 1.6), (GEMM, 0.8), (COMM, 0.5)]


def _worker(rank, world, port, follow_leader, results):
    import torch
    import torch.distributed as dist
    sys.path.insert(0, HERE)
    from conftest import load_package
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    liger = load_package()
    lib = liger.lib()
    cap = liger.capi

    def bcast(ctx, p):
        t = torch.tensor([p[0]], dtype=torch.int32)
        dist.broadcast(t, src=0)
        p[0] = int(t.item())
        return 0

    def barrier(ctx):
        dist.barrier()
        return 0

    cfg = liger.default_config(max_batch_size=2, max_seq_len=128, layer_num=2, factor=8, rq_interval=5000, num_requests=30,
                               ignore_num=3, seq_round=16, poisson=1, seed=5)
    kern = (cap.SimKernel * len(LAYER))(*[cap.SimKernel(t, d) for t, d in LAYER])
    n, capn = C.c_int(0), 100000
    log = (cap.SimLaunch * capn)()
    met = cap.ServingMetrics()
    b_cb, bar_cb = cap.BCAST_INT_FN(bcast), cap.BARRIER_FN(barrier)
    # rank 1's clock runs 3 ms ahead and its device is 40 % slower than profiled
    skew, slow = (0.0, 1.0) if rank == 0 else (3.0, 1.4)
    if follow_leader:
        rc = lib.liger_sim_serve_rank(C.byref(cfg), kern, len(LAYER), cap.MODE_SCHEDULE, 1.0, 0.0, rank, world, b_cb, bar_cb,
                                      None, skew, slow, log, capn, C.byref(n), C.byref(met))
    else:   # every rank decides for itself, as the reference does
        rc = lib.liger_sim_serve_rank(C.byref(cfg), kern, len(LAYER), cap.MODE_SCHEDULE, 1.0, 0.0, 0, 1, cap.BCAST_INT_FN(),
                                      cap.BARRIER_FN(), None, skew, slow, log, capn, C.byref(n), C.byref(met))
    assert rc == 0, lib.liger_last_error()
    # launch order per stream, as the device sees it
    order = {0: [], 1: []}
    for i in range(n.value):
        l = log[i]
        order[l.stream].append((l.request, l.layer, l.name, l.units_begin, l.units_end))
    # the simulator logs on completion; order each stream by start time
    for s_id in (0, 1):
        items = sorted(((log[i].t_start_ms, i) for i in range(n.value) if log[i].stream == s_id))
        order[s_id] = [(log[i].request, log[i].layer, log[i].name, log[i].units_begin, log[i].units_end) for _, i in items]
    results[rank] = (order[0], order[1], met.records)
    dist.barrier()
    dist.destroy_process_group()


def _run(follow_leader, port):
    import torch.multiprocessing as mp
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(2, port, follow_leader, results), nprocs=2, join=True)
    return results[0], results[1]


def test_ranks_issue_identical_launch_sequences_when_rank0_decides_admissions(liger):
    r0, r1 = _run(True, 29561)
    assert r0[2] == r1[2] and r0[2] > 0
    assert r0[0] == r1[0], "main-stream launch order differs between ranks"
    assert r0[1] == r1[1], "secondary-stream launch order differs between ranks"
    comm = [x for x in r0[0] + r0[1] if LAYER[x[2]][0] == COMM]
    assert comm, "the schedule must contain collectives"


def test_without_agreement_the_same_ranks_diverge(liger):
    """Control: the skewed rank deciding on its own admits at different moments (the reference's hazard)."""
    r0, r1 = _run(False, 29562)
    assert r0[0] != r1[0] or r0[1] != r1[1]
