"""The three serving entry points on real GPUs: profile -> Liger's interleaved schedule -> unscheduled
baseline (src/test_schedule.h:19-104), through the C ABI and through the C++ executable."""
import ctypes as C
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def small_cfg(liger, **kw):
    base = dict(max_batch_size=2, max_seq_len=64, head_num=8, size_per_head=64, layer_num=2, factor=4, rq_interval=300,
                graph=1, act=0, ffn_inner=2048, causal=1, num_requests=24, ignore_num=4, seq_round=16, min_seq_len=16,
                schedule_deep=3, workspace_slots=4)
    base.update(kw)
    return liger.default_config(**base)


def test_profile_schedule_and_baseline_single_gpu(gpu, liger, tmp_path):
    cfg = small_cfg(liger)
    model = C.c_void_p()
    liger.check(gpu.liger_model_create(C.byref(model), C.byref(cfg), 0, 1, None))
    d = str(tmp_path).encode()
    nb, nbar = liger.capi.BCAST_INT_FN(), liger.capi.BARRIER_FN()
    liger.check(gpu.liger_serve(model, liger.capi.MODE_PROFILE, nb, nbar, None, d, 0, None))
    main = json.load(open(tmp_path / "Main_1_64_8_2_64.json"))
    sub = json.load(open(tmp_path / "Sub_1_64_8_2_64.json"))
    assert {e["seq_len"] for e in main} == {16, 32, 48, 64}
    assert {e["kernel_name"] for e in main} == {0, 1, 2, 3, 4, 5, 6, 7}       # 7 layer kernels + the first LayerNorm
    assert all(e["duration"] > 0 for e in main)
    assert {e["kernel_name"] for e in sub} == {0, 2, 4, 5} and all(len(e["duration"]) == cfg.factor - 1 for e in sub)
    for mode in (liger.capi.MODE_SCHEDULE, liger.capi.MODE_NO_SCHEDULE):
        met = liger.capi.ServingMetrics()
        liger.check(gpu.liger_serve(model, mode, nb, nbar, None, d, 0, C.byref(met)))
        assert met.records == cfg.num_requests + 1 - cfg.ignore_num
        assert met.launch_errors == 0 and met.tokens_per_s > 0 and met.p50_latency_ms > 0
        assert met.secondary_launches == 0      # no communication kernels at world_size 1: nothing to interleave
    gpu.liger_model_destroy(model)


def _serve_worker(rank, world, port, tmpdir, results):
    import torch
    import torch.distributed as dist
    sys.path.insert(0, HERE)
    sys.path.insert(0, os.path.dirname(HERE))
    from conftest import load_package
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    liger = load_package()
    from liger_b200.dist import Comm
    lib = liger.lib()
    cfg = small_cfg(liger, max_seq_len=128, head_num=16, ffn_inner=4096, rq_interval=150, num_requests=40)
    comm = Comm(rank, world, lib.liger_model_comm_bytes(C.byref(cfg), world), channels=cfg.workspace_slots)
    model = C.c_void_p()
    liger.check(lib.liger_model_create(C.byref(model), C.byref(cfg), rank, world, comm.handle))

    def bcast(ctx, p):
        t = torch.tensor([p[0]], dtype=torch.int32)
        dist.broadcast(t, src=0)
        p[0] = int(t.item())
        return 0

    def barrier(ctx):
        dist.barrier()
        return 0

    b_cb, bar_cb = liger.capi.BCAST_INT_FN(bcast), liger.capi.BARRIER_FN(barrier)
    d = tmpdir.encode()
    liger.check(lib.liger_serve(model, liger.capi.MODE_PROFILE, b_cb, bar_cb, None, d, 0, None))
    out = {}
    for name, mode in (("schedule", liger.capi.MODE_SCHEDULE), ("no_schedule", liger.capi.MODE_NO_SCHEDULE)):
        met = liger.capi.ServingMetrics()
        liger.check(lib.liger_serve(model, mode, b_cb, bar_cb, None, d, 0, C.byref(met)))
        out[name] = dict(records=met.records, tokens_per_s=met.tokens_per_s, p50=met.p50_latency_ms, errors=met.launch_errors,
                         secondary=met.secondary_launches, decompositions=met.decompositions, segments=met.segments)
    st = (C.c_uint * 4)()
    assert lib.liger_device_status(C.byref(st)) == 0, list(st)
    results[rank] = out
    dist.barrier()
    dist.destroy_process_group()


def test_interleaved_schedule_two_ranks(tmp_path):
    """Liger's schedule at world_size 2: all-reduces of one request overlap other requests' GEMMs on the
    secondary stream, every rank issues the same sequence, no wait times out."""
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_serve_worker, args=(2, 29571, str(tmp_path), results), nprocs=2, join=True)
    for r in range(2):
        for name in ("schedule", "no_schedule"):
            m = results[r][name]
            assert m["records"] == 40 + 1 - 4 and m["errors"] == 0 and m["tokens_per_s"] > 0
        assert results[r]["schedule"]["secondary"] > 0
        assert results[r]["no_schedule"]["secondary"] == 0
    assert results[0]["schedule"]["secondary"] == results[1]["schedule"]["secondary"]
    assert results[0]["schedule"]["segments"] == results[1]["schedule"]["segments"]


def test_serving_executable_two_ranks(liger, tmp_path):
    """host/main.cu over the MPI stand-in: the reference's command line, two processes, two GPUs."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    liger.build_all()
    liger.build.build_host()
    cmd = [liger.build.MPIRUN_PATH, "-np", "2", liger.build.MAIN_PATH, "2", "64", "8", "64", "2", "16", "4", "4000",
           "--graph", "preln", "--causal", "1", "--requests", "30", "--ignore", "4", "--seq-round", "16", "--depth", "3"]
    res = subprocess.run(cmd, cwd=str(tmp_path), capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert res.stdout.count("Communication Complete from Rank") == 2
    assert os.path.exists(tmp_path / "Main_2_64_8_2_64.json") and os.path.exists(tmp_path / "Sub_2_64_8_2_64.json")
    assert res.stdout.count("Throughput:") == 2 and res.stdout.count("Average Latency:") == 2   # schedule + no_schedule
    assert "Total 27 records." in res.stdout
