#!/usr/bin/env python
"""Benchmarks of the tensor-parallel layer-stack path.

    python bench.py --gpus N --steps K --warmup W                  (N = 1; the headline: --workload prefill)
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...                           (the reference's own build, same workload)
    python bench.py --workload decode | allreduce_sweep ...

Workloads (synthetic throughout: seeded random weights of the architecture, seeded random hidden states)
  prefill          BASELINE config 2, the one the headline metric is quoted on.  4 decoder layers, hidden 12288,
                   96 heads x 128, GeGLU FFN 32768, pre-LayerNorm with residual adds, causal attention, fp16
                   weights ~N(0, 0.02), fp16 activations ~N(0, 1), seed 0, batch 8 x sequence 512 (4096 tokens per
                   step), tensor parallel over the N GPUs (strong scaling).  A step is one forward pass.
  decode           BASELINE config 3: the same layers, batch 32, one new token each against a seeded KV cache of
                   2048 positions per sequence.  A step is one decode step (32 tokens).
  allreduce_sweep  BASELINE config 5: the fused all-reduce + residual add on fp16 tensors from 8 KB to 512 MB,
                   N >= 2; one record per size (microseconds and bus GB/s).

One JSON line is printed by rank 0, as the last line of stdout:
  value        tokens/s with the input already in HBM (CUDA events around the K timed steps, max over ranks)
  e2e          tokens/s through liger_model_forward_host: pinned host input -> device, the pass, result -> host
  roofline     prefill: the tcgen05 GEMM launches, FLOPs / in-situ duration against the measured cuBLAS peak;
               decode: bytes that must be streamed per step / step time against the measured HBM bandwidth
  parity       rows of the result compared with rows the CPU oracle produced for the same seeded configuration
               (tests/golden/bench_glm130b_rows.npz); the run fails if they differ by more than 1e-2 relative
  cpu_baseline the fp32 host port of the same stack on the box's cores (N = 1, prefill only)
"""
import argparse
import ctypes as C
import importlib.util
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG_DIR = os.path.join(ROOT, "24ppopp-liger_b200")
GOLDEN_ROWS = os.path.join(ROOT, "tests", "golden", "bench_glm130b_rows.npz")

GLM = dict(layers=4, heads=96, head_dim=128, ffn_inner=32768)
WORKLOAD = dict(GLM, name="glm130b_shape_prefill_4layer_b8_s512", batch=8, seq=512)
DECODE = dict(GLM, name="glm130b_shape_decode_4layer_b32_kv2048", batch=32, kv_len=2048, kv_capacity=2112)
PARITY_REL = 1e-2


def load_package():
    if "liger_b200" in sys.modules:
        return sys.modules["liger_b200"]
    spec = importlib.util.spec_from_file_location(
        "liger_b200", os.path.join(PKG_DIR, "__init__.py"), submodule_search_locations=[PKG_DIR])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["liger_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


def measured_peaks():
    """Roofline denominators: the driver-measured figures of this pool when present, else the stated fallback."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        burst = float(p.get("bf16_tflops", 1590.0))
        return dict(burst=burst, sustained=float(p.get("bf16_tflops_sustained", burst)), hbm_gbs=float(p["hbm_gbs"]),
                    source="of measured (MEASURED_PEAKS.json)")
    return dict(burst=1590.0, sustained=1400.0, hbm_gbs=6650.0, source="of fallback (1.59 / 1.4 PFLOP/s, 6.65 TB/s)")


def gemm_peak(peaks, clocks):
    """The cuBLAS figure measured in the regime this run was in: the seconds-long power-capped loop when the GPU
    sat on its power cap during the timed region, the burst figure otherwise."""
    capped = bool(clocks and "sw_power_cap" in (clocks.get("reasons") or []))
    return (peaks["sustained"], "sustained (sw_power_cap active during the timed region)") if capped else \
        (peaks["burst"], "burst (no power cap during the timed region)")


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return dict(sm_mhz=sm[len(sm) // 2] if sm else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=sorted(reasons), samples=len(sm))


def cpu_port_tokens_per_s():
    """fp32 host port of the same stack, timed on this machine's cores on a bounded sample: one
    GLM-shape layer (all tensor-parallel shards) on 512 tokens, the time spent materialising the
    seeded weights excluded, scaled to the 4-layer stack."""
    sys.path.insert(0, ROOT)
    import oracle
    oracle.build()
    H = WORKLOAD["heads"] * WORKLOAD["head_dim"]
    cfg = oracle.Config(hidden=H, heads=WORKLOAD["heads"], head_dim=WORKLOAD["head_dim"], ffn_inner=WORKLOAD["ffn_inner"],
                        layers=1, tp=1, graph=1, act=1, causal=1, round16=0, seed=0)
    s = 512
    x = oracle.fill_normal(s * H, 0, oracle.INPUT).reshape(s, H)
    oracle.fill_seconds(reset=True)
    t0 = time.time()
    oracle.stack_forward(cfg, x, 1, s)
    total = time.time() - t0
    fill = oracle.fill_seconds(reset=True)
    compute = max(total - fill, 1e-9)
    value = s / (compute * WORKLOAD["layers"])
    return dict(value=value, unit="tokens/s", cores=oracle.num_threads(), kind="port",
                sample=(f"oracle/liger_oracle.c (fp32, OpenMP, AVX2): one GLM-130B-shape layer, all shards, one sequence of "
                        f"{s} tokens: {compute:.1f} s of arithmetic ({fill:.1f} s of weight generation excluded); "
                        f"tokens/s = {s} / (t * 4 layers), extrapolated to the 4-layer stack"))


REF_HARNESS = os.path.join(ROOT, "oracle", "_ref", "liger_ref_harness")

# DRAM bytes per GEMM launch at N=1 (read + write, average of the QKV / out-proj / FFN-up / FFN-down launches of
# one layer), from the one-pass ncu capture summarised under profiles/.
GEMM_DRAM_BYTES_PER_LAUNCH_TP1 = 4.44e9
# Decode: DRAM bytes (read + write) per algorithmic byte of the two kernels that make up a step, from ncu captures
# of smaller cases (a full step holds 27 GB): 304.1 + 4.3 MB for the 303.6 MB of the 32 x 12288 x 12288 few-row
# GEMM, 805.6 + 6.3 MB for the 805.3 MB of decode attention over 8 of the 32 sequences.
GEMM_SMALLM_TRAFFIC_RATIO = (304.1 + 4.3) / 303.6
ATTENTION_DECODE_TRAFFIC_RATIO = (805.6 + 6.3) / 805.3


# ---- the reference arm ------------------------------------------------------------------------------------
def run_reference_harness(argv, rank, world, record_key):
    """The reference's own NCCL + cuBLAS build (unmodified sources + oracle/ref_harness/harness.cu, compiled for
    sm_100a into oracle/_ref/), one process per GPU over the MPI stand-in.  Returns rank 0's JSON record."""
    env = dict(os.environ)
    env["LIGER_MPI_RANK"], env["LIGER_MPI_SIZE"] = str(rank), str(world)
    env["LIGER_MPI_JOB"] = "bench_ref_%s" % os.environ.get("MASTER_PORT", "0")
    env.setdefault("LIGER_MPI_TIMEOUT_S", "120")
    try:
        res = subprocess.run([REF_HARNESS] + [str(a) for a in argv], env=env, capture_output=True, text=True, timeout=600)
    except (OSError, subprocess.TimeoutExpired) as e:
        return {"error": f"{type(e).__name__}: {e}"} if rank == 0 else None
    if rank != 0:
        return None
    for ln in res.stdout.splitlines():
        if ln.startswith("{\"" + record_key + "\""):
            rec = json.loads(ln)
            if res.returncode == 0 and rec.get("cuda_error") == "no error":
                return rec
            return {"error": f"exit {res.returncode}, cuda_error {rec.get('cuda_error')}"}
    return {"error": f"exit {res.returncode}: {(res.stderr or res.stdout)[-300:]}"}


def run_reference_arm(args, rank, world):
    """--impl reference.  The reference has no CPU implementation of this path, so the arm is its own GPU build:
    prefill = its layer stack at the benchmark's hidden size (post-LayerNorm, no residual, GELU with a 4H FFN, full
    attention through a mask tensor: the only layer it can express; same GEMM FLOPs as the GeGLU-32768 layer);
    decode = the same stack on 32 sequences of one token (its GEMM chain at the decode batch: it has no KV cache,
    so the cache read is missing from its step); allreduce_sweep = ncclAllReduce + its add_bias_input kernel.
    When the build is missing or fails, the prefill arm times the CPU port of the arithmetic (the oracle)."""
    W = WORKLOAD if args.workload != "decode" else DECODE
    H = W["heads"] * W["head_dim"]
    base = {"impl": "reference", "metric": "tokens/s", "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "data": "synthetic"}
    build = ("unmodified reference sources + oracle/ref_harness/harness.cu, nvcc sm_100a, cuBLAS + NCCL, MPI stand-in; "
             "kernel vector replayed in order on one stream (Scheduler::run_sequential)")
    missing = None if os.path.exists(REF_HARNESS) else "oracle/_ref/liger_ref_harness has not been built"
    if args.workload == "allreduce_sweep":
        rec = {"error": missing} if missing else run_reference_harness(["sweep", args.sweep_max_mb, args.steps], rank, world, "ref_sweep")
        if rank != 0:
            return
        if rec and "error" not in rec:
            line = dict(base, metric="allreduce+residual bus GB/s", unit="GB/s", value=max(r["bus_gbs"] for r in rec["records"]),
                        ms_per_step=None, dtype="fp16", config={"workload": "allreduce_residual_sweep_8KB_512MB", "parallelism": f"tp{world}",
                                                                "build": build, "collective": "ncclAllReduce (in place) + add_bias_input kernel"},
                        records=rec["records"], gpu_launches=2 * len(rec["records"]) * args.steps)
        else:
            line = dict(base, unavailable="reference all-reduce sweep: " + (rec or {}).get("error", "unknown"))
        print(json.dumps(line), flush=True)
        return
    if args.workload == "decode":
        tokens = W["batch"]
        argv = [W["batch"], 1, W["heads"], W["head_dim"], args.layers, args.steps, max(args.warmup, 3)]
        graph = ("the reference's own layer on 32 sequences of ONE token (it has no KV cache or decode path): the GEMM chain of "
                 "a decode step at the same batch, attention over a single key; the 2048-position cache read is absent")
    else:
        tokens = W["batch"] * W["seq"]
        argv = [W["batch"], W["seq"], W["heads"], W["head_dim"], args.layers, args.steps, max(args.warmup, 3)]
        graph = ("the reference's own layer: post-LayerNorm, no residual, GELU FFN 4H (same GEMM FLOPs as the GeGLU-32768 "
                 "layer), full attention with an all-ones mask")
    rec = {"error": missing} if missing else run_reference_harness(argv, rank, world, "ref_harness")
    if rank != 0:
        return
    if rec and "error" not in rec:
        line = dict(base, value=rec["tokens_per_s"], ms_per_step=rec["ms_per_step"], p50_latency_ms=rec["ms_per_step"],
                    dtype="fp16 (fp16 accumulate, CUBLAS_COMPUTE_16F)",
                    config={"workload": W["name"], "tokens_per_step": tokens, "parallelism": f"tp{world}", "graph": graph, "build": build},
                    cpu_baseline={"value": rec["tokens_per_s"], "unit": "tokens/s", "cores": 0, "kind": "reference",
                                  "sample": "the reference's GPU build (it has no CPU path): full workload, all steps"},
                    e2e={"value": rec["tokens_per_s_e2e"], "unit": "tokens/s", "ms_per_step": rec["ms_per_step_e2e"],
                         "h2d_bytes_per_step": tokens * H * 2 * world, "d2h_bytes_per_step": tokens * H * 2,
                         "note": "every rank uploads the whole input (the reference cannot distribute it); rank 0 downloads the result"},
                    gpu_launches=rec["kernels_per_step"] * args.steps)
    elif args.workload == "prefill":
        cpu = cpu_port_tokens_per_s()
        line = dict(base, value=cpu["value"], ms_per_step=1000.0 * tokens / cpu["value"], dtype="f32",
                    config={"workload": W["name"], "tokens_per_step": tokens,
                            "note": "reference GPU build unavailable: " + (rec or {}).get("error", "unknown")},
                    cpu_baseline=cpu,
                    e2e={"value": cpu["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                    gpu_launches=0)
    else:
        line = dict(base, unavailable="reference build: " + (rec or {}).get("error", "unknown"))
    print(json.dumps(line), flush=True)


# ---- this library's arm -------------------------------------------------------------------------------------
class Env:
    """Process-group plumbing shared by the workloads."""

    def __init__(self, args):
        import torch
        self.torch = torch
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", str(self.rank)))
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
        torch.cuda.set_device(self.local_rank)
        self.liger = load_package()
        self.lib = self.liger.lib()   # raises if the CUDA library is missing
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group("nccl", rank=self.rank, world_size=self.world, device_id=torch.device("cuda", self.local_rank))
            self.dist = dist
        self.stream = torch.cuda.current_stream()
        self.sp = C.c_void_p(self.stream.cuda_stream)

    def barrier(self):
        if self.dist:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def all_ok(self, flag):
        if not self.dist:
            return bool(flag)
        t = self.torch.tensor([1 if flag else 0], device="cuda")
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MIN)
        return int(t.item()) == 1

    def max_over_ranks(self, value):
        t = self.torch.tensor([value], dtype=self.torch.float64, device="cuda")
        if self.dist:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def timed(self, fn, steps):
        """K steps between two barriers, CUDA events on the launch stream, max over ranks.  Also returns the median
        of the per-step durations (events between the steps): the latency of one request."""
        torch = self.torch
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        self.barrier()
        ev[0].record(self.stream)
        launches = 0
        for i in range(steps):
            launches += fn()
            ev[i + 1].record(self.stream)
        self.barrier()
        per_step = sorted(ev[i].elapsed_time(ev[i + 1]) for i in range(steps))
        return self.max_over_ranks(ev[0].elapsed_time(ev[steps])), launches, self.max_over_ranks(per_step[len(per_step) // 2])

    def check_device_status(self):
        st = (C.c_uint * 4)()
        if self.lib.liger_device_status(C.byref(st)) != 0:
            raise SystemExit(f"device status word set: {list(st)}")

    def finish(self):
        if self.dist:
            self.dist.barrier()
            self.dist.destroy_process_group()


def check_rows(env, got_rows, want_rows, what):
    """max |got - want| / max |want| over the fixture rows; every rank checks its own copy of the result."""
    import numpy as np
    got = got_rows.float().cpu().numpy().astype(np.float64)
    want = want_rows.astype(np.float64)
    err = float(np.abs(got - want).max() / max(np.abs(want).max(), 1e-30))
    worst = env.max_over_ranks(err if np.isfinite(got).all() else float("inf"))
    if not worst <= PARITY_REL:
        raise SystemExit(f"parity check failed: {what} differs from the oracle's rows by {worst:.3g} relative (bound {PARITY_REL})")
    return {"checked": True, "max_rel": worst, "bound": PARITY_REL, "rows": int(want.shape[0]), "cols": int(want.shape[1]),
            "against": "CPU oracle rows in tests/golden/bench_glm130b_rows.npz (" + what + "), every rank's copy of the result"}


def run_prefill(args, env):
    import numpy as np
    torch, liger, lib, rank, world = env.torch, env.liger, env.lib, env.rank, env.world
    W = WORKLOAD
    H = W["heads"] * W["head_dim"]
    B, S = W["batch"], W["seq"]
    M = B * S
    slots = 4
    cfg = liger.default_config(max_batch_size=B, max_seq_len=S, head_num=W["heads"], size_per_head=W["head_dim"],
                               layer_num=args.layers, graph=1, act=1, ffn_inner=W["ffn_inner"], causal=1, seed=0,
                               workspace_slots=slots, schedule_deep=1)
    comm = None
    if world > 1:
        from liger_b200.dist import Comm
        comm = Comm(rank, world, lib.liger_model_comm_bytes(C.byref(cfg), world), channels=3 * slots)
    model = C.c_void_p()
    liger.check(lib.liger_model_create(C.byref(model), C.byref(cfg), rank, world, comm.handle if comm else None))
    # with more than one GPU the batch runs as two micro-requests whose all-gathers hide under each other's GEMMs
    # Default schedule, from measurements on B200 at N = 2, 4, 8: up to 4 GPUs the whole batch with in-line all-reduces
    # is as fast as either overlapped schedule (overlap removes idle time, the GPU then meets its power cap and the
    # GEMMs slow down by as much); at 8 GPUs two micro-requests with copy-engine all-gathers are slightly ahead.
    micro = args.micro_batches if args.micro_batches > 0 else (2 if world >= 8 and args.overlap == 1 else 1)
    liger.check(lib.liger_model_set_micro_batches(model, micro))
    liger.check(lib.liger_model_set_overlap(model, args.overlap))
    sp, stream = env.sp, env.stream
    x = torch.empty((M, H), dtype=torch.float16, device="cuda")
    liger.check(lib.liger_fill_normal(C.c_void_p(x.data_ptr()), M, H, H, 0, 0, H, 0, 0x10000, 0.0, 1.0, 0, sp))
    out = torch.empty_like(x)
    hin = x.cpu().pin_memory()
    hout = torch.empty((M, H), dtype=torch.float16).pin_memory()
    sharded_out = False
    if world > 1:
        # one host buffer shared by all ranks (a file in /dev/shm mapped by every process and page-locked): every
        # rank downloads the rows it uploaded, so each PCIe link carries 1/N of the result.  Every rank goes
        # through the same collectives whatever fails locally; any failure keeps the private buffer (rank 0
        # then downloads the whole result).
        path = "/dev/shm/liger_bench_out_%s" % os.environ.get("MASTER_PORT", "0")
        created = True
        if rank == 0:
            try:
                with open(path, "wb") as f:
                    f.truncate(M * H * 2)
            except OSError:
                created = False
        shared = None
        if env.all_ok(created):
            try:
                shared = torch.from_file(path, shared=True, size=M * H, dtype=torch.float16).view(M, H)
                if int(torch.cuda.cudart().cudaHostRegister(shared.data_ptr(), M * H * 2, 0)) != 0:
                    shared = None
            except Exception:
                shared = None
            if env.all_ok(shared is not None):
                hout = shared
                sharded_out = True
                liger.check(lib.liger_model_set_output_sharding(model, 1))
        if rank == 0 and created:
            try:
                os.unlink(path)
            except OSError:
                pass

    def step_device():
        return liger.check(lib.liger_model_forward(model, C.c_void_p(x.data_ptr()), C.c_void_p(out.data_ptr()), B, S, 0, sp))

    def step_host():
        n = liger.check(lib.liger_model_forward_host(model, C.c_void_p(hin.data_ptr()), C.c_void_p(hout.data_ptr()), B, S, 2, sp))
        stream.synchronize()   # the caller reads the result on the host every step
        return n

    for _ in range(args.warmup):
        step_device()
    env.barrier()
    sampler = ClockSampler(env.local_rank)
    if rank == 0:
        sampler.start()
    ms_total, launches, p50_ms = env.timed(step_device, args.steps)
    clocks = sampler.stop() if rank == 0 else None

    # in-situ per-kernel durations: events between the kernels of the same schedule the timed region ran (with
    # N > 1: on the compute stream of the pipelined pass, and on the communication stream for the all-gathers)
    lib.liger_model_set_kernel_timing(model, 1)
    env.barrier()
    ksteps = min(args.steps, 10)
    for _ in range(ksteps):
        step_device()
    kms = (C.c_double * 9)()
    kcnt = (C.c_longlong * 9)()
    ov = (C.c_double * 4)()
    liger.check(lib.liger_model_kernel_times(model, C.byref(kms), C.byref(kcnt)))
    liger.check(lib.liger_model_overlap_times(model, C.byref(ov)))
    lib.liger_model_set_kernel_timing(model, 0)
    env.barrier()
    if os.environ.get("LIGER_BENCH_ALL_RANKS"):   # diagnostics: every rank's per-kernel averages and in-kernel all-reduce split
        t4 = (C.c_double * 4)()
        if comm is not None:
            lib.liger_comm_timing(comm.handle, 0, 0, C.byref(t4))
        print(f"rank {rank}: " + " ".join(f"k{k}={kms[k] / max(kcnt[k], 1) * 1e3:.0f}" for k in range(9)) +
              f" wait_ms={ov[0]:.3f} gather_ms={ov[2]:.3f} ar_entry_us={t4[0] / max(t4[3], 1):.0f} ar_work_us={t4[1] / max(t4[3], 1):.0f}",
              file=sys.stderr, flush=True)
    comm_split = None
    if comm is not None:
        t4 = (C.c_double * 4)()
        liger.check(lib.liger_comm_timing(comm.handle, 0, 1, C.byref(t4)))
        if t4[3] > 0:
            comm_split = {"launches": int(t4[3]), "entry_wait_us": t4[0] / t4[3], "work_us": t4[1] / t4[3],
                          "exit_wait_us": t4[2] / t4[3],
                          "note": "per all-reduce launch of workspace slot 0 on rank 0 since model construction: wait for peers "
                                  "(rank skew) / reduce + residual + LayerNorm (+ stores) / wait for peers' stores"}

    for _ in range(2):
        step_host()
    ms_e2e, _, p50_e2e = env.timed(step_host, args.steps)

    env.check_device_status()
    if not bool(torch.isfinite(out.float()).all().item()):
        raise SystemExit("result check failed: non-finite values in the output")
    if rank == 0 and not bool(torch.equal(hout, out.cpu())):
        diff = (hout.float() - out.cpu().float()).abs().max().item()
        raise SystemExit(f"result check failed: host-buffer path differs from device path (max abs diff {diff})")
    parity = {"checked": False, "why": "fixture rows are for the 4-layer stack" if args.layers != W["layers"] else "fixture missing"}
    if args.layers == W["layers"] and os.path.exists(GOLDEN_ROWS):
        g = np.load(GOLDEN_ROWS)
        rows = torch.from_numpy(g["prefill_rows"]).cuda()
        parity = check_rows(env, out[rows], g["prefill"].astype(np.float32), "prefill rows of sequence 0")

    if rank == 0:
        tokens = M * args.steps
        peaks = measured_peaks()
        peak_tf, peak_kind = gemm_peak(peaks, clocks)
        gemm_flops = gemm_ms = 0.0
        gemm_launches = 0
        per_kernel = {}
        names = {0: "qkv_gemm", 1: "attention", 2: "out_proj_gemm", 3: "allreduce_ln_1", 4: "ffn_up_gemm", 5: "ffn_down_gemm",
                 6: "allreduce_ln_2", 7: "first_layernorm", 8: "copy_out"}
        sub_b = B // micro if (world > 1 and micro > 1 and B % micro == 0 and args.overlap != 2) else B
        for k in range(9):
            if kcnt[k] == 0:
                continue
            fl, by = C.c_double(0), C.c_double(0)
            lib.liger_model_kernel_work(model, k, sub_b, S, C.byref(fl), C.byref(by))
            avg_ms = kms[k] / kcnt[k]
            per_kernel[names[k]] = {"avg_us": round(avg_ms * 1e3, 1), "launches_per_step": kcnt[k] // ksteps,
                                    "tflops": round(fl.value / avg_ms / 1e9, 1) if fl.value else None,
                                    "gbs": round(by.value / avg_ms / 1e6, 1)}
            if k in (0, 2, 4, 5):
                gemm_flops += fl.value * kcnt[k]
                gemm_ms += kms[k]
                gemm_launches += kcnt[k]
        achieved = gemm_flops / gemm_ms / 1e9 if gemm_ms else 0.0
        total_k_ms = sum(kms[k] for k in range(9))
        step_ms = ms_total / args.steps
        exposed = None
        if world > 1:
            # what the compute stream spends on communication: the local reductions (with their entry barriers), the
            # final copy of the gathered result, and any time blocked waiting for an all-gather
            comm_ms = (kms[3] + kms[6] + kms[8] + ov[0]) / ksteps
            exposed = {"ms_per_step": comm_ms, "share_of_step": comm_ms / step_ms,
                       "blocked_on_allgather_ms_per_step": ov[0] / ksteps,
                       "allgather_ms_per_step_on_comm_stream": ov[2] / ksteps, "allgathers_per_step": int(ov[3] // ksteps),
                       "note": ("kernel names allreduce_ln_* are the local halves (entry barrier + reduction + residual + LayerNorm "
                                "on the compute stream); their all-gathers run on the copy engines under the other micro-batch's "
                                "GEMMs") if args.overlap == 1 and micro > 1 else
                               ("kernel names allreduce_ln_* are the local halves (entry barrier + reduction + residual + LayerNorm); "
                                "their all-gathers run as a small copy kernel beside the next GEMM, which waits tile by tile for "
                                "its rows (that wait is inside the GEMM's time)") if args.overlap == 2 else "all-reduces run in line"}
        line = {
            "metric": "tokens/s", "value": tokens / (ms_total / 1e3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_ms, "p50_latency_ms": p50_ms,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "fp16 (fp32 accumulate)",
            "data": "synthetic",
            "config": {"workload": W["name"], "layers": args.layers, "hidden": H, "heads": W["heads"], "head_dim": W["head_dim"],
                       "ffn_inner": W["ffn_inner"], "activation": "geglu", "graph": "pre-layernorm + residual, causal",
                       "batch": B, "seq_len": S, "tokens_per_step": M, "parallelism": f"tp{world}",
                       "micro_batches": micro, "overlap_mode": args.overlap if world > 1 else None,
                       "latency": "p50_latency_ms = median duration of one step = one request of 8 x 512 tokens",
                       "l2": "inputs larger than L2: each step streams this rank's weights "
                             f"({(4 * H * H + 3 * H * W['ffn_inner']) * 2 * args.layers / world / 1e9:.1f} GB) and 100 MB activations"},
            "e2e": {"value": tokens / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps,
                    "p50_latency_ms": p50_e2e,
                    "h2d_bytes_per_step": M * H * 2, "d2h_bytes_per_step": M * H * 2,
                    "api": "liger_model_forward_host: pinned host buffers, copies on the launch stream, host sync per step; "
                           "with N > 1 each rank uploads 1/N of the input rows (gathered over NVLink) and " +
                           ("downloads the same rows of the result into one shared pinned host buffer" if sharded_out
                            else "rank 0 downloads the result")},
            "gpu_launches": launches,
            "parity": parity,
            "roofline": {"bound": "tensor", "kernel": "gemm_tcgen05_2cta_wide_kernel / gemm_tcgen05_2cta_kernel (QKV, out-proj, FFN-up, FFN-down launches)",
                         "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s", "frac": achieved / peak_tf,
                         "peak_source": peaks["source"] + ": cuBLAS bf16, " + peak_kind,
                         "frac_of_burst": achieved / peaks["burst"], "frac_of_sustained": achieved / peaks["sustained"],
                         "frac_of_nominal_2250": achieved / 2250.0,
                         "traffic": GEMM_DRAM_BYTES_PER_LAUNCH_TP1 if world == 1 else None,
                         "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum, average over the four GEMM "
                                           "launches of a layer at N=1 (profiles/gemm_tcgen05_2cta_wide_glm130b_tp1.md); "
                                           "not captured for N>1",
                         "launches_timed": gemm_launches,
                         "timing": "CUDA events between the kernels of the schedule that `value` timed (a pass of its own after the timed region)",
                         "share_of_step": gemm_ms / total_k_ms if total_k_ms else None},
            "kernels": per_kernel,
            "exposed_communication": exposed,
            "allreduce_split": comm_split,
            "clocks": clocks,
        }
        if not args.no_cpu_baseline and world == 1:
            line["cpu_baseline"] = cpu_port_tokens_per_s()
        print(json.dumps(line), flush=True)


def run_decode(args, env):
    """BASELINE config 3.  HBM-bound: per step every rank must read its weight shards and its heads of the KV cache
    once; roofline.achieved = those bytes / step time."""
    import numpy as np
    torch, liger, lib, rank, world = env.torch, env.liger, env.lib, env.rank, env.world
    W = DECODE
    H = W["heads"] * W["head_dim"]
    B, L, cap = W["batch"], W["kv_len"], W["kv_capacity"]
    if args.kv_len >= 0:   # 0: every token attends to itself only, the work the reference arm does (it has no cache)
        L = min(args.kv_len, cap - 1)
    cfg = liger.default_config(max_batch_size=B, max_seq_len=8, head_num=W["heads"], size_per_head=W["head_dim"],
                               layer_num=args.layers, graph=1, act=1, ffn_inner=W["ffn_inner"], causal=1, seed=0,
                               workspace_slots=2, schedule_deep=1, kv_capacity=cap)
    comm = None
    if world > 1:
        from liger_b200.dist import Comm
        comm = Comm(rank, world, lib.liger_model_comm_bytes(C.byref(cfg), world), channels=4)
    model = C.c_void_p()
    liger.check(lib.liger_model_create(C.byref(model), C.byref(cfg), rank, world, comm.handle if comm else None))
    liger.check(lib.liger_model_fill_kv_cache(model))
    sp, stream = env.sp, env.stream
    x = torch.empty((B, H), dtype=torch.float16, device="cuda")
    liger.check(lib.liger_fill_normal(C.c_void_p(x.data_ptr()), B, H, H, 0, 0, H, 0, 0x10000, 0.0, 1.0, 0, sp))
    out = torch.empty_like(x)
    hin = x.cpu().pin_memory()
    hout = torch.empty((B, H), dtype=torch.float16).pin_memory()

    def step_device():   # every step appends at position kv_len again: same work each time
        return liger.check(lib.liger_model_decode(model, C.c_void_p(x.data_ptr()), C.c_void_p(out.data_ptr()), B, L, 0, sp))

    def step_host():     # the token's hidden state comes from the host and the result goes back, every step
        x.copy_(hin, non_blocking=True)
        n = step_device()
        if rank == 0:
            hout.copy_(out, non_blocking=True)
        stream.synchronize()
        return n

    for _ in range(args.warmup):
        step_device()
    env.barrier()
    sampler = ClockSampler(env.local_rank)
    if rank == 0:
        sampler.start()
    ms_total, launches, p50_ms = env.timed(step_device, args.steps)
    clocks = sampler.stop() if rank == 0 else None
    # in-situ per-kernel durations (events between the kernels of the step), in a pass of its own
    lib.liger_model_set_kernel_timing(model, 1)
    env.barrier()
    ksteps = min(args.steps, 10)
    for _ in range(ksteps):
        step_device()
    kms = (C.c_double * 9)()
    kcnt = (C.c_longlong * 9)()
    liger.check(lib.liger_model_kernel_times(model, C.byref(kms), C.byref(kcnt)))
    lib.liger_model_set_kernel_timing(model, 0)
    env.barrier()
    for _ in range(2):
        step_host()
    ms_e2e, _, p50_e2e = env.timed(step_host, args.steps)
    env.check_device_status()
    parity = {"checked": False, "why": "fixture rows are for the 4-layer stack" if args.layers != W["layers"] else "fixture missing"}
    if L != W["kv_len"]:
        parity["why"] = "fixture rows are for kv_len %d" % W["kv_len"]
    elif args.layers == W["layers"] and os.path.exists(GOLDEN_ROWS):
        g = np.load(GOLDEN_ROWS)
        assert int(g["decode_kv_len"]) == L and int(g["decode_kv_capacity"]) == cap
        want = g["decode"].astype(np.float32)
        parity = check_rows(env, out[:want.shape[0]], want, "decode step, first sequences")
    if rank == 0:
        peaks = measured_peaks()
        F = W["ffn_inner"]
        weight_bytes = (4 * H * H + 3 * H * F) * 2 / world
        kv_bytes = 2 * B * (W["heads"] / world) * (L + 1) * W["head_dim"] * 2
        step_bytes = args.layers * (weight_bytes + kv_bytes)
        decode_traffic = args.layers * (weight_bytes * GEMM_SMALLM_TRAFFIC_RATIO + kv_bytes * ATTENTION_DECODE_TRAFFIC_RATIO)
        step_ms = ms_total / args.steps
        achieved = step_bytes / (step_ms * 1e-3) / 1e9
        Hl, Fl = H / world, F / world
        kbytes = {0: 2 * H * 3 * Hl, 1: kv_bytes, 2: 2 * Hl * H, 4: 2 * H * 2 * Fl, 5: 2 * Fl * H}   # bytes each kernel must stream
        names = {0: "qkv_gemm", 1: "attention", 2: "out_proj_gemm", 3: "allreduce_ln_1", 4: "ffn_up_gemm", 5: "ffn_down_gemm",
                 6: "allreduce_ln_2", 7: "first_layernorm", 8: "copy_out"}
        per_kernel = {}
        for k in range(9):
            if kcnt[k]:
                avg_ms = kms[k] / kcnt[k]
                per_kernel[names[k]] = {"avg_us": round(avg_ms * 1e3, 1), "launches_per_step": kcnt[k] // ksteps,
                                        "gbs": round(kbytes[k] / avg_ms / 1e6, 1) if k in kbytes else None}
        line = {
            "metric": "tokens/s", "value": B * args.steps / (ms_total / 1e3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_ms, "p50_latency_ms": p50_ms,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "fp16 (fp32 accumulate)", "data": "synthetic",
            "config": {"workload": W["name"].replace("kv%d" % W["kv_len"], "kv%d" % L), "layers": args.layers, "hidden": H,
                       "heads": W["heads"], "head_dim": W["head_dim"],
                       "ffn_inner": F, "activation": "geglu", "batch": B, "kv_len": L, "kv_capacity": cap, "tokens_per_step": B,
                       "parallelism": f"tp{world}",
                       "l2": f"inputs larger than L2: each step streams {step_bytes / 1e9:.2f} GB of weights and KV cache per rank"},
            "e2e": {"value": B * args.steps / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps,
                    "p50_latency_ms": p50_e2e, "h2d_bytes_per_step": B * H * 2, "d2h_bytes_per_step": B * H * 2,
                    "api": "liger_model_decode between a pinned-host upload of the token states and a download of the result"},
            "gpu_launches": launches,
            "parity": parity,
            "kernels": per_kernel,
            "roofline": {"bound": "hbm", "kernel": "whole decode step (weight-streaming GEMMs + split-KV attention)",
                         "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                         "peak_source": peaks["source"] + ": STREAM-style copy",
                         "traffic": decode_traffic if world == 1 and L == W["kv_len"] else None,
                         "traffic_source": "ncu dram read+write of the two kernels on smaller cases, scaled by bytes streamed: "
                                           "few-row GEMM x %.4f (32 x 12288 x 12288), decode attention x %.4f (8 of 32 sequences); "
                                           "see profiles/" % (GEMM_SMALLM_TRAFFIC_RATIO, ATTENTION_DECODE_TRAFFIC_RATIO),
                         "bytes_per_step_per_rank": step_bytes},
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)


def run_allreduce_sweep(args, env):
    """BASELINE config 5: out = sum over ranks of the partials + residual + bias, on every rank, from 8 KB to 512 MB.
    One-shot up to 1 MiB, two-shot (pull, reduce, push) above.  Bus GB/s = 2 (N-1)/N * bytes / time."""
    torch, liger, lib, rank, world = env.torch, env.liger, env.lib, env.rank, env.world
    if world < 2:
        raise SystemExit("--workload allreduce_sweep needs at least 2 GPUs")
    from liger_b200.dist import Comm
    max_bytes = args.sweep_max_mb << 20
    comm = Comm(rank, world, 2 * max_bytes + 512, channels=2)
    sizes = []
    b = 8 << 10
    while b <= max_bytes:
        sizes.append(b)
        b *= 2
    sp = env.sp
    records = []
    hidden = torch.empty(max_bytes // 2, dtype=torch.float16, device="cuda")
    for nbytes in sizes:
        n = 8192 if nbytes >= (1 << 20) else 1024
        m = nbytes // (2 * n)
        part = comm.tensor(0, (m, n))
        liger.check(lib.liger_fill_normal(C.c_void_p(part.data_ptr()), m, n, n, 0, 0, n, 0, 600 + rank, 0.0, 1.0, 0, sp))
        liger.check(lib.liger_fill_normal(C.c_void_p(hidden.data_ptr()), m, n, n, 0, 0, n, 0, 610, 0.0, 1.0, 0, sp))
        bias = torch.zeros(n, dtype=torch.float16, device="cuda")
        one_shot = 1 if nbytes <= (1 << 20) else 0
        iters = max(3, min(args.steps * 4, int(2e9 // nbytes))) if nbytes > (64 << 20) else args.steps * 4

        def call():
            return liger.check(lib.liger_allreduce_fused(comm.handle, 0, 0, max_bytes, None, C.c_void_p(hidden.data_ptr()),
                                                         C.c_void_p(bias.data_ptr()), None, None, m, n, 0, m, one_shot, sp))
        for _ in range(3):
            call()
        t4 = (C.c_double * 4)()
        liger.check(lib.liger_comm_timing(comm.handle, 0, 1, C.byref(t4)))   # reset the in-kernel stamps
        ms, _, _ = env.timed(call, iters)
        us = ms * 1e3 / iters
        liger.check(lib.liger_comm_timing(comm.handle, 0, 1, C.byref(t4)))
        k = max(t4[3], 1.0)
        records.append({"bytes": nbytes, "rows": m, "cols": n, "mode": "one-shot" if one_shot else "two-shot", "us": us,
                        "bus_gbs": 2.0 * (world - 1) / world * nbytes / (us * 1e-6) / 1e9, "iters": iters,
                        "in_kernel_us": {"entry_wait": t4[0] / k, "work": t4[1] / k, "exit_wait": t4[2] / k}})
    env.check_device_status()
    if rank == 0:
        best = max(r["bus_gbs"] for r in records)
        line = {"metric": "allreduce+residual bus GB/s", "value": best, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
                "warmup": 3, "ms_per_step": None, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "fp16 (fp32 sum)",
                "data": "synthetic",
                "config": {"workload": "allreduce_residual_sweep_8KB_512MB", "parallelism": f"tp{world}",
                           "collective": "liger_allreduce_fused: sum + residual + bias in one kernel over peer memory"},
                "roofline": {"bound": "nvlink", "achieved": best, "peak": 900.0, "unit": "GB/s", "frac": best / 900.0,
                             "peak_source": "nominal NVLink 5 per direction per GPU (measured peer copy on this pool: 770)"},
                "records": records, "gpu_launches": 2 * sum(r["iters"] for r in records)}
        print(json.dumps(line), flush=True)
    comm.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="liger", choices=["liger", "reference"])
    ap.add_argument("--workload", default="prefill", choices=["prefill", "decode", "allreduce_sweep"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--layers", type=int, default=WORKLOAD["layers"], help=argparse.SUPPRESS)
    ap.add_argument("--micro-batches", type=int, default=0,
                    help="micro-requests the batch is split into (0 = default: 2 with more than one GPU)")
    ap.add_argument("--overlap", type=int, default=1, choices=[0, 1, 2],
                    help="1: micro-requests on one compute stream + copy-engine all-gathers (default); 0: one stream per "
                         "micro-request; 2: whole batch, all-gather beside the GEMM that consumes it")
    ap.add_argument("--sweep-max-mb", type=int, default=512, help=argparse.SUPPRESS)
    ap.add_argument("--kv-len", type=int, default=-1,
                    help="decode: cached positions per sequence (default: the configuration's 2048); 0 = the reference arm's work")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return
    if world != args.gpus:
        if args.gpus != 1 or world != 1:
            raise SystemExit(f"--gpus {args.gpus} needs {args.gpus} ranks (torch.distributed.run); found WORLD_SIZE={world}")
    args.warmup = max(args.warmup, 3)
    env = Env(args)
    if args.workload == "prefill":
        run_prefill(args, env)
    elif args.workload == "decode":
        run_decode(args, env)
    else:
        run_allreduce_sweep(args, env)
    env.finish()


if __name__ == "__main__":
    main()
