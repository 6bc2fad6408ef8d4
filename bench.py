#!/usr/bin/env python
"""Headline benchmark: tokens/s of the GLM-130B-shape tensor-parallel prefill stack.

    python bench.py --gpus N --steps K --warmup W            (N = 1)
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...                      (the CPU baseline arm)

Workload (fixed for every N, so scaling is strong): 4 decoder layers, hidden 12288, 96 heads x 128,
GeGLU FFN with inner size 32768, pre-LayerNorm with residual adds, causal attention, fp16 weights
~N(0, 0.02) and fp16 activations ~N(0, 1) from seed 0, batch 8 x sequence 512 (4096 tokens per
step), tensor parallel over the N GPUs.  A step is one forward pass of the stack.  Everything is
synthetic: seeded random weights of that architecture and seeded random hidden states.

One JSON line is printed by rank 0:
  value        tokens/s with the input already in HBM (CUDA events around the K timed steps, max over ranks)
  e2e          tokens/s through liger_model_forward_host: pinned host input -> device, the pass, result -> host
  roofline     the tcgen05 GEMM kernel (QKV, out-proj, FFN-up, FFN-down launches), FLOPs / in-situ duration
               against the measured cuBLAS bf16 peak of this pool (MEASURED_PEAKS.json)
  cpu_baseline the fp32 host port of the same stack on the box's cores (N = 1 only)
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

WORKLOAD = dict(name="glm130b_shape_prefill_4layer_b8_s512", layers=4, heads=96, head_dim=128, ffn_inner=32768,
                batch=8, seq=512)


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
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(tflops=float(p.get("bf16_tflops_sustained", p.get("bf16_tflops", 1400.0))), hbm_gbs=float(p["hbm_gbs"]),
                    source="measured (MEASURED_PEAKS.json, sustained cuBLAS bf16)")
    return dict(tflops=1400.0, hbm_gbs=6650.0, source="fallback (1.4 PFLOP/s sustained, 6.65 TB/s)")


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


def run_reference_gpu_build(args, rank, world):
    """The reference's own NCCL + cuBLAS build (unmodified sources + oracle/ref_harness/harness.cu, compiled
    for sm_100a into oracle/_ref/), one process per GPU over the MPI stand-in.  The reference can only
    express its own layer (post-LayerNorm, no residual, GELU with a 4H FFN, full attention through a mask
    tensor); at hidden 12288 that layer has the same GEMM FLOPs as the GeGLU-32768 layer of this
    benchmark, so tokens/s are comparable.  Returns the harness's JSON record (rank 0) or None."""
    env = dict(os.environ)
    env["LIGER_MPI_RANK"], env["LIGER_MPI_SIZE"] = str(rank), str(world)
    env["LIGER_MPI_JOB"] = "bench_ref_%s" % os.environ.get("MASTER_PORT", "0")
    env.setdefault("LIGER_MPI_TIMEOUT_S", "120")
    W = WORKLOAD
    cmd = [REF_HARNESS, str(W["batch"]), str(W["seq"]), str(W["heads"]), str(W["head_dim"]), str(args.layers),
           str(args.steps), str(max(args.warmup, 3))]
    try:
        res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    except (OSError, subprocess.TimeoutExpired) as e:
        return {"error": f"{type(e).__name__}: {e}"} if rank == 0 else None
    if rank != 0:
        return None
    for ln in res.stdout.splitlines():
        if ln.startswith("{\"ref_harness\""):
            rec = json.loads(ln)
            if res.returncode == 0 and rec.get("cuda_error") == "no error":
                return rec
            return {"error": f"exit {res.returncode}, cuda_error {rec.get('cuda_error')}"}
    return {"error": f"exit {res.returncode}: {(res.stderr or res.stdout)[-300:]}"}


def run_reference_arm(args, rank, world):
    """Reference arm.  Preferred: the reference's own GPU build (see run_reference_gpu_build).  The
    reference has no CPU implementation of this path; when its GPU build is not available (not built,
    or it fails on this box) the arm times the CPU port of its arithmetic (the oracle) instead."""
    tokens = WORKLOAD["batch"] * WORKLOAD["seq"]
    H = WORKLOAD["heads"] * WORKLOAD["head_dim"]
    rec = run_reference_gpu_build(args, rank, world) if os.path.exists(REF_HARNESS) else (
        {"error": "oracle/_ref/liger_ref_harness has not been built"} if rank == 0 else None)
    if rank != 0:
        return
    base = {"impl": "reference", "metric": "tokens/s", "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "data": "synthetic"}
    if rec and "error" not in rec:
        line = dict(base, value=rec["tokens_per_s"], ms_per_step=rec["ms_per_step"], dtype="fp16 (fp16 accumulate, CUBLAS_COMPUTE_16F)",
                    config={"workload": WORKLOAD["name"], "tokens_per_step": tokens, "parallelism": f"tp{world}",
                            "graph": "the reference's own layer: post-LayerNorm, no residual, GELU FFN 4H (same GEMM FLOPs as "
                                     "the GeGLU-32768 layer), full attention with an all-ones mask",
                            "build": "unmodified reference sources + oracle/ref_harness/harness.cu, nvcc sm_100a, cuBLAS + NCCL, "
                                     "MPI stand-in; kernel vector replayed in order on one stream (Scheduler::run_sequential)"},
                    cpu_baseline={"value": rec["tokens_per_s"], "unit": "tokens/s", "cores": 0, "kind": "reference",
                                  "sample": "the reference's GPU build (it has no CPU path): full workload, all steps"},
                    e2e={"value": rec["tokens_per_s_e2e"], "unit": "tokens/s", "ms_per_step": rec["ms_per_step_e2e"],
                         "h2d_bytes_per_step": tokens * H * 2 * world, "d2h_bytes_per_step": tokens * H * 2 * world},
                    gpu_launches=rec["kernels_per_step"] * args.steps)
    else:
        cpu = cpu_port_tokens_per_s()
        line = dict(base, value=cpu["value"], ms_per_step=1000.0 * tokens / cpu["value"], dtype="f32",
                    config={"workload": WORKLOAD["name"], "tokens_per_step": tokens,
                            "note": "reference GPU build unavailable: " + (rec or {}).get("error", "unknown")},
                    cpu_baseline=cpu,
                    e2e={"value": cpu["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                    gpu_launches=0)
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="liger", choices=["liger", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--layers", type=int, default=WORKLOAD["layers"], help=argparse.SUPPRESS)
    ap.add_argument("--micro-batches", type=int, default=0,
                    help="batch halves interleaved on two streams (0 = default: 2 with more than one GPU)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", str(rank)))
    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return
    if world != args.gpus:
        if args.gpus != 1 or world != 1:
            raise SystemExit(f"--gpus {args.gpus} needs {args.gpus} ranks (torch.distributed.run); found WORLD_SIZE={world}")
    args.warmup = max(args.warmup, 3)

    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    torch.cuda.set_device(local_rank)
    liger = load_package()
    lib = liger.lib()   # raises if the CUDA library is missing
    import torch.distributed as dist
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ["NCCL_DEBUG"] = "WARN"   # keep NCCL's version banner off stdout: one JSON line only
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local_rank))

    W = WORKLOAD
    H = W["heads"] * W["head_dim"]
    B, S = W["batch"], W["seq"]
    M = B * S
    cfg = liger.default_config(max_batch_size=B, max_seq_len=S, head_num=W["heads"], size_per_head=W["head_dim"],
                               layer_num=args.layers, graph=1, act=1, ffn_inner=W["ffn_inner"], causal=1, seed=0,
                               workspace_slots=4, schedule_deep=1)
    comm = None
    if world > 1:
        from liger_b200.dist import Comm
        comm = Comm(rank, world, lib.liger_model_comm_bytes(C.byref(cfg), world), channels=4)
    model = C.c_void_p()
    liger.check(lib.liger_model_create(C.byref(model), C.byref(cfg), rank, world, comm.handle if comm else None))
    # halves of the batch interleaved on two streams (hides the all-reduces)
    micro = args.micro_batches if args.micro_batches > 0 else (2 if world > 1 else 1)
    liger.check(lib.liger_model_set_micro_batches(model, micro))

    stream = torch.cuda.current_stream()
    sp = C.c_void_p(stream.cuda_stream)
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
        def all_ok(flag):
            t = torch.tensor([1 if flag else 0], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MIN)
            return int(t.item()) == 1
        path = "/dev/shm/liger_bench_out_%s" % os.environ.get("MASTER_PORT", "0")
        created = True
        if rank == 0:
            try:
                with open(path, "wb") as f:
                    f.truncate(M * H * 2)
            except OSError:
                created = False
        shared = None
        if all_ok(created):
            try:
                shared = torch.from_file(path, shared=True, size=M * H, dtype=torch.float16).view(M, H)
                if int(torch.cuda.cudart().cudaHostRegister(shared.data_ptr(), M * H * 2, 0)) != 0:
                    shared = None
            except Exception:
                shared = None
            if all_ok(shared is not None):
                hout = shared
                sharded_out = True
                liger.check(lib.liger_model_set_output_sharding(model, 1))
        if rank == 0 and created:
            try:
                os.unlink(path)
            except OSError:
                pass

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step_device():
        return liger.check(lib.liger_model_forward(model, C.c_void_p(x.data_ptr()), C.c_void_p(out.data_ptr()), B, S, 0, sp))

    def step_host():
        n = liger.check(lib.liger_model_forward_host(model, C.c_void_p(hin.data_ptr()), C.c_void_p(hout.data_ptr()), B, S, 2, sp))
        stream.synchronize()   # the caller reads the result on the host every step
        return n

    def timed(fn, steps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record(stream)
        launches = 0
        for _ in range(steps):
            launches += fn()
        e1.record(stream)
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item()), launches

    for _ in range(args.warmup):
        step_device()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms_total, launches = timed(step_device, args.steps)
    clocks = sampler.stop() if rank == 0 else None

    # in-situ per-kernel durations (events between the kernels of the same pass), separate timed region
    lib.liger_model_set_kernel_timing(model, 1)
    barrier()
    ksteps = min(args.steps, 10)
    for _ in range(ksteps):
        step_device()
    kms = (C.c_double * 9)()
    kcnt = (C.c_longlong * 9)()
    liger.check(lib.liger_model_kernel_times(model, C.byref(kms), C.byref(kcnt)))
    lib.liger_model_set_kernel_timing(model, 0)
    barrier()
    comm_split = None
    if comm is not None:
        t4 = (C.c_double * 4)()
        liger.check(lib.liger_comm_timing(comm.handle, 0, 1, C.byref(t4)))
        if t4[3] > 0:
            comm_split = {"launches": int(t4[3]), "entry_wait_us": t4[0] / t4[3], "work_us": t4[1] / t4[3],
                          "exit_wait_us": t4[2] / t4[3],
                          "note": "per fused all-reduce launch on rank 0 since model construction: wait for peers (rank skew) "
                                  "/ reduce + residual + LayerNorm + stores / wait for peers' stores"}

    for _ in range(2):
        step_host()
    ms_e2e, _ = timed(step_host, args.steps)

    st = (C.c_uint * 4)()
    if lib.liger_device_status(C.byref(st)) != 0:
        raise SystemExit(f"device status word set: {list(st)}")
    if not bool(torch.isfinite(out.float()).all().item()):
        raise SystemExit("result check failed: non-finite values in the output")
    if rank == 0 and not bool(torch.equal(hout, out.cpu())):
        diff = (hout.float() - out.cpu().float()).abs().max().item()
        raise SystemExit(f"result check failed: host-buffer path differs from device path (max abs diff {diff})")

    if rank == 0:
        tokens = M * args.steps
        peaks = measured_peaks()
        gemm_flops = gemm_ms = 0.0
        gemm_launches = 0
        per_kernel = {}
        names = {0: "qkv_gemm", 1: "attention", 2: "out_proj_gemm", 3: "allreduce_ln_1", 4: "ffn_up_gemm", 5: "ffn_down_gemm",
                 6: "allreduce_ln_2", 7: "first_layernorm", 8: "copy_out"}
        for k in range(9):
            if kcnt[k] == 0:
                continue
            fl, by = C.c_double(0), C.c_double(0)
            lib.liger_model_kernel_work(model, k, B, S, C.byref(fl), C.byref(by))
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
        line = {
            "metric": "tokens/s", "value": tokens / (ms_total / 1e3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_total / args.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "fp16 (fp32 accumulate)",
            "data": "synthetic",
            "config": {"workload": W["name"], "layers": args.layers, "hidden": H, "heads": W["heads"], "head_dim": W["head_dim"],
                       "ffn_inner": W["ffn_inner"], "activation": "geglu", "graph": "pre-layernorm + residual, causal",
                       "batch": B, "seq_len": S, "tokens_per_step": M, "parallelism": f"tp{world}",
                       "micro_batches": micro,
                       "l2": "inputs larger than L2: each step streams this rank's weights "
                             f"({(4 * H * H + 3 * H * W['ffn_inner']) * 2 * args.layers / world / 1e9:.1f} GB) and 100 MB activations"},
            "e2e": {"value": tokens / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": M * H * 2, "d2h_bytes_per_step": M * H * 2,
                    "api": "liger_model_forward_host: pinned host buffers, copies on the launch stream, host sync per step; "
                           "with N > 1 each rank uploads 1/N of the input rows (gathered over NVLink) and " +
                           ("downloads the same rows of the result into one shared pinned host buffer" if sharded_out
                            else "rank 0 downloads the result")},
            "gpu_launches": launches,
            "roofline": {"bound": "tensor", "kernel": "gemm_tcgen05_2cta_wide_kernel / gemm_tcgen05_2cta_kernel (QKV, out-proj, FFN-up, FFN-down launches)",
                         "achieved": achieved, "peak": peaks["tflops"], "unit": "TFLOP/s", "frac": achieved / peaks["tflops"],
                         "peak_source": peaks["source"], "frac_of_nominal_2250": achieved / 2250.0,
                         "traffic": GEMM_DRAM_BYTES_PER_LAUNCH_TP1 if world == 1 else None,
                         "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum, average over the four GEMM "
                                           "launches of a layer at N=1 (profiles/gemm_tcgen05_2cta_wide_glm130b_tp1.md); "
                                           "not captured for N>1",
                         "launches_timed": gemm_launches,
                         "share_of_step": gemm_ms / total_k_ms if total_k_ms else None},
            "kernels": per_kernel,
            "allreduce_split": comm_split,
            "clocks": clocks,
        }
        if not args.no_cpu_baseline and world == 1:
            line["cpu_baseline"] = cpu_port_tokens_per_s()
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
