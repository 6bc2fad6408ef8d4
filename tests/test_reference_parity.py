"""Parity against the reference ITSELF: the unmodified reference sources, compiled for sm_100a into
oracle/_ref/liger_ref_harness (oracle/ref_harness/), are run on the GPU on seeded inputs and their output
is compared (i) with the CPU oracle and (ii) with this library called through its C ABI.

Two granularities:
  * per operator -- the reference's own kernels (LayerNorm, bias+GELU, bias+head split, masked softmax,
    head merge, residual+bias(+LayerNorm)) and its cuBLAS-backed Linear_Col / Linear_Row, one at a time;
  * the whole function-assembled layer stack (Bert_Model::forward replayed in order, i.e.
    Scheduler::run_sequential) on shapes the reference's kernels accept (even S, B*S % 4 == 0), at TP = 1
    and, with two GPUs, at TP = 2 over NCCL.

What differs by construction and therefore bounds the tolerance: the reference accumulates its GEMMs in
fp16 (CUBLAS_COMPUTE_16F, src/layer/linear.h:47-53) and scales / masks / exponentiates the softmax in fp16
(src/cuda/attention_kernels.cu:543-573); the oracle is fp32 throughout and this library accumulates in
fp32 and rounds to fp16 only where a tensor is stored.  Data movement is compared bit for bit.  Every
measured error is collected and, when LIGER_PARITY_REPORT names a file, written there as JSON.
"""
import ctypes as C
import json
import os
import subprocess
import uuid

import numpy as np
import pytest

from helpers import assert_close, dev_fill, max_rel_err, ptr, stream_ptr, to_np

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HARNESS = os.path.join(ROOT, "oracle", "_ref", "liger_ref_harness")
REPORT = {}


def _need_harness():
    if not os.path.exists(HARNESS):
        pytest.skip("oracle/_ref/liger_ref_harness is not built (make -C oracle/ref_harness needs the reference sources)")


def _run_harness(argv, world=1, timeout=600):
    """One process per rank over the shared-memory MPI stand-in; returns rank 0's JSON record."""
    job = "refparity_" + uuid.uuid4().hex[:10]
    procs = []
    for r in range(world):
        env = dict(os.environ, LIGER_MPI_RANK=str(r), LIGER_MPI_SIZE=str(world), LIGER_MPI_JOB=job, LIGER_MPI_TIMEOUT_S="120",
                   NCCL_NVLS_ENABLE="0")
        procs.append(subprocess.Popen([HARNESS] + [str(a) for a in argv], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.PIPE, text=True))
    outs = [p.communicate(timeout=timeout) for p in procs]
    for r, p in enumerate(procs):
        assert p.returncode == 0, f"reference harness rank {r} exited {p.returncode}: {outs[r][1][-400:]}"
    for ln in outs[0][0].splitlines():
        if ln.startswith("{\"ref_"):
            rec = json.loads(ln)
            assert rec["cuda_error"] == "no error", rec
            return rec
    raise AssertionError("reference harness printed no record: " + outs[0][0][-400:])


def _note(name, **vals):
    REPORT[name] = {k: float(v) for k, v in vals.items()}
    path = os.environ.get("LIGER_PARITY_REPORT")
    if path:
        with open(path, "w") as f:
            json.dump(REPORT, f, indent=1, sort_keys=True)


@pytest.fixture(scope="module")
def ref_ops(gpu, tmp_path_factory):
    """Every per-operator vector of the reference, as float32 arrays of fp16-representable values."""
    _need_harness()
    d = tmp_path_factory.mktemp("ref_ops")
    rec = _run_harness(["ops", str(d)])
    out = {}
    for name, shape in rec["tensors"].items():
        out[name] = np.fromfile(os.path.join(str(d), name + ".f16"), dtype=np.float16).reshape(shape).astype(np.float32)
    return out


def _host(oracle, rows, cols, tid, mean=0.0, std=1.0):
    """The seeded tensor as the reference harness generated it (fp16 values, as float32)."""
    return oracle.fill_normal_f16(rows * cols, 0, tid, mean=mean, std=std).astype(np.float32).reshape(rows, cols)


def _mask(B, S):
    q = np.arange(S)[:, None]
    k = np.arange(S)[None, :]
    m = np.empty((B, S, S), np.float32)
    m[0] = (k <= q)
    m[1:] = (k < S - S // 4)
    return m


# ---- per operator -----------------------------------------------------------------------------------------
@pytest.mark.parametrize("name,m,n,tid", [("layernorm_1024", 24, 1024, 0x20000), ("layernorm_12288", 8, 12288, 0x20008)])
def test_layernorm_matches_reference_kernel(gpu, liger, oracle, ref_ops, name, m, n, tid):
    import torch
    x, g, b = _host(oracle, m, n, tid, 0.3, 1.5), _host(oracle, 1, n, tid + 1, 1.0, 0.02)[0], _host(oracle, 1, n, tid + 2, 0.0, 0.02)[0]
    ref = ref_ops[name]
    want = oracle.layernorm(x, g, b)
    dx, dg, db = dev_fill(liger, m, n, 0, tid, mean=0.3, std=1.5), dev_fill(liger, 1, n, 0, tid + 1, mean=1.0, std=0.02), \
        dev_fill(liger, 1, n, 0, tid + 2, std=0.02)
    y = torch.empty_like(dx)
    liger.check(gpu.liger_layernorm(ptr(dx), ptr(dg), ptr(db), ptr(y), m, n, stream_ptr()))
    _note(name, ref_vs_oracle=max_rel_err(ref, want), ref_vs_library=max_rel_err(ref, to_np(y)))
    assert_close(ref, want, rel=1e-2, what=f"reference {name} vs oracle")
    assert_close(to_np(y), ref, rel=1e-2, what=f"library {name} vs reference")


def test_bias_gelu_matches_reference_kernel(gpu, liger, oracle, ref_ops):
    m, n = 40, 4096
    x, b = _host(oracle, m, n, 0x20010, 0.0, 1.5), _host(oracle, 1, n, 0x20011, 0.0, 0.5)[0]
    ref = ref_ops["bias_gelu"]
    want = oracle.add_bias_gelu(x, b)
    dx, db = dev_fill(liger, m, n, 0, 0x20010, std=1.5), dev_fill(liger, 1, n, 0, 0x20011, std=0.5)
    liger.check(gpu.liger_add_bias_gelu(ptr(dx), ptr(db), m, n, stream_ptr()))
    _note("bias_gelu", ref_vs_oracle=max_rel_err(ref, want), ref_vs_library=max_rel_err(ref, to_np(dx)))
    assert_close(ref, want, rel=1e-2, what="reference bias+gelu vs oracle")
    assert_close(to_np(dx), ref, rel=1e-2, what="library bias+gelu vs reference")


@pytest.mark.parametrize("tag,B,S,h,D,tid", [("qkv_split_256", 2, 64, 4, 64, 0x20020), ("qkv_split_2048", 2, 64, 16, 128, 0x20028)])
def test_bias_head_split_matches_reference_kernel(gpu, liger, oracle, ref_ops, tag, B, S, h, D, tid):
    import torch
    m, k = B * S, h * D
    src = [_host(oracle, m, k, tid + i) for i in range(3)]
    bias = [_host(oracle, 1, k, tid + 3 + i, 0.0, 0.5)[0] for i in range(3)]
    dsrc = [dev_fill(liger, m, k, 0, tid + i) for i in range(3)]
    dbias = [dev_fill(liger, 1, k, 0, tid + 3 + i, std=0.5) for i in range(3)]
    outs = [torch.empty((B, h, S, D), dtype=torch.float16, device="cuda") for _ in range(3)]
    liger.check(gpu.liger_add_qkv_bias_transpose(ptr(outs[0]), ptr(outs[1]), ptr(outs[2]), ptr(dsrc[0]), ptr(dbias[0]),
                                                 ptr(dsrc[1]), ptr(dbias[1]), ptr(dsrc[2]), ptr(dbias[2]), B, S, h, D, stream_ptr()))
    worst = 0.0
    for i, which in enumerate("qkv"):
        ref = ref_ops[f"{tag}_{which}"]
        want = oracle.round_fp16(oracle.add_bias_split_heads(src[i], bias[i], B, S, h, D))
        # one fp16 add per element on both sides: the reference kernel, the oracle and the library agree exactly
        assert np.array_equal(ref, want), f"reference {tag}_{which} differs from the oracle"
        assert np.array_equal(to_np(outs[i]), ref), f"library {tag}_{which} differs from the reference"
        worst = max(worst, max_rel_err(ref, want))
    _note(tag, ref_vs_oracle=worst, ref_vs_library=0.0)


@pytest.mark.parametrize("name,B,h,S,tid", [("softmax_64", 2, 4, 64, 0x20030), ("softmax_200", 2, 2, 200, 0x20031)])
def test_masked_softmax_matches_reference_kernel(oracle, ref_ops, name, B, h, S, tid):
    """The reference's half path computes scale*s + (1-mask)*-10000 and the exponent argument in fp16; the
    probabilities of a row still sum to one and agree with the fp32 oracle to fp16 accuracy."""
    s = _host(oracle, B * h * S, S, tid, 0.0, 8.0).reshape(B, h, S, S)
    ref = ref_ops[name]
    want = oracle.masked_softmax(s, _mask(B, S), 0.125)
    _note(name, ref_vs_oracle=max_rel_err(ref, want))
    assert_close(ref, want, rel=1e-2, what=f"reference {name} vs oracle")
    assert np.all(ref[0][:, np.triu_indices(S, 1)[0], np.triu_indices(S, 1)[1]] == 0.0)   # masked entries are exactly zero


def test_head_merge_matches_reference_kernel(gpu, liger, oracle, ref_ops):
    import torch
    B, h, S, D = 2, 4, 64, 64
    src = _host(oracle, B * h * S, D, 0x20040).reshape(B, h, S, D)
    ref = ref_ops["merge_heads"]
    assert np.array_equal(ref, oracle.merge_heads(src))
    dsrc = dev_fill(liger, B * h * S, D, 0, 0x20040)
    dst = torch.empty((B * S, h * D), dtype=torch.float16, device="cuda")
    liger.check(gpu.liger_transpose_heads(ptr(dst), ptr(dsrc), B, S, h, D, stream_ptr()))
    assert np.array_equal(to_np(dst), ref)
    _note("merge_heads", ref_vs_oracle=0.0, ref_vs_library=0.0)


def test_residual_layernorm_matches_reference_kernel(gpu, liger, oracle, ref_ops):
    import torch
    m, n = 24, 1024
    inp, g, b = _host(oracle, m, n, 0x20050), _host(oracle, 1, n, 0x20051, 1.0, 0.02)[0], _host(oracle, 1, n, 0x20052, 0.0, 0.02)[0]
    bias, out = _host(oracle, 1, n, 0x20053, 0.0, 0.5)[0], _host(oracle, m, n, 0x20054)
    want_h, want_n = oracle.add_bias_input_layernorm_2(inp, g, b, bias, out)
    d_in, d_g, d_b = dev_fill(liger, m, n, 0, 0x20050), dev_fill(liger, 1, n, 0, 0x20051, mean=1.0, std=0.02), \
        dev_fill(liger, 1, n, 0, 0x20052, std=0.02)
    d_bias, d_out = dev_fill(liger, 1, n, 0, 0x20053, std=0.5), dev_fill(liger, m, n, 0, 0x20054)
    d_norm = torch.empty_like(d_out)
    liger.check(gpu.liger_add_bias_input_layernorm(ptr(d_in), ptr(d_g), ptr(d_b), ptr(d_bias), ptr(d_out), ptr(d_norm), m, n,
                                                   stream_ptr()))
    _note("residual_ln", hidden_ref_vs_oracle=max_rel_err(ref_ops["residual_ln_hidden"], want_h),
          norm_ref_vs_oracle=max_rel_err(ref_ops["residual_ln_norm"], want_n),
          hidden_ref_vs_library=max_rel_err(ref_ops["residual_ln_hidden"], to_np(d_out)),
          norm_ref_vs_library=max_rel_err(ref_ops["residual_ln_norm"], to_np(d_norm)))
    assert_close(ref_ops["residual_ln_hidden"], want_h, rel=1e-2, what="reference residual stream vs oracle")
    assert_close(ref_ops["residual_ln_norm"], want_n, rel=1e-2, what="reference residual LayerNorm vs oracle")
    assert_close(to_np(d_out), ref_ops["residual_ln_hidden"], rel=1e-2, what="library residual stream vs reference")
    assert_close(to_np(d_norm), ref_ops["residual_ln_norm"], rel=1e-2, what="library residual LayerNorm vs reference")
    # residual + bias without LayerNorm (add_bias_input)
    o2, i2, b2 = _host(oracle, m, n, 0x20060), _host(oracle, m, n, 0x20061), _host(oracle, 1, n, 0x20062, 0.0, 0.5)[0]
    want2, _ = oracle.add_bias_input_layernorm_2(i2, None, None, b2, o2, want_norm=False)
    d_o2, d_i2, d_b2 = dev_fill(liger, m, n, 0, 0x20060), dev_fill(liger, m, n, 0, 0x20061), dev_fill(liger, 1, n, 0, 0x20062, std=0.5)
    liger.check(gpu.liger_add_bias_input_layernorm(ptr(d_i2), None, None, ptr(d_b2), ptr(d_o2), None, m, n, stream_ptr()))
    _note("residual_add", ref_vs_oracle=max_rel_err(ref_ops["residual_add"], want2),
          ref_vs_library=max_rel_err(ref_ops["residual_add"], to_np(d_o2)))
    assert_close(ref_ops["residual_add"], want2, rel=1e-2, what="reference residual add vs oracle")
    assert_close(to_np(d_o2), ref_ops["residual_add"], rel=1e-2, what="library residual add vs reference")


@pytest.mark.parametrize("name,m,k,n,tid", [("linear_col", 96, 1024, 512, 0x20070), ("linear_row", 64, 4096, 1024, 0x20072)])
def test_linear_matches_reference_cublas_call(gpu, liger, oracle, ref_ops, name, m, k, n, tid):
    """Linear_Col / Linear_Row as the reference binds cublasGemmEx (fp16 accumulation) against the fp32
    oracle and this library's tcgen05 GEMM (fp32 accumulation in TMEM)."""
    from test_gpu_kernels import gemm
    x, w = _host(oracle, m, k, tid), _host(oracle, k, n, tid + 1, 0.0, 0.02)
    ref = ref_ops[name]
    want = oracle.linear(x, w)
    dx = dev_fill(liger, m, k, 0, tid)
    dwt = dev_fill(liger, k, n, 0, tid + 1, std=0.02, mode=1)
    got = to_np(gemm(liger, dx, dwt))
    _note(name, ref_vs_oracle=max_rel_err(ref, want), ref_vs_library=max_rel_err(ref, got), library_vs_oracle=max_rel_err(got, want))
    assert_close(ref, want, rel=1e-2, what=f"reference {name} vs oracle")
    assert_close(got, ref, rel=1e-2, what=f"library {name} vs reference")


# ---- the whole layer stack ---------------------------------------------------------------------------------
STACKS = {
    "b2_s64_h512": dict(B=2, S=64, heads=8, D=64, layers=2),
    "b2_s128_h1024": dict(B=2, S=128, heads=16, D=64, layers=2),
    "b2_s64_d128": dict(B=2, S=64, heads=8, D=128, layers=1),
    "b4_s128_h1024_3l": dict(B=4, S=128, heads=16, D=64, layers=3),
}
# The reference stack rounds every GEMM accumulation step to fp16; measured on B200 (see the committed report)
# its distance to the fp32 oracle stays below this bound on these shapes.
STACK_REL = 2e-2


def _reference_stack(case, world, tmp_path):
    c = STACKS[case]
    dump = os.path.join(str(tmp_path), f"{case}_tp{world}.f16")
    rec = _run_harness([c["B"], c["S"], c["heads"], c["D"], c["layers"], 1, 1, dump], world=world)
    H = c["heads"] * c["D"]
    assert rec["world_size"] == world and rec["hidden"] == H
    return np.fromfile(dump, dtype=np.float16).reshape(c["B"] * c["S"], H).astype(np.float32)


def _oracle_stack(oracle, case, tp):
    c = STACKS[case]
    H = c["heads"] * c["D"]
    cfg = oracle.Config(hidden=H, heads=c["heads"], head_dim=c["D"], ffn_inner=4 * H, layers=c["layers"], tp=tp, graph=0, act=0,
                        causal=0, round16=0, seed=0)
    M = c["B"] * c["S"]
    x = oracle.fill_normal_f16(M * H, 0, oracle.INPUT).astype(np.float32).reshape(M, H)
    return oracle.stack_forward(cfg, x, c["B"], c["S"])


@pytest.mark.parametrize("case", list(STACKS))
def test_stack_matches_reference_build_single_gpu(gpu, liger, oracle, tmp_path, case):
    import torch
    _need_harness()
    c = STACKS[case]
    H, M = c["heads"] * c["D"], c["B"] * c["S"]
    ref = _reference_stack(case, 1, tmp_path)
    want = _oracle_stack(oracle, case, 1)
    cfg = liger.default_config(max_batch_size=c["B"], max_seq_len=c["S"], head_num=c["heads"], size_per_head=c["D"],
                               layer_num=c["layers"], graph=0, act=0, ffn_inner=0, causal=0, seed=0, workspace_slots=2,
                               schedule_deep=1)
    model = C.c_void_p()
    liger.check(gpu.liger_model_create(C.byref(model), C.byref(cfg), 0, 1, None))
    x = dev_fill(liger, M, H, 0, oracle.INPUT)
    out = torch.zeros((M, H), dtype=torch.float16, device="cuda")
    liger.check(gpu.liger_model_forward(model, ptr(x), ptr(out), c["B"], c["S"], 0, stream_ptr()))
    torch.cuda.synchronize()
    got = to_np(out)
    gpu.liger_model_destroy(model)
    _note("stack_" + case, ref_vs_oracle=max_rel_err(ref, want), ref_vs_library=max_rel_err(ref, got),
          library_vs_oracle=max_rel_err(got, want))
    assert np.isfinite(ref).all()
    assert_close(ref, want, rel=STACK_REL, what=f"reference stack {case} vs oracle")
    assert_close(got, ref, rel=STACK_REL, what=f"library stack {case} vs reference")
    assert_close(got, want, rel=1e-2, what=f"library stack {case} vs oracle")


@pytest.mark.parametrize("case", ["b2_s64_h512", "b2_s128_h1024"])
def test_stack_matches_reference_build_two_gpus(gpu, oracle, tmp_path, case):
    """The reference at TP = 2 (ncclAllReduce of the row-parallel partials) against the oracle's rank-by-rank
    simulation and against its own TP = 1 run."""
    import torch
    _need_harness()
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    ref2 = _reference_stack(case, 2, tmp_path)
    ref1 = _reference_stack(case, 1, tmp_path)
    want = _oracle_stack(oracle, case, 2)
    _note("stack_tp2_" + case, ref_vs_oracle=max_rel_err(ref2, want), ref_tp2_vs_ref_tp1=max_rel_err(ref2, ref1))
    assert_close(ref2, want, rel=STACK_REL, what=f"reference stack {case} TP=2 vs oracle")
    assert_close(ref2, ref1, rel=STACK_REL, what=f"reference stack {case} TP=2 vs TP=1")
