"""Per-kernel parity: every CUDA kernel, called through the C ABI, against the CPU oracle on the same
seeded inputs.  Tolerance for floating-point results: max |got - want| / max |want| <= 1e-2 (fp16
storage, fp32 accumulation on both sides; the GPU sums in a different order).  Seeded tensors
themselves and pure data movement are checked bit for bit."""
import ctypes as C

import numpy as np
import pytest

from helpers import assert_close, dev_fill, max_rel_err, ptr, stream_ptr, to_np

pytestmark = pytest.mark.gpu


def t16(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float16)).cuda()


def gemm(liger, a, wt, n=None, epi=0, bias=None, residual=None, n_begin=0, n_end=None, out=None, qkv=None, seq_len=0,
         heads=0, head_dim=0):
    import torch
    m, k = a.shape
    n = wt.shape[0] if n is None else n
    n_end = n if n_end is None else n_end
    args = liger.GemmArgs()
    args.a, args.wt = a.data_ptr(), wt.data_ptr()
    args.m, args.n, args.k = m, n, k
    args.lda, args.ldw = a.stride(0), wt.stride(0)
    args.n_begin, args.n_end, args.epilogue = n_begin, n_end, epi
    if bias is not None:
        args.bias = bias.data_ptr()
    if epi == liger.capi.EPI_QKV_SPLIT:
        args.q_out, args.k_out, args.v_out = (t.data_ptr() for t in qkv)
        args.seq_len, args.heads, args.head_dim = seq_len, heads, head_dim
    else:
        if out is None:
            cols = n // 2 if epi == liger.capi.EPI_GEGLU else n
            out = torch.zeros((m, cols), dtype=torch.float16, device="cuda")
        args.c, args.ldc = out.data_ptr(), out.stride(0)
        if residual is not None:
            args.residual, args.ldr = residual.data_ptr(), residual.stride(0)
    liger.check(liger.lib().liger_gemm_fp16(C.byref(args), stream_ptr()))
    return out


def check_status(liger):
    import torch
    torch.cuda.synchronize()
    st = (C.c_uint * 4)()
    code = liger.lib().liger_device_status(C.byref(st))
    assert code == 0, f"device status {list(st)}"


# ---------------------------------------------------------------------------------------------------
def test_fill_normal_matches_oracle_bit_for_bit(gpu, liger, oracle):
    rows, cols, ld = 37, 200, 1000
    d = dev_fill(liger, rows, cols, seed=3, tensor_id=17, row0=5, col0=11, src_ld=ld, mean=0.5, std=0.02)
    want = oracle.fill_window(rows, cols, 5, 11, ld, 3, 17, 0.5, 0.02)
    assert np.array_equal(to_np(d), want)
    dt = dev_fill(liger, rows, cols, seed=3, tensor_id=17, row0=5, col0=11, src_ld=ld, mean=0.5, std=0.02, mode=1)
    assert np.array_equal(to_np(dt), want.T)
    # interleaved gate / value placement
    import torch
    k, f = 16, 64
    wt = torch.zeros((2 * f, k), dtype=torch.float16, device="cuda")
    dev_fill(liger, k, f, 1, 4, col0=0, src_ld=2 * f, std=0.02, mode=2, out=wt)
    dev_fill(liger, k, f, 1, 4, col0=f, src_ld=2 * f, std=0.02, mode=3, out=wt)
    full = oracle.fill_window(k, 2 * f, 0, 0, 2 * f, 1, 4, 0.0, 0.02)
    got = to_np(wt)
    for j in range(f):
        assert np.array_equal(got[(j // 32) * 64 + j % 32], full[:, j])
        assert np.array_equal(got[(j // 32) * 64 + 32 + j % 32], full[:, f + j])


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (128, 256, 512), (512, 1536, 1024), (200, 328, 136), (32, 4608, 256),
                                    (1, 8, 8), (4096, 512, 4096)])
def test_gemm_store(gpu, liger, oracle, m, n, k):
    a = dev_fill(liger, m, k, 0, 100)
    w = oracle.fill_window(k, n, 0, 0, n, 0, 101, 0.0, 0.02)     # reference orientation W[k][n]
    wt = dev_fill(liger, k, n, 0, 101, std=0.02, mode=1)         # same tensor, K-contiguous
    assert np.array_equal(to_np(wt), w.T)
    out = gemm(liger, a, wt)
    check_status(liger)
    want = oracle.linear(to_np(a), w)
    assert_close(to_np(out), want, rel=1e-2, what=f"gemm {m}x{n}x{k}")
    # fp32 accumulation: the only error left is the final fp16 rounding
    assert max_rel_err(to_np(out), want) < 2e-3


def test_gemm_decomposed_equals_whole_bitwise(gpu, liger):
    """Slices of N tile the output exactly (src/utils.h:218-260 restarts every slice at column 0)."""
    import torch
    m, n, k, factor = 512, 1536, 1024, 8
    a = dev_fill(liger, m, k, 0, 100)
    wt = dev_fill(liger, k, n, 0, 101, std=0.02, mode=1)
    bias = dev_fill(liger, 1, n, 0, 102, std=0.02).reshape(-1)
    whole = gemm(liger, a, wt, bias=bias)
    for split in (1, 3, 5):   # [split slices, remainder] as Sample::possible_duration creates them
        out = torch.zeros_like(whole)
        step = n // factor
        gemm(liger, a, wt, bias=bias, n_begin=0, n_end=split * step, out=out)
        gemm(liger, a, wt, bias=bias, n_begin=split * step, n_end=n, out=out)
        assert torch.equal(out, whole)
    out = torch.zeros_like(whole)
    for i in range(factor):
        gemm(liger, a, wt, bias=bias, n_begin=i * n // factor, n_end=(i + 1) * n // factor, out=out)
    assert torch.equal(out, whole)
    check_status(liger)


def test_gemm_bias_gelu(gpu, liger, oracle):
    m, n, k = 384, 2048, 1024
    a = dev_fill(liger, m, k, 0, 100)
    wt = dev_fill(liger, k, n, 0, 101, std=0.02, mode=1)
    bias = dev_fill(liger, 1, n, 0, 102, std=0.02).reshape(-1)
    out = gemm(liger, a, wt, epi=liger.capi.EPI_GELU, bias=bias)
    want = oracle.add_bias_gelu(oracle.linear(to_np(a), to_np(wt).T), to_np(bias))
    assert_close(to_np(out), want, rel=1e-2, what="gemm+bias+gelu")
    check_status(liger)


def test_gemm_geglu(gpu, liger, oracle):
    import torch
    m, k, f = 256, 512, 384          # f gate + f value columns
    a = dev_fill(liger, m, k, 0, 100)
    wt = torch.zeros((2 * f, k), dtype=torch.float16, device="cuda")
    dev_fill(liger, k, f, 0, 101, col0=0, src_ld=2 * f, std=0.02, mode=2, out=wt)
    dev_fill(liger, k, f, 0, 101, col0=f, src_ld=2 * f, std=0.02, mode=3, out=wt)
    b_full = oracle.fill_normal(2 * f, 0, 102, std=0.02)
    b_il = np.empty(2 * f, np.float32)
    for j in range(f):
        b_il[(j // 32) * 64 + j % 32] = b_full[j]
        b_il[(j // 32) * 64 + 32 + j % 32] = b_full[f + j]
    out = gemm(liger, a, wt, epi=liger.capi.EPI_GEGLU, bias=t16(b_il))
    w = oracle.fill_window(k, 2 * f, 0, 0, 2 * f, 0, 101, 0.0, 0.02)
    want = oracle.add_bias_geglu(oracle.linear(to_np(a), w), b_full)
    assert_close(to_np(out), want, rel=1e-2, what="gemm+geglu")
    check_status(liger)


def test_gemm_qkv_split(gpu, liger, oracle):
    import torch
    B, S, h, D, k = 2, 96, 4, 64, 512
    n = 3 * h * D
    a = dev_fill(liger, B * S, k, 0, 100)
    wt = dev_fill(liger, k, n, 0, 101, std=0.02, mode=1)
    bias = dev_fill(liger, 1, n, 0, 102, std=0.02).reshape(-1)
    qkv = [torch.zeros((B, h, S, D), dtype=torch.float16, device="cuda") for _ in range(3)]
    gemm(liger, a, wt, epi=liger.capi.EPI_QKV_SPLIT, bias=bias, qkv=qkv, seq_len=S, heads=h, head_dim=D)
    lin = oracle.linear(to_np(a), to_np(wt).T)
    for i in range(3):
        want = oracle.add_bias_split_heads(lin[:, i * h * D:(i + 1) * h * D], to_np(bias)[i * h * D:(i + 1) * h * D], B, S, h, D)
        assert_close(to_np(qkv[i]), want, rel=1e-2, what=f"qkv split {i}")
    check_status(liger)


def test_gemm_residual(gpu, liger, oracle):
    m, n, k = 256, 512, 256
    a = dev_fill(liger, m, k, 0, 100)
    wt = dev_fill(liger, k, n, 0, 101, std=0.02, mode=1)
    bias = dev_fill(liger, 1, n, 0, 102, std=0.02).reshape(-1)
    res = dev_fill(liger, m, n, 0, 103)
    out = gemm(liger, a, wt, epi=liger.capi.EPI_RESIDUAL, bias=bias, residual=res)
    want = oracle.linear(to_np(a), to_np(wt).T) + to_np(bias)[None, :] + to_np(res)
    assert_close(to_np(out), want, rel=1e-2, what="gemm+residual")


SMALLM_KERNELS = {"auto": "1", "cluster": "2", "stream_k": "3"}   # values of LIGER_GEMM_SMALLM (read at every launch)


@pytest.mark.parametrize("kernel", list(SMALLM_KERNELS))
@pytest.mark.parametrize("epi", ["store", "gelu", "residual", "geglu", "qkv", "qkv_cache"])
@pytest.mark.parametrize("m,k", [(32, 1024), (4, 136), (1, 4096), (17, 520)])
def test_gemm_few_rows_weight_streaming_kernel(gpu, liger, oracle, monkeypatch, epi, m, k, kernel):
    """M <= 32 (a decode step) runs on the weight-streaming kernels: operand roles swapped (128 features x 32
    tokens per accumulator), K split either over a thread-block cluster (summed through distributed shared
    memory) or evenly over all CTAs (partial tiles handed over through L2, summed by the last arrival).
    Every epilogue kind against the oracle on either kernel, with K that is not a multiple of the 64-deep
    k-block, N that is not a multiple of the 128-feature tile, and M below the 32-token tile."""
    import torch
    monkeypatch.setenv("LIGER_GEMM_SMALLM", SMALLM_KERNELS[kernel])
    code = {"store": 0, "gelu": liger.capi.EPI_GELU, "residual": liger.capi.EPI_RESIDUAL, "geglu": liger.capi.EPI_GEGLU,
            "qkv": liger.capi.EPI_QKV_SPLIT, "qkv_cache": liger.capi.EPI_QKV_SPLIT}[epi]
    a = dev_fill(liger, m, k, 0, 400)
    if epi == "geglu":
        f = 416                      # 2f = 832 interleaved rows: 6.5 feature tiles
        wt = torch.zeros((2 * f, k), dtype=torch.float16, device="cuda")
        dev_fill(liger, k, f, 0, 401, col0=0, src_ld=2 * f, std=0.02, mode=2, out=wt)
        dev_fill(liger, k, f, 0, 401, col0=f, src_ld=2 * f, std=0.02, mode=3, out=wt)
        b_full = oracle.fill_normal(2 * f, 0, 402, std=0.02)
        b_il = np.empty(2 * f, np.float32)
        for j in range(f):
            b_il[(j // 32) * 64 + j % 32] = b_full[j]
            b_il[(j // 32) * 64 + 32 + j % 32] = b_full[f + j]
        out = gemm(liger, a, wt, epi=code, bias=t16(b_il))
        w = oracle.fill_window(k, 2 * f, 0, 0, 2 * f, 0, 401, 0.0, 0.02)
        want = oracle.add_bias_geglu(oracle.linear(to_np(a), w), b_full)
        assert_close(to_np(out), want, rel=1e-2, what=f"few-row gemm {epi}")
    elif epi.startswith("qkv"):
        h, D, S = 5, 64, 1           # n = 960: 7.5 feature tiles; one token per sequence
        n = 3 * h * D
        wt = dev_fill(liger, k, n, 0, 401, std=0.02, mode=1)
        bias = dev_fill(liger, 1, n, 0, 402, std=0.02).reshape(-1)
        lin = oracle.linear(to_np(a), to_np(wt).T)
        parts = [oracle.add_bias_split_heads(lin[:, i * h * D:(i + 1) * h * D], to_np(bias)[i * h * D:(i + 1) * h * D], m, S, h, D)
                 for i in range(3)]
        if epi == "qkv":
            qkv = [torch.zeros((m, h, S, D), dtype=torch.float16, device="cuda") for _ in range(3)]
            gemm(liger, a, wt, epi=code, bias=bias, qkv=qkv, seq_len=S, heads=h, head_dim=D)
            for i in range(3):
                assert_close(to_np(qkv[i]), parts[i], rel=1e-2, what=f"few-row qkv split {i}")
        else:                        # K and V appended to a cache at position 7 of 12
            cap, pos = 12, 7
            q = torch.zeros((m, h, S, D), dtype=torch.float16, device="cuda")
            kc = torch.zeros((m, h, cap, D), dtype=torch.float16, device="cuda")
            vc = torch.zeros_like(kc)
            args = liger.GemmArgs()
            args.a, args.wt, args.bias = a.data_ptr(), wt.data_ptr(), bias.data_ptr()
            args.m, args.n, args.k, args.lda, args.ldw = m, n, k, k, k
            args.n_begin, args.n_end, args.epilogue = 0, n, code
            args.q_out, args.k_out, args.v_out = q.data_ptr(), kc.data_ptr(), vc.data_ptr()
            args.seq_len, args.heads, args.head_dim, args.kv_stride, args.kv_pos = S, h, D, cap, pos
            liger.check(liger.lib().liger_gemm_fp16(C.byref(args), stream_ptr()))
            assert_close(to_np(q), parts[0], rel=1e-2, what="few-row q")
            assert_close(to_np(kc)[:, :, pos:pos + 1], parts[1], rel=1e-2, what="few-row k append")
            assert_close(to_np(vc)[:, :, pos:pos + 1], parts[2], rel=1e-2, what="few-row v append")
            assert not to_np(kc)[:, :, :pos].any() and not to_np(kc)[:, :, pos + 1:].any()
    else:
        n = 1096                     # 8.56 feature tiles
        wt = dev_fill(liger, k, n, 0, 401, std=0.02, mode=1)
        bias = dev_fill(liger, 1, n, 0, 402, std=0.02).reshape(-1)
        res = dev_fill(liger, m, n, 0, 403) if epi == "residual" else None
        out = gemm(liger, a, wt, epi=code, bias=bias, residual=res)
        want = oracle.linear(to_np(a), to_np(wt).T) + to_np(bias)[None, :]
        if epi == "gelu":
            want = oracle.add_bias_gelu(want, None)
        if epi == "residual":
            want = want + to_np(res)
        assert_close(to_np(out), want, rel=1e-2, what=f"few-row gemm {epi}")
        assert max_rel_err(to_np(out), want) < 2e-3      # fp32 accumulation: only the final rounding is left
        # slices of the feature range give the bits of the whole launch (the K split is chosen from the whole weight)
        out2 = torch.zeros_like(out)
        for lo, hi in [(0, 136), (136, 512), (512, n)]:
            gemm(liger, a, wt, epi=code, bias=bias, residual=res, n_begin=lo, n_end=hi, out=out2)
        assert torch.equal(out2, out)
    check_status(liger)


def test_gemm_few_rows_at_decode_shapes(gpu, liger):
    """The four GEMM shapes of a GLM-130B decode step at TP = 8 (32 tokens): sampled entries against fp64 dot products."""
    import torch
    for (n, k) in [(4608, 12288), (12288, 1536), (8192, 12288), (12288, 4096)]:
        a = dev_fill(liger, 32, k, 0, 410, std=0.5)
        wt = dev_fill(liger, k, n, 0, 411, std=0.02, mode=1)
        y = gemm(liger, a, wt)
        check_status(liger)
        g = torch.Generator().manual_seed(1)
        rows = torch.randint(0, 32, (48,), generator=g).tolist()
        cols = torch.randint(0, n, (48,), generator=g).tolist() + [0, n - 1]
        for r, c in zip(rows + [0, 31], cols):
            want = (a[r].double() * wt[c].double()).sum().item()
            assert abs(y[r, c].item() - want) <= 2e-3 * max(1.0, abs(want)), (n, k, r, c)


def test_gemm_few_rows_stream_k_partitions(gpu, liger, monkeypatch):
    """The stream-K kernel where a CTA's range of k-blocks crosses tile boundaries: a partial head, whole tiles in
    the middle, a partial tail (38400 x 2560: 300 tiles x 40 k-blocks over 148 CTAs), and the two GLM-130B shapes
    with few tiles and a long K.  Against the cluster kernel (same fp32 sums in another order: one rounding apart)
    and against fp64 dot products of sampled entries; twice in a row, since the arrival counters alternate."""
    import torch
    for (n, k) in [(38400, 2560), (12288, 12288), (4608, 12288)]:
        a = dev_fill(liger, 32, k, 0, 420, std=0.5)
        wt = dev_fill(liger, k, n, 0, 421, std=0.02, mode=1)
        monkeypatch.setenv("LIGER_GEMM_SMALLM", SMALLM_KERNELS["cluster"])
        y_cluster = gemm(liger, a, wt)
        monkeypatch.setenv("LIGER_GEMM_SMALLM", SMALLM_KERNELS["stream_k"])
        y1 = gemm(liger, a, wt)
        y2 = gemm(liger, a, wt)
        check_status(liger)
        assert torch.equal(y1, y2)                     # deterministic summation order
        diff = (y1.float() - y_cluster.float()).abs()
        assert bool((diff <= 2e-3 * y_cluster.float().abs().clamp(min=1.0)).all()), (n, k, diff.max().item())
        g = torch.Generator().manual_seed(2)
        rows = torch.randint(0, 32, (32,), generator=g).tolist()
        cols = torch.randint(0, n, (32,), generator=g).tolist()
        for r, c in zip(rows, cols):
            want = (a[r].double() * wt[c].double()).sum().item()
            assert abs(y1[r, c].item() - want) <= 2e-3 * max(1.0, abs(want)), (n, k, r, c)


def test_gemm_few_rows_stream_k_on_two_streams(gpu, liger, monkeypatch):
    """Few-row GEMMs in flight on two streams at once: the stream-K kernel keeps its partial tiles and arrival
    counters per stream, so concurrent launches must not disturb one another (same bits as one after the other)."""
    import torch
    monkeypatch.setenv("LIGER_GEMM_SMALLM", SMALLM_KERNELS["stream_k"])
    n, k = 12288, 4096
    a = [dev_fill(liger, 32, k, 0, 430 + i, std=0.5) for i in range(2)]
    wt = [dev_fill(liger, k, n, 0, 432 + i, std=0.02, mode=1) for i in range(2)]
    want = [gemm(liger, a[i], wt[i]) for i in range(2)]
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream() for _ in range(2)]
    outs = [[torch.zeros_like(want[0]) for _ in range(6)] for _ in range(2)]
    for rep in range(6):
        for i in range(2):
            args = liger.GemmArgs()
            args.a, args.wt, args.c = a[i].data_ptr(), wt[i].data_ptr(), outs[i][rep].data_ptr()
            args.m, args.n, args.k, args.lda, args.ldw, args.ldc = 32, n, k, k, k, n
            args.n_begin, args.n_end, args.epilogue = 0, n, 0
            liger.check(liger.lib().liger_gemm_fp16(C.byref(args), C.c_void_p(streams[i].cuda_stream)))
    torch.cuda.synchronize()
    check_status(liger)
    for i in range(2):
        for rep in range(6):
            assert torch.equal(outs[i][rep], want[i]), (i, rep)


def test_gemm_linearity_at_full_size(gpu, liger):
    """Size-independent property at the GLM-130B TP=8 QKV shape: (A1 + A2) W == A1 W + A2 W up to
    fp16 rounding, and a sampled set of entries against an fp64 dot product."""
    import torch
    m, n, k = 4096, 4608, 12288
    a1 = dev_fill(liger, m, k, 0, 200, std=0.5)
    a2 = dev_fill(liger, m, k, 0, 201, std=0.5)
    wt = dev_fill(liger, k, n, 0, 202, std=0.02, mode=1)
    s = (a1.float() + a2.float()).half()
    y1, y2, ys = gemm(liger, a1, wt), gemm(liger, a2, wt), gemm(liger, s, wt)
    check_status(liger)
    ref = y1.float() + y2.float()
    err = (ys.float() - ref).abs().max().item() / ref.abs().max().item()
    assert err < 1e-2, err
    g = torch.Generator().manual_seed(0)
    rows = torch.randint(0, m, (64,), generator=g).tolist()
    cols = torch.randint(0, n, (64,), generator=g).tolist()
    for r, c in zip(rows, cols):
        want = (a1[r].double() * wt[c].double()).sum().item()
        assert abs(y1[r, c].item() - want) <= 1e-2 * max(1.0, abs(want))


@pytest.mark.parametrize("epi", ["store", "residual", "qkv", "geglu", "gelu"])
@pytest.mark.parametrize("n_end", [12288, 12224])
def test_gemm_long_k_whole_equals_slices_bitwise(gpu, liger, epi, n_end):
    """At long K the whole launch runs on 256x512 tiles (with a split last wave at this shape, and a
    partial last tile for n_end = 12224) while the eight slices are too small for them and take the
    256x256 kernel: every epilogue must give the same bits either way, and sampled entries must match
    an fp64 dot product."""
    import torch
    m, n, k, factor = 4096, 12288, 8192, 8
    B, S, h, D = 8, 512, 32, 128
    a = dev_fill(liger, m, k, 0, 300, std=0.5)
    wt = dev_fill(liger, k, n, 0, 301, std=0.02, mode=1)
    bias = dev_fill(liger, 1, n, 0, 302, std=0.02).reshape(-1)
    res = dev_fill(liger, m, n, 0, 303) if epi == "residual" else None
    code = {"store": 0, "gelu": liger.capi.EPI_GELU, "geglu": liger.capi.EPI_GEGLU, "qkv": liger.capi.EPI_QKV_SPLIT,
            "residual": liger.capi.EPI_RESIDUAL}[epi]

    def run(slices):
        kw = dict(epi=code, bias=bias, residual=res)
        if epi == "qkv":
            qkv = [torch.zeros((B, h, S, D), dtype=torch.float16, device="cuda") for _ in range(3)]
            kw.update(qkv=qkv, seq_len=S, heads=h, head_dim=D)
        else:
            kw.update(out=torch.zeros((m, n // 2 if epi == "geglu" else n), dtype=torch.float16, device="cuda"))
        for lo, hi in slices:
            if lo < hi:
                gemm(liger, a, wt, n_begin=lo, n_end=hi, **kw)
        return kw["qkv"] if epi == "qkv" else [kw["out"]]

    whole = run([(0, n_end)])
    step = n // factor
    parts = run([(i * step, min((i + 1) * step, n_end)) for i in range(factor)])
    check_status(liger)
    for w_, p_ in zip(whole, parts):
        assert torch.equal(w_, p_)
    if epi == "store":
        g = torch.Generator().manual_seed(1)
        rows = torch.randint(0, m, (64,), generator=g).tolist()
        cols = torch.randint(0, n_end, (64,), generator=g).tolist()
        for r, c in zip(rows, cols):
            want = (a[r].double() * wt[c].double()).sum().item() + bias[c].item()
            assert abs(whole[0][r, c].item() - want) <= 1e-2 * max(1.0, abs(want))
        assert whole[0][:, n_end:].abs().max().item() == 0 if n_end < n else True


# ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("m,n", [(7, 1024), (512, 12288), (3, 8), (5, 16384)])
def test_layernorm(gpu, liger, oracle, m, n):
    import torch
    x = dev_fill(liger, m, n, 0, 300, mean=0.3)
    g = dev_fill(liger, 1, n, 0, 301, mean=1.0, std=0.02).reshape(-1)
    b = dev_fill(liger, 1, n, 0, 302, std=0.02).reshape(-1)
    y = torch.empty_like(x)
    liger.check(liger.lib().liger_layernorm(ptr(x), ptr(g), ptr(b), ptr(y), m, n, stream_ptr()))
    want = oracle.layernorm(to_np(x), to_np(g), to_np(b))
    assert_close(to_np(y), want, rel=2e-3, what="layernorm")


@pytest.mark.parametrize("with_norm", [True, False])
def test_add_bias_input_layernorm(gpu, liger, oracle, with_norm):
    import torch
    m, n = 33, 1024
    inp = dev_fill(liger, m, n, 0, 310)
    out = dev_fill(liger, m, n, 0, 311)
    bias = dev_fill(liger, 1, n, 0, 312, std=0.02).reshape(-1)
    g = dev_fill(liger, 1, n, 0, 313, mean=1.0, std=0.02).reshape(-1)
    b = dev_fill(liger, 1, n, 0, 314, std=0.02).reshape(-1)
    want_out, want_norm = oracle.add_bias_input_layernorm_2(to_np(inp), to_np(g), to_np(b), to_np(bias), to_np(out),
                                                            want_norm=with_norm)
    norm = torch.empty_like(out) if with_norm else None
    liger.check(liger.lib().liger_add_bias_input_layernorm(ptr(inp), ptr(g), ptr(b), ptr(bias), ptr(out), ptr(norm),
                                                           m, n, stream_ptr()))
    assert_close(to_np(out), want_out, rel=1e-3, what="residual sum")
    if with_norm:
        assert_close(to_np(norm), want_norm, rel=2e-3, what="residual layernorm")


def test_add_bias_gelu(gpu, liger, oracle):
    m, n = 65, 2048
    x = dev_fill(liger, m, n, 0, 320)
    bias = dev_fill(liger, 1, n, 0, 321, std=0.02).reshape(-1)
    want = oracle.add_bias_gelu(to_np(x), to_np(bias))
    liger.check(liger.lib().liger_add_bias_gelu(ptr(x), ptr(bias), m, n, stream_ptr()))
    assert_close(to_np(x), want, rel=2e-3, what="bias+gelu")


def test_head_split_and_merge(gpu, liger, oracle):
    import torch
    B, S, h, D = 3, 50, 4, 64
    srcs = [dev_fill(liger, B * S, h * D, 0, 330 + i) for i in range(3)]
    biases = [dev_fill(liger, 1, h * D, 0, 340 + i, std=0.02).reshape(-1) for i in range(3)]
    outs = [torch.empty((B, h, S, D), dtype=torch.float16, device="cuda") for _ in range(3)]
    liger.check(liger.lib().liger_add_qkv_bias_transpose(
        ptr(outs[0]), ptr(outs[1]), ptr(outs[2]), ptr(srcs[0]), ptr(biases[0]), ptr(srcs[1]), ptr(biases[1]),
        ptr(srcs[2]), ptr(biases[2]), B, S, h, D, stream_ptr()))
    for i in range(3):
        want = oracle.add_bias_split_heads(to_np(srcs[i]), to_np(biases[i]), B, S, h, D)
        assert_close(to_np(outs[i]), want, rel=1e-3, what="bias+split")
    merged = torch.empty((B * S, h * D), dtype=torch.float16, device="cuda")
    liger.check(liger.lib().liger_transpose_heads(ptr(merged), ptr(outs[0]), B, S, h, D, stream_ptr()))
    assert np.array_equal(to_np(merged), oracle.merge_heads(to_np(outs[0])))


def test_transpose_weight(gpu, liger):
    import torch
    k, n = 100, 192
    w = dev_fill(liger, k, n, 0, 350)
    wt = torch.empty((n, k), dtype=torch.float16, device="cuda")
    liger.check(liger.lib().liger_transpose_weight(ptr(w), ptr(wt), k, n, 0, stream_ptr()))
    assert torch.equal(wt, w.t().contiguous())
    liger.check(liger.lib().liger_transpose_weight(ptr(w), ptr(wt), k, n, 1, stream_ptr()))
    got, src = to_np(wt), to_np(w)
    f = n // 2
    for j in range(f):
        assert np.array_equal(got[(j // 32) * 64 + j % 32], src[:, j])
        assert np.array_equal(got[(j // 32) * 64 + 32 + j % 32], src[:, f + j])


# ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("B,h,S,D,mode", [(2, 3, 128, 64, "causal"), (1, 2, 100, 128, "causal"), (2, 2, 64, 64, "none"),
                                          (1, 2, 130, 64, "mask"), (2, 4, 512, 128, "causal"), (1, 1, 2, 64, "mask"),
                                          (1, 2, 320, 128, "mask"),
                                          # head_dim 128 without a mask tensor, seq >= 128: the tcgen05 kernel (ragged last
                                          # key block / query tile, one and several key blocks, more items than SMs)
                                          (2, 3, 256, 128, "causal"), (1, 2, 200, 128, "causal"), (1, 4, 384, 128, "none"),
                                          (2, 2, 130, 128, "causal"), (1, 3, 128, 128, "none"), (3, 64, 512, 128, "causal"),
                                          (1, 2, 1100, 128, "causal")])
def test_attention_prefill(gpu, liger, oracle, B, h, S, D, mode):
    import torch
    q = dev_fill(liger, B * h * S, D, 0, 400).reshape(B, h, S, D)
    k = dev_fill(liger, B * h * S, D, 0, 401).reshape(B, h, S, D)
    v = dev_fill(liger, B * h * S, D, 0, 402).reshape(B, h, S, D)
    mask_np, mask_t = None, None
    if mode == "mask":   # ragged: per-sequence valid length, plus a causal band (arbitrary 0/1 tensor)
        mask_np = np.zeros((B, S, S), np.float32)
        for b in range(B):
            L = max(1, S - 7 * b - 3)
            mask_np[b, :, :L] = np.tril(np.ones((S, L), np.float32), k=5)
        mask_t = t16(mask_np)
    out = torch.zeros((B * S, h * D), dtype=torch.float16, device="cuda")
    scale = 1.0 / np.sqrt(D)
    liger.check(liger.lib().liger_attention_prefill(ptr(q), ptr(k), ptr(v), ptr(mask_t), ptr(out), B, h, S, D, h * D,
                                                    scale, 1 if mode == "causal" else 0, stream_ptr()))
    want = oracle.merge_heads(oracle.attention(to_np(q), to_np(k), to_np(v), mask=mask_np, causal=(mode == "causal"),
                                               scale=scale))
    assert_close(to_np(out), want, rel=1e-2, what=f"attention {mode}")
    check_status(liger)


def test_attention_decode_cache_larger_than_l2(gpu, liger, oracle):
    """The benchmark's per-layer decode attention at a quarter of its batch: 8 sequences x 96 heads x 2048 cached
    positions x 128 (805 MB of K and V, read once from HBM).  Sixteen sampled (sequence, head) pairs against the
    oracle; the result does not depend on the order in which the 256-key chunks finish (two runs, same bits)."""
    import torch
    B, h, L, D = 8, 96, 2048, 128
    Lmax = L + 64
    q = dev_fill(liger, B * h, D, 0, 410).reshape(B, h, D)
    kc = dev_fill(liger, B * h * Lmax, D, 0, oracle.KCACHE).reshape(B, h, Lmax, D)
    vc = dev_fill(liger, B * h * Lmax, D, 0, oracle.VCACHE).reshape(B, h, Lmax, D)
    nbytes = liger.lib().liger_attention_decode_scratch_bytes(B, h, D, L)
    scratch = torch.empty(nbytes // 4, dtype=torch.float32, device="cuda")
    scale = 1.0 / np.sqrt(D)
    outs = []
    for _ in range(2):
        out = torch.zeros((B, h * D), dtype=torch.float16, device="cuda")
        liger.check(liger.lib().liger_attention_decode(ptr(q), ptr(kc), ptr(vc), ptr(out), ptr(scratch), B, h, L, Lmax, D,
                                                       h * D, scale, stream_ptr()))
        outs.append(out)
    check_status(liger)
    assert torch.equal(outs[0], outs[1])
    g = torch.Generator().manual_seed(3)
    got = to_np(outs[0]).reshape(B, h, D)
    for b, hd in zip(torch.randint(0, B, (16,), generator=g).tolist(), torch.randint(0, h, (16,), generator=g).tolist()):
        want = oracle.attention(to_np(q[b:b + 1, hd:hd + 1])[:, :, None, :], to_np(kc[b:b + 1, hd:hd + 1, :L]),
                                to_np(vc[b:b + 1, hd:hd + 1, :L]), causal=True, scale=scale)
        assert_close(got[b, hd], want.reshape(D), rel=1e-2, what=f"decode attention ({b}, {hd})")


@pytest.mark.parametrize("B,h,L,D", [(2, 3, 300, 128), (4, 2, 2048, 128), (1, 2, 17, 64), (3, 1, 256, 64)])
def test_attention_decode(gpu, liger, oracle, B, h, L, D):
    import torch
    Lmax = L + 5
    q = dev_fill(liger, B * h, D, 0, 410).reshape(B, h, D)
    kc = dev_fill(liger, B * h * Lmax, D, 0, oracle.KCACHE).reshape(B, h, Lmax, D)
    vc = dev_fill(liger, B * h * Lmax, D, 0, oracle.VCACHE).reshape(B, h, Lmax, D)
    nbytes = liger.lib().liger_attention_decode_scratch_bytes(B, h, D, L)
    scratch = torch.empty(nbytes // 4, dtype=torch.float32, device="cuda")
    out = torch.zeros((B, h * D), dtype=torch.float16, device="cuda")
    scale = 1.0 / np.sqrt(D)
    liger.check(liger.lib().liger_attention_decode(ptr(q), ptr(kc), ptr(vc), ptr(out), ptr(scratch), B, h, L, Lmax, D,
                                                   h * D, scale, stream_ptr()))
    want = oracle.attention(to_np(q)[:, :, None, :], to_np(kc)[:, :, :L], to_np(vc)[:, :, :L], causal=True, scale=scale)
    assert_close(to_np(out), want.reshape(B, h * D), rel=1e-2, what="decode attention")
