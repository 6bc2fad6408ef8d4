"""Shared helpers for the GPU parity tests: seeded tensors on both sides, error metrics."""
import ctypes as C

import numpy as np


def stream_ptr():
    import torch
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def dev_fill(liger, rows, cols, seed, tensor_id, row0=0, col0=0, src_ld=None, mean=0.0, std=1.0, mode=0, out=None,
             dst_ld=None, dst_rows=None):
    """Seeded fp16 tensor generated on the device through the C ABI (liger_fill_normal)."""
    import torch
    src_ld = cols if src_ld is None else src_ld
    if out is None:
        shape = (rows, cols) if mode == 0 else ((cols if dst_rows is None else dst_rows), rows)
        out = torch.empty(shape, dtype=torch.float16, device="cuda")
    ld = out.shape[1] if dst_ld is None else dst_ld
    liger.check(liger.lib().liger_fill_normal(ptr(out), rows, cols, ld, row0, col0, src_ld, seed, tensor_id,
                                              mean, std, mode, stream_ptr()))
    return out


def to_np(t):
    return t.detach().float().cpu().numpy()


def max_rel_err(got, want):
    """max |got - want| / max |want| -- the per-tensor relative error used for the 1e-2 bound."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    return float(np.abs(got - want).max() / max(np.abs(want).max(), 1e-30))


def assert_close(got, want, rel=1e-2, abs_floor=None, what=""):
    """Tensor-level bound (max abs diff / max abs oracle <= rel) plus an element-wise check with an
    absolute floor of rel * max|want|."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite values in result"
    scale = max(np.abs(want).max(), 1e-30)
    floor = rel * scale if abs_floor is None else abs_floor
    err = np.abs(got - want)
    tol = floor + rel * np.abs(want)
    bad = err > tol
    assert not bad.any(), (f"{what}: {bad.sum()} elements off; worst abs err {err.max():.4g} at "
                           f"{np.unravel_index(err.argmax(), err.shape)}, tensor scale {scale:.4g}")
    assert err.max() / scale <= rel, f"{what}: max rel err {err.max() / scale:.4g} > {rel}"
