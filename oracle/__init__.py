"""ctypes wrapper around the CPU oracle (oracle/liger_oracle.c).

TEST INFRASTRUCTURE: only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may
import this module.  The product (the package holding the CUDA library) never does.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "liboracle.so")


def build(force=False):
    src = [os.path.join(HERE, "liger_oracle.c"), os.path.join(HERE, "..", "include", "liger_rng.h")]
    if force or not os.path.exists(LIB) or any(os.path.getmtime(s) > os.path.getmtime(LIB) for s in src):
        subprocess.run(["make", "-C", HERE, "-B", "liboracle.so"], check=True, capture_output=True)
    return LIB


class Config(C.Structure):
    _fields_ = [("hidden", C.c_int), ("heads", C.c_int), ("head_dim", C.c_int), ("ffn_inner", C.c_int),
                ("layers", C.c_int), ("tp", C.c_int), ("graph", C.c_int), ("act", C.c_int), ("causal", C.c_int),
                ("round16", C.c_int), ("seed", C.c_uint32)]


# tensor ids (mirrors the enum in liger_oracle.c)
WQ, WK, WV, WO, WUP, WDOWN, BQ, BK, BV, BUP, LN1_G, LN1_B, LN2_G, LN2_B, BO, BDOWN = range(16)
INPUT, KCACHE, VCACHE = 0x10000, 0x10001, 0x10002
W_STD = 0.02

_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB):
            build()
        _lib = C.CDLL(LIB)
        _lib.lo_num_threads.restype = C.c_int
        _lib.lo_fill_seconds.restype = C.c_double
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def fill_seconds(reset=False):
    """Seconds spent generating seeded tensors since the last reset."""
    return lib().lo_fill_seconds(int(reset))


def num_threads():
    return lib().lo_num_threads()


def fill_normal(n, seed, tensor_id, idx0=0, mean=0.0, std=1.0):
    out = np.empty(n, np.float32)
    lib().lo_fill_normal_f32(_p(out), C.c_uint64(n), C.c_uint32(seed), C.c_uint32(tensor_id), C.c_uint64(idx0),
                             C.c_float(mean), C.c_float(std))
    return out


def fill_normal_f16(n, seed, tensor_id, idx0=0, mean=0.0, std=1.0):
    out = np.empty(n, np.uint16)
    lib().lo_fill_normal_f16(_p(out), C.c_uint64(n), C.c_uint32(seed), C.c_uint32(tensor_id), C.c_uint64(idx0),
                             C.c_float(mean), C.c_float(std))
    return out.view(np.float16)


def fill_window(rows, cols, row0, col0, ld, seed, tensor_id, mean=0.0, std=1.0):
    out = np.empty((rows, cols), np.float32)
    lib().lo_fill_normal_window_f32(_p(out), rows, cols, row0, col0, ld, C.c_uint32(seed), C.c_uint32(tensor_id),
                                    C.c_float(mean), C.c_float(std))
    return out


def round_fp16(x):
    x = _f32(x).copy()
    lib().lo_round_fp16(_p(x), C.c_uint64(x.size))
    return x


def linear(x, w):
    x, w = _f32(x), _f32(w)
    m, k = x.shape
    k2, n = w.shape
    assert k == k2
    y = np.empty((m, n), np.float32)
    lib().lo_linear(_p(x), k, _p(w), n, _p(y), n, m, n, k)
    return y


def add_bias_split_heads(src, bias, B, S, h, D):
    src = _f32(src)
    out = np.empty((B, h, S, D), np.float32)
    b = _f32(bias) if bias is not None else None
    lib().lo_add_bias_split_heads(_p(src), src.shape[1], _p(b), _p(out), B, S, h, D)
    return out


def merge_heads(src):
    src = _f32(src)
    B, h, S, D = src.shape
    out = np.empty((B * S, h * D), np.float32)
    lib().lo_merge_heads(_p(src), _p(out), h * D, B, S, h, D)
    return out


def attention(q, k, v, mask=None, causal=False, scale=None):
    q, k, v = _f32(q), _f32(k), _f32(v)
    B, h, Sq, D = q.shape
    Skv = k.shape[2]
    m = _f32(mask) if mask is not None else None
    out = np.empty((B, h, Sq, D), np.float32)
    sc = scale if scale is not None else 1.0 / np.sqrt(D)
    lib().lo_attention(_p(q), _p(k), _p(v), _p(m), int(bool(causal)), _p(out), B, h, Sq, Skv, D, C.c_float(sc))
    return out


def masked_softmax(scores, mask, scale):
    """softmax(scale * scores + (1 - mask) * -10000) over the last axis; scores [B,h,S,S], mask [B,S,S] or None."""
    s = _f32(scores).copy()
    B, h, S, _ = s.shape
    m = _f32(mask) if mask is not None else None
    lib().lo_masked_softmax(_p(s), _p(m), B, h, S, C.c_float(scale))
    return s


def add_bias_gelu(x, bias):
    x = _f32(x).copy()
    b = _f32(bias) if bias is not None else None
    lib().lo_add_bias_gelu(_p(x), _p(b), x.shape[0], x.shape[1])
    return x


def add_bias_geglu(u, bias):
    u = _f32(u)
    m, n2 = u.shape
    out = np.empty((m, n2 // 2), np.float32)
    b = _f32(bias) if bias is not None else None
    lib().lo_add_bias_geglu(_p(u), _p(b), _p(out), m, n2 // 2)
    return out


def layernorm(x, gamma, beta):
    x, gamma, beta = _f32(x), _f32(gamma), _f32(beta)
    y = np.empty_like(x)
    lib().lo_layernorm(_p(x), _p(gamma), _p(beta), _p(y), x.shape[0], x.shape[1])
    return y


def add_bias_input_layernorm_2(inp, gamma, beta, bias, out, want_norm=True, round16=True):
    inp = _f32(inp)
    out = _f32(out).copy()
    norm = np.empty_like(out) if want_norm else None
    g = _f32(gamma) if gamma is not None else None
    b = _f32(beta) if beta is not None else None
    bi = _f32(bias) if bias is not None else None
    lib().lo_add_bias_input_layernorm_2(_p(inp), _p(g), _p(b), _p(bi), _p(out), _p(norm), out.shape[0], out.shape[1],
                                        int(round16))
    return out, norm


def allreduce_sum(partials):
    partials = _f32(partials)
    ws = partials.shape[0]
    out = np.empty(partials.shape[1:], np.float32)
    lib().lo_allreduce_sum(_p(partials), _p(out), ws, C.c_uint64(out.size))
    return out


def stack_forward(cfg: Config, x, B, S, mask=None):
    x = _f32(x)
    out = np.empty_like(x)
    m = _f32(mask) if mask is not None else None
    lib().lo_stack_forward(C.byref(cfg), _p(x), _p(m), _p(out), B, S)
    return out


def stack_decode(cfg: Config, x, B, kv_len, kv_cap):
    """One decode step of the pre-LN stack against the seeded KV cache (see lo_stack_decode)."""
    x = _f32(x)
    out = np.empty_like(x)
    lib().lo_stack_decode(C.byref(cfg), _p(x), _p(out), B, kv_len, kv_cap)
    return out
