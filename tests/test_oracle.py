"""The CPU oracle itself: its seeded generator, each operator against an independent NumPy restatement
(float64), the whole stack for both graphs, tensor-parallel invariance, and the committed fixtures."""
import json
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


# ---- independent NumPy restatement (float64) ---------------------------------------------------------------
def np_gelu(x):
    return x * 0.5 * (1.0 + np.tanh(0.7978845608028654 * (x + 0.044715 * x ** 3)))


def np_layernorm(x, g, b):
    mu = x.mean(-1, keepdims=True)
    var = ((x - mu) ** 2).mean(-1, keepdims=True)
    return (x - mu) / np.sqrt(var + 1e-6) * g + b


def np_attention(q, k, v, mask, scale):
    s = np.einsum("bhqd,bhkd->bhqk", q, k) * scale + (1.0 - mask[:, None]) * -10000.0
    s = s - s.max(-1, keepdims=True)
    p = np.exp(s)
    p = p / (p.sum(-1, keepdims=True) + 1e-6)
    return np.einsum("bhqk,bhkd->bhqd", p, v)


def np_stack(oracle, c, x, B, S):
    """Full (unsharded) weights, float64 -- tensor parallelism must not change the result."""
    H, D, F, heads = c["hidden"], c["head_dim"], c["ffn_inner"], c["heads"]
    upw = 2 * F if c["act"] else F
    mask = np.tril(np.ones((S, S)))[None].repeat(B, 0) if c["causal"] else np.ones((B, S, S))
    h = x.astype(np.float64)

    def w(l, kind, rows, cols):
        return oracle.fill_window(rows, cols, 0, 0, cols, 0, l * 32 + kind, 0.0, 0.02).astype(np.float64)

    def vec(l, kind, n, mean=0.0):
        return oracle.fill_normal(n, 0, l * 32 + kind, 0, mean, 0.02).astype(np.float64)

    for l in range(c["layers"]):
        a_in = np_layernorm(h, vec(l, oracle.LN1_G, H, 1.0), vec(l, oracle.LN1_B, H)) if c["graph"] else h
        qkv = [a_in @ w(l, kind, H, H) + vec(l, bk, H) for kind, bk in
               ((oracle.WQ, oracle.BQ), (oracle.WK, oracle.BK), (oracle.WV, oracle.BV))]
        q, k, v = [t.reshape(B, S, heads, D).transpose(0, 2, 1, 3) for t in qkv]
        att = np_attention(q, k, v, mask, 1.0 / np.sqrt(D)).transpose(0, 2, 1, 3).reshape(B * S, H)
        o = att @ w(l, oracle.WO, H, H)
        if c["graph"]:
            h = h + o + vec(l, oracle.BO, H)
            m_in = np_layernorm(h, vec(l, oracle.LN2_G, H, 1.0), vec(l, oracle.LN2_B, H))
        else:
            m_in = np_layernorm(o, vec(l, oracle.LN1_G, H, 1.0), vec(l, oracle.LN1_B, H))
        u = m_in @ w(l, oracle.WUP, H, upw) + vec(l, oracle.BUP, upw)
        act = np_gelu(u[:, :F]) * u[:, F:] if c["act"] else np_gelu(u)
        d = act @ w(l, oracle.WDOWN, F, H)
        if c["graph"]:
            h = h + d + vec(l, oracle.BDOWN, H)
        else:
            h = np_layernorm(d, vec(l, oracle.LN2_G, H, 1.0), vec(l, oracle.LN2_B, H))
    return h


# ---- the generator -----------------------------------------------------------------------------------------
def test_generator_matches_committed_values(oracle):
    for e in json.load(open(os.path.join(HERE, "golden", "rng_golden.json"))):
        got = oracle.fill_normal_f16(8, e["seed"], e["tensor_id"], e["idx0"], e["mean"], e["std"]).view(np.uint16)
        assert got.tolist() == e["fp16_bits"], e


def test_generator_is_a_pure_function_of_its_index(oracle):
    a = oracle.fill_normal(1000, 3, 9, idx0=0)
    b = oracle.fill_normal(600, 3, 9, idx0=400)
    assert np.array_equal(a[400:], b)
    w = oracle.fill_window(5, 7, 2, 3, 20, 3, 9)
    full = oracle.fill_normal(20 * 20, 3, 9).reshape(20, 20)
    assert np.array_equal(w, full[2:7, 3:10])
    assert not np.array_equal(oracle.fill_normal(100, 3, 9), oracle.fill_normal(100, 4, 9))
    assert not np.array_equal(oracle.fill_normal(100, 3, 9), oracle.fill_normal(100, 3, 10))


def test_generator_is_standard_normal(oracle):
    x = oracle.fill_normal(1 << 20, 0, 77).astype(np.float64)
    assert abs(x.mean()) < 5e-3 and abs(x.std() - 1.0) < 5e-3
    assert abs((x ** 3).mean()) < 2e-2 and abs((x ** 4).mean() - 3.0) < 5e-2
    assert np.isfinite(x).all() and np.abs(x).max() < 6.5
    y = oracle.fill_normal(1 << 16, 0, 78, mean=1.0, std=0.02)
    assert abs(y.mean() - 1.0) < 1e-3 and abs(y.std() - 0.02) < 1e-3


def test_fp16_rounding_is_round_to_nearest_even(oracle):
    x = np.concatenate([np.random.default_rng(0).normal(0, 100, 20000), [0.0, 65504.0, 65519.9, 65520.0, 1e-8, 6e-8, -2.98e-8,
                        2.0 ** -24, 2.0 ** -25, 1.0 + 2.0 ** -11, 1.0 + 3 * 2.0 ** -11]]).astype(np.float32)
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).astype(np.float32)
    assert np.array_equal(oracle.round_fp16(x), want)


# ---- operators ---------------------------------------------------------------------------------------------
def test_linear_layernorm_gelu_against_numpy(oracle):
    rng = np.random.default_rng(1)
    x = rng.normal(size=(37, 100)).astype(np.float32)
    w = rng.normal(size=(100, 53)).astype(np.float32)
    assert np.allclose(oracle.linear(x, w), x.astype(np.float64) @ w, atol=1e-4)
    g, b = rng.normal(1, 0.1, 100).astype(np.float32), rng.normal(0, 0.1, 100).astype(np.float32)
    assert np.allclose(oracle.layernorm(x, g, b), np_layernorm(x.astype(np.float64), g, b), atol=1e-5)
    bias = rng.normal(size=100).astype(np.float32)
    assert np.allclose(oracle.add_bias_gelu(x, bias), np_gelu(x.astype(np.float64) + bias), atol=1e-5)
    u = rng.normal(size=(9, 64)).astype(np.float32)
    b2 = rng.normal(size=64).astype(np.float32)
    t = u.astype(np.float64) + b2
    assert np.allclose(oracle.add_bias_geglu(u, b2), np_gelu(t[:, :32]) * t[:, 32:], atol=1e-5)


@pytest.mark.parametrize("causal", [False, True])
def test_attention_against_numpy(oracle, causal):
    rng = np.random.default_rng(2)
    B, h, S, D = 2, 3, 17, 8
    q, k, v = (rng.normal(size=(B, h, S, D)).astype(np.float32) for _ in range(3))
    mask = np.tril(np.ones((S, S)))[None].repeat(B, 0) if causal else (rng.random((B, S, S)) > 0.3).astype(np.float64)
    mask[:, :, 0] = 1
    got = oracle.attention(q, k, v, mask=None if causal else mask.astype(np.float32), causal=causal)
    want = np_attention(q.astype(np.float64), k.astype(np.float64), v.astype(np.float64), mask, 1 / np.sqrt(D))
    assert np.allclose(got, want, atol=1e-5)


def test_head_split_merge_and_residual(oracle):
    rng = np.random.default_rng(3)
    B, S, h, D = 2, 5, 3, 4
    x = rng.normal(size=(B * S, h * D)).astype(np.float32)
    bias = rng.normal(size=h * D).astype(np.float32)
    sp = oracle.add_bias_split_heads(x, bias, B, S, h, D)
    assert np.allclose(sp, (x + bias).reshape(B, S, h, D).transpose(0, 2, 1, 3))
    assert np.array_equal(oracle.merge_heads(sp), (x + bias).astype(np.float32))
    inp, out = rng.normal(size=(6, 16)).astype(np.float32), rng.normal(size=(6, 16)).astype(np.float32)
    b, g, be = (rng.normal(size=16).astype(np.float32) for _ in range(3))
    o2, n2 = oracle.add_bias_input_layernorm_2(inp, g, be, b, out, round16=False)
    assert np.allclose(o2, inp + out + b, atol=1e-6)
    assert np.allclose(n2, np_layernorm((inp + out + b).astype(np.float64), g, be), atol=1e-5)
    parts = rng.normal(size=(4, 10)).astype(np.float32)
    assert np.allclose(oracle.allreduce_sum(parts), parts.sum(0), atol=1e-6)


# ---- the stack ---------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def golden_mod():
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(HERE, "golden", "make_golden.py"))
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    return m


def test_stack_matches_committed_outputs(oracle, golden_mod):
    gold = np.load(os.path.join(HERE, "golden", "stack_golden.npz"))
    for name in golden_mod.STACK_CASES:
        cfg, x, c = golden_mod.stack_case(name)
        got = oracle.stack_forward(cfg, x, c["B"], c["S"])
        assert np.allclose(got, gold[name], rtol=1e-5, atol=1e-5), name


def test_stack_matches_numpy_restatement(oracle, golden_mod):
    for name in golden_mod.STACK_CASES:
        cfg, x, c = golden_mod.stack_case(name)
        got = oracle.stack_forward(cfg, x, c["B"], c["S"])
        want = np_stack(oracle, c, x, c["B"], c["S"])
        assert np.abs(got - want).max() / np.abs(want).max() < 1e-4, name


def test_stack_is_invariant_under_tensor_parallel_degree(oracle, golden_mod):
    cfg, x, c = golden_mod.stack_case("preln_gelu_causal_tp1")
    outs = []
    for tp in (1, 2, 4):
        cfg.tp = tp
        outs.append(oracle.stack_forward(cfg, x, c["B"], c["S"]))
    for o in outs[1:]:
        assert np.abs(o - outs[0]).max() / np.abs(outs[0]).max() < 1e-5


def test_fp16_rounding_of_intermediates_stays_within_tolerance(oracle, golden_mod):
    cfg, x, c = golden_mod.stack_case("preln_geglu_causal_tp2")
    exact = oracle.stack_forward(cfg, x, c["B"], c["S"])
    cfg.round16 = 1
    rounded = oracle.stack_forward(cfg, x, c["B"], c["S"])
    err = np.abs(rounded - exact).max() / np.abs(exact).max()
    assert 0 < err < 1e-2
