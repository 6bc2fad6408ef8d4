"""Regenerates bench_glm130b_rows.npz, the rows bench.py checks its own output against:

    python tests/golden/make_bench_rows.py            (about two minutes on 8 cores)

The benchmark's configurations are too large for the CPU oracle as a whole, but they do not have to be run as a
whole.  Prefill (GLM-130B shape, 4 layers, pre-LayerNorm + residual, GeGLU 32768, causal, batch 8 x sequence
512): sequences are independent and attention is causal, so the first PREFILL_TOKENS rows of the result depend
only on the first PREFILL_TOKENS rows of the seeded input -- the oracle runs on batch 1 x sequence
PREFILL_TOKENS and PREFILL_ROWS of its output rows are kept.  Decode (same layers, one new token against a
seeded KV cache of DECODE_KV_LEN positions): sequences are independent, so the oracle runs the first
DECODE_SEQS sequences.  Everything is a pure function of (seed 0, tensor id, element index), the same
generator the library uses on the device, so bench.py at any tensor-parallel degree must reproduce these rows
within the 1e-2 relative bound of the parity tests.
"""
import os
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
import oracle  # noqa: E402

GLM = dict(hidden=12288, heads=96, head_dim=128, ffn_inner=32768, layers=4)
PREFILL_TOKENS = 128
PREFILL_ROWS = np.unique(np.round(np.linspace(0, PREFILL_TOKENS - 1, 32)).astype(np.int64))
DECODE_SEQS = 4
DECODE_KV_LEN = 2048
DECODE_KV_CAPACITY = 2112
OUT = os.path.join(HERE, "bench_glm130b_rows.npz")


def main():
    oracle.build()
    H = GLM["hidden"]
    cfg = oracle.Config(hidden=H, heads=GLM["heads"], head_dim=GLM["head_dim"], ffn_inner=GLM["ffn_inner"], layers=GLM["layers"],
                        tp=1, graph=1, act=1, causal=1, round16=0, seed=0)
    t0 = time.time()
    x = oracle.fill_normal(PREFILL_TOKENS * H, 0, oracle.INPUT).reshape(PREFILL_TOKENS, H)
    prefill = oracle.stack_forward(cfg, x, 1, PREFILL_TOKENS)
    print(f"prefill rows: {time.time() - t0:.1f} s", flush=True)
    t0 = time.time()
    xd = oracle.fill_normal(DECODE_SEQS * H, 0, oracle.INPUT).reshape(DECODE_SEQS, H)
    decode = oracle.stack_decode(cfg, xd, DECODE_SEQS, DECODE_KV_LEN, DECODE_KV_CAPACITY)
    print(f"decode rows: {time.time() - t0:.1f} s", flush=True)
    np.savez(OUT, prefill_rows=PREFILL_ROWS, prefill=prefill[PREFILL_ROWS].astype(np.float16),
             prefill_scale=np.float32(np.abs(prefill).max()), decode=decode.astype(np.float16),
             decode_kv_len=np.int64(DECODE_KV_LEN), decode_kv_capacity=np.int64(DECODE_KV_CAPACITY))
    print("wrote", OUT, os.path.getsize(OUT), "bytes")


if __name__ == "__main__":
    main()
