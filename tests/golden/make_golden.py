"""Regenerates the committed fixtures in this directory from the CPU oracle:

    python tests/golden/make_golden.py

rng_golden.json   values of the seeded generator (include/liger_rng.h) at fixed (seed, tensor, index)
stack_golden.npz  outputs of oracle.stack_forward for small configurations of both graphs

The reference itself ships no golden vectors (its tests only time launches over uninitialised memory),
so these pin the oracle and the generator against regressions, not against the reference."""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
import oracle  # noqa: E402

STACK_CASES = {
    "ref_gelu_tp2": dict(hidden=64, heads=4, head_dim=16, ffn_inner=256, layers=2, tp=2, graph=0, act=0, causal=0, B=2, S=8),
    "preln_gelu_causal_tp1": dict(hidden=64, heads=4, head_dim=16, ffn_inner=128, layers=2, tp=1, graph=1, act=0, causal=1, B=2, S=8),
    "preln_geglu_causal_tp2": dict(hidden=64, heads=2, head_dim=32, ffn_inner=128, layers=1, tp=2, graph=1, act=1, causal=1, B=1, S=12),
}


def stack_case(name):
    c = STACK_CASES[name]
    cfg = oracle.Config(hidden=c["hidden"], heads=c["heads"], head_dim=c["head_dim"], ffn_inner=c["ffn_inner"],
                        layers=c["layers"], tp=c["tp"], graph=c["graph"], act=c["act"], causal=c["causal"], round16=0, seed=0)
    M = c["B"] * c["S"]
    x = oracle.fill_normal(M * c["hidden"], 0, oracle.INPUT).reshape(M, c["hidden"])
    return cfg, x, c


def main():
    oracle.build()
    rng = []
    for seed, tid, idx0 in [(0, 0, 0), (0, 5, 1000), (7, 0x10000, 123456789), (1, 33, (1 << 33) + 5)]:
        bits = oracle.fill_normal_f16(8, seed, tid, idx0, 0.0, 1.0).view(np.uint16).tolist()
        rng.append(dict(seed=seed, tensor_id=tid, idx0=idx0, mean=0.0, std=1.0, fp16_bits=bits))
    bits = oracle.fill_normal_f16(8, 0, 4, 0, 1.0, 0.02).view(np.uint16).tolist()
    rng.append(dict(seed=0, tensor_id=4, idx0=0, mean=1.0, std=0.02, fp16_bits=bits))
    with open(os.path.join(HERE, "rng_golden.json"), "w") as f:
        json.dump(rng, f, indent=1)
    out = {}
    for name in STACK_CASES:
        cfg, x, c = stack_case(name)
        out[name] = oracle.stack_forward(cfg, x, c["B"], c["S"])
    np.savez_compressed(os.path.join(HERE, "stack_golden.npz"), **out)
    print("wrote", sorted(os.listdir(HERE)))


if __name__ == "__main__":
    main()
