"""Writes tests/golden/*.npz from the CPU oracle.

The reference cannot run here (Rust, no toolchain) and stores no expected outputs for this path:
its tests recompute them with a scalar loop (nn/moe.rs:2101-2175).  These fixtures hold that
loop's restatement (oracle, left-to-right sums) on the reference's own toy construction, plus the
known-answer vectors the reference's tests spell out as literals.  Run from the repo root:
    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, HERE)

import toy  # noqa: E402
from oracle import oracle as O  # noqa: E402
from mummu_b200 import q4k, synth  # noqa: E402


def main():
    rw = toy.router()
    g, u, d = toy.banks()
    out = {}
    for t, seed, norm in [(5, 2.0, False), (5, 2.0, True), (1, 2.0, False), (1, 2.0, True),
                          (5, 7.0, False), (5, 7.0, True), (3, 0.5, False)]:
        x = toy.inputs(t, seed)
        k = toy.EXPERTS if (t, seed) == (3, 0.5) else toy.TOP_K
        logits = O.router_logits(x, rw, order=O.SUM_SEQUENTIAL)
        ids, w = O.route(logits, k, norm, exp_kind=1)
        y = O.moe_routed(x, ids, w, g, u, d, toy.HIDDEN, toy.INTER, toy.EXPERTS,
                         order=O.SUM_SEQUENTIAL)
        key = f"t{t}_s{seed}_n{int(norm)}_k{k}"
        out[key + "_ids"], out[key + "_w"], out[key + "_y"] = ids, w, y
    np.savez(os.path.join(HERE, "toy_moe.npz"), **out)

    # a small Q4_K layer: bytes, their exact decode, routing and outputs (8-lane sums)
    H, I, E, T, K = 256, 256, 4, 5, 2
    router, gate, up, down, x = synth.moe_layer(H, I, E, T, cfg_seed=7)
    x = x.astype(np.float16).astype(np.float32)
    gq, uq, dq = (q4k.quantize(b) for b in (gate, up, down))
    y, ids, w = O.moe_forward(x, router, gq, uq, dq, K, False, q4k=True)
    np.savez_compressed(os.path.join(HERE, "q4k_small.npz"), router=router, x=x, gate_q=gq, up_q=uq, down_q=dq,
             gate_deq_rows=O.dequant_q4_k(gq[: 4 * 144]), ids=ids, w=w, y=y)
    print("wrote", sorted(os.listdir(HERE)))


if __name__ == "__main__":
    main()
