"""Writes the committed golden fixtures of the packed ternary linear path.

Run from the repository root:  python tests/golden/make_golden.py

Every case is a small seeded problem: the semantic tensor (trits, f16 scale bits, plane counts),
the activations, and the CPU reference port's outputs — the sequential-f32 `salt_v2_matvec_into`
result (bit patterns), and for the int8-activation path the per-token scales, the exact int32
group sums and the fp32 outputs.  The reference itself is a Rust workspace and cannot be run where
these files are made, so the generator is the C restatement under `oracle/`, which
`tests/test_oracle_golden.py` pins to the reference's own known-answer vectors first.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import oracle as orc  # noqa: E402
from tritium_b200.synth import make_activations, make_planes  # noqa: E402
from tritium_b200.format import SaltV2Tensor  # noqa: E402

CASES = [
    # name, rows, cols, planes, tokens, seed
    ("decode_p1", 24, 512, 1, 1, 101),
    ("decode_p3", 40, 768, 3, 4, 102),
    ("prefill_p2", 136, 512, 2, 33, 103),
    ("prefill_p3", 128, 256, 3, 130, 104),
]


def build(rows, cols, planes, tokens, seed):
    trits, scales = make_planes(rows, cols, planes, seed=seed)
    t = SaltV2Tensor.from_matrix_planes("w", trits, scales)
    o = orc.Tensor(rows, cols, 128, t.plane_count.copy(), t.trits.copy(), t.scales.copy())
    x = make_activations(tokens, cols, seed=seed, bf16=True)
    y, acc, act_scale = orc.a8_linear(o, x)
    exact = orc.matmul(o, x, 1) if hasattr(orc, "matmul") else np.stack([orc.matvec(o, x[i]) for i in range(tokens)])
    return dict(plane_count=t.plane_count, trits=t.trits, scales=t.scales, x=x, a8_y=y, a8_acc=acc[..., :planes],
                a8_act_scale=act_scale, exact_y_bits=np.ascontiguousarray(exact, np.float32).view(np.uint32))


def main():
    out = {}
    for name, rows, cols, planes, tokens, seed in CASES:
        for key, value in build(rows, cols, planes, tokens, seed).items():
            out[f"{name}.{key}"] = value
        out[f"{name}.shape"] = np.array([rows, cols, planes, tokens], np.int64)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "linear_cases.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
