"""Committed golden vectors (tests/golden/linear_cases.npz, written by tests/golden/make_golden.py):
the CPU reference port must still reproduce them bit for bit, and the CUDA path is compared with
the committed outputs, not only with a reference port that runs beside it."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(__file__), ".."))

from oracle import oracle as orc  # noqa: E402
from tritium_b200.format import SaltV2Codec, SaltV2Tensor  # noqa: E402

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "linear_cases.npz")
NAMES = ["decode_p1", "decode_p3", "prefill_p2", "prefill_p3"]


def load(name):
    z = np.load(GOLDEN)
    case = {k.split(".", 1)[1]: z[k] for k in z.files if k.startswith(name + ".")}
    rows, cols, planes, tokens = (int(v) for v in case["shape"])
    return case, rows, cols, planes, tokens


def rel_l2(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    return float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))


@pytest.mark.parametrize("name", NAMES)
def test_reference_port_reproduces_the_committed_vectors(name):
    case, rows, cols, planes, tokens = load(name)
    o = orc.Tensor(rows, cols, 128, case["plane_count"].copy(), case["trits"].copy(), case["scales"].copy())
    y, acc, act_scale = orc.a8_linear(o, case["x"])
    assert np.array_equal(acc[..., :planes], case["a8_acc"])
    assert np.array_equal(y.view(np.uint32), case["a8_y"].view(np.uint32))
    assert np.array_equal(act_scale.view(np.uint32), case["a8_act_scale"].view(np.uint32))
    exact = orc.matmul(o, case["x"], 1)
    assert np.array_equal(exact.view(np.uint32), case["exact_y_bits"])


@pytest.fixture(scope="module")
def backend():
    from tritium_b200 import B200Backend
    b = B200Backend(0)
    yield b
    b.close()


@pytest.mark.gpu
@pytest.mark.parametrize("codec", [SaltV2Codec.B3, SaltV2Codec.D2])
@pytest.mark.parametrize("name", NAMES)
def test_cuda_path_matches_the_committed_vectors(backend, name, codec):
    case, rows, cols, planes, tokens = load(name)
    t = SaltV2Tensor("w", rows, cols, case["plane_count"], case["trits"], case["scales"])
    resident = backend.upload_salt_v2(t, codec)
    y, acc, receipt = backend.linear_forward_a8(resident, case["x"], tokens, dump=True)
    assert receipt.kernel == (2 if tokens > 8 else 1)
    assert np.array_equal(acc, case["a8_acc"])                  # int32 group sums: bit exact
    assert rel_l2(y, case["a8_y"]) <= 1e-5                      # fp32 outputs
    out = np.zeros((tokens, rows), np.float32)
    backend.salt_v2_forward_exact_into(resident, case["x"], tokens, out)
    assert np.array_equal(out.view(np.uint32), case["exact_y_bits"])   # sequential-f32 order: bit identical
