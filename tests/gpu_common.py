"""Helpers shared by the GPU parity tests: seeded tensors in product and oracle form, sampled
sub-tensors for the CPU oracle, exact integer group sums with numpy."""
import os

import numpy as np

from oracle import oracle as orc
from tritium_b200.format import SaltV2Tensor
from tritium_b200.synth import make_planes

THREADS = max(1, min(16, os.cpu_count() or 1))


def rel_l2(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    return float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))


def uniform_pair(n, k, planes, seed):
    """(product tensor, oracle tensor) of one seeded uniform-plane [n, k] matrix; the product
    tensor keeps the dense planes in ``raw`` = (trits[P,N,K], scales[P,N,K/128])."""
    trits, scales = make_planes(n, k, planes, seed=seed)
    prod = SaltV2Tensor.from_matrix_planes("w", trits, scales)
    prod.raw = (trits, scales)
    return prod, orc.Tensor(n, k, 128, prod.plane_count.copy(), prod.trits.copy(), prod.scales.copy())


def product_only(n, k, planes, seed):
    trits, scales = make_planes(n, k, planes, seed=seed)
    prod = SaltV2Tensor.from_matrix_planes("w", trits, scales)
    prod.raw = (trits, scales)
    return prod


def oracle_rows(prod, rows):
    """Oracle tensor holding only `rows` of a uniform-plane product tensor (k % 256 == 0)."""
    n, k = prod.rows, prod.cols
    tpr = k // 256
    rows = np.asarray(rows)
    return orc.Tensor(len(rows), k, 128, prod.plane_count.reshape(n, tpr)[rows].reshape(-1).copy(),
                      prod.trits.reshape(n, tpr, 3, 256)[rows].reshape(-1, 3, 256).copy(),
                      prod.scales.reshape(n, tpr, 3, -1)[rows].reshape(-1, 3, prod.scales.shape[-1]).copy())


def sample_rows(n, count=8):
    """First, middle and last rows of an n-row tensor."""
    count = min(count, max(1, n // 3))
    return np.unique(np.r_[0:count, n // 2:n // 2 + count, n - count:n])


def exact_group_sums(trits_pnk, q):
    """int32 [m, n, k/128, P]: sum over each 128-wide group of trit * code, computed with fp32
    matrix products that are exact here (every sum is an integer below 2^24)."""
    p, n, k = trits_pnk.shape
    m, groups = q.shape[0], k // 128
    out = np.zeros((m, n, groups, p), np.int32)
    qf = np.ascontiguousarray(q, np.float32).reshape(m, groups, 128)
    for pl in range(p):
        t = trits_pnk[pl].astype(np.float32).reshape(n, groups, 128)
        for g in range(groups):
            out[:, :, g, pl] = np.rint(qf[:, g, :] @ t[:, g, :].T).astype(np.int32)
    return out
