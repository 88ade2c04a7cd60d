"""GPU parity: the CUDA path, called through the C ABI, against the CPU oracle on the same inputs."""
import numpy as np
import pytest

from oracle import oracle as orc
from tritium_b200 import errors
from tritium_b200 import format as fmt
from tritium_b200.format import SaltV2Codec, SaltV2Tensor
from tritium_b200.synth import bf16_bits_to_f32, f32_to_bf16_bits, make_activations, make_planes

pytestmark = pytest.mark.gpu

CODECS = [(SaltV2Codec.D2, orc.D2), (SaltV2Codec.B3, orc.B3), (SaltV2Codec.S34, orc.S34)]


@pytest.fixture(scope="module")
def backend():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device: there is no CPU path to fall back to")
    from tritium_b200 import B200Backend
    b = B200Backend(0)
    yield b
    b.close()


def f16(v):
    return orc.f32_to_f16(float(np.float32(v)))


def cuda_test_plane(length, plane_index):
    """salt_v2_test_plane (crates/tritium-cuda/src/cuda/tests.rs:67-88): one zero per four (valid S34)."""
    trits = []
    for i in range(length):
        group, slot = divmod(i, 4)
        trits.append(0 if slot == (group + plane_index) % 4 else (1 if (i + plane_index) % 2 == 0 else -1))
    scales = [f16(np.float32(0.25) + np.float32(plane_index) * np.float32(0.125) + np.float32(g) * np.float32(0.0625))
              for g in range((length + 127) // 128)]
    return trits, scales


def cuda_test_tensor(rows, cols, counts):
    coeffs = rows * cols
    tiles = []
    for t, c in enumerate(counts):
        length = min(256, coeffs - t * 256)
        tiles.append([cuda_test_plane(length, p) for p in range(c)])
    return orc.tensor_from_planes(rows, cols, tiles)


def seeded_f32(seed, n, lo, hi):
    """seeded_f32 (crates/tritium-cuda/src/cuda/tests.rs:55-65)."""
    s, out = seed | 1, np.zeros(n, np.float32)
    for i in range(n):
        s ^= (s << 13) & 0xFFFFFFFFFFFFFFFF
        s ^= s >> 7
        s ^= (s << 17) & 0xFFFFFFFFFFFFFFFF
        out[i] = np.float32(lo) + np.float32(s % 1000) / np.float32(1000.0) * np.float32(hi - lo)
    return out


def as_product(t: orc.Tensor, name="w") -> SaltV2Tensor:
    return SaltV2Tensor(name, t.rows, t.cols, t.plane_count.copy(), t.trits.copy(), t.scales.copy(), t.group)


def rel_l2(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    return float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))


# ------------------------------------------------------------------ exact kernel
# crates/tritium-cuda/src/cuda/tests.rs:419-563: GPU output bits == CPU oracle bits
CASES = [(3, 173, [1, 3, 2]), (2, 3, [3]), (1, 1, [1]), (1, 1025 * 256, [1 + i % 3 for i in range(1025)])]


@pytest.mark.parametrize("codec,ocodec", CODECS)
@pytest.mark.parametrize("case", CASES, ids=["3x173", "2x3", "1x1", "1025tiles"])
def test_exact_forward_is_bit_identical_to_cpu_reference(backend, codec, ocodec, case):
    rows, cols, counts = case
    t = cuda_test_tensor(rows, cols, counts)
    m = 2
    x = seeded_f32(0x5A17 + rows * 257 + cols, m * cols, -0.75, 0.75).reshape(m, cols)
    want = np.stack([orc.matvec(t, x[i]) for i in range(m)])
    prod = as_product(t, f"salt-v2-{rows}x{cols}")
    resident = backend.upload_salt_v2(prod, codec)
    streamed = backend.upload_salt_v2_from_package(fmt.write_salt_v2_package(prod, codec), prod.name)
    exact = backend.salt_v2_forward_exact(resident, x, m)
    assert np.array_equal(exact.output.view(np.uint32), want.view(np.uint32))
    again = backend.salt_v2_forward_exact(streamed, x, m)
    assert np.array_equal(again.output.view(np.uint32), want.view(np.uint32))
    fast = backend.salt_v2_forward_fast(resident, x, m)
    assert rel_l2(fast.output, want) <= 1e-5
    plan = orc.resident_plan(t, ocodec)
    alloc = resident.allocation_receipt()
    assert alloc["payload_bytes"] == plan["payload_bytes"] and alloc["scale_bytes"] == plan["scale_bytes"]
    assert alloc["map_bytes"] == len(counts) * 2 // 8 and alloc["rank_prefix_bytes"] == (len(counts) - 1) // 256 * 4
    assert alloc["dense_weight_bytes"] == 0 and exact.receipt.dense_weight_bytes == 0
    assert exact.receipt.activation_bytes == m * cols * 4 and exact.receipt.output_bytes == m * rows * 4


@pytest.mark.parametrize("codec,ocodec", CODECS)
def test_exact_forward_g64_and_straddling_rows(backend, codec, ocodec):
    tiles = []
    for ti in range(9):
        trits = [{0: 0, 1: 1, 2: 1, 3: -1}[(i + ti) % 4] for i in range(256)]
        tiles.append([(trits, [f16(np.float32(0.125) + np.float32(ti * 4 + g) / np.float32(64.0)) for g in range(4)])])
    t = orc.tensor_from_planes(4, 576, tiles, group=64)
    x = ((np.arange(576, dtype=np.float32) - np.float32(283.0)) / np.float32(71.0)).astype(np.float32)
    want = orc.matvec(t, x)
    resident = backend.upload_salt_v2(as_product(t), codec)
    got = backend.salt_v2_forward_exact(resident, x, 1).output[0]
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_exact_forward_rejects_nonfinite_without_touching_output(backend):
    t = cuda_test_tensor(3, 173, [1, 3, 2])
    resident = backend.upload_salt_v2(as_product(t), SaltV2Codec.D2)
    x = np.zeros(173, np.float32)
    x[71] = np.nan
    out = np.full((1, 3), 7.0, np.float32)
    with pytest.raises(errors.InvalidInput):
        backend.salt_v2_forward_exact_into(resident, x, 1, out)
    assert np.all(out == 7.0)
    big = orc.tensor_from_planes(1, 1, [[([1], [0x7BFF])]])
    r2 = backend.upload_salt_v2(as_product(big), SaltV2Codec.D2)
    out = np.full((1, 1), 19.0, np.float32)
    with pytest.raises(errors.InvalidInput):
        backend.salt_v2_forward_exact_into(r2, np.array([np.finfo(np.float32).max], np.float32), 1, out)
    assert out[0, 0] == 19.0
    cancel = orc.tensor_from_planes(1, 2, [[([1, -1], [0x7BFF])]])
    r3 = backend.upload_salt_v2(as_product(cancel), SaltV2Codec.D2)
    fm = np.finfo(np.float32).max
    assert backend.salt_v2_forward_exact(r3, np.array([fm, fm], np.float32), 1).output[0, 0] == 0.0
    with pytest.raises(errors.ShapeMismatch):
        backend.salt_v2_forward_exact(resident, np.zeros(172, np.float32), 1)


def test_upload_rejects_bad_arenas(backend):
    t = cuda_test_tensor(3, 173, [1, 3, 2])
    payload, scales, pmap, terminal, _ = as_product(t).resident(SaltV2Codec.B3)
    with pytest.raises(errors.ShapeMismatch):
        backend.upload_salt_v2_arenas(SaltV2Codec.B3, 128, 3, 173, payload[:-1], scales, pmap, terminal)
    bad = payload.copy()
    bad[0] = 250
    with pytest.raises(errors.InvalidInput):
        backend.upload_salt_v2_arenas(SaltV2Codec.B3, 128, 3, 173, bad, scales, pmap, terminal)
    with pytest.raises(errors.InvalidInput):
        backend.upload_salt_v2_arenas(SaltV2Codec.B3, 32, 3, 173, payload, scales, pmap, terminal)


def test_gather_rows_matches_reference(backend):
    t = cuda_test_tensor(3, 173, [1, 3, 2])
    resident = backend.upload_salt_v2(as_product(t), SaltV2Codec.B3)
    out = np.zeros((2, 173), np.float32)
    backend.salt_v2_gather_rows(resident, [2, 0], out)
    assert np.array_equal(out, orc.gather_rows(t, [2, 0]))
    with pytest.raises(errors.InvalidInput):
        backend.salt_v2_gather_rows(resident, [3], np.zeros((1, 173), np.float32))


# ------------------------------------------------------------------ int8 path (decode kernel)
def uniform_pair(n, k, planes, seed):
    trits, scales = make_planes(n, k, planes, seed=seed)
    prod = SaltV2Tensor.from_matrix_planes("w", trits, scales)
    prod.raw = (trits, scales)
    return prod, orc.Tensor(n, k, 128, prod.plane_count.copy(), prod.trits.copy(), prod.scales.copy())


@pytest.mark.parametrize("codec", [SaltV2Codec.B3, SaltV2Codec.D2])
@pytest.mark.parametrize("planes", [1, 2, 3])
@pytest.mark.parametrize("m", [1, 2, 3, 4, 7])
def test_a8_decode_small_shapes(backend, codec, planes, m):
    n, k = 40, 768   # n is not a multiple of the row block: exercises the padded tail
    prod, orac = uniform_pair(n, k, planes, seed=planes * 10 + m)
    x = make_activations(m, k, seed=m)
    want_y, want_acc, want_scale = orc.a8_linear(orac, x)
    resident = backend.upload_salt_v2(prod, codec)
    y, acc, receipt = backend.linear_forward_a8(resident, x, m, dump=True)
    assert np.array_equal(acc, want_acc[:, :, :, :planes])      # int32 accumulators: bit exact
    assert rel_l2(y, want_y) <= 1e-5                            # fp32 outputs: 1e-5 relative L2
    assert receipt.kernel == 1 and receipt.dense_weight_bytes == 0


def test_a8_extreme_activations_stay_exact(backend):
    n, k = 16, 512
    prod, orac = uniform_pair(n, k, 3, seed=5)
    prod.trits[:, 0, :] = 1
    orac.trits[:, 0, :] = 1
    for fill in (1.0, -1.0):
        x = np.full((1, k), fill, np.float32)           # every code is +-127: largest group sums
        want_y, want_acc, _ = orc.a8_linear(orac, x)
        for codec in (SaltV2Codec.B3, SaltV2Codec.D2):
            resident = backend.upload_salt_v2(prod, codec)
            y, acc, _ = backend.linear_forward_a8(resident, x, 1, dump=True)
            assert np.array_equal(acc, want_acc) and rel_l2(y, want_y) <= 1e-5
    x = np.zeros((2, k), np.float32)
    x[1, 3] = 2.5                                       # a zero row quantises to zeros with a zero scale
    want_y, want_acc, _ = orc.a8_linear(orac, x)
    y, acc, _ = backend.linear_forward_a8(backend.upload_salt_v2(prod, SaltV2Codec.B3), x, 2, dump=True)
    assert np.array_equal(acc, want_acc) and np.all(y[0] == 0) and rel_l2(y, want_y) <= 1e-5


@pytest.mark.parametrize("codec", [SaltV2Codec.B3, SaltV2Codec.D2])
def test_a8_bf16_in_and_out(backend, codec):
    n, k, planes, m = 64, 1024, 3, 4
    prod, orac = uniform_pair(n, k, planes, seed=21)
    x = make_activations(m, k, seed=3, bf16=True)
    want_y, want_acc, _ = orc.a8_linear(orac, x)
    resident = backend.upload_salt_v2(prod, codec)
    y_bits, acc, _ = backend.linear_forward_a8(resident, f32_to_bf16_bits(x), m, y_dtype="bf16", dump=True, x_is_bf16=True)
    assert np.array_equal(acc, want_acc)
    assert rel_l2(bf16_bits_to_f32(y_bits), want_y) <= 1e-2     # bf16 outputs: 1e-2 relative L2


CONFIGS = {
    "c1_k2048_n8192_p1": (8192, 2048, 1),
    "c2_k2560_n6912_p3": (6912, 2560, 3),
}


@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("codec", [SaltV2Codec.B3, SaltV2Codec.D2])
def test_a8_decode_full_size_configs(backend, name, codec):
    n, k, planes = CONFIGS[name]
    prod, orac = uniform_pair(n, k, planes, seed=0)
    for m in (1, 4):
        x = make_activations(m, k, seed=0, bf16=True)
        want_y, want_acc, _ = orc.a8_linear(orac, x)
        resident = backend.upload_salt_v2(prod, codec)
        y, acc, receipt = backend.linear_forward_a8(resident, x, m, dump=True)
        assert np.array_equal(acc, want_acc[:, :, :, :planes])
        assert rel_l2(y, want_y) <= 1e-5
        # linearity in the weights' planes: the output is the sum of the per-plane outputs
        if m == 1 and planes > 1:
            total = np.zeros_like(want_y, dtype=np.float64)
            for p in range(planes):
                single = SaltV2Tensor.from_matrix_planes("p", prod.raw[0][p:p + 1], prod.raw[1][p:p + 1])
                rp = backend.upload_salt_v2(single, codec)
                yp, _, _ = backend.linear_forward_a8(rp, x, 1)
                total += yp.astype(np.float64)
            assert rel_l2(total, want_y) <= 1e-5


# ------------------------------------------------------------------ int8 path (prefill kernel, tcgen05)
@pytest.mark.parametrize("codec", [SaltV2Codec.B3, SaltV2Codec.D2])
@pytest.mark.parametrize("planes", [1, 2, 3])
@pytest.mark.parametrize("m,n,k", [(17, 40, 768), (20, 128, 256), (130, 200, 1024), (257, 129, 512)])
def test_a8_prefill_small_shapes(backend, codec, planes, m, n, k):
    prod, orac = uniform_pair(n, k, planes, seed=planes * 100 + m)
    x = make_activations(m, k, seed=m)
    want_y, want_acc, _ = orc.a8_linear(orac, x)
    resident = backend.upload_salt_v2(prod, codec)
    y, acc, receipt = backend.linear_forward_a8(resident, x, m, dump=True)
    assert receipt.kernel == 2                                  # the tensor-core kernel ran
    assert np.array_equal(acc, want_acc[:, :, :, :planes])      # int32 accumulators: bit exact
    assert rel_l2(y, want_y) <= 1e-5
    # two calls in a row give identical bits (no state left behind in the scratch or in TMEM)
    y2, _, _ = backend.linear_forward_a8(resident, x, m)
    assert np.array_equal(y, y2)


def test_a8_prefill_extreme_activations_stay_exact(backend):
    n, k, m = 130, 512, 32
    prod, orac = uniform_pair(n, k, 3, seed=5)
    prod.trits[:, 0, :] = 1
    orac.trits[:, 0, :] = 1
    x = np.ones((m, k), np.float32)
    x[1::2] = -1.0                                      # every code is +-127: largest group sums
    x[5] = 0.0                                          # a zero row: zero codes, zero scale
    want_y, want_acc, _ = orc.a8_linear(orac, x)
    for codec in (SaltV2Codec.B3, SaltV2Codec.D2):
        y, acc, _ = backend.linear_forward_a8(backend.upload_salt_v2(prod, codec), x, m, dump=True)
        assert np.array_equal(acc, want_acc) and np.all(y[5] == 0) and rel_l2(y, want_y) <= 1e-5


@pytest.mark.parametrize("codec", [SaltV2Codec.B3, SaltV2Codec.D2])
def test_a8_prefill_bf16_in_and_out(backend, codec):
    n, k, planes, m = 192, 1024, 3, 48
    prod, orac = uniform_pair(n, k, planes, seed=22)
    x = make_activations(m, k, seed=4, bf16=True)
    want_y, want_acc, _ = orc.a8_linear(orac, x)
    resident = backend.upload_salt_v2(prod, codec)
    y_bits, acc, _ = backend.linear_forward_a8(resident, f32_to_bf16_bits(x), m, y_dtype="bf16", dump=True, x_is_bf16=True)
    assert np.array_equal(acc, want_acc)
    assert rel_l2(bf16_bits_to_f32(y_bits), want_y) <= 1e-2


@pytest.mark.parametrize("codec", [SaltV2Codec.B3, SaltV2Codec.D2])
def test_a8_prefill_full_size_config(backend, codec):
    """K=2560, N=6912, three planes, 2048 tokens: sampled rows against the CPU reference, and the
    first tokens against the (already pinned) decode kernel on every row."""
    n, k, planes, m = 6912, 2560, 3, 2048
    prod, _ = uniform_pair(n, k, planes, seed=0)
    x = make_activations(m, k, seed=1, bf16=True)
    resident = backend.upload_salt_v2(prod, codec)
    y, _, receipt = backend.linear_forward_a8(resident, x, m)
    assert receipt.kernel == 2
    rows = np.r_[0:8, 3451:3459, n - 8:n]
    sub = orc.Tensor(len(rows), k, 128, prod.plane_count.reshape(n, -1)[rows].reshape(-1).copy(),
                     prod.trits.reshape(n, k // 256, 3, 256)[rows].reshape(-1, 3, 256).copy(),
                     prod.scales.reshape(n, k // 256, 3, -1)[rows].reshape(-1, 3, prod.scales.shape[-1]).copy())
    tokens = np.r_[0:4, 1021:1027, m - 4:m]
    want_y, _, _ = orc.a8_linear(sub, x[tokens])
    assert rel_l2(y[np.ix_(tokens, rows)], want_y) <= 1e-5
    y_dec, _, r_dec = backend.linear_forward_a8(resident, x[:4], 4)
    assert r_dec.kernel == 1 and rel_l2(y[:4], y_dec) <= 1e-5


def test_a8_prefill_sweep_shape_full_accumulator_check(backend):
    """Prefill sweep shape (K=2560, N=2560, one plane) at 512 tokens: every int32 group sum and
    every output against the CPU reference, bf16 outputs."""
    n, k, planes, m = 2560, 2560, 1, 512
    prod, orac = uniform_pair(n, k, planes, seed=3)
    x = make_activations(m, k, seed=2, bf16=True)
    want_y, want_acc, _ = orc.a8_linear(orac, x)
    resident = backend.upload_salt_v2(prod, SaltV2Codec.B3)
    y_bits, acc, receipt = backend.linear_forward_a8(resident, f32_to_bf16_bits(x), m, y_dtype="bf16", dump=True, x_is_bf16=True)
    assert receipt.kernel == 2
    assert np.array_equal(acc, want_acc[:, :, :, :planes])
    assert rel_l2(bf16_bits_to_f32(y_bits), want_y) <= 1e-2


@pytest.mark.parametrize("n,k", [(3840, 2560), (13824, 2560), (2560, 6912)], ids=["qkv", "gate_up", "down"])
def test_a8_decoder_stack_shapes_batch16(backend, n, k):
    """2B-class decoder linears (one plane) at decode batch 16: sampled rows against the reference."""
    planes, m = 1, 16
    prod, _ = uniform_pair(n, k, planes, seed=n % 97)
    x = make_activations(m, k, seed=6, bf16=True)
    resident = backend.upload_salt_v2(prod, SaltV2Codec.B3)
    y, _, _ = backend.linear_forward_a8(resident, x, m)
    rows = np.r_[0:6, n // 2:n // 2 + 6, n - 6:n]
    sub = orc.Tensor(len(rows), k, 128, prod.plane_count.reshape(n, -1)[rows].reshape(-1).copy(),
                     prod.trits.reshape(n, k // 256, 3, 256)[rows].reshape(-1, 3, 256).copy(),
                     prod.scales.reshape(n, k // 256, 3, -1)[rows].reshape(-1, 3, prod.scales.shape[-1]).copy())
    want_y, _, _ = orc.a8_linear(sub, x)
    assert rel_l2(y[:, rows], want_y) <= 1e-5


# ------------------------------------------------------------------ trait path (TQ2_0 conformance)
def conformance_vectors(seed=0xC0FFEE, count=12):
    """generate_vectors (crates/tritium-testkit/src/generate.rs:203-233), TQ2_0 cases only."""
    rng = orc.XorShift64(seed)
    out = []
    for i in range(count):
        rng.perturb(i)
        m, n, k = 1 + rng.below(64), 1 + rng.below(32), 256 * (1 + rng.below(2))
        act = np.array([rng.activation() for _ in range(m * k)], np.float32)
        w = np.array([rng.trit() for _ in range(n * k)], np.int8).reshape(n, k)
        scales = np.array([rng.scale() for _ in range(n)], np.float32)
        if i % 2 == 0:
            out.append((f"rand-{i}", m, n, k, act, w, scales))
    return out


def boundary_vectors():
    """boundary_vectors (generate.rs:108-201): all-zero / all-plus / mixed weights at edge shapes."""
    rng = orc.XorShift64(0xB0117DA47)
    out = []
    for si, (m, n, k) in enumerate([(1, 1, 256), (1, 32, 256), (64, 1, 256), (64, 32, 512), (1, 1, 512)]):
        act = np.array([rng.activation() for _ in range(m * k)], np.float32)
        scales = np.array([rng.scale() for _ in range(n)], np.float32)
        out.append((f"boundary-{si}-allzero", m, n, k, act, np.zeros((n, k), np.int8), scales))
        out.append((f"boundary-{si}-allpos", m, n, k, act, np.ones((n, k), np.int8), scales))
        mixed = np.array([rng.trit() for _ in range(n * k)], np.int8).reshape(n, k)
        out.append((f"boundary-{si}-mixed-tq2", m, n, k, act, mixed, scales))
    return out


def accepts(got, want, relative=1e-4, floor=1.0):
    """Tolerance::accepts_with_floor (crates/tritium-testkit/src/vector.rs:113-126)."""
    return np.all(np.abs(got - want) <= relative * np.maximum(floor, np.abs(want)))


def test_trait_path_conformance(backend):
    from tritium_b200 import GemmShape, MpGemm, TernaryFormat
    for vid, m, n, k, act, w, scales in conformance_vectors() + boundary_vectors():
        packed = fmt.pack_tq2_0_rows(w)
        buf = backend.upload_weights(packed, GemmShape(0, n, k), TernaryFormat.Tq2_0)
        assert buf.len_bytes() == n * (k // 256) * 66
        want = orc.reference_mpgemm(act, w, scales, m, n, k)
        out = np.zeros((m, n), np.float32)
        backend.mpgemm(MpGemm(act, buf, scales, GemmShape(m, n, k), TernaryFormat.Tq2_0, out))
        assert accepts(out, want), vid
        # fused W1.58A8 == host default (run_fused_fallback_contract, crates/tritium-testkit/src/runner.rs:402)
        want_f = orc.mpgemm_with_act_quant(act, w, scales, m, n, k)
        _, s = orc.quantize_act_int8(act, m, k)
        out_f = np.zeros((m, n), np.float32)
        backend.mpgemm_with_act_quant(MpGemm(act, buf, scales, GemmShape(m, n, k), TernaryFormat.Tq2_0, out_f))
        for r in range(m):
            assert accepts(out_f[r], want_f[r], floor=max(float(s[r]), 1e-30)), vid
        # integer-valued activations (what TernaryLinear::forward hands over) are exact
        q, _ = orc.quantize_act_int8(act, m, k)
        out_q = np.zeros((m, n), np.float32)
        backend.mpgemm(MpGemm(q, buf, scales, GemmShape(m, n, k), TernaryFormat.Tq2_0, out_q))
        assert np.array_equal(out_q, orc.reference_mpgemm(q, w, scales, m, n, k)), vid
        # the same weights as TQ1_0 rows give the same bits (crates/tritium-cuda/src/cuda/tests.rs:5520)
        buf1 = backend.upload_weights(orc.tq1_pack_rows(w), GemmShape(0, n, k), TernaryFormat.Tq1_0)
        assert buf1.len_bytes() == n * (k // 256) * 54
        out_1 = np.zeros((m, n), np.float32)
        backend.mpgemm(MpGemm(q, buf1, scales, GemmShape(m, n, k), TernaryFormat.Tq1_0, out_1))
        assert np.array_equal(out_1, out_q), vid
        out_1f = np.zeros((m, n), np.float32)
        backend.mpgemm_with_act_quant(MpGemm(act, buf1, scales, GemmShape(m, n, k), TernaryFormat.Tq1_0, out_1f))
        assert np.array_equal(out_1f, out_f), vid


def test_trait_path_errors(backend):
    from tritium_b200 import GemmShape, MpGemm, TernaryFormat
    w = np.zeros((2, 256), np.int8)
    with pytest.raises(errors.InvalidInput):
        backend.upload_weights(fmt.pack_tq2_0_rows(w)[:-1], GemmShape(0, 2, 256), TernaryFormat.Tq2_0)
    with pytest.raises(errors.UnsupportedFormat):
        backend.upload_weights(b"", GemmShape(0, 2, 256), TernaryFormat.I2sInt8)
    with pytest.raises(errors.InvalidInput):
        backend.upload_weights(b"\x80" * 53, GemmShape(0, 1, 256), TernaryFormat.Tq1_0)
    buf = backend.upload_weights(fmt.pack_tq2_0_rows(w), GemmShape(0, 2, 256), TernaryFormat.Tq2_0)
    out = np.zeros((1, 2), np.float32)
    with pytest.raises(errors.ShapeMismatch):
        backend.mpgemm(MpGemm(np.zeros(255, np.float32), buf, np.ones(2, np.float32), GemmShape(1, 2, 256), TernaryFormat.Tq2_0, out))
    backend.mpgemm(MpGemm(np.zeros(0, np.float32), buf, np.ones(2, np.float32), GemmShape(0, 2, 256), TernaryFormat.Tq2_0, np.zeros((0, 2), np.float32)))
    caps = backend.capabilities()
    assert caps.backend == "b200" and "sm_100a" in caps.features and backend.device_id() == "b200:0"
    assert backend.physical_device_id().startswith("b200:0:GPU-")


# ------------------------------------------------------------------ grouped stack (one launch, many layers)
@pytest.mark.parametrize("codec", [SaltV2Codec.B3, SaltV2Codec.D2])
@pytest.mark.parametrize("m", [1, 3])
def test_grouped_stack_matches_per_layer_oracle(backend, codec, m):
    import torch
    from tritium_b200 import LinearStack
    n, k, planes = 96, 1024, 2
    pairs = [uniform_pair(n, k, planes, seed=100 + i) for i in range(5)]
    weights = [backend.upload_salt_v2(prod, codec) for prod, _ in pairs]
    stack = LinearStack(backend, weights, [0] * len(weights), max_m=4)
    x = make_activations(m, k, seed=17, bf16=True)
    x_dev = torch.from_numpy(f32_to_bf16_bits(x).view(np.int16).copy()).cuda().view(torch.bfloat16).reshape(m, k)
    stream = torch.cuda.Stream()
    for flags in (0, 4):          # plain stream order, then programmatic dependent launch
        with torch.cuda.stream(stream):
            stack.forward_dev(x_dev, flags=flags, stream=stream)
        stream.synchronize()
        backend.check(stream)
        for i, (_, orac) in enumerate(pairs):
            want, _, _ = orc.a8_linear(orac, x, dump=False)
            got = bf16_bits_to_f32(stack.read_output(i, m))
            assert rel_l2(got, want) <= 1e-2, (i, flags)
    stack.close()


def test_stack_host_call_matches_per_layer_calls(backend):
    """One host-pointer call over a stack of projections that read the same activations returns
    what one host-pointer call per projection returns."""
    n, k, planes, m = 96, 512, 2, 3
    tensors = [uniform_pair(n, k, planes, seed=70 + i)[0] for i in range(3)]
    residents = [backend.upload_salt_v2(t, SaltV2Codec.B3) for t in tensors]
    from tritium_b200 import LinearStack
    stack = LinearStack(backend, residents, [0, 0, 0], max_m=4)
    x = make_activations(m, k, seed=8, bf16=True)
    got = stack.forward_host(f32_to_bf16_bits(x), m, x_is_bf16=True)
    assert got.shape == (3, m, n)
    for i, r in enumerate(residents):
        want, _, _ = backend.linear_forward_a8(r, f32_to_bf16_bits(x), m, y_dtype="bf16", x_is_bf16=True)
        assert np.array_equal(got[i], want)
    stack.close()


@pytest.mark.parametrize("codec", [SaltV2Codec.B3, SaltV2Codec.D2])
@pytest.mark.parametrize("m", [1, 6, 24, 200])
def test_mixed_plane_counts_on_aligned_shapes_take_the_fast_kernels(backend, codec, m):
    """A tensor whose tiles hold one to three planes (a plane map with varying counts), on a shape
    the fast kernels take, is stored padded to three plane slots per tile with all-zero planes.
    The int8 path then runs the decode, few-token and many-token kernels with the same exact
    group sums (zero for a padded plane); the fp32 exact kernel still adds only each tile's true
    planes and returns the reference's bits."""
    n, k = 64, 768
    prod, orac = uniform_pair(n, k, 3, seed=91)
    tiles = n * k // 256
    counts = (1 + (np.arange(tiles) * 7 + 2) % 3).astype(np.uint8)
    for t in (prod, orac):
        t.plane_count[:] = counts
        for ti in range(tiles):
            t.trits[ti, counts[ti]:, :] = 0
            t.scales[ti, counts[ti]:, :] = 0
    resident = backend.upload_salt_v2(prod, codec)
    assert resident.info["fast_path"] and resident.info["planes_uniform"] == 3
    slot = 52 if codec == SaltV2Codec.B3 else 64
    assert resident.allocation_receipt()["payload_bytes"] == tiles * 3 * slot
    x = make_activations(m, k, seed=m)
    want_y, want_acc, _ = orc.a8_linear(orac, x)
    y, acc, receipt = backend.linear_forward_a8(resident, x, m, dump=True)
    assert receipt.kernel == (1 if m <= 8 else 2)
    assert np.array_equal(acc, want_acc[:, :, :, :3])
    assert rel_l2(y, want_y) <= 1e-5
    xe = seeded_f32(0x77 + m, min(m, 3) * k, -0.75, 0.75).reshape(min(m, 3), k)
    want = np.stack([orc.matvec(orac, row) for row in xe])
    exact = backend.salt_v2_forward_exact(resident, xe, xe.shape[0])
    assert np.array_equal(exact.output.view(np.uint32), want.view(np.uint32))
    streamed = backend.upload_salt_v2_from_package(fmt.write_salt_v2_package(prod, codec), prod.name)
    again = backend.salt_v2_forward_exact(streamed, xe, xe.shape[0])
    assert np.array_equal(again.output.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("m", [1, 5])
def test_rows_too_long_for_the_decode_kernel_run_on_tensor_cores(backend, m):
    """Three planes at k = 17408 (a 27B-class down projection): two row blocks of the decode
    kernel's ring do not fit in shared memory, so the tensor-core kernel takes the call at every
    token count, with the same exact group sums."""
    n, k, planes = 48, 17408, 3
    prod, orac = uniform_pair(n, k, planes, seed=17)
    x = make_activations(m, k, seed=40 + m)
    want_y, want_acc, _ = orc.a8_linear(orac, x)
    resident = backend.upload_salt_v2(prod, SaltV2Codec.B3)
    y, acc, receipt = backend.linear_forward_a8(resident, x, m, dump=True)
    assert receipt.kernel == 2
    assert np.array_equal(acc, want_acc[:, :, :, :planes])
    assert rel_l2(y, want_y) <= 1e-5
    y32 = backend.salt_v2_forward_fast(resident, x, m)           # fp32 entry: int8 limbs, same route
    want32 = np.stack([orc.matvec(orac, row) for row in x])
    assert rel_l2(y32.output, want32) <= 1e-5


def s34_pair(n, k, planes, seed):
    """Planes with exactly one zero in every four trits (what S34 can hold), random signs and scales."""
    rng = np.random.default_rng(seed)
    prod, orac = uniform_pair(n, k, planes, seed=seed)
    tiles = n * k // 256
    trits = rng.choice(np.array([-1, 1], np.int8), size=(tiles, 3, 64, 4))
    zero_at = rng.integers(0, 4, size=(tiles, 3, 64))
    np.put_along_axis(trits, zero_at[..., None], 0, axis=3)
    trits = trits.reshape(tiles, 3, 256)
    trits[:, planes:, :] = 0
    for t in (prod, orac):
        t.trits[:] = trits
    return prod, orac


@pytest.mark.parametrize("planes,m", [(1, 1), (2, 4), (3, 7), (2, 40), (3, 300)])
def test_s34_tensors_on_aligned_shapes_take_the_fast_kernels(backend, planes, m):
    """An S34 artifact on a shape the fast kernels take is stored as B3 with the same trits: the
    int8 path runs the decode and tensor-core kernels with exact group sums, and the fp32 exact
    kernel still returns the reference's bits.  The package route gives the same resident tensor."""
    n, k = 80, 1024
    prod, orac = s34_pair(n, k, planes, seed=planes * 100 + m)
    resident = backend.upload_salt_v2(prod, SaltV2Codec.S34)
    assert resident.info["fast_path"] and resident.info["planes_uniform"] == planes
    assert resident.allocation_receipt()["payload_bytes"] == (n * k // 256) * planes * 52
    x = make_activations(m, k, seed=m)
    want_y, want_acc, _ = orc.a8_linear(orac, x)
    y, acc, receipt = backend.linear_forward_a8(resident, x, m, dump=True)
    assert receipt.kernel == (1 if m <= 8 else 2)
    assert np.array_equal(acc, want_acc[:, :, :, :planes])
    assert rel_l2(y, want_y) <= 1e-5
    rows = min(m, 2)
    xe = seeded_f32(0x534 + m, rows * k, -0.75, 0.75).reshape(rows, k)
    want = np.stack([orc.matvec(orac, row) for row in xe])
    streamed = backend.upload_salt_v2_from_package(fmt.write_salt_v2_package(prod, SaltV2Codec.S34), prod.name)
    for r in (resident, streamed):
        got = backend.salt_v2_forward_exact(r, xe, rows)
        assert np.array_equal(got.output.view(np.uint32), want.view(np.uint32))


# ------------------------------------------------------------------ int8 path of layouts without a fast kernel
@pytest.mark.parametrize("codec,ocodec", CODECS)
@pytest.mark.parametrize("layout", ["ragged_3x173", "g64_4x576", "mixed_planes_8x256"])
def test_int8_path_of_other_layouts_is_bit_identical_to_cpu(backend, codec, ocodec, layout):
    """Ragged shapes, scale groups of 64, S34 and mixed plane counts on small shapes have no fast kernel: their int8
    path quantises to codes kept as fp32 values and runs the bit-exact kernel on them.  Group sums
    of small integers are exact and the order is the reference's, so the output equals the CPU
    composition (quantise, matvec, token scale) bit for bit."""
    if layout == "ragged_3x173":
        t = cuda_test_tensor(3, 173, [1, 3, 2])
    elif layout == "g64_4x576":
        tiles = []
        for ti in range(9):
            trits = [{0: 0, 1: 1, 2: 1, 3: -1}[(i + ti) % 4] for i in range(256)]
            tiles.append([(trits, [f16(np.float32(0.125) + np.float32(ti * 4 + g) / np.float32(64.0)) for g in range(4)])])
        t = orc.tensor_from_planes(4, 576, tiles, group=64)
    else:
        t = cuda_test_tensor(8, 256, [1, 3, 2, 1, 2, 3, 3, 1])
    m = 3
    x = seeded_f32(0xA8 + t.rows, m * t.cols, -2.5, 2.5).reshape(m, t.cols)
    want, _, scale = orc.a8_linear(t, x, dump=False)
    resident = backend.upload_salt_v2(as_product(t), codec)
    assert not resident.info["fast_path"]
    y, _, receipt = backend.linear_forward_a8(resident, x, m)
    assert receipt.kernel == 0
    assert np.array_equal(y.view(np.uint32), want.view(np.uint32))
    with pytest.raises(errors.UnsupportedFormat, match="accumulator dump"):
        backend.linear_forward_a8(resident, x, m, dump=True)
