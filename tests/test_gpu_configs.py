"""Every cell of the benchmark configurations at full size, through the C ABI, against the CPU
oracle (sampled rows where a full oracle pass would take minutes) and, for the int32 group sums,
against exact integer arithmetic on the host.

C1  K=2048 N=8192, one plane, fp32 activations, M = 1, 32
C2  K=2560 N=6912, three planes, bf16 activations quantised per token, M = 1, 4 (test_gpu_parity), 16, 128, 2048
C3  one plane, (K,N) in {(2560,2560), (2560,6912), (6912,2560), (2048,8192)}, M = 512, 2048, 8192
C4  2B-class decoder linears, one plane, batch 1, 16 (test_gpu_parity), 64
C5  27B-class decoder linears, two planes, batch 1, 32, prefill 4096; tensor-parallel shards of
    ranks 0 and world-1 for world = 2, 4, 8 (each shard runs alone on one GPU with the absmax of
    the whole row passed in, which is what a rank of the group computes)
"""
import numpy as np
import pytest

from oracle import oracle as orc
from tritium_b200 import format as fmt
from tritium_b200.format import SaltV2Codec, SaltV2Tensor
from tritium_b200.synth import bf16_bits_to_f32, f32_to_bf16_bits, make_activations
from tritium_b200.tp import DECODER_27B, DECODER_2B, ShardGeometry

from gpu_common import THREADS, exact_group_sums, oracle_rows, product_only, rel_l2, sample_rows, uniform_pair

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def backend():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device: there is no CPU path to fall back to")
    from tritium_b200 import B200Backend
    b = B200Backend(0)
    yield b
    b.close()


def to_dev_bf16(x):
    import torch
    return torch.from_numpy(f32_to_bf16_bits(x).view(np.int16).copy()).cuda().view(torch.bfloat16).reshape(x.shape)


# ------------------------------------------------------------------ C1: fp32 activations
@pytest.mark.parametrize("codec", [SaltV2Codec.B3, SaltV2Codec.D2], ids=["b3", "d2"])
@pytest.mark.parametrize("m", [1, 32])
def test_c1_fp32_activations_k2048_n8192(backend, codec, m):
    """The exact entry point is bit-identical to salt_v2_matvec_into
    (crates/tritium-cpu/src/salt_v2.rs:316-423); the fast entry point is within 1e-5 relative L2."""
    n, k = 8192, 2048
    prod, orac = uniform_pair(n, k, 1, seed=0)
    x = make_activations(m, k, seed=0)
    want = orc.matmul(orac, x, threads=THREADS)
    resident = backend.upload_salt_v2(prod, codec)
    exact = backend.salt_v2_forward_exact(resident, x, m)
    assert np.array_equal(exact.output.view(np.uint32), want.view(np.uint32))
    fast = backend.salt_v2_forward_fast(resident, x, m)
    assert rel_l2(fast.output, want) <= 1e-5
    assert exact.receipt.dense_weight_bytes == 0 and exact.receipt.activation_bytes == m * k * 4


# ------------------------------------------------------------------ C2: M = 16, 128
@pytest.mark.parametrize("m", [8, 16], ids=["two_decode_passes", "few_token_tensor_kernel"])
@pytest.mark.parametrize("codec", [SaltV2Codec.B3, SaltV2Codec.D2], ids=["b3", "d2"])
def test_c2_three_planes_m16_full_accumulators(backend, codec, m):
    n, k, planes = 6912, 2560, 3
    prod, orac = uniform_pair(n, k, planes, seed=0)
    x = make_activations(m, k, seed=16, bf16=True)
    want_y, want_acc, _ = orc.a8_linear(orac, x)
    y_bits, acc, receipt = backend.linear_forward_a8(backend.upload_salt_v2(prod, codec), f32_to_bf16_bits(x), m,
                                                    y_dtype="bf16", dump=True, x_is_bf16=True)
    assert receipt.kernel == (1 if m <= 8 else 2)
    assert np.array_equal(acc, want_acc)
    assert rel_l2(bf16_bits_to_f32(y_bits), want_y) <= 1e-2


@pytest.mark.parametrize("codec", [SaltV2Codec.B3, SaltV2Codec.D2], ids=["b3", "d2"])
def test_c2_three_planes_m128(backend, codec):
    n, k, planes, m = 6912, 2560, 3, 128
    prod, orac = uniform_pair(n, k, planes, seed=0)
    x = make_activations(m, k, seed=128, bf16=True)
    q, s = orc.quantize_act_int8(x, m, k)
    want_y = orc.matmul(orac, q, threads=THREADS) * s[:, None]
    resident = backend.upload_salt_v2(prod, codec)
    y, _, receipt = backend.linear_forward_a8(resident, x, m)
    assert receipt.kernel == 2
    assert rel_l2(y, want_y) <= 1e-5
    # int32 group sums of a token slice, bit-exact against integer arithmetic on the host
    tok = np.r_[0:8, 60:68, 120:128]
    _, acc, _ = backend.linear_forward_a8(resident, x[tok], len(tok), dump=True)
    # the slice is quantised per token exactly as inside the full call
    assert np.array_equal(acc, exact_group_sums(prod.raw[0], q[tok]))


# ------------------------------------------------------------------ C3: prefill sweep
SWEEP = {"k2560_n2560": (2560, 2560), "k2560_n6912": (6912, 2560), "k6912_n2560": (2560, 6912), "k2048_n8192": (8192, 2048)}


@pytest.mark.parametrize("shape", list(SWEEP))
def test_c3_prefill_sweep_m512_every_accumulator(backend, shape):
    """512 tokens: every int32 group sum bit-exact, bf16 outputs against the oracle on sampled rows."""
    n, k = SWEEP[shape]
    m = 512
    prod = product_only(n, k, 1, seed=3)
    x = make_activations(m, k, seed=2, bf16=True)
    q, s = orc.quantize_act_int8(x, m, k)
    resident = backend.upload_salt_v2(prod, SaltV2Codec.B3)
    y_bits, acc, receipt = backend.linear_forward_a8(resident, f32_to_bf16_bits(x), m, y_dtype="bf16", dump=True, x_is_bf16=True)
    assert receipt.kernel == 2
    assert np.array_equal(acc, exact_group_sums(prod.raw[0], q))
    rows = sample_rows(n)
    want = orc.matmul(oracle_rows(prod, rows), q, threads=THREADS) * s[:, None]
    assert rel_l2(bf16_bits_to_f32(y_bits)[:, rows], want) <= 1e-2


@pytest.mark.parametrize("shape", list(SWEEP))
@pytest.mark.parametrize("m", [2048, 8192])
def test_c3_prefill_sweep_large_m(backend, shape, m):
    """2048 and 8192 tokens: bf16 outputs on sampled rows and tokens against the oracle; the int32
    sums of a 256-token slice (first and last tokens) bit-exact; the slice's outputs are the same
    bits as in the full call (tokens are independent)."""
    n, k = SWEEP[shape]
    prod = product_only(n, k, 1, seed=5)
    x = make_activations(m, k, seed=m, bf16=True)
    resident = backend.upload_salt_v2(prod, SaltV2Codec.B3)
    y_bits, _, receipt = backend.linear_forward_a8(resident, f32_to_bf16_bits(x), m, y_dtype="bf16", x_is_bf16=True)
    assert receipt.kernel == 2
    rows = sample_rows(n)
    tok = np.r_[0:6, m // 2:m // 2 + 6, m - 6:m]
    q, s = orc.quantize_act_int8(x[tok], len(tok), k)
    want = orc.matmul(oracle_rows(prod, rows), q, threads=THREADS) * s[:, None]
    assert rel_l2(bf16_bits_to_f32(y_bits)[np.ix_(tok, rows)], want) <= 1e-2
    sl = np.r_[0:128, m - 128:m]
    qs, _ = orc.quantize_act_int8(x[sl], len(sl), k)
    ys_bits, acc, _ = backend.linear_forward_a8(resident, f32_to_bf16_bits(x[sl]), len(sl), y_dtype="bf16", dump=True, x_is_bf16=True)
    assert np.array_equal(acc, exact_group_sums(prod.raw[0], qs))
    assert np.array_equal(ys_bits, y_bits[sl])


# ------------------------------------------------------------------ C4: 2B-class decoder linears
def decoder_cases(shape):
    return [(name, n, k) for name, _, n, k in shape.linears()]


@pytest.mark.parametrize("name,n,k", decoder_cases(DECODER_2B), ids=[c[0] for c in decoder_cases(DECODER_2B)])
@pytest.mark.parametrize("m", [1, 64])
def test_c4_decoder_2b_linears(backend, name, n, k, m):
    prod = product_only(n, k, DECODER_2B.planes, seed=n % 89)
    x = make_activations(m, k, seed=7 + m, bf16=True)
    y, _, receipt = backend.linear_forward_a8(backend.upload_salt_v2(prod, SaltV2Codec.B3), x, m)
    assert receipt.kernel == (1 if m <= 8 else 2)
    rows = sample_rows(n, 16)
    q, s = orc.quantize_act_int8(x, m, k)
    want = orc.matmul(oracle_rows(prod, rows), q, threads=THREADS) * s[:, None]
    assert rel_l2(y[:, rows], want) <= 1e-5


# ------------------------------------------------------------------ C5: 27B-class decoder linears and their shards
def shard_reference(prod, geometry, rows, q_full, s):
    """Oracle output of `rows` of one rank's shard: trits and scales cut as ShardGeometry says
    (row-parallel: the K slice, padded with zero trits and zero scales to whole tiles), activation
    codes of the whole row's quantisation."""
    trits, scales = prod.raw
    planes = trits.shape[0]
    g = geometry
    t = trits[:, g.n_offset:g.n_offset + g.n][:, rows]
    sc = scales[:, g.n_offset:g.n_offset + g.n][:, rows]
    tp_ = np.zeros((planes, len(rows), g.k), np.int8)
    sp_ = np.zeros((planes, len(rows), g.k // 128), np.float32)
    tp_[:, :, :g.k_valid] = t[:, :, g.k_offset:g.k_offset + g.k_valid]
    sp_[:, :, :g.k_valid // 128] = sc[:, :, g.k_offset // 128:(g.k_offset + g.k_valid) // 128]
    sub = SaltV2Tensor.from_matrix_planes("s", tp_, sp_)
    orac = orc.Tensor(len(rows), g.k, 128, sub.plane_count.copy(), sub.trits.copy(), sub.scales.copy())
    qs = np.zeros((q_full.shape[0], g.k), np.float32)
    qs[:, :g.k_valid] = q_full[:, g.k_offset:g.k_offset + g.k_valid]
    return orc.matmul(orac, qs, threads=THREADS) * s[:, None]


@pytest.fixture(scope="module")
def decoder_27b_tensors():
    return {name: product_only(n, k, DECODER_27B.planes, seed=40 + i)
            for i, (name, _, n, k) in enumerate(DECODER_27B.linears())}


@pytest.mark.parametrize("name,mode,n,k", DECODER_27B.linears(), ids=[c[0] for c in DECODER_27B.linears()])
def test_c5_decoder_27b_linears_and_shards(backend, decoder_27b_tensors, name, mode, n, k):
    import torch
    codec = SaltV2Codec.B3
    prod = decoder_27b_tensors[name]
    payload, scales, _, _, _ = prod.resident(codec)
    xs = {m: make_activations(m, k, seed=90 + m, bf16=True) for m in (1, 32)}
    quant = {m: orc.quantize_act_int8(x, m, k) for m, x in xs.items()}
    stream = torch.cuda.Stream()
    for world, ranks in [(1, [0]), (2, [0, 1]), (4, [0, 3]), (8, [0, 7])]:
        for rank in ranks:
            geo = ShardGeometry.of(mode, n, k, world, rank)
            if world == 1:
                handle = backend.upload_salt_v2(prod, codec)
            else:
                sn, sk, sp, ss, sm, term = fmt.tp_shard(codec, 128, n, k, DECODER_27B.planes, payload, scales, mode == "row", world, rank)
                assert (sn, sk) == (geo.n, geo.k)
                handle = backend.upload_salt_v2_arenas(codec, 128, sn, sk, sp, ss, sm, term)
            rows = sample_rows(geo.n)
            backend.reserve(handle, 32)
            for m, x in xs.items():
                q, s = quant[m]
                want = shard_reference(prod, geo, rows, q, s)
                x_shard = np.zeros((m, geo.k), np.float32)
                x_shard[:, :geo.k_valid] = x[:, geo.k_offset:geo.k_offset + geo.k_valid]
                x_dev = to_dev_bf16(x_shard)
                absmax = torch.from_numpy(np.abs(x).max(axis=1).astype(np.float32)).cuda()
                y_dev = torch.zeros(m, geo.n, dtype=torch.float32, device="cuda")
                with torch.cuda.stream(stream):
                    backend.forward_dev(handle, x_dev, y_dev, a8=True, act_absmax=absmax, stream=stream)
                stream.synchronize()
                backend.check(stream)
                got = y_dev.cpu().numpy()[:, rows]
                assert rel_l2(got, want) <= 1e-5, (name, world, rank, m)
            handle.free()


@pytest.mark.parametrize("name", ["qkv", "down"])
def test_c5_decoder_27b_prefill_4096(backend, decoder_27b_tensors, name):
    m = 4096
    prod = decoder_27b_tensors[name]
    n, k = prod.rows, prod.cols
    x = make_activations(m, k, seed=4096, bf16=True)
    y_bits, _, receipt = backend.linear_forward_a8(backend.upload_salt_v2(prod, SaltV2Codec.B3), f32_to_bf16_bits(x), m,
                                                  y_dtype="bf16", x_is_bf16=True)
    assert receipt.kernel == 2
    rows = sample_rows(n)
    tok = np.r_[0:4, 2047:2051, m - 4:m]
    q, s = orc.quantize_act_int8(x[tok], len(tok), k)
    want = orc.matmul(oracle_rows(prod, rows), q, threads=THREADS) * s[:, None]
    assert rel_l2(bf16_bits_to_f32(y_bits)[np.ix_(tok, rows)], want) <= 1e-2


# ------------------------------------------------------------------ C1 as stated: fp32 activations on the fast entry point
@pytest.mark.parametrize("m", [1, 32])
@pytest.mark.parametrize("codec", [SaltV2Codec.B3, SaltV2Codec.D2], ids=["b3", "d2"])
def test_c1_fp32_fast_entry_point_full_size(backend, codec, m):
    """C1 (K=2048, N=8192, one plane, fp32 activations): the fast fp32 entry point runs the int8
    kernels on four int8 limbs per activation; the exact entry point stays bit-identical."""
    n, k = 8192, 2048
    prod, orac = uniform_pair(n, k, 1, seed=0)
    rng = np.random.default_rng(0)
    x = rng.standard_normal((m, k)).astype(np.float32)
    x[:, 7] *= 50.0                                   # an outlier channel: limbs are relative to the row's absmax
    want = np.stack([orc.matvec(orac, x[i]) for i in range(m)])
    resident = backend.upload_salt_v2(prod, codec)
    fast = backend.salt_v2_forward_fast(resident, x, m)
    assert rel_l2(fast.output, want) <= 1e-5
    assert fast.receipt.kernel in (1, 2)              # a fast kernel ran, not the scalar exact one
    exact = backend.salt_v2_forward_exact(resident, x, m)
    assert np.array_equal(exact.output.view(np.uint32), want.view(np.uint32))
    # tiny activations against one huge one still resolve: 31 bits below the absmax
    x2 = np.full((1, k), 1e-6, np.float32); x2[0, 0] = 1.0
    want2 = orc.matvec(orac, x2[0])[None]
    assert rel_l2(backend.salt_v2_forward_fast(resident, x2, 1).output, want2) <= 1e-5
