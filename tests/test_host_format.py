"""Host logic of the product library against the oracle: byte layouts must be identical."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from oracle import oracle as orc
from tritium_b200 import _lib, errors
from tritium_b200 import format as fmt
from tritium_b200.format import SaltV2Codec, SaltV2Tensor
from tritium_b200.synth import make_planes

CODECS = [(SaltV2Codec.D2, orc.D2), (SaltV2Codec.B3, orc.B3), (SaltV2Codec.S34, orc.S34)]
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "tritium_b200.h")).read()
    declared = set(re.findall(r"\b(tb_[a-z0-9_]+)\s*\(", header))
    declared -= {"tb_status"}
    L = _lib.load()
    assert L.tb_abi_version() == 1
    missing = [name for name in sorted(declared) if not hasattr(L, name)]
    assert not missing, missing
    assert set(_lib.EXPORTS) <= declared


def s34_trits(rng, n):
    t = rng.choice([-1, 1], n).astype(np.int8)
    t[np.arange(0, n, 4) + rng.integers(0, 4, n // 4)] = 0
    return t


@pytest.mark.parametrize("codec,ocodec", CODECS)
def test_codecs_match_oracle_bytes(codec, ocodec):
    rng = np.random.default_rng(11)
    for n in (4, 8, 20, 100, 256, 1024):
        trits = s34_trits(rng, n) if codec == SaltV2Codec.S34 else rng.integers(-1, 2, n).astype(np.int8)
        packed = fmt.pack(codec, trits)
        assert packed == orc.pack(ocodec, trits)
        assert np.array_equal(fmt.unpack(codec, packed, n), trits)
    if codec != SaltV2Codec.S34:
        for n in (1, 5, 6, 7, 87, 173, 255):
            trits = rng.integers(-1, 2, n).astype(np.int8)
            assert fmt.pack(codec, trits) == orc.pack(ocodec, trits)


def test_codec_rejections():
    with pytest.raises(errors.InvalidInput):
        fmt.unpack(SaltV2Codec.D2, bytes([0b01010111]), 1)
    with pytest.raises(errors.InvalidInput):
        fmt.unpack(SaltV2Codec.D2, bytes([0x00]), 1)
    with pytest.raises(errors.InvalidInput):
        fmt.unpack(SaltV2Codec.B3, bytes([243]), 5)
    with pytest.raises(errors.InvalidInput):
        fmt.unpack(SaltV2Codec.B3, bytes([0]), 1)
    with pytest.raises(errors.InvalidInput):
        fmt.unpack(SaltV2Codec.B3, bytes([121, 121]), 1)
    with pytest.raises(errors.InvalidInput):
        fmt.unpack(SaltV2Codec.S34, bytes([0xC9, 0x82]), 8)
    with pytest.raises(errors.InvalidInput):
        fmt.pack(SaltV2Codec.S34, [-1, 1, -1, 1])
    with pytest.raises(errors.InvalidInput):
        fmt.pack(SaltV2Codec.D2, [2])


def ragged_pair(rows, cols, counts, group=128, s34=False, seed=0):
    """The same ragged tensor as a product SaltV2Tensor and as an oracle Tensor."""
    rng = np.random.default_rng(seed)
    tiles = (rows * cols + 255) // 256
    pc = np.array(counts, np.uint8)
    tr = np.zeros((tiles, 3, 256), np.int8)
    sc = np.zeros((tiles, 3, 4), np.uint16)
    for t in range(tiles):
        length = min(256, rows * cols - t * 256)
        for p in range(pc[t]):
            if s34:
                full = (length // 4) * 4
                tr[t, p, :full] = s34_trits(rng, full) if full else []
                tr[t, p, full:length] = rng.choice([-1, 1], length - full)
            else:
                tr[t, p, :length] = rng.integers(-1, 2, length)
            groups = (length + group - 1) // group
            sc[t, p, :groups] = fmt.f16_bits(0.05 + rng.random(groups, dtype=np.float32))
    prod = SaltV2Tensor("w", rows, cols, pc.copy(), tr.copy(), sc.copy(), group)
    orac = orc.Tensor(rows, cols, group, pc.copy(), tr.copy(), sc.copy())
    return prod, orac


@pytest.mark.parametrize("codec,ocodec", CODECS)
@pytest.mark.parametrize("shape", [(3, 173, [1, 3, 2], 128), (2, 3, [3], 128), (1, 1, [1], 128),
                                   (4, 576, [1, 2, 3, 1, 2, 3, 1, 2, 3], 64), (1, 513 * 256, None, 128)])
def test_resident_arenas_and_package_bytes_match_oracle(codec, ocodec, shape):
    rows, cols, counts, group = shape
    if counts is None:
        counts = [1 + i % 3 for i in range(rows * cols // 256)]
    prod, orac = ragged_pair(rows, cols, counts, group, s34=(codec == SaltV2Codec.S34))
    payload, scales, pmap, terminal, sizes = prod.resident(codec)
    o_payload, o_scales, o_meta, o_terminal, plan = orc.resident_build(orac, ocodec)
    assert payload.tobytes() == o_payload.tobytes()
    assert scales.tobytes() == o_scales.tobytes()
    assert pmap.tobytes() == o_meta[: plan["map_bytes"]].tobytes()
    assert terminal == o_terminal
    assert sizes["rank_prefix_bytes"] == plan["rank_prefix_bytes"]
    assert fmt.write_salt_v2_package(prod, codec) == orc.package_write(ocodec, [("w", orac)])


@pytest.mark.parametrize("codec,ocodec", CODECS)
def test_multi_tensor_package_and_seek_reader(codec, ocodec, tmp_path):
    """Several tensors in one package (ragged last tiles, 64- and 128-wide groups, map bits that end in
    the tensor-count word): the writer's bytes equal the oracle's; the seek-backed reader returns, for
    every tensor, the arenas the oracle builds, and touches only the header table and that tensor."""
    s34 = codec == SaltV2Codec.S34
    specs = [("blk.0.q", 3, 173, [1, 3, 2], 128), ("blk.0.k", 4, 576, [1, 2, 3, 1, 2, 3, 1, 2, 3], 64),
             ("blk.1.ffn", 2, 640, [3, 1, 2, 2, 1], 128), ("tiny", 1, 1, [1], 128)]
    pairs = [ragged_pair(r, c, counts, group, s34=s34, seed=10 + i) for i, (_, r, c, counts, group) in enumerate(specs)]
    prods = []
    for (name, *_), (prod, _) in zip(specs, pairs):
        prod.name = name
        prods.append(prod)
    package = fmt.write_salt_v2_package_multi(prods, codec)
    assert package == orc.package_write(ocodec, [(name, orac) for (name, *_), (_, orac) in zip(specs, pairs)])
    path = tmp_path / "model.tslt2"
    path.write_bytes(package)

    class Counting:
        def __init__(self, f): self.f, self.bytes_read = f, 0
        def seek(self, *a): return self.f.seek(*a)
        def tell(self): return self.f.tell()
        def read(self, n):
            self.bytes_read += n
            return self.f.read(n)

    for (name, rows, cols, counts, group), (_, orac) in zip(specs, pairs):
        with open(path, "rb") as f:
            src = Counting(f)
            info, payload, scales, pmap = fmt.package_extract(src, name)
        o_payload, o_scales, o_meta, o_terminal, plan = orc.resident_build(orac, ocodec)
        assert (info["n"], info["k"], info["group"]) == (rows, cols, group)
        assert payload.tobytes() == o_payload.tobytes() and scales.tobytes() == o_scales.tobytes()
        assert pmap.tobytes() == o_meta[: plan["map_bytes"]].tobytes() and info["terminal_map_value"] == o_terminal
        # two passes (sizes, then data): each reads the header table and this tensor's sections only
        others = sum(len(orc.resident_build(o, ocodec)[0]) for (n2, *_), (_, o) in zip(specs, pairs) if n2 != name)
        assert src.bytes_read < 2 * (len(package) - others) + 64
    with open(path, "rb") as f:
        with pytest.raises(errors.InvalidInput, match="no tensor named"):
            fmt.package_extract(f, "absent")
    (tmp_path / "short.tslt2").write_bytes(package[:-8])
    with open(tmp_path / "short.tslt2", "rb") as f:
        with pytest.raises(errors.InvalidInput):
            fmt.package_extract(f, "tiny")


def test_semantic_validation_matches_reference_rules():
    prod, _ = ragged_pair(1, 256, [1])
    for bits in (0x7C00, 0x7E00, 0xBC00, 0x8000):
        bad = SaltV2Tensor("w", 1, 256, prod.plane_count, prod.trits, prod.scales.copy())
        bad.scales[0, 0, 1] = bits
        with pytest.raises(errors.InvalidInput):
            bad.resident(SaltV2Codec.B3)
    bad = SaltV2Tensor("w", 1, 256, prod.plane_count, prod.trits.copy(), prod.scales.copy())
    bad.scales[0, 0, 0] = 0
    bad.trits[0, 0, 5] = 1
    with pytest.raises(errors.InvalidInput):
        bad.resident(SaltV2Codec.B3)
    bad.trits[0, 0, :128] = 0
    bad.resident(SaltV2Codec.B3)  # zero scale over an all-zero group is allowed
    bad = SaltV2Tensor("w", 1, 256, np.array([4], np.uint8), prod.trits, prod.scales)
    with pytest.raises(errors.InvalidInput):
        bad.resident(SaltV2Codec.B3)
    bad = SaltV2Tensor("w", 1, 256, prod.plane_count, prod.trits, prod.scales, 32)
    with pytest.raises(errors.InvalidInput):
        bad.resident(SaltV2Codec.B3)


def test_host_quantiser_matches_oracle():
    rng = np.random.default_rng(2)
    x = (rng.standard_normal((5, 300)) * 3).astype(np.float32)
    x[2] = 0
    q, s = fmt.quantize_act_int8(x, 5, 300)
    oq, os_ = orc.quantize_act_int8(x, 5, 300)
    assert np.array_equal(q, oq) and np.array_equal(s, os_)
    q, s = fmt.quantize_act_int8(np.array([1, -2, 0.5, -0.5, 2, -1], np.float32), 1, 6)
    assert list(q[0]) == [64, -127, 32, -32, 127, -64]


def test_tq1_rows_match_oracle():
    rng = np.random.default_rng(6)
    w = rng.integers(-1, 2, (7, 700)).astype(np.int8)
    assert fmt.pack_tq1_0_rows(w) == orc.tq1_pack_rows(w)


def test_tq2_rows_match_oracle():
    rng = np.random.default_rng(4)
    w = rng.integers(-1, 2, (7, 768)).astype(np.int8)
    assert fmt.pack_tq2_0_rows(w) == orc.tq2_pack_rows(w)


@pytest.mark.parametrize("codec,ocodec", CODECS[:2])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_tensor_parallel_shards_reassemble(codec, ocodec, world):
    n, k, planes = 16, 1024, 2
    trits, scales = make_planes(n, k, planes, seed=3, densities=(0.66, 0.10, 0.03))
    full = SaltV2Tensor.from_matrix_planes("w", trits, scales)
    payload, sc, _, _, _ = full.resident(codec)
    ofull = orc.Tensor(n, k, 128, full.plane_count, full.trits, full.scales)
    x = np.random.default_rng(9).integers(-127, 128, k).astype(np.float32)
    want = orc.matvec(ofull, x)
    # column-parallel: output rows are split, results concatenate
    outs = []
    for r in range(world):
        sn, sk, sp, ss, sm, term = fmt.tp_shard(codec, 128, n, k, planes, payload, sc, False, world, r)
        assert (sn, sk) == (n // world, k)
        outs.append(orc.forward_packed(ocodec, 128, sn, sk, sp, ss, sm, len(sm), term, x)[0])
    assert np.array_equal(np.concatenate(outs), want)
    # row-parallel: k is split (padded to whole tiles with zero trits), partial sums add up.
    # Integer activations keep every partial sum exact, so the total is exact as well.
    dense = np.zeros((n, k), np.float64)
    for p in range(planes):
        dense += trits[p].astype(np.float64) * np.repeat(fmt.f16_bits(scales[p]).view(np.float16).astype(np.float64), 128, axis=1)
    total = np.zeros(n, np.float64)
    for r in range(world):
        sn, sk, sp, ss, sm, term = fmt.tp_shard(codec, 128, n, k, planes, payload, sc, True, world, r)
        kv = k // world
        assert sn == n and sk == (kv + 255) // 256 * 256
        xs = np.zeros(sk, np.float32)
        xs[:kv] = x[r * kv:(r + 1) * kv]
        total += orc.forward_packed(ocodec, 128, sn, sk, sp, ss, sm, len(sm), term, xs)[0].astype(np.float64)
    assert np.allclose(total, dense @ x.astype(np.float64), rtol=1e-5, atol=1e-3)


def test_library_loads_with_full_signatures():
    """Every export carries ctypes argument types, so a call with the wrong arity fails in Python."""
    L = _lib.load()
    for name in _lib.EXPORTS:
        assert getattr(L, name).argtypes is not None, name
    with pytest.raises(TypeError):
        L.tb_fmt_plane_bytes(1)


def test_backend_reports_missing_device_without_aborting():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    from tritium_b200 import B200Backend, Registry
    with pytest.raises(errors.Backend):
        B200Backend(0)
    assert Registry.init().names() == []


def test_stream_handle_names_the_default_stream_explicitly():
    """torch's default stream has the handle 0, which the C ABI reads as "the backend's own stream":
    the wrapper must pass the legacy-stream handle instead, and any other handle unchanged."""
    from types import SimpleNamespace
    from tritium_b200 import _lib
    assert _lib.stream_handle(SimpleNamespace(cuda_stream=0)) == 1
    assert _lib.stream_handle(SimpleNamespace(cuda_stream=0x7F00DEAD)) == 0x7F00DEAD


def test_reference_kernel_weight_layout_and_gate_restatement():
    """The I2sInt8 packer used to feed the reference's own tensor-core kernel (8 x 32 tiles of 2-bit
    codes, n-tile-major then k-tile-major, row-major inside a tile, tq2_0_imma.cu:36-55) and the
    squared-ReLU gate restatement (decode.cu:764-780)."""
    from oracle import oracle as orc
    from oracle import ref_kernels
    rng = np.random.default_rng(4)
    trits = rng.integers(-1, 2, (24, 96)).astype(np.int8)
    packed = ref_kernels.pack_i2s_int8(trits)
    assert packed.size == (24 // 8) * (96 // 32) * 64
    num_kt = 96 // 32
    for nt in range(3):
        for kt in range(num_kt):
            tile = packed[(nt * num_kt + kt) * 64:(nt * num_kt + kt + 1) * 64]
            for e in range(256):
                code = (int(tile[e // 4]) >> (2 * (e % 4))) & 3
                assert code - 1 == int(trits[nt * 8 + e // 32, kt * 32 + e % 32])
    with pytest.raises(ValueError):
        ref_kernels.pack_i2s_int8(trits[:23])
    g = np.array([-2.0, 0.0, 0.5, 3.0], np.float32)
    u = np.array([7.0, 7.0, -4.0, 0.25], np.float32)
    assert np.array_equal(orc.relu2_gate(g, u), np.array([0.0, 0.0, -1.0, 2.25], np.float32))


# ------------------------------------------------------------------ arenas as stored on the device
def _tensor(n, k, counts, rng, s34=False):
    tiles = n * k // 256
    trits = np.zeros((tiles, 3, 256), np.int8)
    scales = np.zeros((tiles, 3, 4), np.uint16)
    for t in range(tiles):
        for p in range(counts[t]):
            trits[t, p] = s34_trits(rng, 256) if s34 else rng.integers(-1, 2, 256)
            scales[t, p, :2] = fmt.f16_bits(rng.uniform(0.01, 1.0, 2).astype(np.float32))
    return SaltV2Tensor("w", n, k, np.asarray(counts, np.uint8), trits, scales, 128)


def test_device_layout_keeps_the_artifact_arenas_of_uniform_tensors():
    rng = np.random.default_rng(3)
    t = _tensor(16, 512, [2] * 32, rng)
    for codec in (SaltV2Codec.B3, SaltV2Codec.D2):
        payload, scales, _, _, _ = t.resident(codec)
        got_p, got_s, info = t.device_layout(codec)
        assert np.array_equal(got_p, payload) and np.array_equal(got_s, scales)
        assert info == dict(codec=int(codec), planes_uniform=2, recoded=0, counts_from_map=0,
                            payload_bytes=payload.size, scale_count=scales.size)


def test_device_layout_stores_s34_as_b3_with_the_same_trits():
    rng = np.random.default_rng(4)
    t = _tensor(16, 512, [3] * 32, rng, s34=True)
    got_p, got_s, info = t.device_layout(SaltV2Codec.S34)
    want_p, want_s, _, _, _ = t.resident(SaltV2Codec.B3)          # the same planes encoded as B3
    assert info["codec"] == int(SaltV2Codec.B3) and info["recoded"] == 1 and info["planes_uniform"] == 3
    assert np.array_equal(got_p, want_p) and np.array_equal(got_s, want_s)
    first = fmt.unpack(SaltV2Codec.B3, bytes(got_p[:52]), 256)
    assert np.array_equal(first, t.trits[0, 0])


@pytest.mark.parametrize("codec", [SaltV2Codec.B3, SaltV2Codec.D2, SaltV2Codec.S34])
def test_device_layout_pads_varying_plane_counts_with_zero_planes(codec):
    rng = np.random.default_rng(5)
    n, k = 16, 512
    counts = [1 + (7 * i + 2) % 3 for i in range(n * k // 256)]
    t = _tensor(n, k, counts, rng, s34=(codec == SaltV2Codec.S34))
    got_p, got_s, info = t.device_layout(codec)
    stored = SaltV2Codec.B3 if codec == SaltV2Codec.S34 else codec
    pb = 52 if stored == SaltV2Codec.B3 else 64
    assert info["counts_from_map"] == 1 and info["planes_uniform"] == 3 and info["codec"] == int(stored)
    assert info["recoded"] == (1 if codec == SaltV2Codec.S34 else 0)
    assert got_p.size == len(counts) * 3 * pb and got_s.size == len(counts) * 3 * 2
    for tile, have in enumerate(counts):
        for p in range(3):
            plane = fmt.unpack(stored, bytes(got_p[(tile * 3 + p) * pb:(tile * 3 + p + 1) * pb]), 256)
            sc = got_s[(tile * 3 + p) * 2:(tile * 3 + p) * 2 + 2]
            if p < have:
                assert np.array_equal(plane, t.trits[tile, p]) and np.array_equal(sc, t.scales[tile, p, :2])
            else:
                assert not plane.any() and not sc.any()


def test_device_layout_leaves_small_and_unaligned_shapes_alone():
    rng = np.random.default_rng(6)
    mixed_small = _tensor(8, 256, [1, 3, 2, 1, 2, 3, 3, 1], rng, s34=True)       # fewer than 16 rows
    for codec in (SaltV2Codec.B3, SaltV2Codec.S34):
        payload, scales, _, _, _ = mixed_small.resident(codec)
        got_p, got_s, info = mixed_small.device_layout(codec)
        assert np.array_equal(got_p, payload) and np.array_equal(got_s, scales)
        assert info["codec"] == int(codec) and not info["recoded"] and not info["counts_from_map"] and info["planes_uniform"] == 0
