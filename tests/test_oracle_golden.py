"""Pins the CPU oracle against the known answers held in the reference's own unit tests.

Every case restates a fixture from the reference (file:line cited per test); nothing here
touches the product library.
"""
import numpy as np
import pytest

from oracle import oracle as orc
from oracle.oracle import B3, D2, S34, CODE, OracleError, Tensor, tensor_from_planes

CODECS = (D2, B3, S34)


def f16(v):
    return orc.f32_to_f16(float(np.float32(v)))


# ---------------------------------------------------------------- codecs
# crates/tritium-format/src/salt_v2.rs:554-611

def test_d2_known_bytes_and_rejections():
    assert orc.pack(D2, [-1, 0, 1, -1, 1]) == bytes([0x24, 0x56])
    assert list(orc.unpack(D2, bytes([0x24, 0x56]), 5)) == [-1, 0, 1, -1, 1]
    with pytest.raises(OracleError) as e:
        orc.unpack(D2, bytes([0b01010111]), 1)
    assert e.value.code == CODE["INVALID_CODE"]
    with pytest.raises(OracleError) as e:
        orc.unpack(D2, bytes([0x00]), 1)
    assert e.value.code == CODE["PADDING"]
    with pytest.raises(OracleError) as e:
        orc.unpack(D2, b"", 1)
    assert e.value.code == CODE["LENGTH"]
    assert orc.ledger(D2, 5) == dict(physical_bytes=2, padding_trits=3, padding_bits=0, encoded_bits=16)


# salt_v2.rs:613-678
def test_b3_known_bytes_and_rejections():
    assert orc.pack(B3, [-1, 0, 1, -1, 1, 1]) == bytes([0xB7, 0x7A])
    assert list(orc.unpack(B3, bytes([0xB7, 0x7A]), 6)) == [-1, 0, 1, -1, 1, 1]
    with pytest.raises(OracleError) as e:
        orc.unpack(B3, bytes([243]), 5)
    assert e.value.code == CODE["INVALID_CODE"]
    with pytest.raises(OracleError) as e:
        orc.unpack(B3, bytes([0]), 1)
    assert e.value.code == CODE["PADDING"]
    with pytest.raises(OracleError) as e:
        orc.unpack(B3, bytes([121, 121]), 1)
    assert e.value.code == CODE["LENGTH"]
    for code in range(243):
        assert orc.pack(B3, orc.unpack(B3, bytes([code]), 5)) == bytes([code])
    assert orc.ledger(B3, 6) == dict(physical_bytes=2, padding_trits=4, padding_bits=0, encoded_bits=16)


# salt_v2.rs:680-753
def test_s34_known_bytes_and_rejections():
    assert orc.pack(S34, [-1, 0, 1, -1, 1, -1, 0, 1]) == bytes([0xC9, 0x02])
    assert list(orc.unpack(S34, bytes([0xC9, 0x02]), 8)) == [-1, 0, 1, -1, 1, -1, 0, 1]
    with pytest.raises(OracleError) as e:
        orc.pack(S34, [-1, 1, -1, 1])
    assert e.value.code == CODE["S34_SHAPE"]
    with pytest.raises(OracleError) as e:
        orc.unpack(S34, bytes([0xC9, 0x82]), 8)
    assert e.value.code == CODE["PADDING"]
    with pytest.raises(OracleError) as e:
        orc.unpack(S34, b"", 4)
    assert e.value.code == CODE["LENGTH"]
    for code in range(32):
        assert orc.pack(S34, orc.unpack(S34, bytes([code]), 4)) == bytes([code])
    with pytest.raises(OracleError):
        orc.ledger(S34, 3)
    assert orc.ledger(S34, 12) == dict(physical_bytes=2, padding_trits=0, padding_bits=1, encoded_bits=15)


def test_f16_conversion_matches_numpy():
    rng = np.random.default_rng(0)
    vals = np.concatenate([rng.standard_normal(2000).astype(np.float32) * 10.0 ** rng.integers(-8, 5, 2000),
                           np.array([0, 65504, 65520, 1e-8, 6e-8, 5.96e-8, 0.25, 0.28125], np.float32)])
    for v in vals:
        with np.errstate(over="ignore"):
            want = int(np.float32(v).astype(np.float16).view(np.uint16))
        assert orc.f32_to_f16(float(v)) == want
    for bits in list(range(0, 0x7C00, 37)) + [0x7BFF, 0x0001, 0x03FF, 0x0400]:
        want = float(np.array([bits], np.uint16).view(np.float16)[0].astype(np.float32))
        assert orc.f16_to_f32(bits) == want


# ---------------------------------------------------------------- format fixtures
# crates/tritium-format/src/salt_v2_package.rs:2960-3020 (test helpers)

def fmt_plane(length, phase):
    trits = [0 if i % 4 == 0 else (1 if (i + phase) % 2 == 0 else -1) for i in range(length)]
    scales = [f16(np.float32(0.5) + np.float32(g + phase) / np.float32(16.0)) for g in range((length + 127) // 128)]
    return trits, scales


def fmt_tile(length, planes, phase):
    return [fmt_plane(length, phase + p) for p in range(planes)]


def ragged_tensor():
    return tensor_from_planes(1, 599, [fmt_tile(256, 1, 0), fmt_tile(256, 3, 1), fmt_tile(87, 2, 2)], rank=1)


# salt_v2_package.rs:3036-3073, 3179-3197
def test_ragged_package_ledgers():
    t = ragged_tensor()
    t.validate()
    plan = orc.resident_plan(t, D2)
    assert plan["payload_bytes"] == 300 and plan["scale_bytes"] == 20
    assert plan["map_bytes"] == 0 and plan["rank_prefix_bytes"] == 0
    payload, scales, meta, terminal, _ = orc.resident_build(t, D2)
    assert len(payload) == 300 and len(scales) == 10 and len(meta) == 0
    # runtime map code is planes-1 per tile: 0, 2, 1
    assert terminal == (0 | (2 << 2) | (1 << 4))
    data = orc.package_write(D2, [("ragged", t)])
    assert len(data) % 8 == 0
    # header: magic, version 1, codec tag 1, flags 0; 4 presence bits (tiles 0,1) ride in the count word
    assert data[:8] == b"TSLT2PKG" and data[8:10] == b"\x01\x00" and data[10] == 1 and data[11] == 0
    word = int.from_bytes(data[12:16], "little")
    assert word & ((1 << 26) - 1) == 1
    assert word >> 26 == 0b1100  # tile0 = 1 plane (00), tile1 = 3 planes (11)
    assert int.from_bytes(data[16:24], "little") == len(data)
    tile_word = int.from_bytes(data[24 + 16:24 + 24], "little")
    assert tile_word & ((1 << 62) - 1) == 3 and tile_word >> 62 == 0b01  # ragged tile has 2 planes
    assert int.from_bytes(data[24 + 24:24 + 32], "little") == 300
    assert int.from_bytes(data[24 + 32:24 + 40], "little") == 20
    name, back, codec = orc.package_read(data, 0)
    assert name == "ragged" and codec == D2
    assert list(back.plane_count) == [1, 3, 2]
    assert np.array_equal(back.trits, t.trits) and np.array_equal(back.scales, t.scales)


# salt_v2_package.rs:3075-3133
@pytest.mark.parametrize("codec", CODECS)
def test_short_final_tile_repack_is_byte_exact(codec):
    for length in list(range(1, 40)) + [63, 64, 65, 127, 128, 129, 199, 255, 256]:
        for planes in (1, 2, 3):
            t = tensor_from_planes(1, length, [fmt_tile(length, planes, length)], rank=1)
            data = orc.package_write(codec, [("tail", t)])
            _, back, _ = orc.package_read(data, 0)
            assert orc.package_write(codec, [("tail", back)]) == data
            stored = (length + 3) // 4 * 4 if codec == S34 else length
            per_plane = orc.ledger(codec, stored)["physical_bytes"]
            assert int.from_bytes(data[24 + 24:24 + 32], "little") == per_plane * planes
            assert int.from_bytes(data[24 + 32:24 + 40], "little") == ((length + 127) // 128) * 2 * planes


# salt_v2_package.rs:3199-3221 and crates/tritium-cuda/src/cuda/tests.rs:523-540
@pytest.mark.parametrize("tiles", [1, 4, 255, 256, 257, 512, 513, 1025])
def test_indexed_runtime_ledger_and_rank_prefixes(tiles):
    t = tensor_from_planes(1, tiles * 256, [fmt_tile(256, 1 + i % 3, i) for i in range(tiles)], rank=1)
    payload, scales, meta, terminal, plan = orc.resident_build(t, D2)
    assert plan["map_bytes"] == tiles * 2 // 8
    assert plan["rank_prefix_bytes"] == (tiles - 1) // 256 * 4
    assert (plan["map_bytes"] * 8 + tiles * 2 % 8) == tiles * 2
    metadata_bits = tiles * 2 + plan["rank_prefix_bytes"] * 8
    assert metadata_bits * 100 <= tiles * 256
    prefixes = np.frombuffer(meta[plan["map_bytes"]:].tobytes(), "<u4")
    counts = np.array([1 + i % 3 for i in range(tiles)])
    for j, v in enumerate(prefixes):
        assert v == counts[: (j + 1) * 256].sum()


# salt_v2_package.rs:3625-3760, 3913-3941: malformed packages fail closed
def test_package_reader_rejections():
    t = ragged_tensor()
    data = bytearray(orc.package_write(B3, [("ragged", t)]))
    for cut in range(0, len(data), 7):
        with pytest.raises(OracleError):
            orc.package_read(bytes(data[:cut]), 0)
    with pytest.raises(OracleError):
        orc.package_read(bytes(data) + b"\0", 0)
    bad = bytearray(data); bad[0] ^= 1
    with pytest.raises(OracleError) as e:
        orc.package_read(bytes(bad), 0)
    assert e.value.code == CODE["MAGIC"]
    bad = bytearray(data); bad[8] = 3
    with pytest.raises(OracleError) as e:
        orc.package_read(bytes(bad), 0)
    assert e.value.code == CODE["VERSION"]
    bad = bytearray(data); bad[10] = 9
    with pytest.raises(OracleError) as e:
        orc.package_read(bytes(bad), 0)
    assert e.value.code == CODE["CODEC"]
    bad = bytearray(data); bad[11] = 1
    with pytest.raises(OracleError) as e:
        orc.package_read(bytes(bad), 0)
    assert e.value.code == CODE["FLAGS"]
    # plane 3 without plane 2 in the embedded map
    bad = bytearray(data)
    word = int.from_bytes(bad[12:16], "little")
    bad[12:16] = ((word & ((1 << 26) - 1)) | (0b0010 << 26)).to_bytes(4, "little")
    with pytest.raises(OracleError):
        orc.package_read(bytes(bad), 0)
    # declared payload length is derived, not trusted
    bad = bytearray(data)
    bad[24 + 24:24 + 32] = (int.from_bytes(bad[24 + 24:24 + 32], "little") - 1).to_bytes(8, "little")
    with pytest.raises(OracleError):
        orc.package_read(bytes(bad), 0)
    with pytest.raises(OracleError) as e:
        orc.package_write(B3, [("a", t), ("a", t)])
    assert e.value.code == CODE["DUPLICATE_NAME"]


# salt_v2_package.rs:3507-3571: semantic construction rules
def test_semantic_validation_rules():
    ok = tensor_from_planes(1, 4, [[([1, 0, -1, 0], [f16(1.0)])]], rank=1)
    ok.validate()
    bad = tensor_from_planes(1, 4, [[([2, 0, -1, 0], [f16(1.0)])]], rank=1)
    with pytest.raises(OracleError) as e:
        bad.validate()
    assert e.value.code == CODE["TRIT"]
    for bits, code in ((0x7C00, "SCALE_NONFINITE"), (0x7E00, "SCALE_NONFINITE"), (0xBC00, "SCALE_NEGATIVE"),
                       (0x8000, "SCALE_NEGATIVE"), (0x0000, "SCALE_ZERO_NONZERO_GROUP")):
        bad = tensor_from_planes(1, 4, [[([1, 0, -1, 0], [bits])]], rank=1)
        with pytest.raises(OracleError) as e:
            bad.validate()
        assert e.value.code == CODE[code], hex(bits)
    zero_ok = tensor_from_planes(1, 4, [[([0, 0, 0, 0], [0])]], rank=1)
    zero_ok.validate()
    bad = tensor_from_planes(1, 4, [[([1, 0, -1, 0], [f16(1.0)])]], rank=1)
    bad.plane_count[0] = 4
    with pytest.raises(OracleError) as e:
        bad.validate()
    assert e.value.code == CODE["PLANE_COUNT"]
    bad = tensor_from_planes(1, 4, [[([1, 0, -1, 0], [f16(1.0)])]], group=32, rank=1)
    with pytest.raises(OracleError) as e:
        bad.validate()
    assert e.value.code == CODE["GROUP_SIZE"]


# ---------------------------------------------------------------- quantiser
# crates/tritium-spec/src/lib.rs:458-478, crates/tritium-nn/src/ops/act_quant.rs:206-299

def test_act_quant_goldens():
    q, s = orc.quantize_act_int8([1, -2, 0.5, -0.5, 2, -1], 1, 6)
    assert list(q[0]) == [64, -127, 32, -32, 127, -64]
    assert abs(s[0] - 2.0 / 127.0) < 1e-9
    q, s = orc.quantize_act_int8([0, 0, 3, -6], 2, 2)
    assert list(q[0]) == [0, 0] and s[0] == 0.0 and abs(s[1] - 6.0 / 127.0) < 1e-9
    q, s = orc.quantize_act_int8([-3.5], 1, 1)
    assert q[0, 0] == -127 and abs(s[0] - 3.5 / 127.0) < 1e-9
    q, s = orc.quantize_act_int8([-5, 5, -2.5, 1.25], 1, 4)
    assert q[0, 0] == -127 and q[0, 1] == 127
    # random rows against an independent numpy restatement (np.rint is round-half-even)
    rng = np.random.default_rng(1)
    x = (rng.random((7, 33), dtype=np.float32) * 8 - 4).astype(np.float32)
    q, s = orc.quantize_act_int8(x, 7, 33)
    g = np.abs(x).max(axis=1)
    want = np.clip(np.rint(x * (np.float32(127.0) / g)[:, None]), -128, 127)
    assert np.array_equal(q, want) and np.array_equal(s, g / np.float32(127.0))


# crates/tritium-spec/src/lib.rs:564-594: [3,-1]·[1,-1]·2.0 -> 338*3/127
def test_fused_default_golden():
    out = orc.mpgemm_with_act_quant([3.0, -1.0], np.array([[1, -1]], np.int8), [2.0], 1, 1, 2)
    assert abs(out[0, 0] - 338.0 * 3.0 / 127.0) < 1e-4


# ---------------------------------------------------------------- matvec fixtures
# crates/tritium-cpu/src/salt_v2.rs:692-763

def cpu_plane(length, plane_index, tile_index):
    trits = [0 if i % 4 == 0 else (1 if (i + plane_index + tile_index) % 2 == 0 else -1) for i in range(length)]
    scales = [f16(np.float32(0.25) + np.float32(plane_index) * np.float32(0.125)
                  + np.float32(tile_index) * np.float32(0.03125) + np.float32(g) * np.float32(0.015625))
              for g in range((length + 127) // 128)]
    return trits, scales


def cpu_matrix():
    tiles = [[cpu_plane(256, p, 0) for p in range(1)], [cpu_plane(256, p, 1) for p in range(3)],
             [cpu_plane(7, p, 2) for p in range(2)]]
    return tensor_from_planes(3, 173, tiles)


def dense_weights(t: Tensor) -> np.ndarray:
    w = np.zeros(t.coeffs, np.float32)
    for c in range(t.coeffs):
        tile, local = divmod(c, 256)
        acc = np.float32(0.0)
        for p in range(t.plane_count[tile]):
            acc = np.float32(acc + np.float32(t.trits[tile, p, local]) *
                             np.float32(orc.f16_to_f32(int(t.scales[tile, p, local // t.group]))))
        w[c] = acc
    return w.reshape(t.rows, t.cols)


def dense_matvec(w, x):
    out = np.zeros(w.shape[0], np.float32)
    for r in range(w.shape[0]):
        s = np.float32(0.0)
        for c in range(w.shape[1]):
            s = np.float32(s + np.float32(w[r, c] * x[c]))
        out[r] = s
    return out


# salt_v2.rs:766-806 (+ receipts 519/1038 checked through the plan)
@pytest.mark.parametrize("codec", CODECS)
def test_ragged_matrix_matches_independent_dense_math(codec):
    t = cpu_matrix()
    x = ((np.arange(173, dtype=np.float32) - np.float32(81.0)) / np.float32(29.0)).astype(np.float32)
    data = orc.package_write(codec, [("projection", t)])
    _, back, _ = orc.package_read(data, 0)
    want = dense_matvec(dense_weights(back), x)
    got = orc.matvec(back, x)
    assert np.all(np.abs(got - want) <= 2.0e-5 * np.maximum(np.abs(want), 1.0))
    assert np.array_equal(got, orc.matvec(back, x))
    assert back.coeffs == 519 and sum(int(back.plane_count[i]) * back.tile_len(i) for i in range(3)) == 1038
    # the packed-arena twin is bit-identical (crates/tritium-nn/src/layers/salt_v2_host.rs:689-730)
    payload, scales, meta, terminal, plan = orc.resident_build(back, codec)
    packed = orc.forward_packed(codec, 128, 3, 173, payload, scales, meta, plan["map_bytes"], terminal, x)
    assert np.array_equal(packed[0].view(np.uint32), got.view(np.uint32))


# salt_v2.rs:735-763, 839-864
@pytest.mark.parametrize("codec", CODECS)
def test_g64_matrix(codec):
    tiles = []
    for ti in range(9):
        trits = [{0: 0, 1: 1, 2: 1, 3: -1}[(i + ti) % 4] for i in range(256)]
        scales = [f16(np.float32(0.125) + np.float32(ti * 4 + g) / np.float32(64.0)) for g in range(4)]
        tiles.append([(trits, scales)])
    t = tensor_from_planes(4, 576, tiles, group=64)
    x = ((np.arange(576, dtype=np.float32) - np.float32(283.0)) / np.float32(71.0)).astype(np.float32)
    data = orc.package_write(codec, [("g64-projection", t)])
    assert data[8:10] == b"\x02\x00"  # version 2 carries the g64 geometry byte
    _, back, _ = orc.package_read(data, 0)
    assert back.group == 64
    want = dense_matvec(dense_weights(back), x)
    got = orc.matvec(back, x)
    assert np.all(np.abs(got - want) <= 2.0e-5 * np.maximum(np.abs(want), 1.0))
    payload, scales, meta, terminal, plan = orc.resident_build(back, codec)
    packed = orc.forward_packed(codec, 64, 4, 576, payload, scales, meta, plan["map_bytes"], terminal, x)
    assert np.array_equal(packed[0].view(np.uint32), got.view(np.uint32))


F32_MAX = float(np.finfo(np.float32).max)
F16_MAX_BITS = 0x7BFF


# salt_v2.rs:951-966
def test_nan_activation_rejected_before_any_write():
    t = cpu_matrix()
    x = np.zeros(173, np.float32)
    x[71] = np.nan
    with pytest.raises(OracleError) as e:
        orc.matvec(t, x)
    assert e.value.code == CODE["NONFINITE_ACTIVATION"] and e.value.column == 71
    assert e.value.bits == int(np.array([np.nan], np.float32).view(np.uint32)[0])


# salt_v2.rs:998-1011
def test_overflow_reports_row_and_column():
    t = tensor_from_planes(1, 1, [[([1], [F16_MAX_BITS])]])
    with pytest.raises(OracleError) as e:
        orc.matvec(t, [F32_MAX])
    assert e.value.code == CODE["NONFINITE_OUTPUT"] and (e.value.row, e.value.column) == (0, 0)


# salt_v2.rs:1013-1025
def test_cancellation_happens_before_the_scale():
    t = tensor_from_planes(1, 2, [[([1, -1], [F16_MAX_BITS])]])
    assert list(orc.matvec(t, [F32_MAX, F32_MAX])) == [0.0]


# crates/tritium-cuda/src/cuda/tests.rs:67-113,428-434: generators for the GPU parity fixtures
def cuda_test_plane(length, plane_index):
    trits = []
    for i in range(length):
        group, slot = divmod(i, 4)
        if slot == (group + plane_index) % 4:
            trits.append(0)
        else:
            trits.append(1 if (i + plane_index) % 2 == 0 else -1)
    scales = [f16(np.float32(0.25) + np.float32(plane_index) * np.float32(0.125) + np.float32(g) * np.float32(0.0625))
              for g in range((length + 127) // 128)]
    return trits, scales


@pytest.mark.parametrize("codec", CODECS)
def test_rank_prefix_crossing_packed_equals_semantic(codec):
    counts = [1 + i % 3 for i in range(1025)]
    cols = 1025 * 256
    t = tensor_from_planes(1, cols, [[cuda_test_plane(256, p) for p in range(c)] for c in counts])
    s, x = 0x5A17 + 257 + cols, []
    s |= 1
    for _ in range(cols):
        s ^= (s << 13) & 0xFFFFFFFFFFFFFFFF
        s ^= s >> 7
        s ^= (s << 17) & 0xFFFFFFFFFFFFFFFF
        x.append(np.float32(-0.75) + np.float32(s % 1000) / np.float32(1000.0) * np.float32(1.5))
    x = np.array(x, np.float32)
    got = orc.matvec(t, x)
    payload, scales, meta, terminal, plan = orc.resident_build(t, codec)
    assert plan["rank_prefix_bytes"] == 16
    packed = orc.forward_packed(codec, 128, 1, cols, payload, scales, meta, plan["map_bytes"], terminal, x)
    assert np.array_equal(packed[0].view(np.uint32), got.view(np.uint32))


# ---------------------------------------------------------------- TQ2_0 + conformance generator
# crates/tritium-format/src/tq2.rs:21-83; crates/tritium-core/src/reference.rs:215-257

def test_tq2_layout_and_reference_mpgemm():
    rng = np.random.default_rng(3)
    w = rng.integers(-1, 2, (5, 512)).astype(np.int8)
    packed = orc.tq2_pack_rows(w)
    assert len(packed) == 5 * 2 * 66
    raw = np.frombuffer(packed, np.uint8).reshape(5, 2, 66)
    # byte c*32+m holds elements c*128 + n*32 + m at bit 2n, code = trit+1
    for c in range(2):
        for m in (0, 7, 31):
            byte = raw[2, 1, c * 32 + m]
            for n in range(4):
                assert ((int(byte) >> (2 * n)) & 3) - 1 == int(w[2, 256 + c * 128 + n * 32 + m])
    assert bytes(raw[0, 0, 64:66]) == b"\x00\x3c"
    assert np.array_equal(orc.tq2_unpack_rows(packed, 5, 512), w)
    act = rng.standard_normal((3, 512)).astype(np.float32)
    scales = rng.random(5).astype(np.float32)
    out = orc.reference_mpgemm(act, w, scales, 3, 5, 512)
    want = (act.astype(np.float64) @ w.T.astype(np.float64)) * scales
    assert np.allclose(out, want, rtol=1e-4, atol=1e-4)


# crates/tritium-testkit/src/generate.rs:18-56,203-233
def test_conformance_generator_is_deterministic():
    def gen(seed, count):
        rng = orc.XorShift64(seed)
        shapes = []
        for i in range(count):
            rng.perturb(i)
            m, n, k = 1 + rng.below(64), 1 + rng.below(32), 256 * (1 + rng.below(2))
            act = [rng.activation() for _ in range(3)]
            shapes.append((m, n, k, tuple(act), rng.trit(), rng.scale()))
            for _ in range(m * k - 3 + n * k - 1 + n - 1):
                rng.below(3)
        return shapes
    a, b = gen(0xC0FFEE, 6), gen(0xC0FFEE, 6)
    assert a == b
    for m, n, k, act, trit, scale in a:
        assert 1 <= m <= 64 and 1 <= n <= 32 and k in (256, 512)
        assert all(-10.0 <= v < 10.0 for v in act) and trit in (-1, 0, 1) and 0 < scale <= 2.0
    # xorshift64 first outputs from seed 1 (x^=x<<13; x^=x>>7; x^=x<<17)
    r = orc.XorShift64(1)
    x = 1
    for _ in range(4):
        x ^= (x << 13) & 0xFFFFFFFFFFFFFFFF
        x ^= x >> 7
        x ^= (x << 17) & 0xFFFFFFFFFFFFFFFF
        assert r.below(1 << 63) == x % (1 << 63)


def test_a8_composition_integers_are_exact():
    rng = np.random.default_rng(5)
    tiles = []
    for _ in range(4):
        tiles.append([(rng.integers(-1, 2, 256).tolist(), [f16(0.02 + 0.01 * g) for g in range(2)]) for _ in range(2)])
    t = tensor_from_planes(2, 512, tiles)
    x = rng.standard_normal((3, 512)).astype(np.float32)
    y, dump, a = orc.a8_linear(t, x)
    q, s = orc.quantize_act_int8(x, 3, 512)
    assert np.array_equal(a, s)
    for m in range(3):
        for r in range(2):
            for g in range(4):
                tile, grp = r * 2 + g // 2, g % 2
                for p in range(2):
                    want = int(np.dot(t.trits[tile, p, grp * 128:(grp + 1) * 128].astype(np.int64),
                                      q[m, g * 128:(g + 1) * 128].astype(np.int64)))
                    assert dump[m, r, g, p] == want
                assert dump[m, r, g, 2] == 0
    assert np.array_equal(y, orc.matmul(t, q) * s[:, None])


def test_gather_rows_reconstructs_weights():
    t = cpu_matrix()
    w = dense_weights(t)
    got = orc.gather_rows(t, [2, 0])
    assert np.allclose(got, w[[2, 0]], rtol=0, atol=1e-6)


def test_salt_v1_restatement_against_dense_math():
    """SALT V1 (packed_salt.rs:612-661, tq2_0_add.cu:640-719): W = sum_p scale_p[block] * trit_p.  The
    reference holds no stored answers for this operator; its own contract is agreement with the dense
    fp32 matmul within 1e-4 (tq2_0_add.cu:650-653), which pins the restatement here."""
    rng = np.random.default_rng(5)
    t, n, k, m = 3, 9, 700, 4
    trits = rng.integers(-1, 2, (t, n, k)).astype(np.int8)
    nb = (k + 255) // 256
    block_scales = (0.01 + 0.05 * rng.random((t, n, nb))).astype(np.float16)
    planes = orc.salt_v1_pack(trits, block_scales.view(np.uint16))
    assert len(planes) == t * n * nb * 66
    act = rng.standard_normal((m, k)).astype(np.float32)
    got = orc.salt_v1_matmul(planes, t, n, k, act)
    dense = np.zeros((n, k), np.float64)
    for p in range(t):
        dense += trits[p].astype(np.float64) * np.repeat(block_scales[p].astype(np.float64), 256, axis=1)[:, :k]
    want = act.astype(np.float64) @ dense.T
    assert np.all(np.abs(got - want) <= 1e-4 * np.maximum(1.0, np.abs(want)))
    # SaltLinear::forward: quantise, project, scale
    q, s_ = orc.quantize_act_int8(act, m, k)
    want_a8 = (q.astype(np.float64) @ dense.T) * s_[:, None].astype(np.float64)
    got_a8 = orc.salt_v1_forward_a8(planes, t, n, k, act)
    assert np.all(np.abs(got_a8 - want_a8) <= 1e-4 * np.maximum(1.0, np.abs(want_a8)))


def test_tq1_block_goldens():
    """crates/tritium-format/src/tq1.rs:130-163: all-zero trits -> qs 0x80, qh 0x7F; all +1 -> qs 0xFF,
    qh 0xFD; all -1 -> 0x00; f16 1.0 scale in the last two bytes; decode of the zero block is zero."""
    for value, qs, qh in ((0, 0x80, 0x7F), (1, 0xFF, 0xFD), (-1, 0x00, 0x00)):
        block = np.frombuffer(orc.tq1_pack_rows(np.full((1, 256), value, np.int8)), np.uint8)
        assert np.all(block[:48] == qs) and np.all(block[48:52] == qh) and bytes(block[52:]) == b"\x00\x3c"
    zero = bytes([0x80] * 48 + [0x7F] * 4 + [0x00, 0x3C])
    assert np.all(orc.tq1_unpack_rows(zero, 1, 256) == 0)
    rng = np.random.default_rng(8)
    w = rng.integers(-1, 2, (5, 700)).astype(np.int8)
    assert np.array_equal(orc.tq1_unpack_rows(orc.tq1_pack_rows(w), 5, 700), w)


def test_rmsnorm_known_answers_and_canonical_order():
    """crates/tritium-nn/src/ops/rmsnorm.rs:101-110 (x = [3, 4], unit weights, eps 0: x / sqrt(12.5))
    and the canonical reduction order of rmsnorm.rs:20-34 restated here in numpy, slot by slot."""
    out = orc.rmsnorm(np.array([[3.0, 4.0]], np.float32), np.ones(2, np.float32), 0.0)
    inv = np.float32(1.0) / np.sqrt(np.float32(12.5))
    assert abs(out[0, 0] - np.float32(3.0) * inv) < 1e-6 and abs(out[0, 1] - np.float32(4.0) * inv) < 1e-6
    rng = np.random.default_rng(12)
    for n in (1, 255, 256, 257, 1000, 2560):
        x = (rng.standard_normal(n) * 5).astype(np.float32)
        w = rng.standard_normal(n).astype(np.float32)
        part = np.zeros(256, np.float32)
        for start in range(0, n, 256):                      # slot t folds x[t], x[t+256], ... ascending
            chunk = x[start:start + 256]
            part[:chunk.size] = part[:chunk.size] + chunk * chunk
        off = 128
        while off:
            part[:off] = part[:off] + part[off:2 * off]
            off >>= 1
        inv = np.float32(1.0) / np.sqrt(part[0] / np.float32(n) + np.float32(1e-5))
        assert np.array_equal(orc.rmsnorm(x[None], w, 1e-5)[0], x * inv * w)
        assert np.array_equal(orc.rmsnorm(x[None], w, 1e-5, zero_centered=True)[0], x * inv * (np.float32(1.0) + w))
