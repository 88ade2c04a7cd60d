"""Host-side mirror of tritium-format's SALT V2 types, backed by the C ABI's ``tb_fmt_*`` helpers.

Names follow the reference (crates/tritium-format/src/salt_v2.rs, src/salt_v2_package.rs):
``SaltV2Codec``, ``SaltV2Tensor``, ``pack_*``/``unpack_*``, ``write_salt_v2_package``.
"""
from __future__ import annotations

import ctypes as C
import enum
from dataclasses import dataclass

import numpy as np

from . import _lib
from .errors import InvalidInput, check

SALT_V2_ALLOCATION_TILE_SIZE = 256
SALT_V2_SCALE_GROUP_SIZE = 128
SALT_V2_SCALE_GROUP_SIZE_64 = 64
SALT_V2_MAX_PLANES = 3


class SaltV2Codec(enum.IntEnum):
    D2 = _lib.TB_CODEC_D2
    B3 = _lib.TB_CODEC_B3
    S34 = _lib.TB_CODEC_S34


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def pack(codec: SaltV2Codec, trits) -> bytes:
    """pack_d2 / pack_b3 / pack_s34 (salt_v2.rs:268-281,333-351,411-440)."""
    t = np.ascontiguousarray(trits, dtype=np.int8)
    L = _lib.load()
    n = L.tb_fmt_pack(int(codec), _ptr(t), C.c_size_t(t.size), None, C.c_size_t(0))
    if n < 0:
        check(-n)
    out = np.zeros(max(int(n), 1), np.uint8)
    n = L.tb_fmt_pack(int(codec), _ptr(t), C.c_size_t(t.size), _ptr(out), C.c_size_t(out.size))
    if n < 0:
        check(-n)
    return out[: int(n)].tobytes()


def unpack(codec: SaltV2Codec, packed: bytes, logical_trits: int) -> np.ndarray:
    """unpack_d2 / unpack_b3 / unpack_s34 with every canonical-form rejection."""
    b = np.frombuffer(bytes(packed), np.uint8).copy()
    out = np.zeros(max(logical_trits, 1), np.int8)
    check(_lib.load().tb_fmt_unpack(int(codec), _ptr(b), C.c_size_t(b.size), C.c_size_t(logical_trits), _ptr(out)))
    return out[:logical_trits]


def f16_bits(values) -> np.ndarray:
    """fp32 -> f16 bit patterns, round to nearest even (half::f16::from_f32)."""
    return np.asarray(values, dtype=np.float32).astype(np.float16).view(np.uint16)


@dataclass
class SaltV2Tensor:
    """A validated semantic tensor in dense host form (SaltV2Tensor, salt_v2_package.rs:520-700).

    ``trits[tile, plane, element]`` int8, ``scales[tile, plane, group]`` f16 bits,
    ``plane_count[tile]``; tiles cut the flattened row-major coefficient index every 256.
    """
    name: str
    rows: int
    cols: int
    plane_count: np.ndarray
    trits: np.ndarray
    scales: np.ndarray
    scale_group_size: int = SALT_V2_SCALE_GROUP_SIZE

    def __post_init__(self):
        self.plane_count = np.ascontiguousarray(self.plane_count, dtype=np.uint8)
        self.trits = np.ascontiguousarray(self.trits, dtype=np.int8)
        self.scales = np.ascontiguousarray(self.scales, dtype=np.uint16)
        tiles = self.tiles
        if self.plane_count.shape != (tiles,) or self.trits.shape != (tiles, 3, 256) or self.scales.shape != (tiles, 3, 4):
            raise InvalidInput(f"tensor arrays do not describe {tiles} tiles")

    @property
    def dims(self):
        return [self.rows, self.cols]

    @property
    def logical_coefficients(self) -> int:
        return self.rows * self.cols

    @property
    def tiles(self) -> int:
        return (self.rows * self.cols + 255) // 256

    @classmethod
    def from_matrix_planes(cls, name: str, trits: np.ndarray, scales_f32: np.ndarray, group: int = 128) -> "SaltV2Tensor":
        """Uniform-plane tensor from ``trits[P, N, K]`` and ``scales_f32[P, N, K // group]`` (K % 256 == 0)."""
        trits = np.asarray(trits, dtype=np.int8)
        p, n, k = trits.shape
        if k % 256:
            raise InvalidInput("from_matrix_planes needs k to be a multiple of 256")
        tiles = n * k // 256
        t = np.zeros((tiles, 3, 256), np.int8)
        t[:, :p, :] = trits.reshape(p, tiles, 256).transpose(1, 0, 2)
        gpt = 256 // group
        s = np.zeros((tiles, 3, 4), np.uint16)
        s[:, :p, :gpt] = f16_bits(scales_f32).reshape(p, tiles, gpt).transpose(1, 0, 2)
        return cls(name, n, k, np.full(tiles, p, np.uint8), t, s, group)

    def resident(self, codec: SaltV2Codec):
        """The indexed runtime arenas (SaltV2IndexedRuntimeLedger, salt_v2_package.rs:889-962):
        returns (payload u8, scales u16, plane_map u8, terminal_map_value, sizes)."""
        L = _lib.load()
        sz = _lib.ResidentSizes()
        check(L.tb_fmt_resident_sizes(int(codec), C.c_uint32(self.scale_group_size), C.c_uint64(self.rows),
                                      C.c_uint64(self.cols), _ptr(self.plane_count), C.byref(sz)))
        payload = np.zeros(max(sz.payload_bytes, 1), np.uint8)
        scales = np.zeros(max(sz.scale_count, 1), np.uint16)
        pmap = np.zeros(max(sz.map_bytes, 1), np.uint8)
        term = C.c_uint32(0)
        check(L.tb_fmt_resident_build(int(codec), C.c_uint32(self.scale_group_size), C.c_uint64(self.rows),
                                      C.c_uint64(self.cols), _ptr(self.plane_count), _ptr(self.trits),
                                      _ptr(self.scales), _ptr(payload), _ptr(scales), _ptr(pmap), C.byref(term)))
        return (payload[: sz.payload_bytes], scales[: sz.scale_count], pmap[: sz.map_bytes], term.value,
                {k: getattr(sz, k) for k, _ in _lib.ResidentSizes._fields_})

    def device_layout(self, codec: SaltV2Codec):
        """The payload and scale arenas as the uploads store them on the device (host-only twin):
        the artifact's own, except that S34 on a shape the fast kernels take is stored as B3 and
        that tiles with different plane counts on such a shape are padded to uniform plane slots
        with all-zero planes.  Returns (payload u8, scales u16, info dict)."""
        L = _lib.load()
        payload, scales, pmap, term, _ = self.resident(codec)
        args = (int(codec), C.c_uint32(self.scale_group_size), C.c_uint32(self.rows), C.c_uint32(self.cols),
                _ptr(payload), C.c_size_t(payload.size), _ptr(scales), C.c_size_t(scales.size),
                _ptr(pmap) if pmap.size else None, C.c_size_t(pmap.size), C.c_uint32(term))
        info = _lib.DeviceLayout()
        check(L.tb_fmt_device_layout(*args, C.byref(info), None, None))
        out_p = np.zeros(max(info.payload_bytes, 1), np.uint8)
        out_s = np.zeros(max(info.scale_count, 1), np.uint16)
        check(L.tb_fmt_device_layout(*args, C.byref(info), _ptr(out_p), _ptr(out_s)))
        return (out_p[: info.payload_bytes], out_s[: info.scale_count],
                {k: getattr(info, k) for k, _ in _lib.DeviceLayout._fields_})


def write_salt_v2_package(tensor: SaltV2Tensor, codec: SaltV2Codec) -> bytes:
    """write_salt_v2_package for a one-tensor package (salt_v2_package.rs:1526-1668)."""
    L = _lib.load()
    args = (int(codec), tensor.name.encode(), C.c_uint32(tensor.scale_group_size), C.c_uint64(tensor.rows),
            C.c_uint64(tensor.cols), _ptr(tensor.plane_count), _ptr(tensor.trits), _ptr(tensor.scales))
    n = L.tb_fmt_package_write(*args, None, C.c_size_t(0))
    if n < 0:
        check(-n)
    out = np.zeros(int(n), np.uint8)
    n = L.tb_fmt_package_write(*args, _ptr(out), C.c_size_t(out.size))
    if n < 0:
        check(-n)
    return out.tobytes()


def write_salt_v2_package_multi(tensors, codec: SaltV2Codec) -> bytes:
    """write_salt_v2_package for several matrix tensors in the given order (salt_v2_package.rs:1526-1668)."""
    L = _lib.load()
    count = len(tensors)
    names = (C.c_char_p * count)(*[t.name.encode() for t in tensors])
    groups = (C.c_uint32 * count)(*[t.scale_group_size for t in tensors])
    ns = (C.c_uint64 * count)(*[t.rows for t in tensors])
    ks = (C.c_uint64 * count)(*[t.cols for t in tensors])
    pcs = (C.c_void_p * count)(*[t.plane_count.ctypes.data for t in tensors])
    trits = (C.c_void_p * count)(*[t.trits.ctypes.data for t in tensors])
    scales = (C.c_void_p * count)(*[t.scales.ctypes.data for t in tensors])
    args = (int(codec), C.c_uint32(count), names, groups, ns, ks, pcs, trits, scales)
    n = L.tb_fmt_package_write_multi(*args, None, C.c_size_t(0))
    if n < 0:
        check(-n)
    out = np.zeros(int(n), np.uint8)
    n = L.tb_fmt_package_write_multi(*args, _ptr(out), C.c_size_t(out.size))
    if n < 0:
        check(-n)
    return out.tobytes()


def package_extract(fileobj, name: str):
    """The resident arenas of one tensor of a package file, read through seeks (the header table and
    that tensor's sections only): (info dict, payload u8, scales u16, plane_map u8)."""
    L = _lib.load()
    fileobj.seek(0, 2)
    length = fileobj.tell()
    cb = _lib.file_read_at(fileobj)
    info = _lib.PackageTensor()
    check(L.tb_fmt_package_extract(cb, None, C.c_uint64(length), name.encode(), C.byref(info), None, None, None))
    payload = np.zeros(max(info.payload_bytes, 1), np.uint8)
    scales = np.zeros(max(info.scale_count, 1), np.uint16)
    pmap = np.zeros(max(info.map_bytes, 1), np.uint8)
    check(L.tb_fmt_package_extract(cb, None, C.c_uint64(length), name.encode(), C.byref(info), _ptr(payload), _ptr(scales), _ptr(pmap)))
    meta = {k: getattr(info, k) for k, _ in _lib.PackageTensor._fields_}
    return meta, payload[: info.payload_bytes], scales[: info.scale_count], pmap[: info.map_bytes]


def pack_tq2_0_rows(trits: np.ndarray) -> bytes:
    """pack_tq2_0_row over [n, k] trits with unit block scales (rows.rs:61-77)."""
    t = np.ascontiguousarray(trits, dtype=np.int8)
    n, k = t.shape
    out = np.zeros(n * ((k + 255) // 256) * 66, np.uint8)
    check(_lib.load().tb_fmt_tq2_pack_rows(_ptr(t), C.c_uint64(n), C.c_uint64(k), _ptr(out)))
    return out.tobytes()


def pack_tq1_0_rows(trits: np.ndarray) -> bytes:
    """pack_tq1_0_block over [n, k] trits with unit block scales (crates/tritium-format/src/tq1.rs:36-78).
    Test vectors only: the product consumes TQ1_0 rows, it never has to produce them on the hot path."""
    trits = np.ascontiguousarray(trits, np.int8)
    n, k = trits.shape
    nb = (k + 255) // 256
    out = np.zeros((n, nb, 54), np.uint8)
    padded = np.zeros((n, nb * 256), np.int64)
    padded[:, :k] = trits
    x = (padded + 1).reshape(n, nb, 256)
    enc = lambda acc: ((acc * 256 + 242) // 243).astype(np.uint8)
    acc = np.zeros((n, nb, 32), np.int64)
    for d in range(5):
        acc = acc * 3 + x[:, :, d * 32:(d + 1) * 32]
    out[:, :, :32] = enc(acc)
    acc = np.zeros((n, nb, 16), np.int64)
    for d in range(5):
        acc = acc * 3 + x[:, :, 160 + d * 16:160 + (d + 1) * 16]
    out[:, :, 32:48] = enc(acc)
    acc = np.zeros((n, nb, 4), np.int64)
    for d in range(4):
        acc = acc * 3 + x[:, :, 240 + d * 4:240 + (d + 1) * 4]
    out[:, :, 48:52] = enc(acc * 3)
    out[:, :, 52], out[:, :, 53] = 0x00, 0x3C
    return out.tobytes()


def quantize_act_int8(act: np.ndarray, m: int, k: int):
    """quantize_act_int8 (crates/tritium-spec/src/lib.rs:351-378), host side."""
    a = np.ascontiguousarray(act, dtype=np.float32)
    q = np.zeros((m, k), np.float32)
    s = np.zeros(m, np.float32)
    _lib.load().tb_fmt_quantize_act_int8(_ptr(a), C.c_uint64(m), C.c_uint64(k), _ptr(q), _ptr(s))
    return q, s


def tp_shard(codec: SaltV2Codec, group: int, n: int, k: int, planes: int, payload: np.ndarray, scales: np.ndarray,
             row_parallel: bool, world: int, rank: int):
    """One rank's shard of a uniform-plane tensor: (n_s, k_s, payload, scales, plane_map, terminal).

    Column-parallel shards are byte slices of the arenas; row-parallel shards are re-encoded
    [n, k/world] tensors whose k is padded to whole tiles with zero trits."""
    L = _lib.load()
    sz = _lib.ShardSizes()
    check(L.tb_tp_shard_sizes(int(codec), C.c_uint32(group), C.c_uint32(n), C.c_uint32(k), C.c_uint32(planes),
                              int(row_parallel), C.c_uint32(world), C.c_uint32(rank), C.byref(sz)))
    payload = np.ascontiguousarray(payload, np.uint8)
    scales = np.ascontiguousarray(scales, np.uint16)
    sp = np.zeros(sz.payload_bytes, np.uint8)
    ss = np.zeros(sz.scale_count, np.uint16)
    sm = np.zeros(max(sz.map_bytes, 1), np.uint8)
    term = C.c_uint32(0)
    check(L.tb_tp_shard(int(codec), C.c_uint32(group), C.c_uint32(n), C.c_uint32(k), C.c_uint32(planes), _ptr(payload),
                        _ptr(scales), int(row_parallel), C.c_uint32(world), C.c_uint32(rank), _ptr(sp), _ptr(ss),
                        _ptr(sm), C.byref(term)))
    return sz.n, sz.k, sp, ss, sm[: sz.map_bytes], term.value
