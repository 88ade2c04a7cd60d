"""ctypes binding of the CPU oracle (``liboracle.so``).  TEST INFRASTRUCTURE ONLY.

Only the test suite, the smoke check and the CPU-baseline leg of the benchmark may import
this module; the product package never does.  Build the library with ``make -C oracle``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")

D2, B3, S34 = 1, 2, 3
TILE = 256


def build(force: bool = False) -> str:
    """Compile ``liboracle.so`` with the committed Makefile (gcc, no FMA contraction)."""
    src = os.path.join(_HERE, "tritium_oracle.c")
    hdr = os.path.join(_HERE, "tritium_oracle.h")
    stale = (not os.path.exists(_LIB_PATH)) or any(
        os.path.exists(p) and os.path.getmtime(p) > os.path.getmtime(_LIB_PATH) for p in (src, hdr)
    )
    if force or stale:
        subprocess.check_call(["make", "-C", _HERE, "-B", "liboracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


# root of the reference checkout: the TRITIUM_REFERENCE variable, else a `reference` folder beside this repository
_REF_ROOT = os.environ.get("TRITIUM_REFERENCE", os.path.normpath(os.path.join(_HERE, "..", "..", "reference")))


def build_reference_kernels() -> list:
    """Compile the reference's own TQ2_0 CUDA kernels into ``_ref/*.fatbin`` with the committed
    Makefile, where the reference checkout exists; otherwise return whatever was built before."""
    ref_dir = os.path.join(_HERE, "_ref")
    if os.path.isdir(os.path.join(_REF_ROOT, "crates", "tritium-cuda", "kernels")):
        subprocess.check_call(["make", "-C", _HERE, f"REF={_REF_ROOT}", "ref-kernels"], stdout=subprocess.DEVNULL)
    return sorted(f for f in (os.listdir(ref_dir) if os.path.isdir(ref_dir) else []) if f.endswith(".fatbin"))


class _CTensor(C.Structure):
    _fields_ = [
        ("rows", C.c_uint64), ("cols", C.c_uint64), ("rank", C.c_uint32), ("group", C.c_uint32),
        ("tiles", C.c_uint64), ("plane_count", C.c_void_p), ("trits", C.c_void_p),
        ("scales", C.c_void_p),
    ]


class _CNamed(C.Structure):
    _fields_ = [("name", C.c_char_p), ("tensor", _CTensor)]


class _CSizes(C.Structure):
    _fields_ = [
        ("payload_bytes", C.c_uint64), ("scale_bytes", C.c_uint64), ("map_bytes", C.c_uint64),
        ("rank_prefix_bytes", C.c_uint64), ("tiles", C.c_uint64), ("present_planes", C.c_uint64),
        ("terminal_map_value", C.c_uint32),
    ]


class _CFail(C.Structure):
    _fields_ = [("row", C.c_uint64), ("column", C.c_uint64), ("bits", C.c_uint32)]


class OracleError(Exception):
    def __init__(self, code: int, fail: "_CFail | None" = None):
        self.code = code
        self.row = fail.row if fail is not None else None
        self.column = fail.column if fail is not None else None
        self.bits = fail.bits if fail is not None else None
        super().__init__(f"oracle error {code} ({ERR.get(code, '?')}) row={self.row} column={self.column}")


ERR = {
    -1: "LENGTH", -2: "INVALID_CODE", -3: "PADDING", -4: "S34_SHAPE", -5: "PLANE_LEN", -6: "TRIT",
    -7: "SCALE_COUNT", -8: "SCALE_NONFINITE", -9: "SCALE_NEGATIVE", -10: "SCALE_ZERO_NONZERO_GROUP",
    -11: "PLANE_COUNT", -12: "GROUP_SIZE", -13: "SHAPE", -14: "MAGIC", -15: "VERSION", -16: "CODEC",
    -17: "FLAGS", -18: "TRUNCATED", -19: "TRAILING", -20: "NON_NESTED_MAP", -21: "NAME",
    -22: "TRANSFORM", -23: "NONFINITE_ACTIVATION", -24: "NONFINITE_OUTPUT", -25: "ALLOC",
    -26: "DUPLICATE_NAME",
}
CODE = {v: k for k, v in ERR.items()}

_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB_PATH)
        L.or_f32_to_f16.restype = C.c_uint16
        L.or_f32_to_f16.argtypes = [C.c_float]
        L.or_f16_to_f32.restype = C.c_float
        L.or_f16_to_f32.argtypes = [C.c_uint16]
        L.or_codec_pack.restype = C.c_long
        L.or_plane_pack.restype = C.c_long
        L.or_package_write.restype = C.c_long
        L.or_plane_payload_bytes.restype = C.c_size_t
        L.or_xs_next.restype = C.c_uint64
        L.or_xs_below.restype = C.c_uint64
        L.or_xs_activation.restype = C.c_float
        L.or_xs_scale.restype = C.c_float
        L.or_xs_trit.restype = C.c_int8
        _lib = L
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def f32_to_f16(v: float) -> int:
    return int(lib().or_f32_to_f16(C.c_float(v)))


def f16_to_f32(b: int) -> float:
    return float(lib().or_f16_to_f32(C.c_uint16(b)))


@dataclass
class Tensor:
    """Dense host form of a semantic SALT V2 tensor (tile, plane, element)."""
    rows: int
    cols: int
    group: int
    plane_count: np.ndarray  # uint8 [tiles]
    trits: np.ndarray        # int8  [tiles, 3, 256]
    scales: np.ndarray       # uint16 [tiles, 3, 4] (f16 bits)
    rank: int = 2

    @property
    def coeffs(self) -> int:
        return self.rows * self.cols

    @property
    def tiles(self) -> int:
        return (self.coeffs + TILE - 1) // TILE

    def c(self) -> _CTensor:
        self.plane_count = np.ascontiguousarray(self.plane_count, dtype=np.uint8)
        self.trits = np.ascontiguousarray(self.trits, dtype=np.int8)
        self.scales = np.ascontiguousarray(self.scales, dtype=np.uint16)
        assert self.trits.shape == (self.tiles, 3, TILE), self.trits.shape
        assert self.scales.shape == (self.tiles, 3, 4), self.scales.shape
        return _CTensor(self.rows, self.cols, self.rank, self.group, self.tiles,
                        _p(self.plane_count).value, _p(self.trits).value, _p(self.scales).value)

    def validate(self) -> None:
        ct = self.c()
        rc = lib().or_tensor_validate(C.byref(ct))
        if rc:
            raise OracleError(rc)

    def tile_len(self, t: int) -> int:
        return min(TILE, self.coeffs - t * TILE)


def tensor_from_planes(rows, cols, tiles_planes, group=128, rank=2) -> Tensor:
    """tiles_planes: list (per tile) of list (per plane) of (trits list, scales list[f16 bits])."""
    nt = (rows * cols + TILE - 1) // TILE
    assert len(tiles_planes) == nt
    pc = np.zeros(nt, np.uint8)
    tr = np.zeros((nt, 3, TILE), np.int8)
    sc = np.zeros((nt, 3, 4), np.uint16)
    for t, planes in enumerate(tiles_planes):
        pc[t] = len(planes)
        for p, (trits, scales) in enumerate(planes):
            tr[t, p, : len(trits)] = trits
            sc[t, p, : len(scales)] = scales
    return Tensor(rows, cols, group, pc, tr, sc, rank)


def ledger(codec: int, n: int):
    out = (C.c_uint64 * 4)()
    rc = lib().or_codec_ledger(codec, C.c_size_t(n), out)
    if rc:
        raise OracleError(rc)
    return dict(physical_bytes=out[0], padding_trits=out[1], padding_bits=out[2], encoded_bits=out[3])


def pack(codec: int, trits) -> bytes:
    t = np.ascontiguousarray(trits, dtype=np.int8)
    n = lib().or_codec_pack(codec, _p(t), C.c_size_t(t.size), None, C.c_size_t(0))
    if n < 0:
        raise OracleError(n)
    out = np.zeros(max(n, 1), np.uint8)
    n2 = lib().or_codec_pack(codec, _p(t), C.c_size_t(t.size), _p(out), C.c_size_t(n))
    if n2 < 0:
        raise OracleError(n2)
    return out[:n].tobytes()


def unpack(codec: int, packed: bytes, n: int) -> np.ndarray:
    b = np.frombuffer(packed, np.uint8).copy()
    out = np.zeros(max(n, 1), np.int8)
    rc = lib().or_codec_unpack(codec, _p(b), C.c_size_t(b.size), C.c_size_t(n), _p(out))
    if rc:
        raise OracleError(rc)
    return out[:n]


def plane_pack(codec: int, trits) -> bytes:
    t = np.ascontiguousarray(trits, dtype=np.int8)
    out = np.zeros(80, np.uint8)
    n = lib().or_plane_pack(codec, _p(t), C.c_size_t(t.size), _p(out), C.c_size_t(80))
    if n < 0:
        raise OracleError(n)
    return out[:n].tobytes()


def plane_unpack(codec: int, packed: bytes, n: int) -> np.ndarray:
    b = np.frombuffer(packed, np.uint8).copy()
    out = np.zeros(TILE, np.int8)
    rc = lib().or_plane_unpack(codec, _p(b), C.c_size_t(b.size), C.c_size_t(n), _p(out))
    if rc:
        raise OracleError(rc)
    return out[:n]


def resident_plan(t: Tensor, codec: int) -> dict:
    s = _CSizes()
    ct = t.c()
    rc = lib().or_resident_plan(C.byref(ct), codec, C.byref(s))
    if rc:
        raise OracleError(rc)
    return {k: getattr(s, k) for k, _ in _CSizes._fields_}


def resident_build(t: Tensor, codec: int):
    """Returns (payload u8, scales u16, index_metadata u8, terminal_map_value, plan)."""
    plan = resident_plan(t, codec)
    payload = np.zeros(plan["payload_bytes"] + 64, np.uint8)
    scales = np.zeros(plan["scale_bytes"] // 2 + 4, np.uint16)
    meta = np.zeros(plan["map_bytes"] + plan["rank_prefix_bytes"] + 8, np.uint8)
    term = C.c_uint32(0)
    ct = t.c()
    rc = lib().or_resident_build(C.byref(ct), codec, _p(payload), _p(scales), _p(meta), C.byref(term))
    if rc:
        raise OracleError(rc)
    return (payload[: plan["payload_bytes"]].copy(), scales[: plan["scale_bytes"] // 2].copy(),
            meta[: plan["map_bytes"] + plan["rank_prefix_bytes"]].copy(), term.value, plan)


def package_write(codec: int, named: list) -> bytes:
    arr = (_CNamed * len(named))()
    keep = []
    for i, (name, t) in enumerate(named):
        nb = name.encode() if isinstance(name, str) else name
        keep.append(nb)
        arr[i].name = nb
        arr[i].tensor = t.c()
    n = lib().or_package_write(codec, arr, C.c_size_t(len(named)), None, C.c_size_t(0))
    if n < 0:
        raise OracleError(n)
    out = np.zeros(n, np.uint8)
    n2 = lib().or_package_write(codec, arr, C.c_size_t(len(named)), _p(out), C.c_size_t(n))
    if n2 < 0:
        raise OracleError(n2)
    return out.tobytes()


def package_probe(data: bytes):
    b = np.frombuffer(data, np.uint8).copy()
    codec, count = C.c_int(0), C.c_uint32(0)
    rc = lib().or_package_probe(_p(b), C.c_size_t(b.size), C.byref(codec), C.byref(count))
    if rc:
        raise OracleError(rc)
    return codec.value, count.value


def package_read(data: bytes, index: int = 0):
    """Returns (name, Tensor, codec) after validating the whole package."""
    b = np.frombuffer(data, np.uint8).copy()
    codec, _ = package_probe(data)
    rows, cols, tiles = C.c_uint64(0), C.c_uint64(0), C.c_uint64(0)
    group, rank = C.c_uint32(0), C.c_uint32(0)
    name = C.create_string_buffer(4096)
    rc = lib().or_package_tensor_info(_p(b), C.c_size_t(b.size), C.c_uint32(index), C.byref(rows),
                                      C.byref(cols), C.byref(group), C.byref(tiles), C.byref(rank),
                                      name, C.c_size_t(4096))
    if rc:
        raise OracleError(rc)
    nt = tiles.value
    pc = np.zeros(nt, np.uint8)
    tr = np.zeros((nt, 3, TILE), np.int8)
    sc = np.zeros((nt, 3, 4), np.uint16)
    rc = lib().or_package_read_tensor(_p(b), C.c_size_t(b.size), C.c_uint32(index), _p(pc), _p(tr), _p(sc))
    if rc:
        raise OracleError(rc)
    return name.value.decode(), Tensor(rows.value, cols.value, group.value, pc, tr, sc, rank.value), codec


def matvec(t: Tensor, x) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    assert x.size == t.cols
    y = np.zeros(t.rows, np.float32)
    fail = _CFail()
    ct = t.c()
    rc = lib().or_matvec(C.byref(ct), _p(x), _p(y), C.byref(fail))
    if rc:
        raise OracleError(rc, fail)
    return y


def matmul(t: Tensor, x, threads: int = 1) -> np.ndarray:
    """[m, cols] -> [m, rows]; per-row arithmetic identical to matvec."""
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, t.cols)
    m = x.shape[0]
    y = np.zeros((m, t.rows), np.float32)
    ct = t.c()
    rc = lib().or_matmul_mt(C.byref(ct), _p(x), C.c_uint64(m), _p(y), C.c_int(threads))
    if rc:
        raise OracleError(rc)
    return y


def forward_packed(codec, group, rows, cols, payload, scales, meta, map_bytes, terminal, x) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, cols)
    m = x.shape[0]
    y = np.zeros((m, rows), np.float32)
    payload = np.ascontiguousarray(payload, np.uint8)
    scales = np.ascontiguousarray(scales, np.uint16)
    meta = np.ascontiguousarray(np.concatenate([meta, np.zeros(8, np.uint8)]), np.uint8)
    fail = _CFail()
    rc = lib().or_forward_packed(codec, C.c_uint32(group), C.c_uint64(rows), C.c_uint64(cols),
                                 _p(payload), _p(scales), _p(meta), C.c_uint64(map_bytes),
                                 C.c_uint32(terminal), _p(x), C.c_uint64(m), _p(y), C.byref(fail))
    if rc:
        raise OracleError(rc, fail)
    return y


def gather_rows(t: Tensor, rows) -> np.ndarray:
    r = np.ascontiguousarray(rows, dtype=np.uint32)
    out = np.zeros((r.size, t.cols), np.float32)
    ct = t.c()
    rc = lib().or_gather_rows(C.byref(ct), _p(r), C.c_uint64(r.size), _p(out))
    if rc:
        raise OracleError(rc)
    return out


def quantize_act_int8(x, m: int, k: int):
    x = np.ascontiguousarray(x, dtype=np.float32)
    q = np.zeros((m, k), np.float32)
    s = np.zeros(m, np.float32)
    lib().or_quantize_act_int8(_p(x), C.c_uint64(m), C.c_uint64(k), _p(q), _p(s))
    return q, s


def a8_linear(t: Tensor, x, dump: bool = True):
    """Returns (y [m, rows] f32, I [m, rows, groups_per_row, 3] int32 or None, act_scale [m])."""
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, t.cols)
    m = x.shape[0]
    y = np.zeros((m, t.rows), np.float32)
    segs = (t.cols + t.group - 1) // t.group
    d = np.zeros((m, t.rows, segs, 3), np.int32) if dump else None
    a = np.zeros(m, np.float32)
    ct = t.c()
    rc = lib().or_a8_linear(C.byref(ct), _p(x), C.c_uint64(m), _p(y), _p(d) if dump else None, _p(a))
    if rc:
        raise OracleError(rc)
    return y, d, a


def tq2_pack_rows(trits: np.ndarray, block_scale_bits: int = 0x3C00) -> bytes:
    """[n, k] int8 -> n rows of ceil(k/256)*66 bytes (block scale defaults to f16 1.0)."""
    trits = np.ascontiguousarray(trits, dtype=np.int8)
    n, k = trits.shape
    nb = (k + 255) // 256
    out = np.zeros((n, nb * 66), np.uint8)
    sc = np.full(nb, block_scale_bits, np.uint16)
    for r in range(n):
        rc = lib().or_tq2_pack_row(_p(trits[r]), C.c_uint64(k), _p(sc), _p(out[r]))
        if rc:
            raise OracleError(rc)
    return out.tobytes()


def tq2_unpack_rows(packed: bytes, n: int, k: int) -> np.ndarray:
    nb = (k + 255) // 256
    b = np.frombuffer(packed, np.uint8).reshape(n, nb * 66).copy()
    out = np.zeros((n, k), np.int8)
    for r in range(n):
        rc = lib().or_tq2_unpack_row(_p(b[r]), C.c_uint64(k), _p(out[r]), None)
        if rc:
            raise OracleError(rc)
    return out


def tq1_pack_rows(trits: np.ndarray, block_scale_bits: int = 0x3C00) -> bytes:
    """[n, k] int8 -> n rows of ceil(k/256)*54 bytes (TQ1_0; block scale defaults to f16 1.0)."""
    trits = np.ascontiguousarray(trits, dtype=np.int8)
    n, k = trits.shape
    nb = (k + 255) // 256
    out = np.zeros((n, nb * 54), np.uint8)
    sc = np.full(nb, block_scale_bits, np.uint16)
    for r in range(n):
        rc = lib().or_tq1_pack_row(_p(trits[r]), C.c_uint64(k), _p(sc), _p(out[r]))
        if rc:
            raise OracleError(rc)
    return out.tobytes()


def tq1_unpack_rows(packed: bytes, n: int, k: int) -> np.ndarray:
    nb = (k + 255) // 256
    b = np.frombuffer(packed, np.uint8).reshape(n, nb * 54).copy()
    out = np.zeros((n, k), np.int8)
    for r in range(n):
        rc = lib().or_tq1_unpack_row(_p(b[r]), C.c_uint64(k), _p(out[r]), None)
        if rc:
            raise OracleError(rc)
    return out


def salt_v1_pack(trits: np.ndarray, block_scales: np.ndarray) -> bytes:
    """trits[T, n, k] int8 and block_scales[T, n, ceil(k/256)] f16 bits -> plane-major TQ2_0 rows."""
    trits = np.ascontiguousarray(trits, np.int8)
    t, n, k = trits.shape
    nb = (k + 255) // 256
    out = np.zeros((t, n, nb * 66), np.uint8)
    for p in range(t):
        for r in range(n):
            sc = np.ascontiguousarray(block_scales[p, r], np.uint16)
            rc = lib().or_tq2_pack_row(_p(trits[p, r]), C.c_uint64(k), _p(sc), _p(out[p, r]))
            if rc:
                raise OracleError(rc)
    return out.tobytes()


def salt_v1_matmul(planes: bytes, t_planes: int, n: int, k: int, act) -> np.ndarray:
    """PackedSaltMatrix::row_dot over every row (packed_salt.rs:612-661); act [m, k] f32."""
    act = np.ascontiguousarray(act, np.float32).reshape(-1, k)
    m = act.shape[0]
    buf = np.frombuffer(planes, np.uint8)
    out = np.zeros((m, n), np.float32)
    rc = lib().or_salt_v1_matmul(_p(buf), C.c_uint32(t_planes), C.c_uint64(n), C.c_uint64(k), _p(act), C.c_uint64(m), _p(out))
    if rc:
        raise OracleError(rc)
    return out


def salt_v1_forward_a8(planes: bytes, t_planes: int, n: int, k: int, act) -> np.ndarray:
    """SaltLinear::forward (crates/tritium-nn/src/layers/salt.rs:114-147): quantise, project, scale."""
    act = np.ascontiguousarray(act, np.float32).reshape(-1, k)
    q, s = quantize_act_int8(act, act.shape[0], k)
    y = salt_v1_matmul(planes, t_planes, n, k, q)
    return y * s[:, None]


def rmsnorm(x, w, eps: float, zero_centered: bool = False) -> np.ndarray:
    """rmsnorm / rmsnorm_zero_centered row by row (crates/tritium-nn/src/ops/rmsnorm.rs:43-94); x [m, k] f32."""
    w = np.ascontiguousarray(w, np.float32)
    x = np.ascontiguousarray(x, np.float32).reshape(-1, w.size)
    out = np.zeros_like(x)
    L = lib()
    for t in range(x.shape[0]):
        L.or_rmsnorm(_p(x[t]), _p(w), C.c_float(eps), C.c_int(int(zero_centered)), C.c_uint64(w.size), _p(out[t]))
    return out


def relu2_gate(gate, up) -> np.ndarray:
    """tritium_nn::layers::mlp gating loop = relu2_gate_f32 (crates/tritium-cuda/kernels/decode.cu:764-780):
    r = max(g, 0); out = (r * r) * u, left-associated single-precision products."""
    g = np.ascontiguousarray(gate, np.float32)
    u = np.ascontiguousarray(up, np.float32)
    r = np.maximum(g, np.float32(0.0))
    return ((r * r).astype(np.float32) * u).astype(np.float32)


def norm_a8_linear(tensor, x, norm_weight, eps: float, zero_centered: bool = False, residual=None):
    """The decode block's fused step: rmsnorm, per-token int8 quantisation, packed linear, then
    ``residual + y`` in one rounding (crates/tritium-cuda/kernels/decode.cu:533-640 for the
    prologue, crates/tritium-cuda/kernels/tq2_0_add.cu:577-637 for the residual epilogue)."""
    y = a8_linear(tensor, rmsnorm(x, norm_weight, eps, zero_centered), dump=False)[0]
    if residual is not None:
        y = (np.ascontiguousarray(residual, np.float32).reshape(y.shape) + y).astype(np.float32)
    return y


def reference_mpgemm(act, w, scales, m, n, k) -> np.ndarray:
    act = np.ascontiguousarray(act, np.float32)
    w = np.ascontiguousarray(w, np.int8)
    scales = np.ascontiguousarray(scales, np.float32)
    out = np.zeros((m, n), np.float32)
    lib().or_reference_mpgemm(_p(act), _p(w), _p(scales), C.c_uint64(m), C.c_uint64(n), C.c_uint64(k), _p(out))
    return out


def mpgemm_with_act_quant(act, w, scales, m, n, k) -> np.ndarray:
    act = np.ascontiguousarray(act, np.float32)
    w = np.ascontiguousarray(w, np.int8)
    scales = np.ascontiguousarray(scales, np.float32)
    out = np.zeros((m, n), np.float32)
    lib().or_mpgemm_with_act_quant(_p(act), _p(w), _p(scales), C.c_uint64(m), C.c_uint64(n), C.c_uint64(k), _p(out))
    return out


class XorShift64:
    """crates/tritium-testkit/src/generate.rs:18-56"""

    class _S(C.Structure):
        _fields_ = [("state", C.c_uint64)]

    def __init__(self, seed: int):
        self.s = XorShift64._S()
        lib().or_xs_seed(C.byref(self.s), C.c_uint64(seed))

    def perturb(self, i: int) -> None:
        self.s.state ^= ((i * 0x9E3779B97F4A7C15) & 0xFFFFFFFFFFFFFFFF) | 1

    def below(self, n: int) -> int:
        return int(lib().or_xs_below(C.byref(self.s), C.c_uint64(n)))

    def activation(self) -> float:
        return float(lib().or_xs_activation(C.byref(self.s)))

    def scale(self) -> float:
        return float(lib().or_xs_scale(C.byref(self.s)))

    def trit(self) -> int:
        return int(lib().or_xs_trit(C.byref(self.s)))
