"""ctypes binding of ``libtritium_b200.so`` (the C ABI declared in ``include/tritium_b200.h``).

The library is the product; there is no Python or CPU fallback for any compute entry point.
Loading fails loudly when the shared object is missing and cannot be built.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_lib", "libtritium_b200.so")

TB_OK, TB_NULL_ARG, TB_SHAPE_MISMATCH, TB_UNSUPPORTED_FORMAT, TB_OUT_OF_MEMORY, TB_INVALID_INPUT, TB_BACKEND, TB_TIMEOUT = range(8)
TB_CODEC_D2, TB_CODEC_B3, TB_CODEC_S34 = 1, 2, 3
TB_F32, TB_BF16, TB_I8 = 0, 1, 2
TB_COMM_HANDLE_BYTES = 64
TB_FWD_A8, TB_FWD_EXACT, TB_FWD_PDL, TB_FWD_FORCE_DECODE, TB_FWD_FORCE_PREFILL = 1, 2, 4, 8, 16

EXPORTS = [
    "tb_abi_version", "tb_last_error", "tb_backend_create", "tb_backend_free", "tb_backend_caps",
    "tb_backend_synchronize", "tb_backend_reserve", "tb_backend_check", "tb_tq2_upload",
    "tb_salt_v2_upload", "tb_salt_v2_upload_package", "tb_weights_info_get", "tb_weights_free",
    "tb_salt_v2_forward_exact", "tb_linear_forward_f32", "tb_linear_forward_a8",
    "tb_salt_v2_gather_rows", "tb_linear_forward_dev", "tb_norm_linear_forward_dev", "tb_act_absmax_dev",
    "tb_linear_forward_tp_dev", "tb_block_linear_forward_tp_dev", "tb_comm_create", "tb_comm_export", "tb_comm_connect", "tb_comm_slot", "tb_comm_allreduce_f32", "tb_comm_set_wait_limit", "tb_comm_disconnect", "tb_comm_free", "tb_mpgemm", "tb_mpgemm_with_act_quant",
    "tb_stack_create", "tb_stack_forward_dev", "tb_stack_forward_host", "tb_stack_bytes_per_step", "tb_stack_read_output", "tb_stack_free",
    "tb_tp_shard_sizes", "tb_tp_shard", "tb_fmt_pack", "tb_fmt_unpack", "tb_fmt_plane_bytes",
    "tb_fmt_resident_sizes", "tb_fmt_resident_build", "tb_fmt_package_write", "tb_fmt_tq2_pack_rows",
    "tb_fmt_quantize_act_int8", "tb_linear_forward_a8_static", "tb_backend_inject_wait_timeout",
    "tb_salt_v2_upload_reader", "tb_fmt_package_write_multi", "tb_fmt_package_extract", "tb_last_shape_mismatch", "tb_salt_v1_upload", "tb_tq1_upload",
    "tb_fmt_device_layout",
]


class Caps(C.Structure):
    _fields_ = [("backend", C.c_char * 16), ("device_name", C.c_char * 128), ("device_id", C.c_char * 32),
                ("physical_id", C.c_char * 96), ("features", C.c_char * 192),
                ("total_memory_bytes", C.c_uint64), ("sm_count", C.c_uint32),
                ("supports_imma", C.c_uint32), ("supports_fp8", C.c_uint32)]


class Receipt(C.Structure):
    _fields_ = [("payload_bytes", C.c_uint64), ("scale_bytes", C.c_uint64), ("map_bytes", C.c_uint64),
                ("rank_prefix_bytes", C.c_uint64), ("activation_bytes", C.c_uint64),
                ("output_bytes", C.c_uint64), ("dense_weight_bytes", C.c_uint64),
                ("kernel", C.c_uint32), ("launches", C.c_uint32)]


class WeightsInfo(C.Structure):
    _fields_ = [("codec", C.c_uint32), ("group", C.c_uint32), ("planes_uniform", C.c_uint32),
                ("n", C.c_uint64), ("k", C.c_uint64), ("tiles", C.c_uint64), ("present_planes", C.c_uint64),
                ("payload_bytes", C.c_uint64), ("scale_bytes", C.c_uint64), ("map_bytes", C.c_uint64),
                ("rank_prefix_bytes", C.c_uint64), ("source_len_bytes", C.c_uint64), ("fast_path", C.c_uint32)]


class ForwardArgs(C.Structure):
    _fields_ = [("x", C.c_void_p), ("x_dtype", C.c_int), ("act_scale", C.c_void_p), ("act_absmax", C.c_void_p),
                ("m", C.c_uint32), ("y", C.c_void_p), ("y_dtype", C.c_int), ("acc_dump", C.c_void_p),
                ("row_scale", C.c_void_p), ("flags", C.c_uint32), ("stream", C.c_void_p)]


class NormLinearArgs(C.Structure):
    _fields_ = [("x", C.c_void_p), ("x_dtype", C.c_int), ("norm_weight", C.c_void_p), ("norm_eps", C.c_float),
                ("norm_flags", C.c_uint32), ("residual", C.c_void_p), ("m", C.c_uint32), ("y", C.c_void_p),
                ("y_dtype", C.c_int), ("flags", C.c_uint32), ("stream", C.c_void_p), ("relu2_up", C.c_void_p)]


TB_NORM_ZERO_CENTERED = 1


def stream_handle(stream) -> int:
    """cudaStream_t of a torch stream for the C ABI.  The ABI reads NULL as "the backend's own
    stream", which is non-blocking and therefore not ordered with anything torch does; torch's
    default stream has the handle 0, so it is passed as cudaStreamLegacy (0x1), which names the
    legacy default stream explicitly."""
    handle = int(stream.cuda_stream)
    return handle if handle else 1

READ_AT_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_uint64, C.c_void_p, C.c_size_t)


class PackageTensor(C.Structure):
    _fields_ = [("codec", C.c_uint32), ("group", C.c_uint32), ("terminal_map_value", C.c_uint32), ("planes_uniform", C.c_uint32),
                ("n", C.c_uint64), ("k", C.c_uint64), ("payload_bytes", C.c_uint64), ("scale_count", C.c_uint64),
                ("map_bytes", C.c_uint64)]


class DeviceLayout(C.Structure):
    _fields_ = [("codec", C.c_uint32), ("planes_uniform", C.c_uint32), ("recoded", C.c_uint32), ("counts_from_map", C.c_uint32),
                ("payload_bytes", C.c_uint64), ("scale_count", C.c_uint64)]


def file_read_at(fileobj):
    """A tb_read_at_fn over a seekable binary file object; keep the returned object alive while it is in use."""
    def read_at(_user, offset, dst, length):
        try:
            fileobj.seek(offset)
            data = fileobj.read(length)
            if len(data) != length:
                return 1
            C.memmove(dst, data, length)
            return 0
        except Exception:
            return 2
    return READ_AT_FN(read_at)


class ShardSizes(C.Structure):
    _fields_ = [("n", C.c_uint32), ("k", C.c_uint32), ("payload_bytes", C.c_uint64),
                ("scale_count", C.c_uint64), ("map_bytes", C.c_uint64)]


class ResidentSizes(C.Structure):
    _fields_ = [("payload_bytes", C.c_uint64), ("scale_count", C.c_uint64), ("map_bytes", C.c_uint64),
                ("rank_prefix_bytes", C.c_uint64), ("tiles", C.c_uint64), ("present_planes", C.c_uint64)]


_lib = None

# (restype, argtypes) of every export, in the order of include/tritium_b200.h.  Pointers to
# opaque handles, structs and buffers are all c_void_p: ctypes then accepts byref(), arrays,
# c_void_p values, ints and None alike, and checks the argument count and the integer widths.
_P, _U32, _U64, _SZ, _I = C.c_void_p, C.c_uint32, C.c_uint64, C.c_size_t, C.c_int
_ST = C.c_int
_SIGNATURES = {
    "tb_abi_version": (C.c_uint32, []),
    "tb_last_error": (C.c_char_p, []),
    "tb_last_shape_mismatch": (_ST, [_P, _P]),
    "tb_backend_create": (_ST, [_I, _P]),
    "tb_backend_free": (None, [_P]),
    "tb_backend_caps": (_ST, [_P, _P]),
    "tb_backend_synchronize": (_ST, [_P]),
    "tb_tq2_upload": (_ST, [_P, _P, _SZ, _U32, _U32, _P]),
    "tb_tq1_upload": (_ST, [_P, _P, _SZ, _U32, _U32, _P]),
    "tb_salt_v1_upload": (_ST, [_P, _P, _SZ, _U32, _U32, _U32, _P]),
    "tb_salt_v2_upload": (_ST, [_P, _I, _U32, _U32, _U32, _P, _SZ, _P, _SZ, _P, _SZ, _U32, _P]),
    "tb_salt_v2_upload_package": (_ST, [_P, _P, _SZ, C.c_char_p, _P]),
    "tb_weights_info_get": (_ST, [_P, _P]),
    "tb_weights_free": (None, [_P]),
    "tb_salt_v2_forward_exact": (_ST, [_P, _P, _P, _U32, _P, _P]),
    "tb_linear_forward_f32": (_ST, [_P, _P, _P, _U32, _P, _P]),
    "tb_linear_forward_a8": (_ST, [_P, _P, _P, _I, _U32, _P, _I, _P, _P]),
    "tb_salt_v2_gather_rows": (_ST, [_P, _P, _P, _SZ, _P]),
    "tb_linear_forward_dev": (_ST, [_P, _P, _P, _P]),
    "tb_norm_linear_forward_dev": (_ST, [_P, _P, _P, _P]),
    "tb_linear_forward_a8_static": (_ST, [_P, _P, _P, _I, _P, _U32, _P, _I, _P]),
    "tb_act_absmax_dev": (_ST, [_P, _P, _I, _U32, _U32, _P, _P]),
    "tb_backend_reserve": (_ST, [_P, _P, _U32]),
    "tb_backend_check": (_ST, [_P, _P]),
    "tb_backend_inject_wait_timeout": (_ST, [_P, _U32]),
    "tb_mpgemm": (_ST, [_P, _P, _P, _P, _U32, _U32, _U32, _P]),
    "tb_mpgemm_with_act_quant": (_ST, [_P, _P, _P, _P, _U32, _U32, _U32, _P]),
    "tb_stack_create": (_ST, [_P, _P, _P, _U32, _U32, _P]),
    "tb_stack_forward_dev": (_ST, [_P, _P, _I, _U32, _P, _I, _U32, _P]),
    "tb_stack_forward_host": (_ST, [_P, _P, _I, _U32, _P, _U32]),
    "tb_stack_bytes_per_step": (C.c_uint64, [_P, _U32]),
    "tb_stack_read_output": (_ST, [_P, _U32, _U32, _P]),
    "tb_stack_free": (None, [_P]),
    "tb_block_linear_forward_tp_dev": (_ST, [_P, _P, _P, _U32, _U32, _P]),
    "tb_comm_create": (_ST, [_P, _U32, _U32, _SZ, _U32, _U32, _P]),
    "tb_comm_export": (_ST, [_P, _P]),
    "tb_comm_connect": (_ST, [_P, _P]),
    "tb_comm_slot": (C.c_void_p, [_P, _U32]),
    "tb_comm_allreduce_f32": (_ST, [_P, _U32, _U32, _I, _P, _P]),
    "tb_linear_forward_tp_dev": (_ST, [_P, _P, _P, _U32, _U32, _P, _I, _U32, _P, _I, _U32, _P]),
    "tb_comm_set_wait_limit": (_ST, [_P, C.c_uint64]),
    "tb_comm_disconnect": (_ST, [_P]),
    "tb_comm_free": (None, [_P]),
    "tb_tp_shard_sizes": (_ST, [_I, _U32, _U32, _U32, _U32, _I, _U32, _U32, _P]),
    "tb_tp_shard": (_ST, [_I, _U32, _U32, _U32, _U32, _P, _P, _I, _U32, _U32, _P, _P, _P, _P]),
    "tb_fmt_pack": (C.c_int64, [_I, _P, _SZ, _P, _SZ]),
    "tb_fmt_unpack": (_ST, [_I, _P, _SZ, _SZ, _P]),
    "tb_fmt_plane_bytes": (C.c_size_t, [_I, _SZ]),
    "tb_fmt_resident_sizes": (_ST, [_I, _U32, _U64, _U64, _P, _P]),
    "tb_fmt_resident_build": (_ST, [_I, _U32, _U64, _U64, _P, _P, _P, _P, _P, _P, _P]),
    "tb_fmt_package_write": (C.c_int64, [_I, C.c_char_p, _U32, _U64, _U64, _P, _P, _P, _P, _SZ]),
    "tb_fmt_tq2_pack_rows": (_ST, [_P, _U64, _U64, _P]),
    "tb_salt_v2_upload_reader": (_ST, [_P, _P, _P, _U64, C.c_char_p, _P]),
    "tb_fmt_package_write_multi": (C.c_int64, [_I, _U32, _P, _P, _P, _P, _P, _P, _P, _P, _SZ]),
    "tb_fmt_package_extract": (_ST, [_P, _P, _U64, C.c_char_p, _P, _P, _P, _P]),
    "tb_fmt_quantize_act_int8": (None, [_P, _U64, _U64, _P, _P]),
    "tb_fmt_device_layout": (_ST, [_I, _U32, _U32, _U32, _P, _SZ, _P, _SZ, _P, _SZ, _U32, _P, _P, _P]),
}


def _declare(L: C.CDLL) -> None:
    missing = [name for name in EXPORTS if name not in _SIGNATURES]
    if missing:
        raise RuntimeError(f"no signature recorded for {missing}")
    for name, (restype, argtypes) in _SIGNATURES.items():
        fn = getattr(L, name)
        fn.restype = restype
        fn.argtypes = argtypes


def load(build_if_missing: bool = True) -> C.CDLL:
    """Load the shared library, building it in-tree first when it is absent."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        if not build_if_missing:
            raise RuntimeError(f"{LIB_PATH} is missing: run tritium_b200/build.py (there is no fallback path)")
        from . import build as _build
        _build.build()
    L = C.CDLL(LIB_PATH)
    _declare(L)
    _lib = L
    return L


def last_error() -> str:
    msg = load().tb_last_error()
    return msg.decode() if msg else ""
