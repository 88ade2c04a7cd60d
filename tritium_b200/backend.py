"""Python host side of the B200 backend, mirroring the reference's backend interface.

``B200Backend`` carries the ``TernaryBackend`` trait methods (crates/tritium-spec/src/lib.rs:166-333)
and the concrete SALT V2 methods callers reach by downcast
(crates/tritium-cuda/src/cuda/backend.rs:7463-7701); every compute call goes through the C ABI in
``libtritium_b200.so``.  torch is used only for device memory and streams.
"""
from __future__ import annotations

import ctypes as C
import enum
from dataclasses import dataclass, field

import numpy as np

from . import _lib
from .errors import BackendError, InvalidInput, ShapeMismatch, UnsupportedFormat, check
from .format import SaltV2Codec, SaltV2Tensor


class TernaryFormat(enum.Enum):
    """crates/tritium-core/src/dtype.rs:89-108"""
    Tq1_0 = "tq1_0"
    Tq2_0 = "tq2_0"
    I2sInt8 = "i2s_int8"


@dataclass(frozen=True)
class GemmShape:
    """crates/tritium-core/src/shape.rs:10-38: act [M,K], weights [N,K], out [M,N]."""
    m: int
    n: int
    k: int


@dataclass
class DeviceCaps:
    """crates/tritium-spec/src/caps.rs:7-68"""
    backend: str
    device_name: str
    features: list
    total_memory_bytes: int
    supports_imma: bool
    supports_fp8: bool
    sm_count: int = 0


@dataclass
class MpGemm:
    """crates/tritium-spec/src/lib.rs:64-78"""
    act: np.ndarray
    weights: "DeviceBuffer"
    scales: np.ndarray
    shape: GemmShape
    format: TernaryFormat
    out: np.ndarray


@dataclass
class SaltV2ForwardReceipt:
    """Byte receipt of one forward call (crates/tritium-cuda/src/cuda/backend.rs:321-405)."""
    payload_bytes: int = 0
    scale_bytes: int = 0
    map_bytes: int = 0
    rank_prefix_bytes: int = 0
    activation_bytes: int = 0
    output_bytes: int = 0
    dense_weight_bytes: int = 0
    kernel: int = 0
    launches: int = 0
    mode: str = "Exact"

    def steady_resident_bytes(self) -> int:
        return self.payload_bytes + self.scale_bytes + self.map_bytes + self.rank_prefix_bytes

    def algorithmic_bytes(self) -> int:
        return self.steady_resident_bytes() + self.activation_bytes + self.output_bytes


@dataclass
class SaltV2Forward:
    output: np.ndarray
    receipt: SaltV2ForwardReceipt


class DeviceBuffer:
    """Opaque owner of device-resident weights (crates/tritium-spec/src/lib.rs:147-158)."""

    def __init__(self, backend: "B200Backend", handle: int):
        self._backend = backend
        self._h = C.c_void_p(handle)
        info = _lib.WeightsInfo()
        check(_lib.load().tb_weights_info_get(self._h, C.byref(info)))
        self.info = {k: getattr(info, k) for k, _ in _lib.WeightsInfo._fields_}

    def len_bytes(self) -> int:
        return int(self.info["source_len_bytes"])

    def is_empty(self) -> bool:
        return self.len_bytes() == 0

    @property
    def rows(self) -> int:
        return int(self.info["n"])

    @property
    def columns(self) -> int:
        return int(self.info["k"])

    def free(self) -> None:
        if self._h:
            _lib.load().tb_weights_free(self._h)
            self._h = C.c_void_p(None)

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class SaltV2ResidentTensor(DeviceBuffer):
    """crates/tritium-cuda/src/cuda/backend.rs:196-265"""

    def allocation_receipt(self) -> dict:
        i = self.info
        return dict(payload_bytes=i["payload_bytes"], scale_bytes=i["scale_bytes"], map_bytes=i["map_bytes"],
                    rank_prefix_bytes=i["rank_prefix_bytes"], dense_weight_bytes=0,
                    steady_resident_bytes=i["payload_bytes"] + i["scale_bytes"] + i["map_bytes"] + i["rank_prefix_bytes"])


_NP_DTYPE = {np.dtype(np.float32): _lib.TB_F32, np.dtype(np.int8): _lib.TB_I8}


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


class B200Backend:
    """The backend a registry entry named ``b200`` constructs."""

    def __init__(self, ordinal: int = 0):
        self._L = _lib.load()
        h = C.c_void_p(None)
        check(self._L.tb_backend_create(int(ordinal), C.byref(h)))
        self._h = h
        self.ordinal = ordinal
        caps = _lib.Caps()
        check(self._L.tb_backend_caps(self._h, C.byref(caps)))
        self._caps = caps

    # ---- TernaryBackend --------------------------------------------------------------
    def device_id(self) -> str:
        return self._caps.device_id.decode()

    def physical_device_id(self) -> str:
        return self._caps.physical_id.decode()

    def capabilities(self) -> DeviceCaps:
        c = self._caps
        return DeviceCaps(c.backend.decode(), c.device_name.decode(), c.features.decode().split(","),
                          int(c.total_memory_bytes), bool(c.supports_imma), bool(c.supports_fp8), int(c.sm_count))

    def upload_weights(self, packed: bytes, shape: GemmShape, format: TernaryFormat) -> DeviceBuffer:
        if format not in (TernaryFormat.Tq2_0, TernaryFormat.Tq1_0):
            raise UnsupportedFormat(f"unsupported ternary format: {format}")
        buf = np.frombuffer(bytes(packed), np.uint8)
        h = C.c_void_p(None)
        upload = self._L.tb_tq2_upload if format == TernaryFormat.Tq2_0 else self._L.tb_tq1_upload
        check(upload(self._h, _ptr(buf), C.c_size_t(buf.size), C.c_uint32(shape.n), C.c_uint32(shape.k), C.byref(h)))
        out = DeviceBuffer(self, h.value)
        out.format = format
        return out

    def _check_mpgemm(self, p: MpGemm):
        m, n, k = p.shape.m, p.shape.n, p.shape.k
        if not isinstance(p.weights, DeviceBuffer) or p.weights._backend is not self:
            raise InvalidInput("buffer is not a B200 buffer of this backend")
        if p.format not in (TernaryFormat.Tq2_0, TernaryFormat.Tq1_0) or getattr(p.weights, "format", p.format) != p.format:
            raise UnsupportedFormat(f"unsupported ternary format: {p.format}")
        for arr, want in ((p.act, m * k), (p.scales, n), (p.out, m * n)):
            if arr.size != want:
                raise ShapeMismatch(f"shape mismatch: expected {want}, got {arr.size}")
        if p.out.dtype != np.float32 or not p.out.flags.c_contiguous:
            raise InvalidInput("out must be a contiguous float32 array")
        return m, n, k

    def mpgemm(self, p: MpGemm) -> None:
        m, n, k = self._check_mpgemm(p)
        act = np.ascontiguousarray(p.act, np.float32)
        scales = np.ascontiguousarray(p.scales, np.float32)
        check(self._L.tb_mpgemm(self._h, p.weights._h, _ptr(act), _ptr(scales), C.c_uint32(m), C.c_uint32(n), C.c_uint32(k), _ptr(p.out)))

    def mpgemm_with_act_quant(self, p: MpGemm) -> None:
        m, n, k = self._check_mpgemm(p)
        act = np.ascontiguousarray(p.act, np.float32)
        scales = np.ascontiguousarray(p.scales, np.float32)
        check(self._L.tb_mpgemm_with_act_quant(self._h, p.weights._h, _ptr(act), _ptr(scales), C.c_uint32(m), C.c_uint32(n), C.c_uint32(k), _ptr(p.out)))

    def mpgemm_projected_vjp(self, *_args, **_kw):
        raise BackendError(f"backend `{self.device_id()}` does not implement packed mpGEMM VJP")

    def as_concrete(self):
        return self

    # ---- SALT V2 (reached by downcast in the reference) ---------------------------------
    def upload_salt_v2(self, tensor: SaltV2Tensor, codec: SaltV2Codec) -> SaltV2ResidentTensor:
        payload, scales, pmap, terminal, _ = tensor.resident(codec)
        return self.upload_salt_v2_arenas(codec, tensor.scale_group_size, tensor.rows, tensor.cols, payload, scales, pmap, terminal)

    def upload_salt_v2_arenas(self, codec, group, n, k, payload, scales, plane_map, terminal) -> SaltV2ResidentTensor:
        payload = np.ascontiguousarray(payload, np.uint8)
        scales = np.ascontiguousarray(scales, np.uint16)
        plane_map = np.ascontiguousarray(plane_map, np.uint8)
        h = C.c_void_p(None)
        check(self._L.tb_salt_v2_upload(self._h, int(codec), C.c_uint32(group), C.c_uint32(n), C.c_uint32(k), _ptr(payload),
                                        C.c_size_t(payload.size), _ptr(scales), C.c_size_t(scales.size),
                                        _ptr(plane_map) if plane_map.size else None, C.c_size_t(plane_map.size),
                                        C.c_uint32(terminal), C.byref(h)))
        return SaltV2ResidentTensor(self, h.value)

    def upload_salt_v1(self, planes: bytes, t_planes: int, n: int, k: int) -> SaltV2ResidentTensor:
        """SALT V1 plane-major TQ2_0 planes with per-block f16 scales (tq2_0_add.cu:640-719,
        packed_salt.rs:612-678); the handle's K is k rounded up to whole 256-blocks."""
        buf = np.frombuffer(bytes(planes), np.uint8)
        h = C.c_void_p(None)
        check(self._L.tb_salt_v1_upload(self._h, _ptr(buf), C.c_size_t(buf.size), C.c_uint32(t_planes), C.c_uint32(n), C.c_uint32(k), C.byref(h)))
        return SaltV2ResidentTensor(self, h.value)

    def upload_salt_v2_from_package(self, package: bytes, name: str) -> SaltV2ResidentTensor:
        buf = np.frombuffer(bytes(package), np.uint8)
        h = C.c_void_p(None)
        check(self._L.tb_salt_v2_upload_package(self._h, _ptr(buf), C.c_size_t(buf.size), name.encode(), C.byref(h)))
        return SaltV2ResidentTensor(self, h.value)

    def upload_salt_v2_from_reader(self, fileobj, name: str) -> SaltV2ResidentTensor:
        """upload_salt_v2_from_reader (crates/tritium-cuda/src/cuda/backend/salt_v2_reader_upload.rs:32): the
        package is a seekable binary file object; only the header table and the named tensor's sections are read."""
        fileobj.seek(0, 2)
        length = fileobj.tell()
        cb = _lib.file_read_at(fileobj)
        h = C.c_void_p(None)
        check(self._L.tb_salt_v2_upload_reader(self._h, cb, None, C.c_uint64(length), name.encode(), C.byref(h)))
        return SaltV2ResidentTensor(self, h.value)

    def _receipt(self, r: _lib.Receipt, mode: str) -> SaltV2ForwardReceipt:
        out = SaltV2ForwardReceipt(**{k: int(getattr(r, k)) for k, _ in _lib.Receipt._fields_})
        out.mode = mode
        return out

    def _f32_forward(self, fn, t, activation, m, output, mode):
        act = np.ascontiguousarray(activation, np.float32)
        if act.size != m * t.columns:
            raise ShapeMismatch(f"shape mismatch: expected {m * t.columns}, got {act.size}")
        if output.size != m * t.rows:
            raise ShapeMismatch(f"shape mismatch: expected {m * t.rows}, got {output.size}")
        staged = np.empty(m * t.rows, np.float32)   # the caller's buffer is untouched on any error
        r = _lib.Receipt()
        check(fn(self._h, t._h, _ptr(act), C.c_uint32(m), _ptr(staged), C.byref(r)))
        output.reshape(-1)[:] = staged
        return self._receipt(r, mode)

    def salt_v2_forward_exact_into(self, t, activation, m, output) -> SaltV2ForwardReceipt:
        return self._f32_forward(self._L.tb_salt_v2_forward_exact, t, activation, m, output, "Exact")

    def salt_v2_forward_exact(self, t, activation, m) -> SaltV2Forward:
        out = np.zeros((m, t.rows), np.float32)
        return SaltV2Forward(out, self.salt_v2_forward_exact_into(t, activation, m, out))

    def salt_v2_forward_fast(self, t, activation, m) -> SaltV2Forward:
        out = np.zeros((m, t.rows), np.float32)
        return SaltV2Forward(out, self._f32_forward(self._L.tb_linear_forward_f32, t, activation, m, out, "Fast"))

    def salt_v2_gather_rows(self, t, rows, output) -> None:
        r = np.ascontiguousarray(rows, np.uint32)
        if output.size != r.size * t.columns:
            raise ShapeMismatch(f"shape mismatch: expected {r.size * t.columns}, got {output.size}")
        check(self._L.tb_salt_v2_gather_rows(self._h, t._h, _ptr(r), C.c_size_t(r.size), _ptr(output)))

    def linear_forward_a8(self, t, x: np.ndarray, m: int, y_dtype: str = "f32", dump: bool = False, x_is_bf16: bool = False):
        """Fused per-token int8 quantisation + exact int32 contraction + scale fold.

        ``x`` is [m, k] float32, or bfloat16 bit patterns (uint16) when ``x_is_bf16``.  Returns
        (y, accumulators or None, receipt); y is float32 or bf16 bit patterns (uint16)."""
        n, k = t.rows, t.columns
        if x_is_bf16:
            xa = np.ascontiguousarray(x, np.uint16)
            xd = _lib.TB_BF16
        else:
            xa = np.ascontiguousarray(x, np.float32)
            xd = _lib.TB_F32
        if xa.size != m * k:
            raise ShapeMismatch(f"shape mismatch: expected {m * k}, got {xa.size}")
        y = np.zeros((m, n), np.float32 if y_dtype == "f32" else np.uint16)
        yd = _lib.TB_F32 if y_dtype == "f32" else _lib.TB_BF16
        planes = int(t.info["planes_uniform"])
        acc = np.zeros((m, n, k // 128, max(planes, 1)), np.int32) if dump else None
        r = _lib.Receipt()
        check(self._L.tb_linear_forward_a8(self._h, t._h, _ptr(xa), xd, C.c_uint32(m), _ptr(y), yd,
                                           _ptr(acc) if dump else None, C.byref(r)))
        return y, acc, self._receipt(r, "A8")

    # ---- device-pointer path (torch tensors) --------------------------------------------
    def forward_dev(self, t, x, y, *, a8=True, act_scale=None, act_absmax=None, acc_dump=None, row_scale=None,
                    flags: int = 0, stream=None) -> None:
        """Launches on device tensors without synchronising.  ``x``/``y`` are torch CUDA tensors."""
        import torch
        dt = {torch.float32: _lib.TB_F32, torch.bfloat16: _lib.TB_BF16, torch.int8: _lib.TB_I8}
        args = _lib.ForwardArgs()
        args.x = x.data_ptr(); args.x_dtype = dt[x.dtype]
        args.act_scale = act_scale.data_ptr() if act_scale is not None else None
        args.act_absmax = act_absmax.data_ptr() if act_absmax is not None else None
        args.m = x.shape[0] if x.dim() > 1 else 1
        args.y = y.data_ptr(); args.y_dtype = dt[y.dtype]
        args.acc_dump = acc_dump.data_ptr() if acc_dump is not None else None
        args.row_scale = row_scale.data_ptr() if row_scale is not None else None
        args.flags = flags | (_lib.TB_FWD_A8 if a8 else 0)
        s = stream if stream is not None else torch.cuda.current_stream()
        args.stream = _lib.stream_handle(s)
        check(self._L.tb_linear_forward_dev(self._h, t._h, C.byref(args), None))

    def norm_linear_forward_dev(self, t, x, y, *, norm_weight=None, eps: float = 0.0, zero_centered: bool = False,
                                residual=None, relu2_up=None, flags: int = 0, stream=None) -> None:
        """RMSNorm -> int8 quantiser -> packed linear -> ``residual + y`` on device tensors, without synchronising.

        The decode block's fused step (crates/tritium-cuda/kernels/decode.cu:533-640 in front,
        crates/tritium-cuda/kernels/tq2_0_add.cu:577-637 behind).  ``norm_weight`` fp32 [k] or None,
        ``residual`` fp32 [m, n] or None.
        """
        import torch
        dt = {torch.float32: _lib.TB_F32, torch.bfloat16: _lib.TB_BF16}
        args = _lib.NormLinearArgs()
        args.x = x.data_ptr(); args.x_dtype = dt[x.dtype]
        args.norm_weight = norm_weight.data_ptr() if norm_weight is not None else None
        args.norm_eps = eps
        args.norm_flags = _lib.TB_NORM_ZERO_CENTERED if zero_centered else 0
        args.residual = residual.data_ptr() if residual is not None else None
        # squared-ReLU gate (crates/tritium-cuda/kernels/decode.cu:772-780): x = gate projection, relu2_up = up projection
        args.relu2_up = relu2_up.data_ptr() if relu2_up is not None else None
        args.m = x.shape[0] if x.dim() > 1 else 1
        args.y = y.data_ptr(); args.y_dtype = dt[y.dtype]
        args.flags = flags
        s = stream if stream is not None else torch.cuda.current_stream()
        args.stream = _lib.stream_handle(s)
        check(self._L.tb_norm_linear_forward_dev(self._h, t._h, C.byref(args), None))

    def act_absmax_dev(self, x, out, stream=None) -> None:
        """Per-token max|x| of a [m, k] fp32/bf16 CUDA tensor into ``out`` (fp32 [m]); no sync."""
        import torch
        dt = {torch.float32: _lib.TB_F32, torch.bfloat16: _lib.TB_BF16}
        s = stream if stream is not None else torch.cuda.current_stream()
        check(self._L.tb_act_absmax_dev(self._h, C.c_void_p(x.data_ptr()), dt[x.dtype], C.c_uint32(x.shape[0]),
                                        C.c_uint32(x.shape[1]), C.c_void_p(out.data_ptr()), C.c_void_p(_lib.stream_handle(s))))

    def reserve(self, t, max_m: int) -> None:
        check(self._L.tb_backend_reserve(self._h, t._h, C.c_uint32(max_m)))

    def check(self, stream=None) -> None:
        """Reads the device status word (bounded-wait timeouts, non-finite values); synchronises."""
        check(self._L.tb_backend_check(self._h, C.c_void_p(_lib.stream_handle(stream)) if stream is not None else None))

    def synchronize(self) -> None:
        check(self._L.tb_backend_synchronize(self._h))

    def close(self) -> None:
        if self._h:
            self._L.tb_backend_free(self._h)
            self._h = C.c_void_p(None)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class LinearStack:
    """Resident sequence of linears run back to back (decoder QKV / O / gate+up / down)."""

    def __init__(self, backend: B200Backend, weights: list, chain: list, max_m: int):
        self._backend = backend
        self._weights = list(weights)
        arr = (C.c_void_p * len(weights))(*[w._h for w in weights])
        ch = (C.c_uint8 * len(weights))(*[1 if c else 0 for c in chain])
        h = C.c_void_p(None)
        check(backend._L.tb_stack_create(backend._h, arr, ch, C.c_uint32(len(weights)), C.c_uint32(max_m), C.byref(h)))
        self._h = h

    def forward_dev(self, x, y_last=None, flags: int = 0, stream=None) -> None:
        import torch
        dt = {torch.float32: _lib.TB_F32, torch.bfloat16: _lib.TB_BF16, torch.int8: _lib.TB_I8}
        s = stream if stream is not None else torch.cuda.current_stream()
        check(self._backend._L.tb_stack_forward_dev(
            self._h, C.c_void_p(x.data_ptr()), dt[x.dtype], C.c_uint32(x.shape[0]),
            C.c_void_p(y_last.data_ptr()) if y_last is not None else None,
            dt[y_last.dtype] if y_last is not None else _lib.TB_BF16, C.c_uint32(flags), C.c_void_p(_lib.stream_handle(s))))

    def forward_host(self, x: np.ndarray, m: int, x_is_bf16: bool = False, flags: int = 0) -> np.ndarray:
        """Host buffers in and out: every layer's bf16 output bits as [layers, m, n] (uint16); the
        layers must all read the stack input and share n."""
        xa = np.ascontiguousarray(x, np.uint16 if x_is_bf16 else np.float32)
        n = self._weights[0].rows
        y = np.zeros((len(self._weights), m, n), np.uint16)
        check(self._backend._L.tb_stack_forward_host(self._h, _ptr(xa), _lib.TB_BF16 if x_is_bf16 else _lib.TB_F32, C.c_uint32(m), _ptr(y),
                                            C.c_uint32(flags)))
        return y

    def read_output(self, layer: int, m: int) -> np.ndarray:
        """bf16 bit patterns [m, n] of a grouped layer's output (synchronises)."""
        out = np.zeros((m, self._weights[layer].rows), np.uint16)
        check(self._backend._L.tb_stack_read_output(self._h, C.c_uint32(layer), C.c_uint32(m), out.ctypes.data_as(C.c_void_p)))
        return out

    def bytes_per_step(self, m: int) -> int:
        return int(self._backend._L.tb_stack_bytes_per_step(self._h, C.c_uint32(m)))

    def close(self) -> None:
        if self._h:
            self._backend._L.tb_stack_free(self._h)
            self._h = C.c_void_p(None)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
