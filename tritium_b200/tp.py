"""Tensor-parallel ternary linears over the GPUs of one node (one process per GPU).

The reference has no tensor-parallel inference path; its only collective is the training
gradient all-reduce (crates/tritium-cuda/src/nccl.rs:530-625).  The sharding rules here follow
the artifact layout (crates/tritium-format/src/salt_v2_package.rs:607-631: tiles cut the flattened
row-major index, so rows may straddle tiles) and the per-token quantiser
(crates/tritium-spec/src/lib.rs:351-378):

* column-parallel (QKV, gate/up): output rows are split.  A rank's shard is a byte slice of the
  arenas; no communication; outputs stay sharded.
* row-parallel (O, down): K is split.  A rank's shard is a re-encoded [N, K/world] tensor whose K
  is padded to whole tiles with zero trits.  The int8 quantiser must see the absmax of the whole
  row, so the ranks take one small MAX all-reduce over their local absmax, run the contraction
  on their slice, and SUM all-reduce the fp32 partial outputs.

`ShardExecutor` is the seam between the collective logic and the device.  `CudaExecutor` is the
only executor this package ships (B200 kernels through the C ABI, NCCL on CUDA tensors); tests
of the collective logic run the same classes over `gloo` with an executor of their own.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from . import format as fmt
from .format import SaltV2Codec, SaltV2Tensor


@dataclass(frozen=True)
class ShardGeometry:
    """Shape of one rank's shard of an [n, k] linear."""
    mode: str          # "column" | "row"
    n: int             # output rows held by this rank
    k: int             # K of the shard tensor (row-parallel: padded to whole tiles)
    k_valid: int       # activations of the unsharded row that this rank consumes
    k_offset: int      # first activation column of the unsharded row
    n_offset: int      # first output row of the unsharded tensor

    @staticmethod
    def of(mode: str, n: int, k: int, world: int, rank: int) -> "ShardGeometry":
        if mode == "column":
            if n % world:
                raise ValueError(f"column-parallel: {n} rows do not split over {world} ranks")
            return ShardGeometry(mode, n // world, k, k, 0, rank * (n // world))
        if mode == "row":
            if k % (128 * world):
                raise ValueError(f"row-parallel: K={k} over {world} ranks breaks the 128-wide scale groups")
            kv = k // world
            return ShardGeometry(mode, n, (kv + 255) // 256 * 256, kv, rank * kv, 0)
        raise ValueError(f"unknown mode {mode!r}")


class ShardExecutor:
    """What a TP linear needs from the device.  Tensors are torch tensors on the executor's device."""

    def upload(self, codec, group, n, k, payload, scales, plane_map, terminal):
        raise NotImplementedError

    def alloc(self, shape, dtype):
        raise NotImplementedError

    def row_absmax(self, x, out) -> None:
        raise NotImplementedError

    def linear(self, handle, x, y, act_absmax) -> None:
        raise NotImplementedError


class CudaExecutor(ShardExecutor):
    """B200 kernels through the C ABI; every call is asynchronous on the current torch stream."""

    def __init__(self, backend, flags: int = 0, comm=None):
        self.backend = backend
        self.flags = flags
        self.comm = comm    # PeerComm or None (NCCL only)
        self._side = None

    def upload(self, codec, group, n, k, payload, scales, plane_map, terminal):
        return self.backend.upload_salt_v2_arenas(codec, group, n, k, payload, scales, plane_map, terminal)

    def alloc(self, shape, dtype):
        import torch
        return torch.zeros(shape, dtype=dtype, device=f"cuda:{self.backend.ordinal}")

    def reserve(self, handle, max_m: int) -> None:
        self.backend.reserve(handle, max_m)

    def side_stream(self):
        """Second stream of this executor, for collectives that overlap the next chunk's kernel."""
        import torch
        if self._side is None:
            self._side = torch.cuda.Stream(device=self.backend.ordinal)
        return self._side

    def row_absmax(self, x, out) -> None:
        self.backend.act_absmax_dev(x, out)

    def linear(self, handle, x, y, act_absmax) -> None:
        self.backend.forward_dev(handle, x, y, a8=True, act_absmax=act_absmax, flags=self.flags)


class PeerComm:
    """Slots of device memory that the ranks of one node map into each other (CUDA IPC) and reduce
    with one kernel launch (`tb_comm_allreduce_f32`): the small-message all-reduce of decode."""

    def __init__(self, backend, rank: int, world: int, slot_bytes: int, slots: int, group=None, counters_per_slot: int = 1024):
        import ctypes as C
        import torch.distributed as dist
        from . import _lib
        from .errors import check
        self._L, self._check, self.backend = _lib.load(), check, backend
        self.rank, self.world, self.slots, self.slot_bytes = rank, world, slots, (slot_bytes + 255) // 256 * 256
        self._next, self._group = 0, group
        h = C.c_void_p(None)
        check(self._L.tb_comm_create(backend._h, C.c_uint32(world), C.c_uint32(rank), C.c_size_t(slot_bytes), C.c_uint32(slots),
                                     C.c_uint32(counters_per_slot), C.byref(h)))
        self._h = h
        if world > 1:
            mine = (C.c_uint8 * _lib.TB_COMM_HANDLE_BYTES)()
            check(self._L.tb_comm_export(self._h, mine))
            gathered = [None] * world
            dist.all_gather_object(gathered, bytes(mine), group=group)
            blob = (C.c_uint8 * (_lib.TB_COMM_HANDLE_BYTES * world)).from_buffer_copy(b"".join(gathered))
            check(self._L.tb_comm_connect(self._h, blob))
            dist.barrier(group=group)

    def take_slot(self) -> int:
        if self._next >= self.slots:
            raise RuntimeError("communicator has no free slot left")
        self._next += 1
        return self._next - 1

    def slot_tensor(self, slot: int, shape):
        """fp32 torch view of a slot (zero-copy)."""
        import torch
        ptr = self._L.tb_comm_slot(self._h, slot)
        count = int(np.prod(shape))
        if not ptr or count * 4 > self.slot_bytes:
            raise ValueError("slot index or shape out of range")

        class _Raw:
            __cuda_array_interface__ = {"shape": (count,), "typestr": "<f4", "data": (int(ptr), False), "version": 2}
        return torch.as_tensor(_Raw(), device=f"cuda:{self.backend.ordinal}").view(*shape)

    def all_reduce(self, slot: int, count: int, out, op_max: bool = False, stream=None) -> None:
        import ctypes as C
        import torch
        from . import _lib
        s = stream if stream is not None else torch.cuda.current_stream()
        self._check(self._L.tb_comm_allreduce_f32(self._h, C.c_uint32(slot), C.c_uint32(count), int(op_max),
                                                  C.c_void_p(out.data_ptr()), C.c_void_p(_lib.stream_handle(s))))

    def linear_fused(self, handle, slot_absmax: int, slot_y: int, x, y, stream=None, flags: int = 0) -> None:
        """Row-parallel forward of up to 8 tokens (`tb_linear_forward_tp_dev`): the absmax exchange
        and the output sum over the ranks both happen inside the kernels (one launch per four
        tokens when the activation tables are small)."""
        import ctypes as C
        import torch
        from . import _lib
        dt = {torch.float32: _lib.TB_F32, torch.bfloat16: _lib.TB_BF16}
        s = stream if stream is not None else torch.cuda.current_stream()
        self._check(self._L.tb_linear_forward_tp_dev(self.backend._h, handle._h, self._h, C.c_uint32(slot_absmax), C.c_uint32(slot_y),
                                                     C.c_void_p(x.data_ptr()), dt[x.dtype], C.c_uint32(x.shape[0]),
                                                     C.c_void_p(y.data_ptr()), dt[y.dtype], C.c_uint32(flags),
                                                     C.c_void_p(_lib.stream_handle(s))))

    def block_linear_fused(self, handle, slot_absmax: int, slot_y: int, x, y, *, relu2_up=None, residual=None, stream=None,
                           flags: int = 0) -> None:
        """`linear_fused` with the block's fused steps (`tb_block_linear_forward_tp_dev`): the
        squared-ReLU gate on this rank's slice in front, the residual behind the sum over the ranks."""
        import ctypes as C
        import torch
        from . import _lib
        dt = {torch.float32: _lib.TB_F32, torch.bfloat16: _lib.TB_BF16}
        s = stream if stream is not None else torch.cuda.current_stream()
        args = _lib.NormLinearArgs()
        args.x = x.data_ptr(); args.x_dtype = dt[x.dtype]
        args.relu2_up = relu2_up.data_ptr() if relu2_up is not None else None
        args.residual = residual.data_ptr() if residual is not None else None
        args.m = x.shape[0]
        args.y = y.data_ptr(); args.y_dtype = dt[y.dtype]
        args.flags = flags
        args.stream = _lib.stream_handle(s)
        self._check(self._L.tb_block_linear_forward_tp_dev(self.backend._h, handle._h, self._h, C.c_uint32(slot_absmax),
                                                           C.c_uint32(slot_y), C.byref(args)))

    def set_wait_limit(self, sm_cycles: int) -> None:
        """Bound of every wait on a peer, in SM clock cycles (default about two seconds)."""
        import ctypes as C
        self._check(self._L.tb_comm_set_wait_limit(self._h, C.c_uint64(sm_cycles)))

    def close(self) -> None:
        """Collective teardown: every rank must call it.  No rank frees its buffer while a peer may
        still have it mapped or a kernel may still touch it: quiesce, barrier, unmap, barrier, free."""
        if not self._h:
            return
        h, self._h = self._h, None
        if self.world > 1:
            import torch
            import torch.distributed as dist
            torch.cuda.synchronize(self.backend.ordinal)
            dist.barrier(group=self._group)
            self._L.tb_comm_disconnect(h)
            dist.barrier(group=self._group)
        self._L.tb_comm_free(h)

    def __del__(self):
        # A collective cannot run from a finaliser (the peers may be gone): a communicator that was
        # never closed only releases this rank's side.
        try:
            if self._h:
                h, self._h = self._h, None
                self._L.tb_comm_free(h)
        except Exception:
            pass


class TPLinear:
    """One rank's share of a tensor-parallel ternary linear."""

    def __init__(self, executor: ShardExecutor, tensor: SaltV2Tensor, codec: SaltV2Codec, mode: str, rank: int, world: int,
                 group=None, max_m: int = 1, act_dtype=None, full_shape=None):
        """``tensor`` is the whole [n, k] tensor (it is sharded here), or, when ``full_shape`` =
        (n, k) is given, this rank's shard already cut and padded as `ShardGeometry` says."""
        import torch
        self.executor, self.rank, self.world, self.group, self.max_m = executor, rank, world, group, max_m
        planes = int(tensor.plane_count[0])
        if np.any(tensor.plane_count != planes):
            raise ValueError("tensor-parallel sharding needs the same plane count in every tile")
        if full_shape is None:
            n, k = tensor.rows, tensor.cols
            self.geometry = ShardGeometry.of(mode, n, k, world, rank)
            payload, scales, _, _, _ = tensor.resident(codec)
            sn, sk, sp, ss, sm, term = fmt.tp_shard(codec, tensor.scale_group_size, n, k, planes, payload, scales,
                                                    mode == "row", world, rank)
        else:
            self.geometry = ShardGeometry.of(mode, full_shape[0], full_shape[1], world, rank)
            sn, sk = tensor.rows, tensor.cols
            sp, ss, sm, term, _ = tensor.resident(codec)
        if (sn, sk) != (self.geometry.n, self.geometry.k):
            raise ValueError(f"shard is [{sn}, {sk}], expected [{self.geometry.n}, {self.geometry.k}]")
        self.handle = executor.upload(codec, tensor.scale_group_size, sn, sk, sp, ss, sm, term)
        if hasattr(executor, "reserve"):
            executor.reserve(self.handle, max_m)
        act_dtype = act_dtype or torch.bfloat16
        # activations live in a buffer as wide as the shard tensor's (padded) K: the padding
        # columns stay zero and meet zero trits
        self.x = executor.alloc((max_m, self.geometry.k), act_dtype)
        self.y = executor.alloc((max_m, self.geometry.n), torch.float32)
        self.absmax = executor.alloc((max_m,), torch.float32) if mode == "row" else None
        # small messages (decode) are reduced over peer memory when the executor carries a
        # communicator: the kernels write their partials straight into its slots
        comm = getattr(executor, "comm", None) if mode == "row" and world > 1 else None
        # `fused` (decode-sized batches): False = separate absmax and one-shot reduce kernels around
        # the ordinary forward; True = both exchanges happen inside the linear's own kernels.
        # Switch only while every rank is idle (a barrier): the two ways share the slots.
        self.comm, self.peer_m, self.fused = comm, 0, False
        # > 0: row-parallel batches of at least two chunks of this many tokens reduce chunk by chunk
        # on a second stream.  Off by default: on two GPUs the smaller kernels and the reduce's SMs
        # cost more (15.0k tok/s at 1024 tokens) than the exposed reduce (17.3k tok/s).
        self.reduce_chunk_tokens = 0
        if comm is not None:
            self.peer_m = min(max_m, comm.slot_bytes // (4 * self.geometry.n))
            if self.peer_m:
                self.slot_absmax, self.slot_y = comm.take_slot(), comm.take_slot()
                self.peer_absmax = comm.slot_tensor(self.slot_absmax, (self.peer_m,))
                self.peer_y = comm.slot_tensor(self.slot_y, (self.peer_m, self.geometry.n))

    @property
    def mode(self) -> str:
        return self.geometry.mode

    def input_view(self, m: int):
        """[m, k_valid] view of the activation buffer: write this rank's slice of the row here."""
        return self.x[:m, : self.geometry.k_valid]

    def forward(self, m: int):
        """Runs on the first ``m`` rows of the activation buffer.  Returns the fp32 output:
        column-parallel [m, n / world] (this rank's rows), row-parallel [m, n] (reduced)."""
        import torch.distributed as dist
        x, y = self.x[:m], self.y[:m]
        if self.mode == "column":
            self.executor.linear(self.handle, x, y, None)
            return y
        absmax = self.absmax[:m]
        if self.comm is not None and self.fused and m <= 8 and \
                2 * self.world * min(m, 4) * self.geometry.n * 8 <= self.comm.slot_bytes:
            self.comm.linear_fused(self.handle, self.slot_absmax, self.slot_y, x, y, flags=getattr(self.executor, "flags", 0))
            return y
        if self.comm is not None and m <= self.peer_m:
            self.executor.row_absmax(x, self.peer_absmax[:m])
            self.comm.all_reduce(self.slot_absmax, m, absmax, op_max=True)
            self.executor.linear(self.handle, x, self.peer_y[:m], absmax)
            self.comm.all_reduce(self.slot_y, m * self.geometry.n, y)
            return y
        self.executor.row_absmax(x, absmax)
        if self.world > 1:
            dist.all_reduce(absmax, op=dist.ReduceOp.MAX, group=self.group)
        chunk = self.reduce_chunk_tokens
        if self.world == 1 or not chunk or m < 2 * chunk or not hasattr(self.executor, "side_stream"):
            self.executor.linear(self.handle, x, y, absmax)
            if self.world > 1:
                dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.group)
            return y
        # Prefill-sized batches: the sum of one chunk of tokens travels on a second stream while the
        # tensor-core kernel works on the next chunk, so that only the last chunk's reduce is exposed.
        import torch
        main, side = torch.cuda.current_stream(), self.executor.side_stream()
        side.wait_stream(main)               # y's previous readers are done before a reduce overwrites it
        for m0 in range(0, m, chunk):
            m1 = min(m, m0 + chunk)
            self.executor.linear(self.handle, x[m0:m1], y[m0:m1], absmax[m0:m1])
            ready = torch.cuda.Event()
            ready.record(main)
            side.wait_event(ready)
            with torch.cuda.stream(side):
                dist.all_reduce(y[m0:m1], op=dist.ReduceOp.SUM, group=self.group)
        main.wait_stream(side)
        return y


@dataclass(frozen=True)
class DecoderShape:
    """Linear shapes of one decoder layer: QKV, O, gate+up (fused), down."""
    hidden: int
    q_heads: int
    kv_heads: int
    head_dim: int
    ffn: int
    planes: int
    layers: int

    def linears(self):
        qkv = (self.q_heads + 2 * self.kv_heads) * self.head_dim
        return [("qkv", "column", qkv, self.hidden), ("o", "row", self.hidden, self.q_heads * self.head_dim),
                ("gate_up", "column", 2 * self.ffn, self.hidden), ("down", "row", self.hidden, self.ffn)]


DECODER_2B = DecoderShape(hidden=2560, q_heads=20, kv_heads=5, head_dim=128, ffn=6912, planes=1, layers=30)
DECODER_27B = DecoderShape(hidden=5120, q_heads=40, kv_heads=8, head_dim=128, ffn=17408, planes=2, layers=64)


class TPDecoderStack:
    """The linears of a decoder, layer by layer, each fed its own fixed input (no attention,
    norm or activation function between them): QKV and gate/up column-parallel, O and down
    row-parallel with the all-reduce behind them."""

    def __init__(self, executor: ShardExecutor, shape: DecoderShape, codec: SaltV2Codec, rank: int, world: int, group=None,
                 max_m: int = 1, make_tensor=None, distinct_layers: int | None = None, act_dtype=None,
                 synthetic_shards: bool = False):
        """``synthetic_shards`` draws each rank's shard directly from the seeded generator instead of
        building and cutting the whole tensor (benchmarks: 1/world of the host work per rank)."""
        from .synth import make_shard_tensor, make_tensor as synth_tensor
        make_tensor = make_tensor or synth_tensor
        self.shape, self.rank, self.world = shape, rank, world
        built = distinct_layers or shape.layers
        self.layers = []
        for layer in range(built):
            row = []
            for idx, (name, mode, n, k) in enumerate(shape.linears()):
                if synthetic_shards:
                    t = make_shard_tensor(f"l{layer}.{name}", n, k, shape.planes, mode, rank, world, seed=layer * 4 + idx)
                    row.append(TPLinear(executor, t, codec, mode, rank, world, group, max_m, act_dtype, full_shape=(n, k)))
                else:
                    t = make_tensor(f"l{layer}.{name}", n, k, shape.planes, seed=layer * 4 + idx)
                    row.append(TPLinear(executor, t, codec, mode, rank, world, group, max_m, act_dtype))
                del t
            self.layers.append(row)

    def fill_inputs(self, m: int, seed: int = 0) -> None:
        """Seeded activations, identical on every rank before slicing (a rank keeps its K slice)."""
        import torch
        from .synth import make_activations
        for li, row in enumerate(self.layers):
            for idx, lin in enumerate(row):
                g = lin.geometry
                k_full = g.k_valid * (self.world if lin.mode == "row" else 1)
                full = make_activations(m, k_full, seed=seed + li * 4 + idx, bf16=True)
                part = full[:, g.k_offset:g.k_offset + g.k_valid]
                lin.input_view(m).copy_(torch.from_numpy(np.ascontiguousarray(part)).to(lin.x.dtype))

    def use_peer_reduce(self, enabled: bool) -> None:
        """Switches the row-parallel linears between the peer-memory reduce and NCCL."""
        for row in self.layers:
            for lin in row:
                if lin.mode == "row" and getattr(lin, "_comm_built", lin.comm) is not None:
                    lin._comm_built = getattr(lin, "_comm_built", lin.comm)
                    lin.comm = lin._comm_built if enabled else None

    def use_fused_reduce(self, enabled: bool) -> None:
        """Row-parallel decode: absmax exchange inside the prepare kernel, or separate one-shot kernels."""
        for row in self.layers:
            for lin in row:
                lin.fused = enabled

    def forward(self, m: int) -> list:
        """One pass over every layer; returns the outputs of the last layer's four linears."""
        out = []
        for row in self.layers:
            out = [lin.forward(m) for lin in row]
        return out

    def weight_bytes(self) -> int:
        """Resident arena bytes this rank streams per pass."""
        total = 0
        for row in self.layers:
            for lin in row:
                r = lin.handle.allocation_receipt()
                total += int(r["steady_resident_bytes"])
        return total
