"""Tensor-parallel host logic on CPU: two `gloo` ranks shard, run and reduce; the reduced result
must equal the unsharded CPU reference.  The per-shard contraction is done by the reference port
here (there is no GPU); the classes under test are the ones the CUDA path uses."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

sys.path.insert(0, os.path.join(os.path.dirname(__file__), ".."))

from oracle import oracle as orc  # noqa: E402
from tritium_b200 import tp  # noqa: E402
from tritium_b200.format import SaltV2Codec  # noqa: E402
from tritium_b200.synth import make_activations, make_tensor  # noqa: E402

OCODEC = {SaltV2Codec.D2: orc.D2, SaltV2Codec.B3: orc.B3}


class OracleExecutor(tp.ShardExecutor):
    """Shard arenas decoded and multiplied by the CPU reference port (test double for the device)."""

    def upload(self, codec, group, n, k, payload, scales, plane_map, terminal):
        return dict(codec=OCODEC[codec], group=group, n=n, k=k, payload=payload, scales=scales, map=plane_map, term=terminal)

    def alloc(self, shape, dtype):
        return torch.zeros(shape, dtype=dtype)

    def row_absmax(self, x, out) -> None:
        out.copy_(x.float().abs().amax(dim=1))

    def linear(self, h, x, y, act_absmax) -> None:
        xf = x.float().numpy()
        gamma = act_absmax.numpy() if act_absmax is not None else np.abs(xf).max(axis=1)
        for t in range(xf.shape[0]):
            # quantize_act_int8 with the given absmax, then the exact f32 kernel on the dequantised codes
            s = np.float32(127.0) / gamma[t] if gamma[t] > 0 else np.float32(0)
            q = np.clip(np.rint(xf[t] * np.float32(s)), -128, 127).astype(np.float32)
            deq = q * (np.float32(gamma[t]) / np.float32(127.0))
            out = orc.forward_packed(h["codec"], h["group"], h["n"], h["k"], h["payload"], h["scales"], h["map"],
                                     len(h["map"]), h["term"], deq)[0]
            y[t].copy_(torch.from_numpy(out))


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def rel_l2(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    return float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))


def reference(tensor, x):
    o = orc.Tensor(tensor.rows, tensor.cols, 128, tensor.plane_count.copy(), tensor.trits.copy(), tensor.scales.copy())
    return orc.a8_linear(o, x, dump=False)[0]


def rank_main(rank, world, port, codec_value, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        codec = SaltV2Codec(codec_value)
        ex = OracleExecutor()
        m, n, k, planes = 3, 64, 1024, 2
        tensor = make_tensor("w", n, k, planes, seed=11)
        x = make_activations(m, k, seed=5, bf16=True)
        want = reference(tensor, x)

        col = tp.TPLinear(ex, tensor, codec, "column", rank, world, max_m=m, act_dtype=torch.float32)
        col.input_view(m).copy_(torch.from_numpy(x))
        y_col = col.forward(m).numpy()
        g = col.geometry
        err_col = rel_l2(y_col, want[:, g.n_offset:g.n_offset + g.n])

        row = tp.TPLinear(ex, tensor, codec, "row", rank, world, max_m=m, act_dtype=torch.float32)
        g = row.geometry
        row.input_view(m).copy_(torch.from_numpy(np.ascontiguousarray(x[:, g.k_offset:g.k_offset + g.k_valid])))
        y_row = row.forward(m).numpy()
        err_row = rel_l2(y_row, want)
        # the global absmax every rank used equals the unsharded one
        absmax_ok = bool(np.array_equal(row.absmax[:m].numpy(), np.abs(x).max(axis=1)))

        # a small decoder stack: shapes and modes line up, every rank ends with the same reduced rows
        shape = tp.DecoderShape(hidden=256, q_heads=2, kv_heads=1, head_dim=128, ffn=512, planes=1, layers=2)
        stack = tp.TPDecoderStack(ex, shape, codec, rank, world, max_m=2, act_dtype=torch.float32)
        stack.fill_inputs(2, seed=3)
        outs = stack.forward(2)
        o_full = outs[1].clone()
        gathered = [torch.zeros_like(o_full) for _ in range(world)]
        dist.all_gather(gathered, o_full)
        same = all(torch.equal(gathered[0], t) for t in gathered)
        shapes = [tuple(o.shape) for o in outs]
        # shards drawn directly by each rank (the benchmark's way) go through the same classes
        direct = tp.TPDecoderStack(ex, shape, codec, rank, world, max_m=2, act_dtype=torch.float32, distinct_layers=1,
                                   synthetic_shards=True)
        direct.fill_inputs(2, seed=4)
        d_outs = direct.forward(2)
        gathered = [torch.zeros_like(d_outs[3]) for _ in range(world)]
        dist.all_gather(gathered, d_outs[3].clone())
        same = same and all(torch.equal(gathered[0], t) for t in gathered) and [tuple(o.shape) for o in d_outs] == shapes
        results[rank] = (err_col, err_row, absmax_ok, same, shapes)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("codec", [SaltV2Codec.B3, SaltV2Codec.D2])
def test_two_rank_tensor_parallel_matches_unsharded_reference(codec):
    world = 2
    port = free_port()
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(rank_main, args=(world, port, int(codec), results), nprocs=world, join=True)
        assert sorted(results.keys()) == [0, 1]
        for rank in range(world):
            err_col, err_row, absmax_ok, same, shapes = results[rank]
            assert err_col <= 1e-5 and err_row <= 1e-5, (err_col, err_row)
            assert absmax_ok and same
            assert shapes == [(2, 512 // world), (2, 256), (2, 1024 // world), (2, 256)]


def test_shard_geometry_rules():
    g = tp.ShardGeometry.of("row", 5120, 5120, 8, 3)
    assert (g.n, g.k, g.k_valid, g.k_offset) == (5120, 768, 640, 1920)      # half-tile shards are padded
    g = tp.ShardGeometry.of("column", 7168, 5120, 8, 7)
    assert (g.n, g.k, g.n_offset) == (896, 5120, 6272)
    with pytest.raises(ValueError):
        tp.ShardGeometry.of("row", 16, 640, 8, 0)                          # 80-wide shards cut scale groups
    with pytest.raises(ValueError):
        tp.ShardGeometry.of("column", 30, 256, 4, 0)
    assert [l[2:] for l in tp.DECODER_27B.linears()] == [(7168, 5120), (5120, 5120), (34816, 5120), (5120, 17408)]
    assert [l[2:] for l in tp.DECODER_2B.linears()] == [(3840, 2560), (2560, 2560), (13824, 2560), (2560, 6912)]
