"""Tensor-parallel linears on two GPUs over NCCL: the reduced result equals the unsharded CPU
reference; per-shard int8 codes use the absmax of the whole row."""
import os
import socket
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(__file__), ".."))

pytestmark = pytest.mark.gpu


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def rel_l2(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    return float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))


def rank_main(rank, world, port, codec_value, use_peer, results):
    import torch.distributed as dist
    from oracle import oracle as orc
    from tritium_b200 import B200Backend, tp
    from tritium_b200.format import SaltV2Codec
    from tritium_b200.synth import make_activations, make_tensor

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        codec = SaltV2Codec(codec_value)
        backend = B200Backend(rank)
        from tritium_b200 import _lib
        comm = tp.PeerComm(backend, rank, world, slot_bytes=64 * 384 * 4, slots=10) if use_peer else None
        ex = tp.CudaExecutor(backend, comm=comm, flags=_lib.TB_FWD_PDL if use_peer == 3 else 0)
        stream = torch.cuda.Stream()
        out = {}
        # decode kernel with its own tables (one and two passes), tables from the preparation kernel, tensor-core kernel
        for m, n, k, planes in [(3, 256, 1024, 2), (7, 200, 1536, 3), (4, 256, 8192, 2), (40, 384, 2048, 1)]:
            tensor = make_tensor("w", n, k, planes, seed=11 + m)
            x = make_activations(m, k, seed=5, bf16=True)
            otensor = orc.Tensor(n, k, 128, tensor.plane_count.copy(), tensor.trits.copy(), tensor.scales.copy())
            want = orc.a8_linear(otensor, x, dump=False)[0]
            with torch.cuda.stream(stream):
                col = tp.TPLinear(ex, tensor, codec, "column", rank, world, max_m=m)
                col.input_view(m).copy_(torch.from_numpy(x).to(torch.bfloat16))
                y_col = col.forward(m)
                row = tp.TPLinear(ex, tensor, codec, "row", rank, world, max_m=m)
                g = row.geometry
                row.input_view(m).copy_(torch.from_numpy(np.ascontiguousarray(x[:, g.k_offset:g.k_offset + g.k_valid])).to(torch.bfloat16))
                assert (row.comm is not None) == bool(use_peer)
                row.fused = use_peer >= 2
                row.reduce_chunk_tokens = 16      # m = 40 without a communicator: three chunks, reduced on the second stream
                for _ in range(3):          # repeated rounds on the same slots
                    y_row = row.forward(m)
                stream.synchronize()
                backend.check(stream)
                # every rank must hold the same bits of the reduced rows
                bits = [torch.zeros_like(y_row) for _ in range(world)]
                dist.all_gather(bits, y_row.contiguous())
                stream.synchronize()
                assert all(torch.equal(bits[0], b) for b in bits), (m, "ranks disagree on the reduced rows")
            gc = col.geometry
            # the in-kernel exchange keeps the row absmax to itself; the output parity covers it
            absmax_ok = (use_peer >= 2 and m <= 8) or bool(np.array_equal(row.absmax[:m].cpu().numpy(), np.abs(x).max(axis=1)))
            out[m] = (rel_l2(y_col.cpu().numpy(), want[:, gc.n_offset:gc.n_offset + gc.n]), rel_l2(y_row.cpu().numpy(), want), absmax_ok)
        results[rank] = out
        if comm is not None:
            comm.close()
    finally:
        dist.destroy_process_group()


def timeout_main(rank, world, port, in_kernel, results):
    """Rank 1 leaves one exchange out.  Rank 0's wait has a short limit: its kernel returns by
    itself, the status word says so, and both contexts stay usable.  Nothing is in flight on the
    rank that stays away, and nothing traps or faults."""
    import torch.distributed as dist
    from tritium_b200 import B200Backend, errors, tp
    from tritium_b200.format import SaltV2Codec
    from tritium_b200.synth import make_activations, make_tensor

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        backend = B200Backend(rank)
        comm = tp.PeerComm(backend, rank, world, slot_bytes=64 * 256 * 4, slots=4)
        comm.set_wait_limit(200_000_000)             # about a tenth of a second of SM clocks
        ex = tp.CudaExecutor(backend, comm=comm)
        m, n, k = 2, 256, 1024
        tensor = make_tensor("w", n, k, 2, seed=3)
        x = make_activations(m, k, seed=5, bf16=True)
        row = tp.TPLinear(ex, tensor, SaltV2Codec.B3, "row", rank, world, max_m=m)
        g = row.geometry
        row.input_view(m).copy_(torch.from_numpy(np.ascontiguousarray(x[:, g.k_offset:g.k_offset + g.k_valid])).to(torch.bfloat16))
        row.fused = bool(in_kernel)
        first = row.forward(m).clone()                # a complete round on both ranks
        torch.cuda.synchronize()
        backend.check()
        dist.barrier()
        outcome = "ok"
        if rank == 0:
            row.forward(m)                            # the peer never joins this round
            torch.cuda.synchronize()
            try:
                backend.check()
            except errors.Timeout:
                outcome = "timeout"
        dist.barrier()
        # the context still runs kernels: a linear without peers gives the same result twice
        single = tp.TPLinear(tp.CudaExecutor(backend), tensor, SaltV2Codec.B3, "column", 0, 1, max_m=m)
        single.input_view(m).copy_(torch.from_numpy(x).to(torch.bfloat16))
        a = single.forward(m).clone()
        b = single.forward(m)
        torch.cuda.synchronize()
        backend.check()
        results[rank] = (outcome, bool(torch.equal(a, b)), bool(torch.isfinite(first).all()))
        comm.close()
    finally:
        dist.destroy_process_group()


def block_main(rank, world, port, results):
    """Down-projection shape of an MLP block on two GPUs: squared-ReLU gate on each rank's slice in
    front of the row-parallel linear, residual behind the sum over the ranks, one call."""
    import torch.distributed as dist
    from oracle import oracle as orc
    from tritium_b200 import B200Backend, tp
    from tritium_b200.format import SaltV2Codec
    from tritium_b200.synth import make_tensor

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        backend = B200Backend(rank)
        comm = tp.PeerComm(backend, rank, world, slot_bytes=64 * 512 * 4, slots=8)
        ex = tp.CudaExecutor(backend, comm=comm)
        out = {}
        for m, n, k, planes in [(1, 256, 1024, 2), (4, 320, 6912, 1), (7, 200, 1536, 3)]:   # in-kernel tables, preparation kernel, two passes
            tensor = make_tensor("down", n, k, planes, seed=3 + m)
            rng = np.random.default_rng(m)
            gate = rng.standard_normal((m, k)).astype(np.float32)
            up = rng.standard_normal((m, k)).astype(np.float32)
            residual = rng.standard_normal((m, n)).astype(np.float32)
            otensor = orc.Tensor(n, k, 128, tensor.plane_count.copy(), tensor.trits.copy(), tensor.scales.copy())
            want = (residual + orc.a8_linear(otensor, orc.relu2_gate(gate, up), dump=False)[0]).astype(np.float32)
            row = tp.TPLinear(ex, tensor, SaltV2Codec.B3, "row", rank, world, max_m=m, act_dtype=torch.float32)
            g = row.geometry
            up_dev = torch.zeros_like(row.x)
            row.input_view(m).copy_(torch.from_numpy(np.ascontiguousarray(gate[:, g.k_offset:g.k_offset + g.k_valid])))
            up_dev[:m, :g.k_valid].copy_(torch.from_numpy(np.ascontiguousarray(up[:, g.k_offset:g.k_offset + g.k_valid])))
            r_dev = torch.from_numpy(residual).cuda()
            for _ in range(2):
                comm.block_linear_fused(row.handle, row.slot_absmax, row.slot_y, row.x[:m], row.y[:m], relu2_up=up_dev[:m], residual=r_dev)
            torch.cuda.synchronize()
            backend.check()
            bits = [torch.zeros_like(row.y[:m]) for _ in range(world)]
            dist.all_gather(bits, row.y[:m].contiguous())
            torch.cuda.synchronize()
            out[m] = (rel_l2(row.y[:m].cpu().numpy() - residual, want - residual), bool(all(torch.equal(bits[0], b2) for b2 in bits)))
        results[rank] = out
        comm.close()
    finally:
        dist.destroy_process_group()


def test_two_gpu_block_linear_with_gate_and_residual():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(block_main, args=(2, free_port(), results), nprocs=2, join=True)
        for rank in range(2):
            for m, (err, same) in results[rank].items():
                assert err <= 1e-5 and same, (rank, m, err, same)


@pytest.mark.parametrize("in_kernel", [0, 1], ids=["one_shot_reduce", "in_kernel_exchange"])
def test_two_gpu_wait_on_an_absent_peer_runs_out(in_kernel):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(timeout_main, args=(2, free_port(), in_kernel, results), nprocs=2, join=True)
        assert results[0] == ("timeout", True, True), results[0]
        assert results[1] == ("ok", True, True), results[1]


@pytest.mark.parametrize("use_peer", [0, 1, 2, 3], ids=["nccl", "peer_one_shot", "peer_in_kernel", "peer_in_kernel_pdl"])
@pytest.mark.parametrize("codec", [2, 1], ids=["b3", "d2"])
def test_two_gpu_tensor_parallel_matches_unsharded_reference(codec, use_peer):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(rank_main, args=(world, free_port(), codec, use_peer, results), nprocs=world, join=True)
        assert sorted(results.keys()) == [0, 1]
        for rank in range(world):
            for m, (err_col, err_row, absmax_ok) in results[rank].items():
                assert err_col <= 1e-5 and err_row <= 1e-5, (rank, m, err_col, err_row)
                assert absmax_ok, (rank, m)
