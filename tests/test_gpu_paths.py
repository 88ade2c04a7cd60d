"""GPU tests of the paths around the kernels: chained and grouped layer stacks, non-finite
activations on the device-pointer entry points, activations that are not 16-byte aligned, and a
bounded device wait that is made to run out (the kernel returns by itself, the call reports
TB_TIMEOUT, the next call works)."""
import ctypes as C

import numpy as np
import pytest

from oracle import oracle as orc
from tritium_b200 import _lib, errors
from tritium_b200.format import SaltV2Codec
from tritium_b200.synth import bf16_bits_to_f32, f32_to_bf16_bits, make_activations

from gpu_common import rel_l2, uniform_pair

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


def bf16_round(v):
    return bf16_bits_to_f32(f32_to_bf16_bits(np.ascontiguousarray(v, np.float32)))


# ------------------------------------------------------------------ layer stacks
@pytest.mark.parametrize("chain", [[0, 0, 1], [0, 1, 1]], ids=["group_then_chain", "chain_of_three"])
@pytest.mark.parametrize("m", [2, 6, 20])
def test_chained_stack_matches_layer_by_layer_oracle(backend, chain, m):
    """chain[i] = 1 feeds layer i with the bf16 output of layer i-1; the others read the stack input.
    Decode kernel (one and two passes) and tensor-core kernel."""
    import torch
    from tritium_b200 import LinearStack
    k = 512
    pairs = [uniform_pair(k, k, 2, seed=200 + i) for i in range(3)]
    weights = [backend.upload_salt_v2(prod, SaltV2Codec.B3) for prod, _ in pairs]
    stack = LinearStack(backend, weights, chain, max_m=m)
    x = make_activations(m, k, seed=23, bf16=True)
    y_last = torch.zeros(m, k, dtype=torch.float32, device="cuda")
    stream = torch.cuda.Stream()
    for flags in (0, _lib.TB_FWD_PDL):
        y_last.zero_()
        with torch.cuda.stream(stream):
            stack.forward_dev(to_dev_bf16(x), y_last=y_last, flags=flags, stream=stream)
        stream.synchronize()
        backend.check(stream)
        prev, want = None, None
        for i, (_, orac) in enumerate(pairs):
            want = orc.a8_linear(orac, bf16_round(prev) if chain[i] else x, dump=False)[0]
            prev = want
        assert rel_l2(y_last.cpu().numpy(), want) <= 2e-2, flags   # two bf16 hand-offs on the way
    stack.close()


@pytest.mark.parametrize("m,flags", [(6, 0), (6, _lib.TB_FWD_PDL), (20, 0)], ids=["m6", "m6_pdl", "m20_tensor_core"])
def test_grouped_stack_beyond_four_tokens(backend, m, flags):
    """A grouped run (layers that read the stack input) takes more than four tokens: the grouped
    launch is repeated per pass of four tokens; above sixteen the tensor-core kernel runs per layer.
    Every layer's output is read back from the group buffer."""
    import torch
    from tritium_b200 import LinearStack
    n, k, planes = 96, 1024, 2
    pairs = [uniform_pair(n, k, planes, seed=300 + i) for i in range(4)]
    weights = [backend.upload_salt_v2(prod, SaltV2Codec.B3) for prod, _ in pairs]
    stack = LinearStack(backend, weights, [0] * 4, max_m=max(m, 8))
    x = make_activations(m, k, seed=29, bf16=True)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        stack.forward_dev(to_dev_bf16(x), flags=flags, stream=stream)
    stream.synchronize()
    backend.check(stream)
    for i, (_, orac) in enumerate(pairs):
        want = orc.a8_linear(orac, x, dump=False)[0]
        assert rel_l2(bf16_bits_to_f32(stack.read_output(i, m)), want) <= 1e-2, i
    got = stack.forward_host(f32_to_bf16_bits(x), m, x_is_bf16=True)
    for i, (_, orac) in enumerate(pairs):
        assert rel_l2(bf16_bits_to_f32(got[i]), orc.a8_linear(orac, x, dump=False)[0]) <= 1e-2, i
    # the last layer belongs to a group: a y_last pointer is refused, not ignored
    with pytest.raises(errors.InvalidInput):
        stack.forward_dev(to_dev_bf16(x), y_last=torch.zeros(m, n, dtype=torch.float32, device="cuda"), stream=stream)
    stack.close()


# ------------------------------------------------------------------ input checks on device pointers
@pytest.mark.parametrize("bad", [float("nan"), float("inf")], ids=["nan", "inf"])
@pytest.mark.parametrize("m", [2, 24], ids=["decode", "tensor_core"])
def test_nonfinite_bf16_activation_is_reported(backend, bad, m):
    """quantize_act_int8 (crates/tritium-spec/src/lib.rs:351-378) would carry a NaN through to the
    output; the device paths report it instead of returning clamped codes."""
    import torch
    n, k = 64, 512
    prod, _ = uniform_pair(n, k, 1, seed=9)
    resident = backend.upload_salt_v2(prod, SaltV2Codec.B3)
    backend.reserve(resident, m)
    x = make_activations(m, k, seed=3, bf16=True)
    x[m - 1, 77] = bad
    x_dev = torch.from_numpy(x).cuda().to(torch.bfloat16)
    y_dev = torch.zeros(m, n, dtype=torch.float32, device="cuda")
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        backend.forward_dev(resident, x_dev, y_dev, a8=True, stream=stream)
    with pytest.raises(errors.InvalidInput, match="non-finite"):
        backend.check(stream)
    if m <= 4:
        L = _lib.load()
        errors.check(L.tb_linear_forward_a8_static(backend._h, resident._h, C.c_void_p(x_dev.data_ptr()), _lib.TB_BF16, None,
                                                   C.c_uint32(m), C.c_void_p(y_dev.data_ptr()), _lib.TB_F32, C.c_void_p(stream.cuda_stream)))
        with pytest.raises(errors.InvalidInput, match="non-finite"):
            backend.check(stream)
    # the status word is clear again and the next call is clean
    x[m - 1, 77] = 1.0
    with torch.cuda.stream(stream):
        backend.forward_dev(resident, torch.from_numpy(x).cuda().to(torch.bfloat16), y_dev, a8=True, stream=stream)
    backend.check(stream)


def test_unaligned_activation_pointer_takes_the_scratch_path(backend):
    """The one-launch path reads activations with 16-byte loads; a pointer that is only 2-byte
    aligned goes through the preparation kernel and gives the same bits."""
    import torch
    n, k, m = 80, 768, 3
    prod, orac = uniform_pair(n, k, 3, seed=13)
    resident = backend.upload_salt_v2(prod, SaltV2Codec.B3)
    x = make_activations(m, k, seed=4, bf16=True)
    flat = torch.zeros(m * k + 8, dtype=torch.bfloat16, device="cuda")
    aligned, shifted = flat[:m * k].view(m, k), flat[1:m * k + 1].view(m, k)
    want_dev = torch.zeros(m, n, dtype=torch.float32, device="cuda")
    got_dev = torch.zeros(m, n, dtype=torch.float32, device="cuda")
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        aligned.copy_(torch.from_numpy(x))
        backend.forward_dev(resident, aligned, want_dev, a8=True, stream=stream)
        stream.synchronize()
        shifted.copy_(torch.from_numpy(x))
        assert shifted.data_ptr() % 16 != 0
        backend.forward_dev(resident, shifted, got_dev, a8=True, stream=stream)
    stream.synchronize()
    backend.check(stream)
    assert torch.equal(want_dev, got_dev)
    assert rel_l2(got_dev.cpu().numpy(), orc.a8_linear(orac, x, dump=False)[0]) <= 1e-5


# ------------------------------------------------------------------ a bounded wait that runs out
def test_bounded_wait_runs_out_and_the_context_stays_usable(backend):
    """The hook makes one kernel wait for bytes that nobody copies.  The wait has a limit: the kernel
    returns by itself (no trap, no fault), the status word says so, tb_backend_check turns it into
    TB_TIMEOUT, and the same backend computes correct results right after."""
    import torch
    L = _lib.load()
    n, k, m = 64, 512, 2
    prod, orac = uniform_pair(n, k, 2, seed=17)
    resident = backend.upload_salt_v2(prod, SaltV2Codec.B3)
    x = make_activations(m, k, seed=5, bf16=True)
    x_dev = to_dev_bf16(x)
    y_dev = torch.zeros(m, n, dtype=torch.float32, device="cuda")
    stream = torch.cuda.Stream()

    def static_call():
        errors.check(L.tb_linear_forward_a8_static(backend._h, resident._h, C.c_void_p(x_dev.data_ptr()), _lib.TB_BF16, None,
                                                   C.c_uint32(m), C.c_void_p(y_dev.data_ptr()), _lib.TB_F32, C.c_void_p(stream.cuda_stream)))

    static_call()                       # resolves the scratch address; clean
    backend.check(stream)
    errors.check(L.tb_backend_inject_wait_timeout(backend._h, 1))
    static_call()
    with pytest.raises(errors.Timeout, match="bounded device wait"):
        backend.check(stream)
    y_dev.zero_()
    static_call()                       # the hook disarmed itself
    backend.check(stream)
    assert rel_l2(y_dev.cpu().numpy(), orc.a8_linear(orac, x, dump=False)[0]) <= 1e-5


# ------------------------------------------------------------------ package file -> device through seeks
def test_upload_from_seekable_package_file(backend, tmp_path):
    """upload_salt_v2_from_reader: a multi-tensor package on disk, one tensor uploaded through seeks,
    forward bit-identical to the upload from arenas."""
    from tritium_b200 import format as fmt
    a, oa = uniform_pair(48, 512, 2, seed=61)
    b2, ob = uniform_pair(32, 768, 3, seed=62)
    a.name, b2.name = "blk.0.attn_q", "blk.0.ffn_up"
    path = tmp_path / "two.tslt2"
    path.write_bytes(fmt.write_salt_v2_package_multi([a, b2], SaltV2Codec.B3))
    x = make_activations(2, 768, seed=6)
    with open(path, "rb") as f:
        streamed = backend.upload_salt_v2_from_reader(f, "blk.0.ffn_up")
    want = np.stack([orc.matvec(ob, x[i]) for i in range(2)])
    got = backend.salt_v2_forward_exact(streamed, x, 2).output
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    y, acc, _ = backend.linear_forward_a8(streamed, x, 2, dump=True)
    want_y, want_acc, _ = orc.a8_linear(ob, x)
    assert np.array_equal(acc, want_acc) and rel_l2(y, want_y) <= 1e-5
    with open(path, "rb") as f:
        with pytest.raises(errors.InvalidInput):
            backend.upload_salt_v2_from_reader(f, "blk.9.none")


# ------------------------------------------------------------------ SALT V1 multi-plane operator
@pytest.mark.parametrize("t_planes", [1, 2, 3])
@pytest.mark.parametrize("m", [1, 4, 24])
def test_salt_v1_planes_match_the_reference_row_dot(backend, t_planes, m):
    """Plane-major TQ2_0 planes with per-block f16 scales (tq2_0_add.cu:640-719): the int8 path against
    SaltLinear::forward (quantise, PackedSaltMatrix::row_dot, scale), the fp32 path against row_dot on
    the raw activations, both under the reference's own 1e-4 rule (crates/tritium-testkit/src/vector.rs:113-126)."""
    rng = np.random.default_rng(100 + t_planes)
    n, k = 72, 700                                       # k is not a multiple of 256: rows are padded with zero trits
    trits = rng.integers(-1, 2, (t_planes, n, k)).astype(np.int8)
    nb = (k + 255) // 256
    block_scales = (0.01 + 0.05 * rng.random((t_planes, n, nb))).astype(np.float16).view(np.uint16)
    planes = orc.salt_v1_pack(trits, block_scales)
    handle = backend.upload_salt_v1(planes, t_planes, n, k)
    assert handle.rows == n and handle.columns == nb * 256
    x = make_activations(m, k, seed=40 + m)
    xp = np.zeros((m, nb * 256), np.float32)
    xp[:, :k] = x
    want = orc.salt_v1_forward_a8(planes, t_planes, n, k, x)
    _, s = orc.quantize_act_int8(x, m, k)
    y, _, receipt = backend.linear_forward_a8(handle, xp, m)
    assert receipt.kernel == (1 if m <= 8 else 2)
    for r in range(m):
        assert np.all(np.abs(y[r] - want[r]) <= 1e-4 * np.maximum(max(float(s[r]), 1e-30), np.abs(want[r])))
    want_f32 = orc.salt_v1_matmul(planes, t_planes, n, k, x)
    got_f32 = backend.salt_v2_forward_fast(handle, xp, m).output
    assert np.all(np.abs(got_f32 - want_f32) <= 1e-4 * np.maximum(1.0, np.abs(want_f32)))
    with pytest.raises(errors.UnsupportedFormat):
        backend.upload_salt_v1(planes + planes[: len(planes) // t_planes], t_planes + 3, n, k)


# ------------------------------------------------------------------ RMSNorm prologue, residual epilogue
@pytest.mark.parametrize("codec", [SaltV2Codec.B3, SaltV2Codec.D2])
@pytest.mark.parametrize("n,k,planes,m,x_bf16,zero_centered,with_residual", [
    (192, 2560, 3, 1, False, False, True),     # one launch: the norm runs inside the decode kernel's table builder
    (192, 2560, 2, 2, True, True, False),
    (200, 768, 1, 3, False, True, True),
    (192, 1280, 3, 4, True, False, True),
    (96, 8192, 2, 4, False, False, True),      # large tables: norm kernel, preparation kernel, decode kernel
    (160, 2560, 3, 6, False, True, True),      # two passes
    (256, 1024, 2, 40, False, False, True),    # tensor-core kernel behind the norm kernel
])
def test_norm_linear_matches_the_reference_arithmetic(backend, codec, n, k, planes, m, x_bf16, zero_centered, with_residual):
    """RMSNorm in the canonical reduction order, the int8 quantiser, the packed linear and
    ``residual + y`` in one rounding.  Every float operation of the prologue is the reference's, so
    the result must equal, bit for bit, the plain int8 forward of rows the oracle normalised, with
    the residual added once in fp32; and it must agree with the oracle's whole chain."""
    import torch
    prod, orac = uniform_pair(n, k, planes, seed=91)
    resident = backend.upload_salt_v2(prod, codec)
    backend.reserve(resident, m)
    rng = np.random.default_rng(5 + m)
    x = make_activations(m, k, seed=17, bf16=x_bf16) * np.float32(3.7)
    if x_bf16:
        x = bf16_bits_to_f32(f32_to_bf16_bits(x))
    w_norm = (rng.standard_normal(k) * 0.3 + (0.0 if zero_centered else 1.0)).astype(np.float32)
    residual = rng.standard_normal((m, n)).astype(np.float32) if with_residual else None
    eps = 1e-6
    normed = orc.rmsnorm(x, w_norm, eps, zero_centered)
    stream = torch.cuda.Stream()
    x_dev = torch.from_numpy(x).cuda()
    if x_bf16:
        x_dev = x_dev.to(torch.bfloat16)
    plain = torch.zeros(m, n, dtype=torch.float32, device="cuda")
    got = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    got_bf16 = torch.zeros(m, n, dtype=torch.bfloat16, device="cuda")
    w_dev = torch.from_numpy(w_norm).cuda()
    r_dev = torch.from_numpy(residual).cuda() if with_residual else None
    with torch.cuda.stream(stream):
        backend.forward_dev(resident, torch.from_numpy(normed).cuda(), plain, a8=True, stream=stream)
        backend.norm_linear_forward_dev(resident, x_dev, got, norm_weight=w_dev, eps=eps, zero_centered=zero_centered,
                                        residual=r_dev, stream=stream)
        backend.norm_linear_forward_dev(resident, x_dev, got_bf16, norm_weight=w_dev, eps=eps, zero_centered=zero_centered,
                                        residual=r_dev, stream=stream)
    stream.synchronize()
    backend.check(stream)
    want = plain.cpu().numpy()
    if with_residual:
        want = (residual + want).astype(np.float32)
    assert np.array_equal(got.cpu().numpy(), want)
    assert np.array_equal(got_bf16.view(torch.int16).cpu().numpy().view(np.uint16), f32_to_bf16_bits(want))
    chain = orc.norm_a8_linear(orac, x, w_norm, eps, zero_centered, residual)
    plain_chain = orc.norm_a8_linear(orac, x, w_norm, eps, zero_centered, None)
    # the tolerance belongs to the linear's output; the residual is added exactly once on both sides
    assert rel_l2(got.cpu().numpy() - (residual if with_residual else 0), plain_chain) <= 1e-5
    assert np.allclose(got.cpu().numpy(), chain, rtol=0, atol=1e-4 * float(np.abs(plain_chain).max()))


def test_residual_epilogue_alone_and_argument_checks(backend):
    import torch
    n, k, m = 128, 1024, 2
    prod, orac = uniform_pair(n, k, 3, seed=8)
    resident = backend.upload_salt_v2(prod, SaltV2Codec.B3)
    x = make_activations(m, k, seed=3, bf16=True)
    residual = np.random.default_rng(1).standard_normal((m, n)).astype(np.float32)
    x_dev = torch.from_numpy(x).cuda().to(torch.bfloat16)
    y = torch.from_numpy(residual).cuda()          # residual aliases the fp32 output: x = x + linear(h)
    plain = torch.zeros(m, n, dtype=torch.float32, device="cuda")
    backend.forward_dev(resident, x_dev, plain, a8=True)
    backend.norm_linear_forward_dev(resident, x_dev, y, residual=y)
    torch.cuda.synchronize()
    backend.check()
    assert np.array_equal(y.cpu().numpy(), (residual + plain.cpu().numpy()).astype(np.float32))
    with pytest.raises(errors.InvalidInput, match="non-negative"):
        backend.norm_linear_forward_dev(resident, x_dev, y, norm_weight=torch.ones(k, device="cuda"), eps=float("nan"))
    with pytest.raises(KeyError):
        backend.norm_linear_forward_dev(resident, torch.zeros(m, k, dtype=torch.int8, device="cuda"), y)


def test_backend_freed_before_its_weights():
    """Handles may be dropped in any order: freeing the backend first leaves the weights' free call
    valid, refuses further work on the released context, and poisons nothing for the next context."""
    import torch
    from tritium_b200 import B200Backend
    first = B200Backend(0)
    prod, orac = uniform_pair(64, 512, 2, seed=3)
    resident = first.upload_salt_v2(prod, SaltV2Codec.B3)
    released = C.c_void_p(first._h.value)
    first.close()                                   # the context is only marked released
    x_dev = torch.zeros(1, 512, dtype=torch.bfloat16, device="cuda")
    y_dev = torch.zeros(1, 64, dtype=torch.float32, device="cuda")
    args = _lib.ForwardArgs()
    args.x, args.x_dtype, args.m, args.y, args.y_dtype, args.flags = x_dev.data_ptr(), _lib.TB_BF16, 1, y_dev.data_ptr(), _lib.TB_F32, _lib.TB_FWD_A8
    # the pointer stays valid while the weights live, and work on it is refused
    assert _lib.load().tb_linear_forward_dev(released, resident._h, C.byref(args), None) == _lib.TB_INVALID_INPUT
    assert "freed" in _lib.last_error()
    resident.free()                                 # the last dependant destroys the released context
    second = B200Backend(0)
    prod2, orac2 = uniform_pair(64, 512, 2, seed=4)
    again = second.upload_salt_v2(prod2, SaltV2Codec.B3)
    x = make_activations(40, 512, seed=1, bf16=True)   # the tensor-core route checks the runtime's last error first
    y, _, _ = second.linear_forward_a8(again, x, 40, x_is_bf16=False)
    assert rel_l2(y, orc.a8_linear(orac2, x, dump=False)[0]) <= 1e-5
    second.close()


# ------------------------------------------------------------------ few tokens on the tensor cores (9..64 tokens)
@pytest.mark.parametrize("codec", [SaltV2Codec.B3, SaltV2Codec.D2])
@pytest.mark.parametrize("m,n,k,planes", [
    (9, 200, 768, 3),       # smallest batch that takes the tensor-core route; K split three ways; ragged rows
    (20, 256, 1024, 2),
    (32, 6912, 2560, 3),    # the benchmark's layer: 54 row tiles, two K splits
    (33, 384, 2560, 3),     # 64-token tile
    (64, 1000, 1536, 1),
    (48, 19200, 512, 2),    # more row tiles than SMs: no split, several tiles per CTA
])
def test_few_token_tensor_core_kernel_is_exact(backend, codec, m, n, k, planes):
    """Batches of 9 to 64 tokens run one pass of the few-token tensor-core kernel (accumulator ring,
    sums in registers, K split over CTAs with a fixed-order combine).  The int32 group sums must be
    the oracle's bit for bit, with and without the dump, and two runs must give the same bits."""
    import torch
    prod, orac = uniform_pair(n, k, planes, seed=m + planes)
    resident = backend.upload_salt_v2(prod, codec)
    backend.reserve(resident, m)
    x = make_activations(m, k, seed=3, bf16=True)
    x_dev = torch.from_numpy(x).cuda().to(torch.bfloat16)
    residual = np.random.default_rng(m).standard_normal((m, n)).astype(np.float32)
    r_dev = torch.from_numpy(residual).cuda()
    y = torch.zeros(m, n, dtype=torch.float32, device="cuda")
    y2 = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    y3 = torch.zeros(m, n, dtype=torch.float32, device="cuda")
    dump = torch.zeros(m, n, k // 128, planes, dtype=torch.int32, device="cuda")
    backend.forward_dev(resident, x_dev, y, a8=True, acc_dump=dump)
    backend.forward_dev(resident, x_dev, y2, a8=True)
    backend.norm_linear_forward_dev(resident, x_dev, y3, residual=r_dev)      # residual epilogue, also behind the split combine
    torch.cuda.synchronize()
    backend.check()
    # the oracle is a scalar program: the big layers are checked on their last 300 rows
    if n <= 2048:
        sample = slice(0, n)
        want, want_dump, _ = orc.a8_linear(orac, x, dump=True)
    else:
        from gpu_common import oracle_rows
        sample = slice(n - 300, n)
        want, want_dump, _ = orc.a8_linear(oracle_rows(prod, np.arange(n - 300, n)), x, dump=True)
    assert np.array_equal(dump.cpu().numpy()[:, sample], want_dump[..., :planes])
    assert torch.equal(y, y2)
    assert rel_l2(y.cpu().numpy()[:, sample], want) <= 1e-5
    assert np.array_equal(y3.cpu().numpy(), (residual + y.cpu().numpy()).astype(np.float32))


# ------------------------------------------------------------------ squared-ReLU gate in front of the down projection
@pytest.mark.parametrize("codec", [SaltV2Codec.B3, SaltV2Codec.D2])
@pytest.mark.parametrize("n,k,planes,m", [
    (192, 1024, 2, 1),      # tables built in the decode kernel
    (160, 6912, 1, 4),      # the 2B-class down projection's width: preparation kernel
    (256, 2560, 3, 6),      # two passes
    (256, 1536, 2, 40),     # few-token tensor-core kernel
    (128, 1024, 1, 200),    # many-token kernel
])
def test_relu2_gate_prologue_is_bit_identical(backend, codec, n, k, planes, m):
    """(max(gate, 0)^2) * up is computed where the activations are quantised; elementwise and
    association-preserving, so the result equals the plain int8 forward of gated rows bit for bit."""
    import torch
    prod, orac = uniform_pair(n, k, planes, seed=21)
    resident = backend.upload_salt_v2(prod, codec)
    backend.reserve(resident, m)
    rng = np.random.default_rng(m)
    gate = rng.standard_normal((m, k)).astype(np.float32)
    up = rng.standard_normal((m, k)).astype(np.float32)
    gated = orc.relu2_gate(gate, up)
    plain = torch.zeros(m, n, dtype=torch.float32, device="cuda")
    got = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    backend.forward_dev(resident, torch.from_numpy(gated).cuda(), plain, a8=True)
    backend.norm_linear_forward_dev(resident, torch.from_numpy(gate).cuda(), got, relu2_up=torch.from_numpy(up).cuda())
    torch.cuda.synchronize()
    backend.check()
    assert torch.equal(got, plain)
    assert rel_l2(got.cpu().numpy(), orc.a8_linear(orac, gated, dump=False)[0]) <= 1e-5
    with pytest.raises(errors.InvalidInput, match="not combined"):
        backend.norm_linear_forward_dev(resident, torch.from_numpy(gate).cuda(), got, relu2_up=torch.from_numpy(up).cuda(),
                                        norm_weight=torch.ones(k, device="cuda"))
