"""The allocation-free forward entry point against the regular device-pointer entry point and the CPU oracle.

Some users of this library may not allocate device memory while they run (a serving loop with a
fixed memory plan, a thread that must stay out of the driver's allocator).  For them the library
offers one call whose scratch is a fixed array inside the library image.  This file checks, through
the C ABI, that the call gives the same bits as the regular path (both run the same arithmetic on
the same codes) and agrees with the CPU oracle, twice in a row (the array is shared and keeps the
previous call's contents), and that oversize shapes are refused.

Collected last on purpose: a failure here must not hide the result of any other test.
"""
import ctypes as C

import numpy as np
import pytest

from oracle import oracle as orc
from tritium_b200 import _lib, errors
from tritium_b200.format import SaltV2Codec, SaltV2Tensor
from tritium_b200.synth import f32_to_bf16_bits, make_activations, make_planes

pytestmark = pytest.mark.gpu


def rel_l2(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    return float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))


@pytest.mark.parametrize("codec", [SaltV2Codec.B3, SaltV2Codec.D2])
def test_static_scratch_forward_matches_regular_path_twice(codec):
    import torch
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device: there is no CPU path to fall back to")
    from tritium_b200 import B200Backend
    backend = B200Backend(0)
    L = _lib.load()
    n, k, planes = 200, 1536, 3
    trits, scales = make_planes(n, k, planes, seed=31)
    tensor = SaltV2Tensor.from_matrix_planes("w", trits, scales)
    oracle_tensor = orc.Tensor(n, k, 128, tensor.plane_count.copy(), tensor.trits.copy(), tensor.scales.copy())
    resident = backend.upload_salt_v2(tensor, codec)
    stream = torch.cuda.Stream()
    for call, m in enumerate((1, 3)):                      # two calls in a row, different inputs
        x = make_activations(m, k, seed=50 + call, bf16=True)
        x_dev = torch.from_numpy(f32_to_bf16_bits(x).view(np.int16).copy()).cuda().view(torch.bfloat16).reshape(m, k)
        want = torch.zeros(m, n, dtype=torch.float32, device="cuda")
        got = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
        with torch.cuda.stream(stream):
            backend.forward_dev(resident, x_dev, want, a8=True, stream=stream)
        stream.synchronize()
        backend.check(stream)
        errors.check(L.tb_linear_forward_a8_static(backend._h, resident._h, C.c_void_p(x_dev.data_ptr()), _lib.TB_BF16,
                                                   None, C.c_uint32(m), C.c_void_p(got.data_ptr()), _lib.TB_F32,
                                                   C.c_void_p(stream.cuda_stream)))
        stream.synchronize()
        backend.check(stream)
        assert torch.equal(got, want), (call, m)                                  # same bits as the regular path
        assert rel_l2(got.cpu().numpy(), orc.a8_linear(oracle_tensor, x, dump=False)[0]) <= 1e-5, (call, m)
    # shapes beyond the fixed scratch, or beyond four tokens, are refused with a clear message
    x_dev = torch.zeros(5, k, dtype=torch.bfloat16, device="cuda")
    y_dev = torch.zeros(5, n, dtype=torch.float32, device="cuda")
    with pytest.raises(errors.InvalidInput, match="at most 4 tokens"):
        errors.check(L.tb_linear_forward_a8_static(backend._h, resident._h, C.c_void_p(x_dev.data_ptr()), _lib.TB_BF16, None,
                                                   C.c_uint32(5), C.c_void_p(y_dev.data_ptr()), _lib.TB_F32, None))
    big_k = 64 * 1024
    t2, s2 = make_planes(16, big_k, 1, seed=2)
    wide = backend.upload_salt_v2(SaltV2Tensor.from_matrix_planes("wide", t2, s2), codec)
    x_dev = torch.zeros(4, big_k, dtype=torch.bfloat16, device="cuda")
    y_dev = torch.zeros(4, 16, dtype=torch.float32, device="cuda")
    with pytest.raises(errors.InvalidInput, match="fixed scratch holds"):
        errors.check(L.tb_linear_forward_a8_static(backend._h, wide._h, C.c_void_p(x_dev.data_ptr()), _lib.TB_BF16, None,
                                                   C.c_uint32(4), C.c_void_p(y_dev.data_ptr()), _lib.TB_F32, None))
    backend.close()
