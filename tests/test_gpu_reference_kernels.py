"""The B200 kernels against the reference's own CUDA kernels on the same GPU and inputs.

The reference's decode GEMV (tq2_0_add.cu:439-498) and AOT tensor-core GEMM (tq2_0_imma.cu:156-285)
are compiled from its sources into oracle/_ref (a build step of the oracle; the files travel with
the repository snapshot, the sources do not).  Both compute (float)acc * scale[n] * act_scale[m] on
exact int32 sums, so the int8 path here must agree to the last multiply's rounding.
"""
import numpy as np
import pytest

from oracle import oracle as orc
from oracle import ref_kernels
from tritium_b200.format import pack_tq2_0_rows
from tritium_b200.backend import GemmShape, TernaryFormat

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,n,k", [(1, 6912, 2560), (4, 2560, 6912), (48, 256, 1024)])
def test_int8_path_agrees_with_the_reference_cuda_kernels(m, n, k):
    import torch
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device: there is no CPU path to fall back to")
    if not ref_kernels.available():
        pytest.skip("oracle/_ref holds no built reference kernels (build() makes them where the reference checkout exists)")
    from tritium_b200 import B200Backend
    backend = B200Backend(0)
    rng = np.random.default_rng(m * 7 + 1)
    trits = rng.integers(-1, 2, (n, k)).astype(np.int8)
    scales = rng.uniform(0.5, 2.0, n).astype(np.float32)
    x = (rng.standard_normal((m, k)) * 2).astype(np.float32)
    q, act_scale = orc.quantize_act_int8(x, m, k)              # int8 codes as float values, and gamma / 127
    q8 = q.astype(np.int8)
    acc = q8.astype(np.int64) @ trits.astype(np.int64).T       # exact integers
    want = (acc.astype(np.float32) * scales[None, :]) * act_scale[:, None]

    ref = ref_kernels.ReferenceKernels()
    stream = torch.cuda.current_stream()
    q_dev = torch.from_numpy(q8).cuda()
    as_dev = torch.from_numpy(act_scale.astype(np.float32)).cuda()
    sc_dev = torch.from_numpy(scales).cuda()
    w_rows = torch.from_numpy(np.frombuffer(pack_tq2_0_rows(trits), np.uint8).copy()).cuda()
    w_tiles = torch.from_numpy(ref_kernels.pack_i2s_int8(trits)).cuda()
    out_gemv = torch.zeros(m, n, dtype=torch.float32, device="cuda")
    out_imma = torch.zeros(m, n, dtype=torch.float32, device="cuda")
    ref.decode_gemv(q_dev, w_rows, sc_dev, as_dev, out_gemv, m, n, k, stream)
    ref.imma_gemm(q_dev, w_tiles, as_dev, sc_dev, out_imma, m, n, k, stream)
    torch.cuda.synchronize()
    assert np.array_equal(out_gemv.cpu().numpy(), want)         # the reference kernels reproduce their own contract
    assert np.array_equal(out_imma.cpu().numpy(), want)

    handle = backend.upload_weights(pack_tq2_0_rows(trits), GemmShape(m, n, k), TernaryFormat.Tq2_0)
    ours = torch.zeros(m, n, dtype=torch.float32, device="cuda")
    backend.reserve(handle, m)
    backend.forward_dev(handle, q_dev, ours, a8=True, act_scale=as_dev, row_scale=sc_dev)
    torch.cuda.synchronize()
    backend.check()
    got = ours.cpu().numpy()
    # same exact integer sums; (acc * a) * s against (acc * s) * a differ by the last rounding only
    assert np.allclose(got, want, rtol=3e-7, atol=0)
    backend.close()
