"""Seeded random sweep over shapes, token counts, codecs and options of the int8 linear: every
route (decode passes, few-token and many-token tensor-core kernels; RMSNorm or squared-ReLU gate
in front, residual behind; bf16 output) against the CPU oracle.  Temporaries are handed to the
library and dropped at once on purpose: calls run on torch's current stream, so the allocator's
stream-ordered reuse must be safe."""
import numpy as np
import pytest

from oracle import oracle as orc
from tritium_b200.format import SaltV2Codec
from tritium_b200.synth import make_activations

from gpu_common import rel_l2, uniform_pair

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_random_shapes_and_options_against_the_oracle(seed):
    import torch
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device: there is no CPU path to fall back to")
    from tritium_b200 import B200Backend
    backend = B200Backend(0)
    rng = np.random.default_rng(seed)
    for case in range(14):
        m = int(rng.choice([rng.integers(1, 9), rng.integers(9, 65), rng.integers(65, 300)]))
        n, k, planes = int(rng.integers(1, 1200)), 256 * int(rng.integers(1, 11)), int(rng.integers(1, 4))
        codec = SaltV2Codec.B3 if rng.integers(2) else SaltV2Codec.D2
        mode = case % 4
        prod, orac = uniform_pair(n, k, planes, seed=int(rng.integers(1 << 30)))
        resident = backend.upload_salt_v2(prod, codec)
        backend.reserve(resident, m)
        x = (make_activations(m, k, seed=int(rng.integers(1 << 30)), bf16=False) * np.float32(rng.uniform(0.1, 10))).astype(np.float32)
        x_dev = torch.from_numpy(x).cuda()
        y = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
        what = dict(case=case, m=m, n=n, k=k, planes=planes, codec=codec.name, mode=mode)
        if mode == 0:      # accumulator dump: int32 sums bit-exact
            dump = torch.zeros(m, n, k // 128, planes, dtype=torch.int32, device="cuda")
            backend.forward_dev(resident, x_dev, y, a8=True, acc_dump=dump)
            torch.cuda.synchronize()
            backend.check()
            want, want_dump, _ = orc.a8_linear(orac, x, dump=True)
            assert np.array_equal(dump.cpu().numpy(), want_dump[..., :planes]), what
            assert rel_l2(y.cpu().numpy(), want) <= 1e-5, what
        elif mode == 1:    # RMSNorm in front, residual behind: bit-identical to the plain forward of normalised rows
            w = (rng.standard_normal(k) * 0.3 + 1).astype(np.float32)
            r = rng.standard_normal((m, n)).astype(np.float32)
            backend.norm_linear_forward_dev(resident, x_dev, y, norm_weight=torch.from_numpy(w).cuda(), eps=1e-6,
                                            residual=torch.from_numpy(r).cuda())
            plain = torch.zeros_like(y)
            backend.forward_dev(resident, torch.from_numpy(orc.rmsnorm(x, w, 1e-6)).cuda(), plain, a8=True)
            torch.cuda.synchronize()
            backend.check()
            assert np.array_equal(y.cpu().numpy(), (r + plain.cpu().numpy()).astype(np.float32)), what
        elif mode == 2:    # squared-ReLU gate in front
            up = rng.standard_normal((m, k)).astype(np.float32)
            backend.norm_linear_forward_dev(resident, x_dev, y, relu2_up=torch.from_numpy(up).cuda())
            plain = torch.zeros_like(y)
            backend.forward_dev(resident, torch.from_numpy(orc.relu2_gate(x, up)).cuda(), plain, a8=True)
            torch.cuda.synchronize()
            backend.check()
            assert torch.equal(y, plain), what
        else:              # bf16 in and out
            y16 = torch.zeros(m, n, dtype=torch.bfloat16, device="cuda")
            x16 = x_dev.to(torch.bfloat16)
            backend.forward_dev(resident, x16, y16, a8=True)
            torch.cuda.synchronize()
            backend.check()
            want = orc.a8_linear(orac, x16.float().cpu().numpy(), dump=False)[0]
            assert rel_l2(y16.float().cpu().numpy(), want) <= 1e-2, what
        resident.free()
    backend.close()
