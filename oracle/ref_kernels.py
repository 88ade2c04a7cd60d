"""Launcher for the reference's own CUDA kernels of this path, built into ``oracle/_ref/*.fatbin``.

TEST AND BENCHMARK INFRASTRUCTURE ONLY: the product never imports this.  It exists so that the
B200 kernels can be compared, on the same GPU and the same inputs, with what the reference would
run there: its decode GEMV on int8 activations and its AOT tensor-core GEMM, both over 1-plane
TQ2_0-class weights with a per-channel scale.  The kernels are launched through the CUDA driver
API (cuda-python) on a torch stream; tensors are torch CUDA tensors.

Kernels and their launch geometry, from the reference's sources:
  * ``tq2_0_add_mpgemm_tiled_i8_scaled`` (crates/tritium-cuda/kernels/tq2_0_add.cu:439-498):
    grid (ceil(N/8), M), block 256, one warp per output; weights are rows of 66-byte TQ2_0 blocks.
  * ``tq2_0_imma_mpgemm`` (crates/tritium-cuda/kernels/tq2_0_imma.cu:156-285): grid
    (ceil(N/8), ceil(M/16)), block 32; weights in the I2sInt8 layout (8 x 32 tiles of 2-bit
    codes, n-tile-major then k-tile-major, row-major inside a tile, tq2_0_imma.cu:36-55).
The reference's autotuned tiles are rendered by its Rust host at run time
(crates/tritium-cuda/src/codegen.rs, autotune.rs) and cannot be built without its toolchain.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_REF = os.path.join(_HERE, "_ref")


def available() -> bool:
    return all(os.path.exists(os.path.join(_REF, f)) for f in ("tq2_0_add.fatbin", "tq2_0_imma.fatbin"))


def pack_i2s_int8(trits: np.ndarray) -> np.ndarray:
    """[n, k] trits -> I2sInt8 bytes (tq2_0_imma.cu:36-55); n % 8 == 0 and k % 32 == 0."""
    n, k = trits.shape
    if n % 8 or k % 32:
        raise ValueError("pad n to a multiple of 8 and k to a multiple of 32")
    codes = (trits.astype(np.int16) + 1).astype(np.uint8).reshape(n // 8, 8, k // 32, 32)
    tiles = codes.transpose(0, 2, 1, 3).reshape(-1, 4)          # (nt, kt, n_in, k_in), four codes per byte
    return (tiles[:, 0] | (tiles[:, 1] << 2) | (tiles[:, 2] << 4) | (tiles[:, 3] << 6)).astype(np.uint8)


class ReferenceKernels:
    """The two modules, loaded into the current CUDA context (torch must have created it)."""

    def __init__(self):
        from cuda.bindings import driver
        self._d = driver
        self._mods = []
        self.gemv = self._function("tq2_0_add.fatbin", b"tq2_0_add_mpgemm_tiled_i8_scaled")
        self.imma = self._function("tq2_0_imma.fatbin", b"tq2_0_imma_mpgemm")

    def _check(self, result):
        err = result[0]
        if int(err) != 0:
            raise RuntimeError(f"CUDA driver call failed: {err}")
        return result[1] if len(result) > 1 else None

    def _function(self, file: str, name: bytes):
        with open(os.path.join(_REF, file), "rb") as f:
            image = f.read()
        mod = self._check(self._d.cuModuleLoadData(image))
        self._mods.append(mod)
        return self._check(self._d.cuModuleGetFunction(mod, name))

    def _launch(self, fn, grid, block, args, stream) -> None:
        # kernel parameters: pointers and ints, passed as an array of pointers to the values
        holders = [C.c_void_p(a) if kind == "p" else C.c_int(a) for kind, a in args]
        ptrs = (C.c_void_p * len(holders))(*[C.addressof(h) for h in holders])
        self._check(self._d.cuLaunchKernel(fn, grid[0], grid[1], 1, block, 1, 1, 0, stream.cuda_stream, C.addressof(ptrs), 0))

    def decode_gemv(self, qact, weights, scales, act_scale, out, m: int, n: int, k: int, stream) -> None:
        """out[m, n] = (float)acc * scales[n] * act_scale[m]; qact int8 [m, k], weights TQ2_0 rows."""
        row_bytes = (k + 255) // 256 * 66
        self._launch(self.gemv, ((n + 7) // 8, m), 256,
                     [("p", qact.data_ptr()), ("p", weights.data_ptr()), ("p", scales.data_ptr()), ("p", act_scale.data_ptr()),
                      ("p", out.data_ptr()), ("i", m), ("i", n), ("i", k), ("i", row_bytes)], stream)

    def imma_gemm(self, qact, weights, act_scale, weight_scale, out, m: int, n: int, k: int, stream) -> None:
        """Same contract through mma.sync m16n8k32; weights I2sInt8 (see pack_i2s_int8)."""
        self._launch(self.imma, ((n + 7) // 8, (m + 15) // 16), 32,
                     [("p", qact.data_ptr()), ("p", weights.data_ptr()), ("p", act_scale.data_ptr()), ("p", weight_scale.data_ptr()),
                      ("p", out.data_ptr()), ("i", m), ("i", n), ("i", k), ("i", (k + 31) // 32)], stream)
