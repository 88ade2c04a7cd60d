#!/usr/bin/env python
"""Benchmark of the packed additive-ternary linear layer on B200.

Workload (N=1): BASELINE config 2 — 3-plane additive ternary linear, K=2560, N=6912, B3 packed,
per-128-group f16 scales, bf16 activations with outlier channels, int8-quantised per token,
decode M=1.  One "step" is one forward of every layer copy in a rotating set of distinct weight
buffers that is larger than L2, so every step streams its weights from HBM.

The metric is HBM GB/s: algorithmic bytes (resident arenas read once + activations in + outputs
out) divided by device time.  `value` is timed with inputs resident in HBM; `e2e` goes through the
host-pointer C ABI call with host buffers, copies included.

`--impl reference` times the CPU restatement of the reference's scalar algorithm (the oracle) on
the host cores for the same configuration.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

N_ROWS, K_COLS, PLANES = 6912, 2560, 3
METRIC = "ternary linear HBM GB/s (M=1)"
UNIT = "GB/s"
PLANE_BYTES = {"b3": 52, "d2": 64}
# dram__bytes_read.sum + dram__bytes_write.sum of ONE grouped decode launch, from an ncu capture of
# this command (decode kernel, C2, B3, M=1); key = (codec, tokens, weight copies per launch).  The
# figure belongs to the kernel it was captured on; `traffic_source` in the output says so.
NCU_TRAFFIC_BYTES = {("b3", 1, 26): 302_004_224 + 3_978_496}
NCU_TRAFFIC_SOURCE = "ncu capture of one grouped launch of this command (dram__bytes_read.sum + dram__bytes_write.sum); constant, not re-measured per run"


def algorithmic_bytes(codec: str, m: int, x_size: int = 2, y_size: int = 2) -> int:
    from tritium_b200.synth import algorithmic_bytes as ab
    return ab(N_ROWS, K_COLS, PLANES, PLANE_BYTES[codec], m, x_size, y_size)


def measured_peaks() -> tuple[float, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                      "-i", str(self.index)], capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.samples.append([f.strip() for f in out.split(",")])
            except Exception:
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=6)

    def summary(self) -> dict:
        sm = [int(s[0]) for s in self.samples if s and s[0].isdigit()]
        mx = [int(s[1]) for s in self.samples if len(s) > 1 and s[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(s) > 2 + i and s[2 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": int(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def build_inputs(m: int):
    from tritium_b200 import SaltV2Tensor
    from tritium_b200.synth import f32_to_bf16_bits, make_activations, make_planes
    trits, scales = make_planes(N_ROWS, K_COLS, PLANES, seed=0)
    tensor = SaltV2Tensor.from_matrix_planes("ffn_up", trits, scales)
    x = make_activations(m, K_COLS, seed=0, bf16=True)
    return tensor, x, f32_to_bf16_bits(x)


# ---------------------------------------------------------------------------------------- CPU arm
def cpu_forward_time(tensor, x: np.ndarray, threads: int, repeats: int) -> float:
    """Seconds per forward of the oracle: quantise, contract row by row, fold scales."""
    from oracle import oracle as orc
    orac = orc.Tensor(tensor.rows, tensor.cols, 128, tensor.plane_count, tensor.trits, tensor.scales)
    m = x.shape[0]
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        if threads <= 1:
            orc.a8_linear(orac, x, dump=False)
        else:
            q, s = orc.quantize_act_int8(x, m, tensor.cols)
            y = orc.matmul(orac, q, threads=threads)
            y *= s[:, None]
        best = min(best, time.perf_counter() - t0)
    return best


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    tensor, x, _ = build_inputs(1)
    cores = os.cpu_count() or 1
    for _ in range(max(args.warmup, 1)):
        cpu_forward_time(tensor, x, cores, 1)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_forward_time(tensor, x, cores, 1)
    dt = (time.perf_counter() - t0) / args.steps
    value = algorithmic_bytes("b3", 1) / dt / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": "c2_3plane_k2560_n6912_b3_m1"},
        "setup": {"sample": "one layer forward per step"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"one C2 layer forward (M=1) per step; scalar port of salt_v2_matvec_into, rows split over {cores} POSIX threads"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------- GPU arm
def time_graph(torch, stream, launch, steps: int, warmup: int, sampler=None):
    """Capture one step in a CUDA graph, replay it `warmup` + `steps` times, time with events on `stream`."""
    with torch.cuda.stream(stream):
        launch()                      # eager once: module load, attribute setup
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            launch()
        for _ in range(warmup):
            graph.replay()
        stream.synchronize()
    return graph


def measure_prefill(torch, backend, weights, m: int, codec_name: str, steps: int, warmup: int, stream) -> dict:
    """INT8 tensor-core leg: Y[m, N] for m tokens through the tcgen05 kernel (quantisation pre-pass
    included), one weight copy per iteration out of the rotating set, CUDA events on `stream`."""
    from tritium_b200.synth import f32_to_bf16_bits, make_activations
    x = make_activations(m, K_COLS, seed=1, bf16=True)
    x_dev = torch.from_numpy(f32_to_bf16_bits(x).view(np.int16).copy()).cuda().view(torch.bfloat16).reshape(m, K_COLS)
    y_dev = torch.zeros((m, N_ROWS), dtype=torch.bfloat16, device="cuda")
    backend.reserve(weights[0], m)
    with torch.cuda.stream(stream):
        for i in range(max(warmup, 3)):
            backend.forward_dev(weights[i % len(weights)], x_dev, y_dev, stream=stream)
        stream.synchronize()
        backend.check(stream)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(stream)
        for i in range(steps):
            backend.forward_dev(weights[i % len(weights)], x_dev, y_dev, stream=stream)
        stop.record(stream)
        stream.synchronize()
        backend.check(stream)
    ms = start.elapsed_time(stop) / steps
    ops = 2.0 * m * N_ROWS * K_COLS * PLANES
    tops = ops / (ms * 1e-3) / 1e12
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peak, kind = 2.0 * float(json.load(f)["bf16_tflops"]), "2 x measured cuBLAS bf16 burst (INT8 issues at twice the bf16 rate)"
    except Exception:
        peak, kind = 2.0 * 1590.0, "2 x fallback bf16 figure"
    return {"metric": f"INT8 TOPS (M={m})", "value": tops, "unit": "TOPS", "ms_per_call": ms, "launches_per_call": 2,
            "ops_per_call": ops, "workload": f"c2_3plane_k2560_n6912_{codec_name}_m{m}", "out_dtype": "bf16",
            "l2_policy": f"weights rotate over {len(weights)} copies; activations stay L2-resident as they would after the previous layer",
            "roofline": {"bound": "tensor", "achieved": tops, "peak": peak, "unit": "TOPS", "frac": tops / peak,
                         "peak_kind": kind, "frac_of_nominal_4500": tops / 4500.0, "kernel": "prefill_kernel"}}


def measure_single_layer(torch, backend, weights, x_dev, m: int, layer_bytes: int, steps: int, stream, pdl_flag: int) -> dict:
    """One linear per launch (the call shape of a decoder's ModelRunner): every layer of the rotating
    set through tb_linear_forward_dev, eagerly and as a CUDA graph whose launches chain with
    programmatic dependent launch.  GB/s = algorithmic bytes of one layer / time per launch."""
    y_dev = torch.zeros((m, N_ROWS), dtype=torch.bfloat16, device="cuda")
    out = {"workload": f"c2_3plane_k2560_n6912_m{m}, one linear per launch over {len(weights)} weight copies", "launches_per_linear": 1}

    def sweep(flags):
        for w in weights:
            backend.forward_dev(w, x_dev, y_dev, flags=flags, stream=stream)

    with torch.cuda.stream(stream):
        for name, flags, use_graph in (("eager", 0, False), ("graph_pdl", pdl_flag, True)):
            sweep(flags)
            stream.synchronize()
            run = lambda: sweep(flags)
            if use_graph:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    sweep(flags)
                run = graph.replay
            for _ in range(3):
                run()
            stream.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(steps):
                run()
            e1.record(stream)
            stream.synchronize()
            backend.check(stream)
            us = e0.elapsed_time(e1) * 1e3 / (steps * len(weights))
            out[name] = {"us_per_linear": us, "gbs": layer_bytes / (us * 1e-6) / 1e9}
    return out


def measure_e2e_per_linear(torch, backend, weights, x_bits, m: int, layer_bytes: int, rounds: int) -> dict:
    """The reference's call shape: one host-pointer call per linear (tb_linear_forward_a8: x host ->
    device, kernel, y device -> host, one synchronisation), over the rotating weight set."""
    for w in weights[:3]:
        backend.linear_forward_a8(w, x_bits, m, y_dtype="bf16", x_is_bf16=True)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(rounds):
        for w in weights:
            backend.linear_forward_a8(w, x_bits, m, y_dtype="bf16", x_is_bf16=True)
    dt = (time.perf_counter() - t0) / (rounds * len(weights))
    return {"value": layer_bytes / dt / 1e9, "unit": UNIT, "us_per_call": dt * 1e6, "api": "tb_linear_forward_a8 (one call per linear)",
            "h2d_bytes_per_call": m * K_COLS * 2, "d2h_bytes_per_call": m * N_ROWS * 2}


def measure_int8_peak(torch) -> dict | None:
    """Dense INT8 GEMM rate of the library GEMM on this GPU (torch._int_mm, 8192^3, best of 10):
    the INT8 denominator of the tensor-core leg's roofline, measured in the same run."""
    try:
        n = 8192
        a = torch.randint(-8, 8, (n, n), dtype=torch.int8, device="cuda")
        bm = torch.randint(-8, 8, (n, n), dtype=torch.int8, device="cuda")
        for _ in range(3):
            torch._int_mm(a, bm)
        torch.cuda.synchronize()
        best = float("inf")
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch._int_mm(a, bm)
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        return {"tops": 2.0 * n ** 3 / (best * 1e-3) / 1e12, "how": "torch._int_mm int8 8192^3, best of 10, CUDA events"}
    except Exception as exc:  # the library GEMM may not offer int8 on this build
        return {"tops": None, "how": f"torch._int_mm unavailable: {type(exc).__name__}: {exc}"[:200]}


def measure_few_tokens(torch, backend, codec, stream, shapes=None, batches=(16, 32, 64), copies_cap: int = 0) -> dict:
    """Batches of 9 to 64 tokens (batched decode): one call of the few-token tensor-core kernel per
    linear against chained 4-token decode passes, on the benchmark's layer and on a 27B-class gate/up
    linear, weights rotating over copies larger than L2, eager calls (quantisation pre-pass included)."""
    from tritium_b200 import _lib
    from tritium_b200.synth import make_activations, make_tensor
    shapes = shapes or [("c2_3plane", N_ROWS, K_COLS, PLANES), ("gate_up_27b_2plane", 34816, 5120, 2)]
    out = {"timing": "CUDA events over back-to-back calls on one stream, bf16 in and out, weight copies > 126 MB L2"}
    for name, n, k, planes in shapes:
        t = make_tensor(name, n, k, planes, seed=1)
        payload, scales, pmap, terminal, _ = t.resident(codec)
        layer = len(payload) + len(scales)
        copies = max(2, int(np.ceil(300e6 / layer)))
        if copies_cap:
            copies = min(copies, copies_cap)
        hs = [backend.upload_salt_v2_arenas(codec, 128, n, k, payload, scales, pmap, terminal) for _ in range(copies)]
        backend.reserve(hs[0], max(batches))
        entry = {"n": n, "k": k, "planes": planes, "packed_bytes": layer, "weight_copies": copies}
        for m in batches:
            x = torch.from_numpy(make_activations(m, k, seed=2, bf16=True)).cuda().to(torch.bfloat16)
            y = torch.zeros(m, n, dtype=torch.bfloat16, device="cuda")
            res = {}
            for label, flags in (("tensor_core_us", _lib.TB_FWD_FORCE_PREFILL), ("decode_passes_us", _lib.TB_FWD_FORCE_DECODE | _lib.TB_FWD_PDL)):
                if label == "decode_passes_us" and m > 32:
                    continue
                with torch.cuda.stream(stream):
                    for i in range(3):
                        backend.forward_dev(hs[i % copies], x, y, a8=True, flags=flags, stream=stream)
                    stream.synchronize()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    iters = 2 * copies
                    e0.record(stream)
                    for i in range(iters):
                        backend.forward_dev(hs[i % copies], x, y, a8=True, flags=flags, stream=stream)
                    e1.record(stream)
                    stream.synchronize()
                    backend.check(stream)
                res[label] = e0.elapsed_time(e1) / iters * 1e3
            res["tensor_core_weight_gbs"] = layer / res["tensor_core_us"] / 1e3
            entry[f"m{m}"] = res
        out[name] = entry
        del hs
    return out


def measure_c1_fp32(torch, backend, codec, stream, peak: float, peak_kind: str) -> dict:
    """BASELINE config 1 as stated: one-plane linear, K=2048, N=8192, fp32 activations, M=1 and 32, on
    the fast fp32 entry point (four int8 limbs per activation through the int8 kernels) and on the
    bit-exact entry point, device pointers, weights rotating over copies larger than L2."""
    from tritium_b200 import _lib
    from tritium_b200.synth import make_tensor
    n, k = 8192, 2048
    t = make_tensor("c1", n, k, 1, seed=0)
    payload, scales, pmap, terminal, _ = t.resident(codec)
    layer = len(payload) + len(scales)
    copies = max(2, int(np.ceil(300e6 / layer)))
    hs = [backend.upload_salt_v2_arenas(codec, 128, n, k, payload, scales, pmap, terminal) for _ in range(copies)]
    out = {"workload": "c1_1plane_k2048_n8192_fp32", "weight_copies": copies, "packed_bytes": layer,
           "timing": "CUDA events over back-to-back eager calls on one stream"}
    for m in (1, 32):
        x = torch.randn(m, k, device="cuda", dtype=torch.float32)
        y = torch.zeros(m, n, device="cuda", dtype=torch.float32)
        res = {}
        for label, flags in (("fast", _lib.TB_FWD_PDL), ("exact", _lib.TB_FWD_EXACT)):
            with torch.cuda.stream(stream):
                for i in range(3):
                    backend.forward_dev(hs[i % copies], x, y, a8=False, flags=flags, stream=stream)
                stream.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                iters = copies if label == "fast" else min(copies, 8)
                e0.record(stream)
                for i in range(iters):
                    backend.forward_dev(hs[i % copies], x, y, a8=False, flags=flags, stream=stream)
                e1.record(stream)
                stream.synchronize()
                backend.check(stream)
            us = e0.elapsed_time(e1) / iters * 1e3
            algorithmic = layer + m * k * 4 + m * n * 4
            res[label] = {"us_per_call": us, "gbs": algorithmic / us / 1e3}
        res["roofline"] = {"bound": "hbm", "achieved": res["fast"]["gbs"], "peak": peak, "unit": UNIT, "frac": res["fast"]["gbs"] / peak,
                           "peak_kind": peak_kind, "note": "one 3.7 MB layer per call: bound by launches, not bytes"}
        out[f"m{m}"] = res
    del hs
    return out


def measure_mlp_block(torch, backend, codec, stream) -> dict:
    """A decoder's MLP block at M=1 on the 2B-class shapes (hidden 2560, ffn 6912, one plane), chained
    through 30 distinct blocks (> L2): RMSNorm -> gate+up projection (one launch, the norm runs in the
    kernel's table builder), then squared-ReLU gate -> down projection -> + residual (preparation kernel
    + decode kernel, gate and residual fused).  Three launches per block, none of them elementwise."""
    from tritium_b200 import _lib
    from tritium_b200.synth import make_tensor
    hidden, ffn, blocks = 2560, 6912, 30
    ws = []
    total = 0
    for i in range(blocks):
        row = []
        for name, n, k in (("gate_up", 2 * ffn, hidden), ("down", hidden, ffn)):
            t = make_tensor(f"b{i}.{name}", n, k, 1, seed=2 * i + (name == "down"))
            payload, scales, pmap, terminal, _ = t.resident(codec)
            total += len(payload) + len(scales)
            row.append(backend.upload_salt_v2_arenas(codec, 128, n, k, payload, scales, pmap, terminal))
        ws.append(row)
    norm_w = torch.ones(hidden, device="cuda") + 0.01 * torch.randn(hidden, device="cuda")
    xs = [torch.zeros(1, hidden, device="cuda") for _ in range(2)]
    xs[0].normal_()
    y_gu = torch.zeros(1, 2 * ffn, device="cuda")
    gate, up = y_gu[:, :ffn], y_gu[:, ffn:]
    flags = _lib.TB_FWD_PDL

    def step():
        for i, (w_gu, w_down) in enumerate(ws):
            src, dst = xs[i & 1], xs[(i + 1) & 1]
            backend.norm_linear_forward_dev(w_gu, src, y_gu, norm_weight=norm_w, eps=1e-6, flags=flags, stream=stream)
            backend.norm_linear_forward_dev(w_down, gate, dst, relu2_up=up, residual=src, flags=flags, stream=stream)

    out = {"workload": "mlp_block_2b_1plane_m1", "blocks": blocks, "packed_bytes_per_block": total // blocks, "launches_per_block": 3}
    with torch.cuda.stream(stream):
        step()
        stream.synchronize()
        backend.check(stream)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            step()
        for label, fn in (("eager", step), ("graph_pdl", graph.replay)):
            for _ in range(3):
                fn()
            stream.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(5):
                fn()
            e1.record(stream)
            stream.synchronize()
            backend.check(stream)
            us = e0.elapsed_time(e1) / 5 / blocks * 1e3
            out[label] = {"us_per_block": us, "weight_gbs": (total / blocks) / us / 1e3}
    out["finite"] = bool(torch.isfinite(xs[0]).all() and torch.isfinite(xs[1]).all())
    return out


def measure_reference_gpu_kernels(torch, backend, stream) -> dict:
    """The reference's own CUDA kernels (built from its sources into oracle/_ref) beside this
    library's kernels, on the same GPU, the same 1-plane TQ2_0-class weights with a per-channel
    scale, the same int8 activations.  Decode: tq2_0_add_mpgemm_tiled_i8_scaled against the decode
    kernel; many tokens: tq2_0_imma_mpgemm (the ahead-of-time tile; the reference's autotuned tiles
    are rendered by its Rust host and cannot be built here) against the tensor-core kernel.
    A set of distinct weight copies larger than L2 rotates under both."""
    from oracle import ref_kernels
    from tritium_b200 import _lib
    from tritium_b200.backend import GemmShape, TernaryFormat
    from tritium_b200.format import pack_tq2_0_rows
    if not ref_kernels.available():
        return {"unavailable": "oracle/_ref holds no built reference kernels"}
    ref = ref_kernels.ReferenceKernels()
    out = {"weights": "1 plane, TQ2_0 rows (66 bytes per 256 trits), per-channel fp32 scale; int8 activations resident",
           "timing": "CUDA events over back-to-back launches on one stream, rotating weight copies > 126 MB L2"}
    rng = np.random.default_rng(3)

    def timed(fn, iters):
        for _ in range(3):
            fn(0)
        stream.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(iters):
            fn(i)
        e1.record(stream)
        stream.synchronize()
        return e0.elapsed_time(e1) / iters * 1e3      # microseconds per launch

    for name, m, n, k in [("c2_shape_m1", 1, 6912, 2560), ("gate_up_27b_m1", 1, 34816, 5120), ("c2_shape_m2048", 2048, 6912, 2560)]:
        trits = rng.integers(-1, 2, (n, k)).astype(np.int8)
        rows = pack_tq2_0_rows(trits)
        copies = max(2, int(np.ceil(300e6 / len(rows)))) if m == 1 else 2
        with torch.cuda.stream(stream):
            w_rows = [torch.from_numpy(np.frombuffer(rows, np.uint8).copy()).cuda() for _ in range(copies)]
            handles = [backend.upload_weights(rows, GemmShape(m, n, k), TernaryFormat.Tq2_0) for _ in range(copies)]
            backend.reserve(handles[0], m)
            q = torch.randint(-127, 128, (m, k), dtype=torch.int8, device="cuda")
            a_s = torch.rand(m, device="cuda") + 0.5
            w_s = torch.rand(n, device="cuda") + 0.5
            y_ref = torch.zeros(m, n, device="cuda")
            y_own = torch.zeros(m, n, device="cuda")
            entry = {"m": m, "n": n, "k": k, "weight_copies": copies, "packed_row_bytes": len(rows)}
            if m == 1:
                us_ref = timed(lambda i: ref.decode_gemv(q, w_rows[i % copies], w_s, a_s, y_ref, m, n, k, stream), 20 * copies)
                entry["reference_kernel"] = "tq2_0_add_mpgemm_tiled_i8_scaled"
            else:
                w_tiles = [torch.from_numpy(ref_kernels.pack_i2s_int8(trits)).cuda() for _ in range(copies)]
                us_ref = timed(lambda i: ref.imma_gemm(q, w_tiles[i % copies], a_s, w_s, y_ref, m, n, k, stream), 4)
                entry["reference_kernel"] = "tq2_0_imma_mpgemm (ahead-of-time tile)"
            us_own = timed(lambda i: backend.forward_dev(handles[i % copies], q, y_own, a8=True, act_scale=a_s, row_scale=w_s,
                                                         stream=stream), 20 * copies if m == 1 else 10)
            backend.check(stream)
            if m == 1:
                # what a caller of this library gets on a stream of dependent launches: the weight
                # stream of a launch starts under the previous launch's tail
                entry["this_library_pdl_us"] = timed(lambda i: backend.forward_dev(
                    handles[i % copies], q, y_own, a8=True, act_scale=a_s, row_scale=w_s, flags=_lib.TB_FWD_PDL, stream=stream), 20 * copies)
                backend.check(stream)
            entry["same_result"] = bool(torch.allclose(y_ref, y_own, rtol=3e-7, atol=0))
        entry.update({"reference_us": us_ref, "this_library_us": us_own, "speedup": us_ref / us_own})
        if m == 1:
            entry["reference_gbs"] = len(rows) / us_ref / 1e3
            entry["this_library_gbs"] = len(rows) / us_own / 1e3
        else:
            entry["reference_tops"] = 2.0 * m * n * k / us_ref / 1e6
            entry["this_library_tops"] = 2.0 * m * n * k / us_own / 1e6
        out[name] = entry
        del w_rows, handles
    return out


def measure_tp(torch, dist, backend, rank: int, world: int, codec, codec_name: str, args, stream,
               shape_name: str = "27b", batches=(1,), m_prefill: int = 0, reduce_variants: bool = True) -> dict:
    """Tensor-parallel leg: the linears of the 27B-class decoder (64 layers x {QKV 5120->7168,
    O 5120->5120, gate+up 5120->34816, down 17408->5120}, 2 planes) sharded over `world` GPUs:
    QKV and gate/up column-parallel, O and down row-parallel with a MAX all-reduce of the per-token
    absmax before and a SUM all-reduce of the fp32 partial outputs after.  `L` = 2 x world distinct
    layers are built and timed (each rank streams 2 x 144 MB > L2 per step); the 64-layer step
    time is L-layer time x 64 / L, stated in the output."""
    from tritium_b200 import _lib, tp
    shape = tp.DECODER_27B if shape_name == "27b" else tp.DECODER_2B
    # enough distinct layers that one rank's weights of a timed step exceed L2 (126 MB)
    built = 2 * world if shape_name == "27b" else 12 * world
    out = {"workload": f"{'c5_27b_2plane' if shape_name == '27b' else 'c4_2b_1plane'}_tp{world}_{codec_name}", "layers_timed": built,
           "layers_model": shape.layers,
           "collective": "nccl all_reduce (fp32 sum after O and down; fp32 max of the row absmax before them)" if world > 1 else "none"}
    batches = list(batches)
    max_m = max([1, m_prefill] + batches)
    comm = None
    if world > 1:
        # two slots (row absmax, partial outputs) per row-parallel linear, sized for decode batches up to 32
        # (the in-kernel exchange keeps every rank's partial rows of a four-token pass in two alternating copies)
        comm = tp.PeerComm(backend, rank, world, slot_bytes=max(32, 2 * world * 4 * 2) * shape.hidden * 4, slots=4 * built)
    ex = tp.CudaExecutor(backend, flags=0 if args.no_pdl else _lib.TB_FWD_PDL, comm=comm)
    t0 = time.perf_counter()
    stack = tp.TPDecoderStack(ex, shape, codec, rank, world, max_m=max_m, distinct_layers=built, synthetic_shards=True)
    out["build_seconds"] = time.perf_counter() - t0
    if args.tp_reduce_chunk:
        for row in stack.layers:
            for lin in row:
                lin.reduce_chunk_tokens = args.tp_reduce_chunk
        out["prefill_reduce_chunk_tokens"] = args.tp_reduce_chunk
    bytes_rank = stack.weight_bytes()
    steps = max(3, min(args.steps, 20))

    def timed(m: int, use_graph: bool):
        stack.fill_inputs(m, seed=m)
        with torch.cuda.stream(stream):
            stack.forward(m)
            stream.synchronize()
            backend.check(stream)
            step = lambda: stack.forward(m)
            graph = None
            if use_graph:
                try:
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph, stream=stream):
                        stack.forward(m)
                    step = graph.replay
                except Exception as exc:  # capture of a collective is refused on some setups: time eagerly
                    out.setdefault("notes", []).append(f"graph capture failed ({type(exc).__name__}); eager launches")
                    graph = None
                    step = lambda: stack.forward(m)
            for _ in range(3):
                step()
            stream.synchronize()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(steps):
                step()
            e1.record(stream)
            stream.synchronize()
            backend.check(stream)
        t = torch.tensor([e0.elapsed_time(e1) / steps], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()), graph is not None

    def decode_entry(ms, graphed, reduce_kind):
        full_ms = ms * shape.layers / built
        return {"ms_per_step_timed_layers": ms, "ms_per_model_step": full_ms, "tokens_per_s": 1e3 / full_ms,
                "weight_gbs_all_ranks": world * bytes_rank / (ms * 1e-3) / 1e9, "cuda_graph": graphed,
                "all_reduces_per_timed_step": 4 * built if world > 1 else 0, "reduce": reduce_kind}

    # row-parallel linears exchange the absmax and sum their outputs inside their own kernels
    # (batches up to 8 tokens; larger ones use the separate one-shot kernels or NCCL)
    stack.use_fused_reduce(True)
    ms, graphed = timed(1, not args.no_graph)
    out["decode_m1"] = decode_entry(ms, graphed, "absmax exchange and output sum inside the linear's kernels (pushes into peer memory)" if world > 1 else "none")
    if world > 1 and reduce_variants:
        stack.use_fused_reduce(False)
        dist.barrier()
        ms, graphed = timed(1, not args.no_graph)
        out["decode_m1_one_shot"] = decode_entry(ms, graphed, "separate absmax and one-shot reduce kernels over peer memory")
        stack.use_peer_reduce(False)
        ms, graphed = timed(1, not args.no_graph)
        out["decode_m1_nccl"] = decode_entry(ms, graphed, "nccl all_reduce")
        stack.use_peer_reduce(True)
        stack.use_fused_reduce(True)
        dist.barrier()
    for mb in batches:
        if mb == 1:
            continue
        ms, graphed = timed(mb, not args.no_graph)
        full_ms = ms * shape.layers / built
        out[f"decode_m{mb}"] = {"ms_per_step_timed_layers": ms, "ms_per_model_step": full_ms, "tokens_per_s": mb * 1e3 / full_ms,
                                "weight_gbs_all_ranks": world * bytes_rank / (ms * 1e-3) / 1e9, "cuda_graph": graphed}
    if m_prefill > 0:
        ms, _ = timed(m_prefill, False)
        full_ms = ms * shape.layers / built
        ops = 2.0 * m_prefill * shape.planes * sum(n * k for _, _, n, k in shape.linears()) * built
        out[f"prefill_m{m_prefill}"] = {"ms_per_step_timed_layers": ms, "ms_per_model_step": full_ms,
                                        "tokens_per_s": m_prefill * 1e3 / full_ms, "tops_all_ranks": ops / (ms * 1e-3) / 1e12}
    del stack
    if comm is not None:
        comm.close()
    return out


def run_b200(args) -> None:
    import torch
    import torch.distributed as dist
    from tritium_b200 import B200Backend, LinearStack, SaltV2Codec, _lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    codec_name = args.codec
    codec = SaltV2Codec.B3 if codec_name == "b3" else SaltV2Codec.D2
    m = args.m
    tensor, x, x_bits = build_inputs(m)
    backend = B200Backend(local)
    payload, scales, pmap, terminal, _ = tensor.resident(codec)
    layer_bytes = algorithmic_bytes(codec_name, m)
    copies = args.copies or max(2, int(np.ceil(300e6 / layer_bytes)))   # rotating set > 126 MB L2
    weights = [backend.upload_salt_v2_arenas(codec, 128, N_ROWS, K_COLS, payload, scales, pmap, terminal)
               for _ in range(copies)]
    stack = LinearStack(backend, weights, [0] * copies, max_m=max(m, 1))

    stream = torch.cuda.Stream()
    if args.only_few_tokens:
        # profiling aid: the few-token tensor-core kernel alone, on the 27B-class gate/up linear
        print(json.dumps(measure_few_tokens(torch, backend, codec, stream, shapes=[("gate_up_27b_2plane", 34816, 5120, 2)],
                                            batches=(args.only_few_tokens,), copies_cap=3)), flush=True)
        return
    if args.only_prefill:
        # profiling aid: the tensor-core leg alone (no decode leg, no CPU leg)
        print(json.dumps(measure_prefill(torch, backend, weights[:2], args.prefill_m, codec_name, args.steps, args.warmup, stream)), flush=True)
        return
    x_dev = torch.from_numpy(x_bits.view(np.int16).copy()).cuda().view(torch.bfloat16).reshape(m, K_COLS)
    flags = _lib.TB_FWD_PDL if not args.no_pdl else 0

    def launch():
        stack.forward_dev(x_dev, flags=flags, stream=stream)

    with torch.cuda.stream(stream):
        launch()
        stream.synchronize()
        backend.check(stream)
        graph = None
        if not args.no_graph:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                launch()
        step = graph.replay if graph is not None else launch
        for _ in range(max(args.warmup, 3)):
            step()
        stream.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(local) as clocks:
            start.record(stream)
            for _ in range(args.steps):
                step()
            stop.record(stream)
            stream.synchronize()
            elapsed_ms = start.elapsed_time(stop)
            # keep the sampler alive long enough to see the clocks under load on short runs
            t_end = time.time() + 0.6
            while time.time() < t_end and len(clocks.samples) < 2:
                step()
            stream.synchronize()
        backend.check(stream)
    t = torch.tensor([elapsed_ms], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    elapsed_ms = float(t.item())
    ms_per_step = elapsed_ms / args.steps
    bytes_per_step = layer_bytes * copies
    value = world * bytes_per_step / (ms_per_step * 1e-3) / 1e9
    # One step = ONE grouped decode launch that quantises x itself and streams every layer copy.
    per_launch_us = ms_per_step * 1e3
    peak, peak_kind = measured_peaks()
    achieved = bytes_per_step / (per_launch_us * 1e-6) / 1e9

    # ---- end to end through the host-pointer C ABI call of the same step (tb_stack_forward_host):
    # x goes host -> device from a pinned bounce buffer, every layer's bf16 output comes back
    y_dtype = "bf16"
    e2e_steps = max(3, min(args.steps, 20))
    for _ in range(3):
        stack.forward_host(x_bits, m, x_is_bf16=True)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        y_host = stack.forward_host(x_bits, m, x_is_bf16=True)
    e2e_dt = (time.perf_counter() - t0) / e2e_steps
    assert y_host.shape == (copies, m, N_ROWS)
    e2e_t = torch.tensor([e2e_dt], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(e2e_t, op=dist.ReduceOp.MAX)
    e2e_value = world * bytes_per_step / float(e2e_t.item()) / 1e9

    prefill = None
    if args.prefill_m > 0:
        prefill = measure_prefill(torch, backend, weights, args.prefill_m, codec_name, max(5, min(args.steps, 20)), args.warmup, stream)
        pt = torch.tensor([prefill["ms_per_call"]], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(pt, op=dist.ReduceOp.MAX)
            scale = prefill["ms_per_call"] / float(pt.item())
            prefill["ms_per_call"] = float(pt.item())
            prefill["value"] *= scale * world
            prefill["roofline"]["achieved"] *= scale
            prefill["roofline"]["frac"] *= scale
            prefill["roofline"]["frac_of_nominal_4500"] *= scale

    single = e2e_linear = int8_peak = None
    if not args.quick:
        single = measure_single_layer(torch, backend, weights, x_dev, m, layer_bytes, max(3, min(args.steps, 10)), stream, _lib.TB_FWD_PDL)
        e2e_linear = measure_e2e_per_linear(torch, backend, weights, x_bits, m, layer_bytes, 3)
        if prefill is not None:
            int8_peak = measure_int8_peak(torch)
            if int8_peak and int8_peak.get("tops"):
                prefill["roofline"]["int8_gemm_peak_measured"] = int8_peak
                prefill["roofline"]["frac_of_measured_int8_gemm"] = prefill["roofline"]["achieved"] / int8_peak["tops"]

    def extra_leg(fn, *leg_args, **leg_kwargs):
        """An explanatory leg beside the headline must not take the benchmark line down with it."""
        try:
            return fn(*leg_args, **leg_kwargs)
        except Exception as exc:
            torch.cuda.synchronize()
            return {"unavailable": f"{type(exc).__name__}: {exc}"[:300]}

    few_tokens = c1_fp32 = mlp_block = None
    if world == 1 and not args.quick:
        few_tokens = extra_leg(measure_few_tokens, torch, backend, codec, stream)
        c1_fp32 = extra_leg(measure_c1_fp32, torch, backend, codec, stream, peak, peak_kind)
        mlp_block = extra_leg(measure_mlp_block, torch, backend, codec, stream)

    ref_gpu = None
    if world == 1 and not args.quick:
        try:
            ref_gpu = measure_reference_gpu_kernels(torch, backend, stream)
        except Exception as exc:  # a measuring stick must not take the benchmark down with it
            ref_gpu = {"unavailable": f"{type(exc).__name__}: {exc}"[:300]}

    tp_leg = stack_2b = None
    if not args.no_tp:
        batches = [int(v) for v in args.tp_batches.split(",") if v]
        if world > 1:
            # the same decoder unsharded on this rank's GPU: the baseline of the efficiency figures below
            base = measure_tp(torch, None, backend, 0, 1, codec, codec_name, args, stream, shape_name=args.tp_shape, batches=batches,
                              m_prefill=args.tp_prefill_m, reduce_variants=False)
        # (on several GPUs a leg that raised on one rank would leave the others in a collective: no guard there)
        tp_leg = (measure_tp if world > 1 else lambda *a2, **k2: extra_leg(measure_tp, *a2, **k2))(
            torch, dist, backend, rank, world, codec, codec_name, args, stream, shape_name=args.tp_shape,
            batches=batches, m_prefill=args.tp_prefill_m)
        if world > 1:
            eff = {}
            for key, entry in tp_leg.items():
                if isinstance(entry, dict) and "tokens_per_s" in entry:
                    ref = base.get(key if key in base else "decode_m1")
                    if ref:
                        eff[key] = entry["tokens_per_s"] / (world * ref["tokens_per_s"])
            tp_leg["one_gpu_same_run"] = {k2: v for k2, v in base.items() if isinstance(v, dict) and "tokens_per_s" in v}
            tp_leg["efficiency_vs_one_gpu"] = eff
        if world == 1 and not args.quick and args.tp_shape == "27b":
            stack_2b = extra_leg(measure_tp, torch, dist, backend, rank, world, codec, codec_name, args, stream, shape_name="2b", batches=[1, 16, 64])

    if rank == 0:
        cpu = None
        if world == 1 and not args.skip_cpu:
            reps = 3
            sec = cpu_forward_time(tensor, x, 1, reps)
            cpu = {"value": layer_bytes / sec / 1e9, "unit": UNIT, "cores": 1, "kind": "port",
                   "sample": f"best of {reps} single-thread oracle forwards of one C2 layer (M={m}), {sec * 1e3:.0f} ms each"}
            # the reference's default host path for TQ2_0 weights (mpgemm_with_act_quant,
            # crates/tritium-spec/src/lib.rs:266-318) on the same shape, one plane
            from oracle import oracle as orc
            rng = np.random.default_rng(9)
            trits1 = rng.integers(-1, 2, (N_ROWS, K_COLS)).astype(np.int8)
            ch_scale = rng.uniform(0.5, 2.0, N_ROWS).astype(np.float32)
            t_best = float("inf")
            for _ in range(reps):
                t0 = time.perf_counter()
                orc.mpgemm_with_act_quant(x[:1], trits1, ch_scale, 1, N_ROWS, K_COLS)
                t_best = min(t_best, time.perf_counter() - t0)
            cpu["tq2_0_trait_path"] = {"ms_per_forward": t_best * 1e3, "packed_gbs": N_ROWS * (K_COLS // 256) * 66 / t_best / 1e9,
                                       "what": "oracle port of mpgemm_with_act_quant, 1 plane, per-channel scale, M=1, single thread"}
        line = {
            "metric": METRIC if m == 1 else f"ternary linear HBM GB/s (M={m})", "value": value, "unit": UNIT,
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
            "config": {"workload": f"c2_3plane_k2560_n6912_{codec_name}_m{m}"},
            "setup": {"layer_copies_per_step": copies,
                      "l2_policy": f"rotating set of {copies} distinct weight buffers ({bytes_per_step / 1e6:.0f} MB > 126 MB L2)",
                      "launch": ("cuda graph" if graph is not None else "eager") + (" + programmatic dependent launch" if flags else "")},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": UNIT, "frac": achieved / peak,
                         "traffic": NCU_TRAFFIC_BYTES.get((codec_name, m, copies)),
                         "traffic_source": NCU_TRAFFIC_SOURCE if (codec_name, m, copies) in NCU_TRAFFIC_BYTES else None, "peak_kind": peak_kind, "kernel": "decode_kernel", "us_per_launch": per_launch_us,
                         "algorithmic_bytes_per_launch": bytes_per_step, "layers_per_launch": copies,
                         "algorithmic_bytes_per_layer": layer_bytes},
            "cpu_baseline": cpu,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": m * K_COLS * 2,
                    "d2h_bytes_per_step": copies * m * N_ROWS * 2, "api": "tb_stack_forward_host (one call per step)"},
            "gpu_launches": args.steps,
            "clocks": clocks.summary(),
            "single_layer": single,
            "e2e_per_linear": e2e_linear,
            "prefill": prefill,
            "few_tokens": few_tokens,
            "c1_fp32": c1_fp32,
            "mlp_block": mlp_block,
            "reference_gpu_kernels": ref_gpu,
            "tp": tp_leg,
            "stack_2b": stack_2b,
        }
        print(json.dumps(line), flush=True)
    stack.close()
    for w in weights:
        w.free()
    backend.close()
    if world > 1:
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--codec", default="b3", choices=["b3", "d2"])
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--copies", type=int, default=0)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-pdl", action="store_true")
    ap.add_argument("--skip-cpu", action="store_true")
    ap.add_argument("--prefill-m", type=int, default=2048, help="tokens of the tensor-core leg (0 = skip)")
    ap.add_argument("--only-prefill", action="store_true")
    ap.add_argument("--only-few-tokens", type=int, default=0, metavar="M", help="profiling aid: only the few-token kernel at M tokens (9..64)")
    ap.add_argument("--no-tp", action="store_true", help="skip the tensor-parallel decoder-stack leg")
    ap.add_argument("--tp-prefill-m", type=int, default=4096, help="tokens of the tensor-parallel prefill pass (0 = skip)")
    ap.add_argument("--tp-shape", default="27b", choices=["27b", "2b"], help="decoder whose linears the tensor-parallel leg runs")
    ap.add_argument("--tp-reduce-chunk", type=int, default=0, help="tensor-parallel prefill: reduce chunks of this many tokens on a second stream (0 = one reduce per linear)")
    ap.add_argument("--tp-batches", default="1,32", help="comma-separated decode batch sizes of the tensor-parallel leg")
    ap.add_argument("--quick", action="store_true", help="headline legs only (no single-layer, per-linear, INT8-peak and 2B-stack legs)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
