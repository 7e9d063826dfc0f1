"""Benchmark of the quantized-weight matmul hot path.

Workload (BASELINE.json configs[4]): the Qwen3-8B-shaped decode matmul stack —
hidden 4096, 36 layers x {q,k,v,o,gate,up,down}, lm_head 151936 — int8
per-channel weights (f32 scales, w = q*s), f16 activations, f32 accumulate,
random init, synthetic activations.  One "step" = one pass of the whole stack
over a batch of `--batch` tokens (default 8): 253 quantized matmuls, 7.57 GB of
int8 weight streamed from HBM per step (far larger than L2, so nothing is
flushed between steps).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch M] [--tp-mode chained|gather]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference ...      # the CPU arm (oracle port on the host cores)

Prints ONE JSON line on rank 0.  `value` = tokens/s of the whole job, timed on
the device with CUDA events on the library's stream (max over ranks); `e2e` =
the same metric through the public API with the activations copied from pinned
host memory and the logits read back every step; `roofline` = algorithmic bytes
per GEMV launch / measured duration against the measured HBM peak.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "qwen3_8b_decode_matmul_stack_tokens_per_s"
UNIT = "tok/s"
FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            d = json.load(open(p))
            return float(d["hbm_gbs"]), float(d.get("bf16_tflops", FALLBACK_BF16_TFLOPS)), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, FALLBACK_BF16_TFLOPS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed
    region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc, self.thread = index, [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "20", "-i",
                 str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, cell in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if cell.lower().startswith("active"):
                    reasons.add(name)
        pw = []
        for r in self.rows:
            try:
                pw.append(float(r[2]))
            except (ValueError, IndexError):
                continue
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "power_w_median": statistics.median(pw) if pw else None, "reasons": sorted(reasons)}


# ---------------------------------------------------------------------------
# CPU arm: the oracle port of the reference's CPU path, on the host cores
# ---------------------------------------------------------------------------

class CpuArm:
    """The reference CPU arithmetic (dequantize once, untimed; then matmul +
    epilogue with f64 accumulation) on a bounded sample of the stack: one layer's
    seven projections plus `lm_rows` rows of lm_head, extrapolated to a step."""

    def __init__(self, batch: int, lm_rows: int = 8192, threads: int = 0):
        import numpy as np

        from oracle import oracle as orc
        from torchlette_b200.decode_stack import QWEN3_8B as cfg

        self.orc, self.cfg, self.batch, self.lm_rows = orc, cfg, batch, lm_rows
        # explicit: under torch.distributed.run OMP_NUM_THREADS is 1, which is not the box's core count
        self.threads = threads or len(os.sched_getaffinity(0)) or orc.max_threads()
        rng = np.random.Generator(np.random.PCG64(0))
        self.items = []
        shapes = [(name, k, n) for name, k, n, _ in cfg.projections()] + [("lm_head", cfg.hidden, lm_rows)]
        for name, k, n in shapes:
            q = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
            s = rng.uniform(0.001, 0.01, size=(n, 1)).astype(np.float32)
            w = orc.dequantize_direct_f32(q.view(np.uint32).reshape(n, k // 4), s, k, k)  # the reference holds f32
            x = rng.standard_normal((batch, k)).astype(np.float16).astype(np.float32)
            self.items.append((name, w, x))

    def step_seconds(self, threads: int = 0) -> float:
        threads = threads or self.threads
        t_layer = t_lm = 0.0
        for name, w, x in self.items:
            t0 = time.perf_counter()
            y = self.orc.matmul_nt(x, w, threads)
            if name == "gate":
                self.orc.unary("silu", y)
            dt = time.perf_counter() - t0
            if name == "lm_head":
                t_lm = dt * (self.cfg.vocab / self.lm_rows)
            else:
                t_layer += dt
        return t_layer * self.cfg.layers + t_lm

    def describe(self, value: float):
        return {"value": value, "unit": UNIT, "cores": self.threads, "kind": "port",
                "sample": f"1 of {self.cfg.layers} layers (7 projections) + {self.lm_rows} of {self.cfg.vocab} lm_head "
                          f"rows, batch {self.batch}, extrapolated to a full step; f32 weights dequantized once, untimed"}


def cpu_sample(batch: int, seconds: float = 10.0):
    """About `seconds` of CPU work on all host threads: the sample is repeated and the median kept."""
    arm = CpuArm(batch)
    arm.step_seconds()
    t0 = time.perf_counter()
    vals = []
    while len(vals) < 3 or time.perf_counter() - t0 < seconds:
        vals.append(arm.step_seconds())
    d = arm.describe(batch / statistics.median(vals))
    d["sample"] += f"; {len(vals)} repetitions in {time.perf_counter() - t0:.1f} s, median"
    # the reference's JavaScript CPU backend is single-threaded: the faithful figure beside the all-core one
    d["value_1_thread"] = batch / statistics.median([arm.step_seconds(threads=1) for _ in range(3)])
    return d


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    arm = CpuArm(args.batch)
    for _ in range(args.warmup):
        arm.step_seconds()
    times = [arm.step_seconds() for _ in range(args.steps)]
    step_s = statistics.mean(times)
    val = args.batch / step_s
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": step_s * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f64 accumulate over f32 (CPU)", "data": "synthetic",
        "config": {"workload": "qwen3-8b-decode-matmul-stack", "batch": args.batch, "layers": 36, "hidden": 4096,
                   "intermediate": 12288, "vocab": 151936, "weights": "int8 per-channel, f32 scales, random init",
                   "note": "the reference is TypeScript and no node runtime exists here; this arm is the C port of its "
                           "CPU path (oracle/tl_oracle.c) on all host cores, each step a bounded sample extrapolated"},
        "cpu_baseline": {**arm.describe(val), "value_1_thread": args.batch / arm.step_seconds(threads=1)},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------

def single_matrix_extras(be, hbm_peak, tf_peak):
    """The two single-kernel figures the path's targets are stated on: the int8
    GEMV on 4096x14336 (rotating over enough weight copies to defeat L2) and the
    prefill GEMM M=2048 (tensor roofline)."""
    import torch

    from torchlette_b200 import binding as B

    lib, ctx = be._lib, be._ctx
    dev = torch.device("cuda", be.device)
    out = {}
    k, n = 4096, 14336
    copies = 6  # 6 x 58.7 MB = 352 MB > 2 x L2
    w = torch.randint(-127, 128, (copies, n, k), dtype=torch.int8, device=dev)
    s = torch.empty(copies, n, dtype=torch.float32, device=dev).uniform_(0.001, 0.01)
    bias = torch.randn(n, device=dev) * 0.02
    q = B.QuantDesc(B.TL_SCHEME_INT8_GROUPED, k, B.TL_F32, B.TL_SCALE_DIRECT)
    e = B.Epilogue()
    e.n_ops, e.n_inputs = 2, 1
    e.ops[0] = B.EpilogueOp(B.TL_EPI_BIAS, 0, 0, 0)
    e.ops[1] = B.EpilogueOp(B.TL_EPI_UNARY, B.TL_UNARY["gelu"], 0, 0)
    e.inputs[0] = bias.data_ptr()
    ev0, ev1 = C.c_void_p(), C.c_void_p()
    B.check(ctx, lib.tl_event_create(ctx, C.byref(ev0)))
    B.check(ctx, lib.tl_event_create(ctx, C.byref(ev1)))
    torch.cuda.synchronize(dev)

    def time_sweep(sweep_fn, n_copies, reps=20):
        """One sweep over the weight copies captured as a graph and replayed: the launches arrive back
        to back however slow the host's call path is.  Returns microseconds per launch."""
        sweep_fn(2)
        be.sync()
        B.check(ctx, lib.tl_graph_begin(ctx))
        sweep_fn(1)
        gh = C.c_void_p()
        B.check(ctx, lib.tl_graph_end(ctx, C.byref(gh)))
        for _ in range(3):
            B.check(ctx, lib.tl_graph_launch(ctx, gh))
        be.sync()
        B.check(ctx, lib.tl_event_record(ctx, ev0))
        for _ in range(reps):
            B.check(ctx, lib.tl_graph_launch(ctx, gh))
        B.check(ctx, lib.tl_event_record(ctx, ev1))
        ms = C.c_float()
        B.check(ctx, lib.tl_event_elapsed_ms(ctx, ev0, ev1, C.byref(ms)))
        B.check(ctx, lib.tl_graph_destroy(ctx, gh))
        return ms.value * 1e3 / (reps * n_copies)

    for m in (1, 16):
        x = torch.randn(m, k, device=dev).to(torch.float16)
        y = torch.empty(m, n, dtype=torch.float16, device=dev)
        torch.cuda.synchronize(dev)

        def sweep(reps):
            for _ in range(reps):
                for c in range(copies):
                    B.check(ctx, lib.tl_qgemv_nt(ctx, x.data_ptr(), B.TL_F16, w[c].data_ptr(), s[c].data_ptr(),
                                                 y.data_ptr(), B.TL_F16, m, n, k, C.byref(q), 1.0, C.byref(e)))
        us = time_sweep(sweep, copies)
        nbytes = n * k + n * 4 + n * 4 + m * k * 2 + m * n * 2
        gbs = nbytes / us / 1e3
        out[f"gemv_4096x14336_m{m}"] = {"us_per_launch": us, "algorithmic_bytes": nbytes, "GBps": gbs,
                                       "frac_of_hbm_peak": gbs / hbm_peak, "epilogue": "bias+gelu, f16 out",
                                       "l2": f"rotating over {copies} weight copies (352 MB)",
                                       "launch": "replayed graph of one sweep over the copies"}
    del w, s
    # the dense (unquantized f16) counterpart through tl_matmul: the tensor-core GEMV at the same
    # shape (2 bytes per weight, so twice the traffic), and the tiled kernel on a square product
    copies = 3  # 3 x 117.4 MB = 352 MB
    wd = (torch.randn(copies, n, k, device=dev) * 0.02).to(torch.float16)
    for m in (1, 16):
        x = torch.randn(m, k, device=dev).to(torch.float16)
        y = torch.empty(m, n, dtype=torch.float16, device=dev)

        def sweep_dense(reps):
            for _ in range(reps):
                for c in range(copies):
                    B.check(ctx, lib.tl_matmul(ctx, x.data_ptr(), wd[c].data_ptr(), y.data_ptr(), m, n, k, 1, 0, 0, m * n, 0, 1,
                                               1.0, B.TL_F16, B.TL_F16, B.TL_F16, -1, -1, C.byref(e), None))
        us = time_sweep(sweep_dense, copies)
        nbytes = 2 * n * k + n * 4 + m * k * 2 + m * n * 2
        out[f"dense_gemv_f16_4096x14336_m{m}"] = {"us_per_launch": us, "algorithmic_bytes": nbytes, "GBps": nbytes / us / 1e3,
                                                 "frac_of_hbm_peak": nbytes / us / 1e3 / hbm_peak, "epilogue": "bias+gelu, f16 out",
                                                 "l2": f"rotating over {copies} weight copies (352 MB)"}
    del wd
    # int4-grouped (G = 128, f16 abs-max scales): half a byte per weight
    copies4 = 12  # 12 x 29.4 MB = 352 MB
    w4 = torch.randint(-2 ** 31, 2 ** 31 - 1, (copies4, n, k // 8), dtype=torch.int32, device=dev)
    s4 = torch.empty(n, k // 128, device=dev).uniform_(0.01, 0.1).to(torch.float16)
    q4 = B.QuantDesc(B.TL_SCHEME_INT4_GROUPED, 128, B.TL_F16, B.TL_SCALE_SNORM127)
    for m in (1, 16):
        x = torch.randn(m, k, device=dev).to(torch.float16)
        y = torch.empty(m, n, dtype=torch.float16, device=dev)

        def sweep4(reps):
            for _ in range(reps):
                for c in range(copies4):
                    B.check(ctx, lib.tl_qmatmul_nt(ctx, x.data_ptr(), B.TL_F16, w4[c].data_ptr(), s4.data_ptr(), y.data_ptr(), B.TL_F16,
                                                   m, n, k, C.byref(q4), 1.0, C.byref(e)))
        us = time_sweep(sweep4, copies4, reps=10)
        nbytes = n * k // 2 + n * (k // 128) * 2 + n * 4 + m * k * 2 + m * n * 2
        out[f"int4_gemv_g128_4096x14336_m{m}"] = {"us_per_launch": us, "algorithmic_bytes": nbytes, "GBps": nbytes / us / 1e3,
                                                  "frac_of_hbm_peak": nbytes / us / 1e3 / hbm_peak, "epilogue": "bias+gelu, f16 out",
                                                  "l2": f"rotating over {copies4} weight copies (352 MB)"}
    del w4, s4
    # dense products on the tensor cores (tl_matmul's tcgen05 kernel): the prefill shape in the NT layout
    # `linear` produces, a square NN product (B is transposed into scratch first), and the tiled
    # CUDA-core kernel forced on the same square for reference
    def time_dense(m_, n_, k_, trans_b, dt, tdt, epi_ptr, reps=10):
        xa = (torch.randn(m_, k_, device=dev) * 0.05).to(tdt)
        xb = (torch.randn(*((n_, k_) if trans_b else (k_, n_)), device=dev) * 0.05).to(tdt)
        yc = torch.empty(m_, n_, dtype=tdt, device=dev)

        def run():
            B.check(ctx, lib.tl_matmul(ctx, xa.data_ptr(), xb.data_ptr(), yc.data_ptr(), m_, n_, k_, 1, 0, 0, m_ * n_, 0,
                                       1 if trans_b else 0, 1.0, dt, dt, dt, -1, -1, epi_ptr, None))
        for _ in range(3):
            run()
        be.sync()
        B.check(ctx, lib.tl_event_record(ctx, ev0))
        for _ in range(reps):
            run()
        B.check(ctx, lib.tl_event_record(ctx, ev1))
        ms = C.c_float()
        B.check(ctx, lib.tl_event_elapsed_ms(ctx, ev0, ev1, C.byref(ms)))
        tf = 2.0 * m_ * n_ * k_ / (ms.value / reps * 1e-3) / 1e12
        return {"ms": ms.value / reps, "TFLOPs": tf, "frac_of_bf16_peak": tf / tf_peak}
    eg = B.Epilogue()
    eg.n_ops = 1
    eg.ops[0] = B.EpilogueOp(B.TL_EPI_UNARY, B.TL_UNARY["gelu"], 0, 0)
    out["dense_tc_bf16_2048x4096x14336_nt_gelu"] = dict(time_dense(2048, 14336, 4096, True, B.TL_BF16, torch.bfloat16, C.byref(eg)),
                                                        kernel="tcgen05, A and B from shared memory")
    out["dense_tc_f16_2048x2048x2048_nn"] = dict(time_dense(2048, 2048, 2048, False, B.TL_F16, torch.float16, None),
                                                 kernel="tcgen05, B stored [K, N] and multiplied MN-major as it lies (no transposed copy)")
    be.forceVariant((B.TL_FAMILY_MATMUL, 0, 0, 0, 0, 0))
    try:
        out["dense_tiled_f16_2048x2048x2048"] = dict(time_dense(2048, 2048, 2048, False, B.TL_F16, torch.float16, None, reps=3),
                                                     kernel="tiled (CUDA cores): the always-applicable kernel, forced")
    finally:
        be.forceVariant(None)
    # prefill GEMM, config 3
    for (m, kk, nn) in ((2048, 4096, 14336), (2048, 14336, 4096)):
        w = torch.randint(-127, 128, (nn, kk), dtype=torch.int8, device=dev)
        s = torch.empty(nn, dtype=torch.float32, device=dev).uniform_(0.001, 0.01)
        x = torch.randn(m, kk, device=dev).to(torch.bfloat16)
        y = torch.empty(m, nn, dtype=torch.bfloat16, device=dev)
        q = B.QuantDesc(B.TL_SCHEME_INT8_GROUPED, kk, B.TL_F32, B.TL_SCALE_DIRECT)
        e2 = B.Epilogue()
        e2.n_ops = 1
        e2.ops[0] = B.EpilogueOp(B.TL_EPI_UNARY, B.TL_UNARY["gelu"], 0, 0)
        torch.cuda.synchronize(dev)

        def run():
            return lib.tl_qgemm_nt(ctx, x.data_ptr(), B.TL_BF16, w.data_ptr(), s.data_ptr(), y.data_ptr(), B.TL_BF16,
                                   m, nn, kk, C.byref(q), 1.0, C.byref(e2))
        rc = run()
        if rc != 0:
            out[f"qgemm_{m}x{kk}x{nn}"] = {"unavailable": lib.tl_last_error(ctx).decode()}
            continue
        for _ in range(3):
            run()
        be.sync()
        reps = 10
        B.check(ctx, lib.tl_event_record(ctx, ev0))
        for _ in range(reps):
            run()
        B.check(ctx, lib.tl_event_record(ctx, ev1))
        ms = C.c_float()
        B.check(ctx, lib.tl_event_elapsed_ms(ctx, ev0, ev1, C.byref(ms)))
        tf = 2.0 * m * nn * kk / (ms.value / reps * 1e-3) / 1e12
        rcpt = B.PlanReceipt()
        B.check(ctx, lib.tl_plan_qmatmul(ctx, m, nn, kk, B.TL_BF16, B.TL_BF16, C.byref(q), C.byref(e2), C.byref(rcpt)))
        out[f"qgemm_{m}x{kk}x{nn}"] = {"ms": ms.value / reps, "TFLOPs": tf, "frac_of_bf16_peak": tf / tf_peak,
                                       "epilogue": "gelu, bf16 out",
                                       "variant": lib.tl_variant_name(C.byref(rcpt.choice)).decode()}
        # both int8 routes on every shape, forced: converting on the operand path (tcgen05, A from TMEM)
        # against writing the weight out as bf16 once and running the dense kernel
        for label, forced in (("fused", (B.TL_FAMILY_QGEMM, 0, 192, 128, 3, 8)), ("dequant_dense", (B.TL_FAMILY_QGEMM, 2, 0, 0, 0, 0))):
            be.forceVariant(forced)
            try:
                for _ in range(3):
                    run()
                be.sync()
                B.check(ctx, lib.tl_event_record(ctx, ev0))
                for _ in range(reps):
                    run()
                B.check(ctx, lib.tl_event_record(ctx, ev1))
                B.check(ctx, lib.tl_event_elapsed_ms(ctx, ev0, ev1, C.byref(ms)))
                out[f"qgemm_{m}x{kk}x{nn}"][label + "_ms"] = ms.value / reps
            finally:
                be.forceVariant(None)
        del w, s, x, y
    # the two small configurations: a 2048 x 2048 f32 GEMV, and the seven 0.6B-shaped decode
    # projections (q, k, v, gate, up on K=1024; o on K=2048; down on K=3072) replayed as ONE
    # captured graph.  1-4 MB of weights per launch is under a microsecond of HBM time (and fits
    # L2), so these are launch-latency figures, not bandwidth figures.
    def timed_graph(enqueue, reps=200):
        enqueue()
        be.sync()
        B.check(ctx, lib.tl_graph_begin(ctx))
        enqueue()
        g = C.c_void_p()
        B.check(ctx, lib.tl_graph_end(ctx, C.byref(g)))
        for _ in range(5):
            B.check(ctx, lib.tl_graph_launch(ctx, g))
        be.sync()
        B.check(ctx, lib.tl_event_record(ctx, ev0))
        for _ in range(reps):
            B.check(ctx, lib.tl_graph_launch(ctx, g))
        B.check(ctx, lib.tl_event_record(ctx, ev1))
        ms = C.c_float()
        B.check(ctx, lib.tl_event_elapsed_ms(ctx, ev0, ev1, C.byref(ms)))
        B.check(ctx, lib.tl_graph_destroy(ctx, g))
        return ms.value * 1e3 / reps

    def make_proj(nn, kk):
        return (torch.randint(-127, 128, (nn, kk), dtype=torch.int8, device=dev),
                torch.empty(nn, dtype=torch.float32, device=dev).uniform_(0.001, 0.01))
    w0, s0 = make_proj(2048, 2048)
    x0 = torch.randn(1, 2048, device=dev)
    y0 = torch.empty(1, 2048, device=dev)
    q0 = B.QuantDesc(B.TL_SCHEME_INT8_GROUPED, 2048, B.TL_F32, B.TL_SCALE_DIRECT)
    us0 = timed_graph(lambda: B.check(ctx, lib.tl_qgemv_nt(ctx, x0.data_ptr(), B.TL_F32, w0.data_ptr(), s0.data_ptr(), y0.data_ptr(),
                                                           B.TL_F32, 1, 2048, 2048, C.byref(q0), 1.0, None)))
    b0 = 2048 * 2048 + 2048 * 4 * 3
    out["config0_gemv_2048x2048_f32"] = {"us_per_launch": us0, "algorithmic_bytes": b0, "GBps": b0 / us0 / 1e3,
                                         "bound": "launch latency (4 MB of weights, L2-resident across replays)"}
    shapes = [("q", 2048, 1024), ("k", 1024, 1024), ("v", 1024, 1024), ("gate", 3072, 1024), ("up", 3072, 1024),
              ("o", 1024, 2048), ("down", 1024, 3072)]
    projs = {nm: make_proj(nn, kk) + (torch.empty(1, nn, dtype=torch.float16, device=dev), nn, kk) for nm, nn, kk in shapes}
    acts = {kk: torch.randn(1, kk, device=dev).to(torch.float16) for kk in (1024, 2048, 3072)}

    def one(nm):
        wq, sq, yq, nn, kk = projs[nm]
        qd = B.QuantDesc(B.TL_SCHEME_INT8_GROUPED, kk, B.TL_F32, B.TL_SCALE_DIRECT)
        B.check(ctx, lib.tl_qgemv_nt(ctx, acts[kk].data_ptr(), B.TL_F16, wq.data_ptr(), sq.data_ptr(), yq.data_ptr(), B.TL_F16,
                                     1, nn, kk, C.byref(qd), 1.0, None))

    def group(names):
        items = (B.QGemvItem * len(names))()
        for i, nm in enumerate(names):
            wq, sq, yq, nn, kk = projs[nm]
            items[i] = B.QGemvItem(wq.data_ptr(), sq.data_ptr(), yq.data_ptr(), nn, 1.0, None)
        kk = projs[names[0]][4]
        qd = B.QuantDesc(B.TL_SCHEME_INT8_GROUPED, kk, B.TL_F32, B.TL_SCALE_DIRECT)
        B.check(ctx, lib.tl_qgemv_nt_batched(ctx, acts[kk].data_ptr(), B.TL_F16, items, len(names), B.TL_F16, 1, kk, C.byref(qd)))
    us7 = timed_graph(lambda: [one(nm) for nm, _, _ in shapes])
    us4 = timed_graph(lambda: (group(["q", "k", "v"]), group(["gate", "up"]), one("o"), one("down")))
    b1 = sum(nn * kk + nn * 4 + nn * 2 for _, nn, kk in shapes) + 2 * (1024 + 2048 + 3072)
    out["config1_seven_projections_graph"] = {
        "us_per_replay_7_launches": us7, "us_per_replay_4_launches_batched": us4, "algorithmic_bytes": b1,
        "GBps_4_launches": b1 / us4 / 1e3, "bound": "launch latency (12.6 MB of weights per replay, L2-resident)"}
    lib.tl_event_destroy(ctx, ev0)
    lib.tl_event_destroy(ctx, ev1)
    return out


def stack_parity(stack, dist):
    """The stack's last step against the CPU oracle, on its own intermediate values, at any N:
    (a) 64 lm_head columns spread over all ranks' shards, oracle on the final hidden state
    (column-parallel path and the logits gather; f32 logits, gate 1e-3);
    (b) 64 output columns of the LAST layer's down projection, oracle partial products of every rank
    summed over the ranks (row-parallel path and its all-reduce; f16 hand-over, gate 1e-2);
    (c) the gathered logits and the reduced hidden state are bit-identical on all ranks."""
    import numpy as np
    import torch

    from oracle import oracle as orc

    world, dev = stack.world, stack.dev
    per = max(8, 64 // world)

    def rel(got, ref):
        got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
        return float(np.max(np.abs(got - ref) / np.maximum(1.0, np.abs(ref))))

    def rows_of(n):
        return torch.as_tensor(np.unique(np.linspace(0, n - 1, per).astype(np.int64)), device=dev)

    # (a) lm_head: this rank's own columns
    lm = stack.lm_head
    rows = rows_of(lm.n)
    w = lm.w[rows].cpu().numpy().astype(np.float32) * lm.s[rows].cpu().numpy().astype(np.float32)[:, None]
    h = stack.h2.float().cpu().numpy()
    ref = orc.linear_reference(h, w, None, None, alpha=lm.alpha)
    err_lm = rel(stack.logits_local[:, rows].float().cpu().numpy(), ref)
    # (b) last layer's down projection: partial reference per rank, summed over ranks
    pd = stack.layers[-1][6]
    rows_d = rows_of(pd.n)
    wd = pd.w[rows_d].cpu().numpy().astype(np.float32) * pd.s[rows_d].cpu().numpy().astype(np.float32)[:, None]
    part = orc.linear_reference(stack.g.float().cpu().numpy(), wd, None, None, alpha=pd.alpha).astype(np.float64)
    if dist is not None:
        t = torch.as_tensor(part, device=dev)
        dist.all_reduce(t)
        part = t.cpu().numpy()
    err_down = rel(stack.h2[:, rows_d].float().cpu().numpy(), part)
    identical = True
    if dist is not None:
        # (c) every rank holds the same gathered logits and the same reduced hidden state, and the
        # gathered logits hold this rank's own slice at its column offset
        nl = stack.logits_local.shape[1]
        own = torch.equal(stack.logits[:, stack.rank * nl:(stack.rank + 1) * nl], stack.logits_local)
        sums = torch.stack([stack.logits.double().sum(), stack.logits.double().abs().sum(), stack.h2.double().sum(),
                            stack.h2.double().abs().sum()])
        lo, hi = sums.clone(), sums.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        flag = torch.tensor([1.0 if (own and torch.equal(lo, hi)) else 0.0], device=dev, dtype=torch.float64)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        identical = bool(flag.item() == 1.0)
        e = torch.tensor([err_lm, err_down], device=dev, dtype=torch.float64)
        dist.all_reduce(e, op=dist.ReduceOp.MAX)
        err_lm, err_down = float(e[0]), float(e[1])
    return {"rows": int(per * world), "rel_err": err_lm, "lm_head_rel_err": err_lm, "down_rows": int(len(rows_d)),
            "down_rel_err": err_down, "ranks_identical": identical,
            "oracle": "CPU restatement of the reference (oracle/tl_oracle.c) on the stack's own intermediate values"}


def run_gpu(args):
    import numpy as np
    import torch
    import torch.distributed as dist

    from torchlette_b200 import backend as tb
    from torchlette_b200 import binding as B
    from torchlette_b200.decode_stack import QWEN3_8B, DecodeStack, StackConfig

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run for N>1")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback on this path")
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        B.preload_nccl()
    be = tb.CudaBackend(local_rank)
    lib, ctx = be._lib, be._ctx
    if world > 1:
        ident = [None]
        if rank == 0:
            buf = (C.c_char * B.TL_COMM_ID_BYTES)()
            B.check(None, lib.tl_comm_unique_id(buf))
            ident[0] = bytes(buf)
        dist.broadcast_object_list(ident, src=0)
        idbuf = (C.c_char * B.TL_COMM_ID_BYTES).from_buffer_copy(ident[0])
        B.check(ctx, lib.tl_comm_init(ctx, rank, world, idbuf))
        if args.allreduce in ("p2p", "fused", "push"):
            # exchange buffers for the one-shot peer all-reduce: [batch, hidden] partial sums.
            # If any rank cannot map its peers (no peer access between some pair of GPUs), every
            # rank switches to the NCCL all-reduce and the JSON line says so.
            ok = 1
            try:
                hbuf = (C.c_char * 64)()
                B.check(ctx, lib.tl_p2p_create(ctx, args.batch * 4096 * 8, hbuf))  # {f32 partial, epoch} per value
                mine = bytes(hbuf)
            except tb.TlError as ex:
                ok, mine = 0, bytes(64)
                sys.stderr.write(f"rank {rank}: peer all-reduce unavailable ({ex})\n")
            handles = [None] * world
            dist.all_gather_object(handles, (ok, mine))
            if all(h[0] for h in handles):
                try:
                    allh = (C.c_char * (64 * world)).from_buffer_copy(b"".join(h[1] for h in handles))
                    B.check(ctx, lib.tl_p2p_attach(ctx, allh))
                except tb.TlError as ex:
                    ok = 0
                    sys.stderr.write(f"rank {rank}: peer all-reduce unavailable ({ex})\n")
            else:
                ok = 0
            flags = [None] * world
            dist.all_gather_object(flags, ok)
            if not all(flags):
                args.allreduce = "nccl (peer buffers could not be mapped)"
            dist.barrier()

    if args.push_poll_ranks:
        be.setOption("push_poll_ranks", args.push_poll_ranks)
    cfg = StackConfig(**{**QWEN3_8B.__dict__, "batch": args.batch})
    stack = DecodeStack(be, cfg, rank, world, args.tp_mode, allreduce=args.allreduce if (world > 1 and args.allreduce in ("p2p", "fused", "push")) else "nccl",
                        fuse=not args.no_fuse, chain=args.step_launch == "chain")
    chained = stack.uses_chain()
    if args.autotune:
        shapes = sorted({(cfg.batch, p.n, p.k) for p in stack.layers[0]} | {(cfg.batch, stack.lm_head.n, stack.lm_head.k)})
        be.setAutotuneEnabled(True)
        for (m, n, k) in shapes:
            be.pretuneMatmulShapes([(m, n, k)], cfg.act_dtype, cfg.act_dtype, tb.QuantPacking("int8-grouped", k, "f32", "direct"))
    if chained and args.chain_shape:
        w, d = (int(v) for v in args.chain_shape.split(","))
        be.forceVariant((B.TL_FAMILY_QGEMV, 7, w, d, 0, 0))
        try:
            stack.build_chain()
        finally:
            be.forceVariant(None)
    stack.capture()

    def barrier():
        if world > 1:
            dist.barrier()
        be.sync()
        torch.cuda.synchronize()

    def max_over_ranks(v: float) -> float:
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=torch.device("cuda", local_rank))
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    ev0, ev1 = C.c_void_p(), C.c_void_p()
    B.check(ctx, lib.tl_event_create(ctx, C.byref(ev0)))
    B.check(ctx, lib.tl_event_create(ctx, C.byref(ev1)))

    # ---- device-timed steps ------------------------------------------------
    # Blocks of exactly --steps steps, each bracketed by a barrier + synchronize on both sides and
    # timed with CUDA events on the library's stream; repeated until at least 0.5 s has been timed
    # (3 blocks at least) and the MEDIAN block (of the max over ranks) is reported.  The clock sampler
    # starts before the barrier, and one untimed step right behind the barrier aligns the ranks on
    # the device (it holds all-reduces), so host start-up skew never lands inside a timed block.
    def timed_blocks(st, min_seconds):
        blocks, total = [], 0.0
        while len(blocks) < 3 or (total < min_seconds and len(blocks) < 200):
            barrier()
            st.step()
            B.check(ctx, lib.tl_event_record(ctx, ev0))
            for _ in range(args.steps):
                st.step()
            B.check(ctx, lib.tl_event_record(ctx, ev1))
            barrier()
            ms = C.c_float()
            B.check(ctx, lib.tl_event_elapsed_ms(ctx, ev0, ev1, C.byref(ms)))
            blocks.append(max_over_ranks(ms.value))
            total += blocks[-1] * 1e-3
        return blocks

    for _ in range(args.warmup):
        stack.step()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = be.getKernelLaunchCount()
    block_ms = timed_blocks(stack, 0.5)
    launches = (be.getKernelLaunchCount() - launches0) * args.steps // ((args.steps + 1) * len(block_ms))
    dev_ms = statistics.median(block_ms)
    ms_per_step = dev_ms / args.steps
    value = cfg.batch * args.steps / (dev_ms * 1e-3)

    # ---- end to end: pinned host activations in, logits out, every step -----
    act_np = np.random.default_rng(1).standard_normal((cfg.batch, cfg.hidden)).astype(np.float16)
    hx = torch.from_numpy(act_np).pin_memory()
    hlogits = torch.empty(cfg.batch, cfg.vocab, dtype=torch.float32).pin_memory()
    h2d, d2h = hx.numel() * 2, hlogits.numel() * 4

    # Every rank uploads its copy of the step's activations; the step's result -- the gathered logits --
    # is read back where a sampler would sit: on rank 0 (the other ranks only synchronise).  With every
    # rank downloading all 4.9 MB the eight copies shared the host's PCIe paths: +0.2 ms per step at N = 8.
    def e2e_step():
        B.check(ctx, lib.tl_upload(ctx, stack.x.data_ptr(), hx.data_ptr(), h2d))
        stack.step()
        if rank == 0:
            B.check(ctx, lib.tl_download(ctx, hlogits.data_ptr(), stack.logits.data_ptr(), d2h))
        be.sync()

    for _ in range(max(1, args.warmup)):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    clocks = sampler.stop() if rank == 0 else None
    e2e_value = cfg.batch * args.steps / e2e_s
    finite = rank != 0 or (bool(torch.isfinite(hlogits).all().item()) and float(hlogits.abs().max()) > 0)

    parity = stack_parity(stack, dist if world > 1 else None)

    # ---- the same stack at batch 1, and (N > 1) with the gathered column-parallel layout -------
    def algorithmic_bytes(st, m):
        b = sum(p.n * p.k + p.n * 4 + m * p.k * 2 + m * p.n * 2 for p in st.layers[0]) * cfg.layers
        return b + st.lm_head.n * st.lm_head.k + st.lm_head.n * 4 + m * st.lm_head.k * 2 + m * st.lm_head.n * 4

    def secondary(batch, tp_mode):
        c2 = StackConfig(**{**QWEN3_8B.__dict__, "batch": batch})
        st = DecodeStack(be, c2, rank, world, tp_mode, allreduce=stack.allreduce, fuse=not args.no_fuse, chain=False)
        st.capture()
        for _ in range(max(3, args.warmup)):
            st.step()
        blocks = timed_blocks(st, 0.2)
        par = stack_parity(st, dist if world > 1 else None)
        ms_step = statistics.median(blocks) / args.steps
        res = {"batch": batch, "tp_mode": tp_mode if world > 1 else "none", "ms_per_step": ms_step, "tok_s": batch / (ms_step * 1e-3),
               "GBps_per_rank": algorithmic_bytes(st, batch) / (ms_step * 1e-3) / 1e9, "timed_blocks": len(blocks), "parity": par}
        st.destroy()
        return res
    stack_m1 = None if (args.no_extras or cfg.batch == 1) else secondary(1, args.tp_mode)
    stack_gather = None if (args.no_extras or world == 1 or args.tp_mode == "gather") else secondary(cfg.batch, "gather")

    hbm_peak, tf_peak, which = measured_peaks()
    # Per rank: the algorithmic bytes of its own shard, summed over the 253 launches of a step.
    m, a = cfg.batch, 2
    alg = 0
    for p in stack.layers[0]:
        alg += p.n * p.k + p.n * 4 + m * p.k * a + m * p.n * a
    alg *= cfg.layers
    alg += stack.lm_head.n * stack.lm_head.k + stack.lm_head.n * 4 + m * stack.lm_head.k * a + m * stack.lm_head.n * 4
    gemv_launches = stack.launches_per_step()
    achieved = alg / (ms_per_step * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                "traffic": None, "peak_source": f"{which} (MEASURED_PEAKS.json hbm_gbs)" if which == "measured" else "fallback 6650 GB/s",
                "kernel": "qgemv_chain_kernel" if chained else "qgemv_ring_kernel", "algorithmic_bytes_per_launch": alg / gemv_launches,
                "avg_launch_us": ms_per_step * 1e3 / gemv_launches,
                "note": ("per rank; one persistent launch runs all 253 projections of a step (145 phases), events on the launching stream"
                         if chained else
                         f"per rank; all {gemv_launches} small-batch GEMV launches of one step (253 projections), events on the launching stream")
                        + ("" if world == 1 else "; at N>1 the step time also holds the NCCL collectives")}
    tpath = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(tpath):
        try:
            # one ncu capture of the dominant kernel on a 58.9 MB matrix; DRAM traffic grows in
            # proportion to the matrix, so the measured traffic/algorithmic ratio is scaled to a launch
            roofline["traffic"] = json.load(open(tpath))["qgemv_dram_over_algorithmic_bytes"] * alg / gemv_launches
        except Exception:
            pass

    extras = {}
    cpu = None
    if rank == 0 and world == 1:
        if not args.no_extras:
            try:
                extras = single_matrix_extras(be, hbm_peak, tf_peak)
            except tb.TlError as ex:  # reported, never hidden
                extras = {"error": str(ex)}
        if not args.no_cpu:
            cpu = cpu_sample(cfg.batch)

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "int8 weights x f16 activations, f32 accumulate", "data": "synthetic",
            "config": {"workload": "qwen3-8b-decode-matmul-stack", "batch": cfg.batch, "layers": cfg.layers,
                       "hidden": cfg.hidden, "intermediate": cfg.inter, "vocab": cfg.vocab,
                       "weights": "int8 per-channel, f32 scales, random init", "parallelism": f"tp{world}",
                       "tp_mode": args.tp_mode if world > 1 else "none",
                       "allreduce": args.allreduce if world > 1 else "none",
                       "replay": "one persistent cooperative launch per step (tl_qgemv_chain)" if chained else "cuda graph",
                       "fusion": ("vertical: all 253 projections in one launch, weight prefetch runs across phase boundaries" if chained
                                  else "none" if args.no_fuse else "q+k+v and gate+up share one launch each (same activations)"),
                       "l2": "inputs larger than L2: 7.57 GB of weights per step, no flush needed",
                       "autotune": bool(args.autotune)},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_s / args.steps * 1e3, "logits_finite": finite,
                    "result_read_on": "rank 0 (every rank uploads the step's activations)"},
            "gpu_launches": int(launches), "timed_blocks": len(block_ms), "clocks": clocks, "roofline": roofline,
            "parity": parity,
            "weight_GB_per_step": cfg.weight_bytes_per_step() / 1e9,
        }
        if stack_m1 is not None:
            stack_m1["frac_of_hbm_peak"] = stack_m1["GBps_per_rank"] / hbm_peak
            line["stack_m1"] = stack_m1
        if stack_gather is not None:
            line["stack_tp_gather"] = stack_gather
        if cpu is not None:
            line["cpu_baseline"] = cpu
        if extras:
            line["kernels"] = extras
        print(json.dumps(line))
    stack.destroy()
    parity_ok = parity["lm_head_rel_err"] <= 1e-3 and parity["down_rel_err"] <= 1e-2 and parity["ranks_identical"]
    if world > 1:
        lib.tl_comm_destroy(ctx)
        dist.barrier()
        dist.destroy_process_group()
    if not parity_ok:
        raise SystemExit(f"bench.py: parity check failed: {parity}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tp-mode", default="chained", choices=["chained", "gather"])
    ap.add_argument("--autotune", action="store_true")
    ap.add_argument("--allreduce", default="push", choices=["p2p", "fused", "push", "nccl"],
                    help="row-parallel sums: push = the projection pushes f32 partial sums to every rank and the next "
                         "launch reduces them on read (no collective launch; default, fastest measured at 2, 4 and 8 GPUs); "
                         "p2p = the library's one-shot peer-memory all-reduce kernel; fused = the GEMV fused with its "
                         "all-reduce (tl_qgemv_nt_allreduce); nccl")
    ap.add_argument("--push-poll-ranks", type=int, default=0, help="reduce-on-read: ranks polled together (1..4; 0 = the library's default)")
    ap.add_argument("--step-launch", default="graph", choices=["chain", "graph"],
                    help="graph: a replayed CUDA graph of per-projection launches (the measured-faster default); "
                         "chain: the whole step as one persistent cooperative launch (one GPU, batch <= 16)")
    ap.add_argument("--chain-shape", default="", help="warps,depth of the chain kernel's CTAs (default: the library's)")
    ap.add_argument("--no-fuse", action="store_true", help="one launch per projection (no q/k/v and gate/up fusion)")
    ap.add_argument("--no-extras", action="store_true", help="skip the single-matrix GEMV / prefill GEMM figures")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline sample")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
