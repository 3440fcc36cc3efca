#!/usr/bin/env python
"""Benchmark of the arbitrary-bit quantized GEMM path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload at every N (one replica per GPU, no data-path collective): the decode-shape sweep
W2A8, W3A8, W4A8 x M in {1, 4, 16} over the LLaMA-7B linear shapes (N, K) in {(4096, 4096),
(12288, 4096), (11008, 4096), (4096, 11008)}; weights unsigned uniform over their bit range with a
per-128-group fp16 scale ~U(0.001, 0.02) and an integer zero point, activations int8 ~N(0, 30)
clipped, fp16 dequantised output.  One step = one pass over the 36 GEMMs.  All data is synthetic and
seeded; it stands in for real checkpoints, which are not needed to time a GEMM.

Metric: algorithmic GB/s (weight planes + activation planes + scales + zero points + output, each
counted once per GEMM) summed over the sweep -- the decode path is HBM-bound, so this is the number
its roofline is stated in; effective TOPS (2*M*N*K / t) per WxAy is reported beside it.

The line also carries `e2e` (same metric through the C ABI with host buffers: activation planes are
copied from pinned host memory and the fp16 result is copied back inside the timed region),
`roofline` (dominant kernel against the measured HBM peak) and `cpu_baseline` (the reference's CPU
loop on a bounded sample, rank 0, N=1 only).
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

SHAPES = [(4096, 4096), (12288, 4096), (11008, 4096), (4096, 11008)]
WBITS = [2, 3, 4]
MS = [1, 4, 16]
XBITS = 8
GROUP = 128
WEIGHT_COPIES = 2  # every weight exists twice and the copies alternate, so a pass never finds its planes in L2
METRIC = "quant_gemm_decode_sweep_algorithmic_GBps"
# dram__bytes_read + dram__bytes_write over algorithmic bytes, from the ncu capture of decode_kernel summarised in
# profiles/decode_kernel_sweep_and_w4a8_m1_32768x4096.md (a smaller single-shape case; traffic grows with the bytes)
DRAM_TRAFFIC_PER_ALGORITHMIC_BYTE = 1.018


def load_package():
    pkg = ROOT / "abq-llm_b200"
    spec = importlib.util.spec_from_file_location("abq_llm_b200", pkg / "__init__.py", submodule_search_locations=[str(pkg)])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["abq_llm_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


def algorithmic_bytes(M, N, K, p, q, group=GROUP):
    """Bytes one GEMM must move: W planes, X planes, fp16 output, fp16 scales, u8 zero points."""
    return q * N * K // 8 + p * M * K // 8 + 2 * M * N + 2 * N * (K // group) + N * (K // group)


def measured_peaks():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        d = json.loads(f.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [x.strip() for x in ln.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                smax = float(parts[1])
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": smax, "reasons": sorted(reasons), "samples": len(sm)}


def build_workload(abq, torch, seed):
    """Seeded device-resident operands (packed by the library's own pack kernel) and one launch plan per GEMM."""
    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed)
    B = abq.binding

    def pack(codes, bits):
        rows, K = codes.shape
        planes = torch.empty((bits, rows, K // 32), dtype=torch.int32, device="cuda")
        abq.pack_int32(codes.contiguous(), planes, rows, K, bits)
        return planes

    weights = {}
    for q in WBITS:
        for (N, K) in SHAPES:
            copies = []
            for c in range(WEIGHT_COPIES):
                codes = torch.randint(0, 1 << q, (N, K), dtype=torch.int32, device="cuda", generator=gen)
                planes = pack(codes, q)
                ws = (torch.rand((N, K // GROUP), device="cuda", generator=gen) * 0.019 + 0.001).to(torch.float16)
                wz = torch.randint(0, 1 << q, (N, K // GROUP), dtype=torch.int32, device="cuda", generator=gen).to(torch.uint8)
                copies.append((planes, ws, wz))
            weights[(q, N, K)] = copies
    acts = {}
    for M in MS:
        for K in sorted({k for _, k in SHAPES}):
            x = torch.clamp(torch.round(torch.randn((M, K), device="cuda", generator=gen) * 30.0), -128, 127).to(torch.int32)
            dev_x = pack(x, XBITS)
            host = torch.empty(dev_x.shape, dtype=torch.int32).pin_memory()
            host.copy_(dev_x)
            acts[(M, K)] = (host, dev_x)
    torch.cuda.synchronize()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    gemms = []
    # e2e mode: the activation planes of a whole pass travel in ONE pinned host buffer -> one device buffer, the fp16
    # results of a pass in one device buffer -> one pinned host buffer; every GEMM works on its views of the two
    order = [(q, M, N, K) for q in WBITS for M in MS for (N, K) in SHAPES]
    x_words = sum(XBITS * M * (K // 32) for (_, M, _, K) in order)
    out_elems = sum(M * N for (_, M, N, _) in order)
    e2e = {"x_host": torch.empty(x_words, dtype=torch.int32).pin_memory(), "x_dev": torch.empty(x_words, dtype=torch.int32, device="cuda"),
           "out_dev": torch.empty(out_elems, dtype=torch.float16, device="cuda"), "out_host": torch.empty(out_elems, dtype=torch.float16).pin_memory()}
    x_at = out_at = 0
    # one bit width after the other, as a model with one weight format runs them: consecutive GEMMs use the same kernel
    for (q, M, N, K) in order:
        ws_bytes = abq.gemm_workspace_bytes(M, N, K, XBITS, q)
        host_x, dev_x = acts[(M, K)]
        nx, no = XBITS * M * (K // 32), M * N
        e2e["x_host"][x_at:x_at + nx].copy_(host_x.view(-1))
        stage_x = e2e["x_dev"][x_at:x_at + nx].view(XBITS, M, K // 32)
        out_e2e = e2e["out_dev"][out_at:out_at + no].view(M, N)
        x_at, out_at = x_at + nx, out_at + no
        for c in range(WEIGHT_COPIES):
            planes, wsc, wz = weights[(q, N, K)][c]
            out = torch.empty((M, N), dtype=torch.float16, device="cuda")
            work = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
            states = {}
            for name, xbuf, obuf in (("resident", dev_x, out), ("e2e", stage_x, out_e2e)):
                p = B.make_params(M, N, K, xbuf, planes, obuf, x_bits=XBITS, w_bits=q, x_signed=True, w_signed=False,
                                  out_dtype=abq.OUT_FP16, scale_mode=abq.SCALE_GROUP, group_size=GROUP, w_scale=wsc, w_zero=wz,
                                  flags=abq.FLAG_PDL if os.environ.get("ABQ_BENCH_PDL", "1") == "1" else 0, workspace=work,
                                  status_word=status)
                states[name] = abq.gemm_init(p)
            gemms.append(dict(M=M, N=N, K=K, q=q, copy=c, states=states, out=out, host_x=host_x,
                              keep=(planes, wsc, wz, work, dev_x), bytes=algorithmic_bytes(M, N, K, XBITS, q), ops=2 * M * N * K))
    for g in gemms:
        g["e2e"] = e2e
    return gemms, status


def one_pass(abq, gemms, copy, mode):
    """One pass over the 36 GEMMs (weight copy `copy`).  mode 'resident': operands already in HBM;
    mode 'e2e': the pass's activation planes come from pinned host memory in one copy and its results go back to
    pinned host memory in one copy, both inside the pass."""
    mine = [g for g in gemms if g["copy"] == copy]
    if mode == "e2e" and mine:
        mine[0]["e2e"]["x_dev"].copy_(mine[0]["e2e"]["x_host"], non_blocking=True)      # this pass's activation planes, host -> device
    for g in mine:
        abq.gemm_exec(g["states"]["e2e" if mode == "e2e" else "resident"])
    if mode == "e2e" and mine:
        mine[0]["e2e"]["out_host"].copy_(mine[0]["e2e"]["out_dev"], non_blocking=True)  # this pass's results, device -> host


def capture_passes(torch, abq, gemms, mode):
    """One CUDA graph per weight copy holding a whole pass (72 kernels, plus the copies in e2e mode), so that the
    timed region measures the device and not the Python launch loop.  Returns a callable step(i)."""
    side = torch.cuda.Stream()
    graphs = []
    with torch.cuda.stream(side):
        for c in range(WEIGHT_COPIES):
            one_pass(abq, gemms, c, mode)  # first launches outside capture: kernel attributes get set here
        side.synchronize()
        for c in range(WEIGHT_COPIES):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                one_pass(abq, gemms, c, mode)
            graphs.append(g)
    torch.cuda.synchronize()
    return lambda i: graphs[i % WEIGHT_COPIES].replay()


def max_over_ranks(torch, dist, value: float, device) -> float:
    """The slowest rank's figure (timing rule for every multi-GPU number); identity without a process group."""
    if dist is None:
        return value
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def whole_job_rate(world: int, units_per_rank_step: float, steps: int, ms_max: float) -> float:
    """Replicas do not exchange data: the job processed world * units in the time of its slowest rank."""
    return world * units_per_rank_step * steps / (ms_max * 1e-3)


def timed(torch, dist, fn, steps, warmup):
    """W warm-up calls, then K timed calls between device events, barrier + synchronize on both sides; max over ranks."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for i in range(steps):
        fn(warmup + i)
    e1.record()
    torch.cuda.synchronize()
    wall_ms = (time.perf_counter() - t0) * 1e3
    ms = e0.elapsed_time(e1)
    if dist is not None:
        dist.barrier()
        torch.cuda.synchronize()
    return max_over_ranks(torch, dist, ms, "cuda"), wall_ms


def per_config_detail(torch, abq, gemms, reps=20):
    """Device time of every (WxAy, M, shape) GEMM alone, alternating the weight copies: TOPS and GB/s per config."""
    rows = []
    by_key = {}
    for g in gemms:
        by_key.setdefault((g["q"], g["M"], g["N"], g["K"]), []).append(g)
    for (q, M, N, K), gs in sorted(by_key.items()):
        for i in range(4):
            abq.gemm_exec(gs[i % len(gs)]["states"]["resident"])
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(reps):
            abq.gemm_exec(gs[i % len(gs)]["states"]["resident"])
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / reps
        rows.append({"wxay": f"W{q}A{XBITS}", "M": M, "N": N, "K": K, "us": round(us, 3), "GBps": round(gs[0]["bytes"] / us / 1e3, 1),
                     "TOPS": round(gs[0]["ops"] / us / 1e6, 3)})
    return rows


PREFILL_CASES = [(4, 4, 4096, 4096, 4096, 0), (4, 4, 4096, 11008, 4096, 0), (2, 8, 4096, 12288, 4096, 0), (8, 8, 4096, 4096, 11008, 0),
                 (4, 4, 2048, 4096, 4096, 0), (4, 4, 512, 12288, 4096, 0),
                 (4, 8, 4096, 4096, 4096, 128), (2, 8, 2048, 11008, 4096, 128)]  # (w bits, x bits, M, N, K, scale group: 0 = per channel)


def prefill_leg(torch, abq, reps=10):
    """Prefill shapes (M >= 512) on the tcgen05 kind::i8 route, per-channel or per-group fp16 scale, fp16 output: device time of the
    whole call (plane -> int8 expansion of both operands, the GEMM with its fused epilogue) per case, effective
    TOPS = 2*M*N*K / t, and the fraction of twice the measured dense bf16 rate (the int8 rate of the same pipe)."""
    peak = None
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        peak = 2.0 * float(json.loads(f.read_text())["bf16_tflops"])
    gen = torch.Generator(device="cuda")
    gen.manual_seed(7)
    B = abq.binding
    rows = []
    for (q, p, M, N, K, group) in PREFILL_CASES:
        def planes_of(rows_, bits):
            codes = torch.randint(0, 1 << bits, (rows_, K), dtype=torch.int32, device="cuda", generator=gen)
            out = torch.empty((bits, rows_, K // 32), dtype=torch.int32, device="cuda")
            abq.pack_int32(codes, out, rows_, K, bits)
            return out
        xp, wp = planes_of(M, p), planes_of(N, q)
        shape = (N, K // group) if group else (N,)
        wsc = (torch.rand(shape, device="cuda", generator=gen) * 0.019 + 0.001).to(torch.float16)
        wz = torch.randint(0, 1 << q, shape, dtype=torch.int32, device="cuda", generator=gen).to(torch.uint8) if group else None
        out = torch.empty((M, N), dtype=torch.float16, device="cuda")
        work = torch.empty(abq.gemm_workspace_bytes(M, N, K, p, q), dtype=torch.uint8, device="cuda")
        prm = B.make_params(M, N, K, xp, wp, out, x_bits=p, w_bits=q, x_signed=bool(group), w_signed=False, out_dtype=abq.OUT_FP16,
                            scale_mode=abq.SCALE_GROUP if group else abq.SCALE_CHANNEL, group_size=group, w_scale=wsc, w_zero=wz,
                            workspace=work)
        st = abq.gemm_init(prm)
        for _ in range(3):
            abq.gemm_exec(st)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            abq.gemm_exec(st)
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / reps
        tops = 2.0 * M * N * K / us / 1e6
        # the same call with the weight codes expanded once beforehand (weights that stay the same from call to call)
        prm.flags = abq.FLAG_WEIGHTS_PREPARED
        st2 = abq.gemm_init(prm)
        abq.gemm_prepare_weights(st2)
        for _ in range(3):
            abq.gemm_exec(st2)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(reps):
            abq.gemm_exec(st2)
        e1.record()
        torch.cuda.synchronize()
        us2 = e0.elapsed_time(e1) * 1e3 / reps
        tops2 = 2.0 * M * N * K / us2 / 1e6
        # ... and with fp16 activations handed to the call (quantised straight to int8 codes): the FasterTransformer wrapper's path
        xh = (torch.randn((M, K), device="cuda", generator=gen) * 2).to(torch.float16)
        qs = torch.full((1,), 1.5 if p < 8 else 12.0, dtype=torch.float32, device="cuda")
        prm3 = B.make_params(M, N, K, xh, wp, out, x_bits=p, w_bits=q, x_signed=True, w_signed=False, out_dtype=abq.OUT_FP16,
                             scale_mode=abq.SCALE_GROUP if group else abq.SCALE_CHANNEL, group_size=group, w_scale=wsc, w_zero=wz,
                             workspace=work, flags=abq.FLAG_WEIGHTS_PREPARED | abq.FLAG_X_HALF, x_quant_scale=qs)
        st3 = abq.gemm_init(prm3)
        abq.gemm_prepare_weights(st3)
        for _ in range(3):
            abq.gemm_exec(st3)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(reps):
            abq.gemm_exec(st3)
        e1.record()
        torch.cuda.synchronize()
        us3 = e0.elapsed_time(e1) * 1e3 / reps
        tops3 = 2.0 * M * N * K / us3 / 1e6
        rows.append({"wxay": f"W{q}A{p}", "scales": f"g{group} + zero" if group else "channel", "M": M, "N": N, "K": K, "us": round(us, 2),
                     "TOPS": round(tops, 1),
                     "frac_of_int8_peak": round(tops / peak, 3) if peak else None, "us_weights_prepared": round(us2, 2),
                     "TOPS_weights_prepared": round(tops2, 1), "frac_weights_prepared": round(tops2 / peak, 3) if peak else None,
                     "us_half_x_prepared_w": round(us3, 2), "TOPS_half_x_prepared_w": round(tops3, 1),
                     "frac_half_x_prepared_w": round(tops3 / peak, 3) if peak else None})
        del xp, wp, out, work, xh
    return {"route": "tcgen05 kind::i8 (plane->int8 expansion included in the time)", "int8_peak_TOPS": peak,
            "peak_source": "2 x MEASURED_PEAKS.json bf16_tflops" if peak else None, "cases": rows}


def _time_calls(torch, fn, reps=10, warm=3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / reps


def routes_leg(torch, abq):
    """The two formulations side by side on one decode and one prefill shape (int32 output, so that the numbers are the
    contraction alone): route A = 1-bit mma.sync AND+POPC over the stacked planes as the reference does it, against the
    int8 routes that the planner picks."""
    gen = torch.Generator(device="cuda")
    gen.manual_seed(11)
    B = abq.binding
    rows = []
    for (q, p, M, N, K, fast) in [(2, 8, 1, 4096, 4096, abq.ROUTE_I8_MMA), (2, 8, 16, 4096, 4096, abq.ROUTE_I8_MMA),
                                  (4, 4, 512, 4096, 4096, abq.ROUTE_I8_UMMA)]:
        def planes_of(r, bits):
            codes = torch.randint(0, 1 << bits, (r, K), dtype=torch.int32, device="cuda", generator=gen)
            out = torch.empty((bits, r, K // 32), dtype=torch.int32, device="cuda")
            abq.pack_int32(codes, out, r, K, bits)
            return out
        xp, wp = planes_of(M, p), planes_of(N, q)
        out = torch.empty((M, N), dtype=torch.int32, device="cuda")
        res = {}
        for name, route in (("b1_mma", abq.ROUTE_B1_MMA), ("int8", fast)):
            work = torch.empty(max(256, abq.gemm_workspace_bytes(M, N, K, p, q, route)), dtype=torch.uint8, device="cuda")
            st = abq.gemm_init(B.make_params(M, N, K, xp, wp, out, x_bits=p, w_bits=q, x_signed=False, w_signed=False, route=route, workspace=work))
            res[name] = _time_calls(torch, lambda: abq.gemm_exec(st), reps=5 if name == "b1_mma" else 20)
        rows.append({"wxay": f"W{q}A{p}", "M": M, "N": N, "K": K, "us_route_a_b1_mma": round(res["b1_mma"], 1),
                     "us_int8_route": round(res["int8"], 1), "int8_route": "I8_MMA" if fast == abq.ROUTE_I8_MMA else "I8_UMMA",
                     "ratio": round(res["b1_mma"] / res["int8"], 1)})
    return rows


def pack_leg(torch, abq):
    """The pack kernels against the HBM roofline: bytes read + planes written per launch over the launch time, on inputs
    larger than L2 (a prefill batch of activations, a weight matrix)."""
    peak, _ = measured_peaks()
    gen = torch.Generator(device="cuda")
    gen.manual_seed(5)
    rows = []
    M, K = 16384, 8192  # 268 MB of fp16 activations, 537 MB of int32 codes
    x16 = (torch.randn((M, K), device="cuda", generator=gen) * 3).to(torch.float16)
    scale = torch.full((1,), 8.0, dtype=torch.float32, device="cuda")
    for bits in (8, 4):
        planes = torch.empty((bits, M, K // 32), dtype=torch.int32, device="cuda")
        us = _time_calls(torch, lambda: abq.quantize_pack_half(x16, scale, planes, M, K, bits, 0))
        nbytes = 2 * M * K + bits * M * K // 8
        rows.append({"kernel": f"quantize_pack_half_kernel<{bits}>", "rows": M, "K": K, "us": round(us, 1), "GBps": round(nbytes / us / 1e3, 1),
                     "frac_of_hbm": round(nbytes / us / 1e3 / peak, 3)})
    del x16
    codes = torch.randint(0, 16, (M, K), dtype=torch.int32, device="cuda", generator=gen)
    for bits in (4, 2):
        planes = torch.empty((bits, M, K // 32), dtype=torch.int32, device="cuda")
        us = _time_calls(torch, lambda: abq.pack_int32(codes, planes, M, K, bits))
        nbytes = 4 * M * K + bits * M * K // 8
        rows.append({"kernel": f"pack_int32_kernel<{bits}>", "rows": M, "K": K, "us": round(us, 1), "GBps": round(nbytes / us / 1e3, 1),
                     "frac_of_hbm": round(nbytes / us / 1e3 / peak, 3)})
    return rows


def cpu_baseline_sample(kind_pref: str, budget_s: float = 12.0):
    """The reference's CPU loop (`compute_ref`) on a bounded sample of the sweep: its W2A8, M=16, N=4096,
    K=4096 GEMM, repeated until about `budget_s` seconds of host time are spent; all host cores."""
    from oracle import oracle as O
    O.build()
    use_ref = O.ref_available() and kind_pref != "port"
    M, N, K, q, p = 16, 4096, 4096, 2, XBITS
    rng = np.random.default_rng(1)
    cores = os.cpu_count() or 1
    x = np.clip(np.rint(rng.normal(0, 30, size=(M, K))), -128, 127).astype(np.int32)
    xp = O.pack(x, p)
    rows = (N + cores - 1) // cores
    slabs = [O.pack(rng.integers(0, 1 << q, size=(rows, K), dtype=np.int32), q) for _ in range(cores)]
    whole = np.concatenate(slabs, axis=1)

    def run():
        def work(i):
            O.ref_compute_ref(slabs[i], xp, True)

        t0 = time.perf_counter()
        if use_ref:  # the reference loop is single-threaded: one slab of weight rows per core
            threads = [threading.Thread(target=work, args=(i,)) for i in range(cores)]
            for th in threads:
                th.start()
            for th in threads:
                th.join()
        else:        # the C restatement splits the output range over pthreads itself
            O.set_threads(cores)
            O.compute_ref(whole, xp, True, True)
        return time.perf_counter() - t0

    first = run()
    reps = int(max(1, min(64, budget_s / max(first, 1e-3))))
    t = sum(run() for _ in range(reps))
    n_rows = rows * cores
    nbytes = algorithmic_bytes(M, n_rows, K, p, q) * reps
    return {"value": nbytes / t / 1e9, "unit": "GB/s", "cores": cores, "kind": "reference" if use_ref else "port",
            "sample": f"W2A8 M=16 N={n_rows} K=4096 (signed planes, as the reference's driver runs it), compute_ref x{reps} "
                      f"in {t:.2f} s = {2 * M * n_rows * K * reps / t / 1e12:.6f} effective TOPS",
            "seconds": t}


WORKLOAD = ("decode sweep (BASELINE configs[1]): W{2,3,4}A8 x M{1,4,16} x (N,K) in "
            "{(4096,4096),(12288,4096),(11008,4096),(4096,11008)}, g128 fp16 scale + u8 zero, fp16 out")


REF_GPU_CASES = [(1, 1, 4096, 4096), (1, 1, 12288, 4096), (1, 1, 11008, 4096), (3, 8, 12288, 4096)]  # (kernel id, M, N, K), unsigned W2A8


def reference_gpu_kernels():
    """Device time of the reference's own W2A8 GPU kernels (the two tiles its FasterTransformer wrapper hard-codes,
    compiled from its headers into oracle/_ref/libabq_ref_gpu.so) on sweep shapes: int32 output, no scales (it has
    none), weight copies rotating so that no launch finds its planes in L2, one CUDA graph of all launches."""
    from oracle import oracle as O
    try:
        import torch
    except ImportError:
        return None
    if not (O.ref_gpu_available() and torch.cuda.is_available()):
        return None
    rng = np.random.default_rng(3)
    rows = []
    for (cfg, M, N, K) in REF_GPU_CASES:
        p, q, signed = O.ref_gpu_config(cfg)
        copies = max(2, int(160e6 // (q * N * K // 8)) + 1)
        xp = torch.from_numpy(O.pack(rng.integers(0, 1 << p, size=(M, K), dtype=np.int32), p).view(np.int32)).cuda()
        base = torch.from_numpy(O.pack(rng.integers(0, 1 << q, size=(N, K), dtype=np.int32), q).view(np.int32)).cuda()
        ws = [base] + [torch.roll(base, c, dims=1) for c in range(1, copies)]
        out = torch.empty((M, N), dtype=torch.int32, device="cuda")
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            O.ref_gpu_gemm(cfg, xp.data_ptr(), ws[0].data_ptr(), M, N, K, out.data_ptr(), 1, side.cuda_stream)
            side.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                for w in ws:
                    O.ref_gpu_gemm(cfg, xp.data_ptr(), w.data_ptr(), M, N, K, out.data_ptr(), 1, side.cuda_stream)
        torch.cuda.synchronize()
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(3):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (3 * copies)
        nbytes = q * N * K // 8 + p * M * K // 8 + 4 * M * N
        rows.append({"kernel": O.REF_GPU_CONFIGS[cfg], "M": M, "N": N, "K": K, "us": round(us, 2), "GBps": round(nbytes / us / 1e3, 1),
                     "TOPS": round(2 * M * N * K / us / 1e6, 3)})
        del ws, base
    return rows


def run_tp_decode(args, rank, world, local):
    """`--workload tp_decode`: one decode step through the quantized linear layers of LLaMA-7B (32 blocks: fused QKV, O,
    fused gate+up, down; W4A4, per-channel scale + zero point, static activation scale), tensor parallel over the
    ranks: column-parallel QKV / gate+up, row-parallel O / down with an NCCL all-reduce after each.  Attention, norms,
    embedding and lm_head are outside the path (elementwise torch stand-ins keep the data flowing).  Strong scaling:
    the model is fixed, every rank holds 1/N of every weight."""
    import torch
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local))
        dist = dist_mod
    abq = load_package()
    spec = importlib.util.spec_from_file_location("abq_llm_b200.tp_linear", ROOT / "abq-llm_b200" / "tp_linear.py")
    tp = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = tp
    spec.loader.exec_module(tp)
    hidden, ffn, layers, q, p = 4096, 11008, args.layers, 4, 4
    gen = torch.Generator(device="cuda")
    backend = tp.AbqBackend(abq, torch, dist, x_bits=p, x_scale=2.0, max_tokens=32)
    blocks = []
    for layer in range(layers):
        gen.manual_seed(1000 + layer)  # the same full weights on every rank; each keeps its shard
        weights = []
        for sp in tp.llama_block_specs(hidden, ffn):
            codes = torch.randint(0, 1 << q, (sp.out_features, sp.in_features), dtype=torch.int32, device="cuda", generator=gen)
            scale = (torch.rand((sp.out_features,), device="cuda", generator=gen) * 0.002 + 0.0005).to(torch.float16)
            zero = torch.randint(0, 1 << q, (sp.out_features,), dtype=torch.int32, device="cuda", generator=gen).to(torch.uint8)
            weights.append((codes, scale, zero))
        blocks.append(tp.TensorParallelBlockLinears(backend, hidden, ffn, rank, world, weights, q, 0))
        del weights
    results = []
    for M in (1, 8, 32):
        gen.manual_seed(7)
        x = (torch.randn((M, hidden), device="cuda", generator=gen)).to(torch.float16)

        def step():
            h = x
            for b in blocks:
                h = b.forward(h)
            return h
        for _ in range(2):
            step()  # plans and buffers are made here
        torch.cuda.synchronize()
        if rank == 0:
            print(f"tp_decode: batch {M} warmed up", file=sys.stderr, flush=True)
        graph = None
        pieces = None
        # The whole step as one CUDA graph: on one GPU, and on several ranks when the all-reduce is the library's own
        # one-shot kernel over peer memory.  With NCCL all-reduces (ABQ_TP_NCCL=1): the pieces between them as graphs
        # and the collectives launched in between (a capture that contained NCCL collectives did not finish on this stack)
        if not args.no_graph and (world == 1 or backend.peer_reduce) and not args.tp_pieces:
            try:
                side = torch.cuda.Stream()
                with torch.cuda.stream(side):
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph, stream=side):
                        step()
                torch.cuda.synchronize()
            except Exception as e:
                graph = None
                if rank == 0:
                    print(f"graph capture failed ({type(e).__name__}): timing eager launches", file=sys.stderr)
        elif not args.no_graph:
            side = torch.cuda.Stream()
            pieces, pool = [], None
            with torch.cuda.stream(side):
                cur, pend = x, None
                for b in blocks:
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=side, pool=pool):
                        xin = cur if pend is None else backend.glue_residual(pend[0], pend[1], None)
                        o = b.attention_part(xin)
                    pool = pool or g.pool()
                    pieces.append((g, o))
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=side, pool=pool):
                        h, d = b.ffn_part(xin, o)
                    pieces.append((g, d))
                    pend = (h, d)
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side, pool=pool):
                    y = backend.glue_residual(pend[0], pend[1], None)
                pieces.append((g, None))
            torch.cuda.synchronize()

        def step_pieces():
            for g, t in pieces:
                g.replay()
                if t is not None:
                    backend.all_reduce(t)
        fn = (lambda i: graph.replay()) if graph is not None else ((lambda i: step_pieces()) if pieces else (lambda i: step()))
        ms, _ = timed(torch, dist, fn, max(3, args.steps // 10), 3)
        n = max(3, args.steps // 10)
        results.append({"batch": M, "ms_per_step": ms / n, "tokens_per_s": M * n / (ms * 1e-3), "cuda_graph": "whole step" if graph is not None else ("between the all-reduces" if pieces else "no")})
    if rank == 0:
        wbytes = layers * sum(sp.out_features * sp.in_features for sp in tp.llama_block_specs(hidden, ffn)) * q // 8
        best = results[0]
        line = {"metric": "llama7b_w4a4_linear_stack_decode_tokens_per_s", "value": best["tokens_per_s"], "unit": "tokens/s", "n_gpus": world,
                "steps": max(3, args.steps // 10), "warmup": 3, "ms_per_step": best["ms_per_step"], "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
                "config": {"workload": f"LLaMA-7B linear layers only, {layers} blocks, W4A4 per-channel, tensor parallel {world}, batch 1 "
                                       "(value); batches 8 and 32 in `batches`", "weight_bytes_all_ranks": wbytes},
                "batches": results,
                "hbm_bound_tokens_per_s_batch1": world * measured_peaks()[0] * 1e9 / wbytes}
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


def run_reference(args, rank, world):
    """`--impl reference`: the reference's own CPU implementation of the path on the host cores."""
    if rank != 0:
        return
    steps, warm = max(1, args.steps), max(0, args.warmup)
    per = max(1.0, min(10.0, 60.0 / (steps + warm)))
    vals = []
    base = None
    for i in range(warm + steps):
        base = cpu_baseline_sample("reference", budget_s=per)
        if i >= warm:
            vals.append(base)
    total_t = sum(v["seconds"] for v in vals)
    value = statistics.mean(v["value"] for v in vals)
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": args.gpus, "steps": steps, "warmup": warm,
            "ms_per_step": total_t / steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int32",
            "data": "synthetic", "config": {"workload": WORKLOAD + "; each step a bounded sample (one M=16 W2A8 4096x4096 GEMM of the sweep, "
                                                                   "repeated) on the host cores, reference compute_ref"},
            "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    line["cpu_baseline"]["value"] = value
    gpu_rows = reference_gpu_kernels()  # context only: the arm's value stays the reference's CPU implementation
    if gpu_rows:
        line["reference_gpu_kernels"] = gpu_rows
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--detail", action="store_true", help="also time every GEMM of the sweep alone")
    ap.add_argument("--only", default="", help="profiling aid: restrict the sweep to GEMMs 'q:M:N:K[,q:M:N:K...]' (0 = any)")
    ap.add_argument("--shape", default="", help="profiling aid: replace the sweep by the single GEMM 'q:M:N:K' (any size the route takes)")
    ap.add_argument("--no-prefill", action="store_true", help="skip the short prefill-shape (tcgen05 route) leg")
    ap.add_argument("--workload", default="decode_sweep", choices=["decode_sweep", "tp_decode"],
                    help="decode_sweep (default, the headline metric) or tp_decode: tensor-parallel LLaMA-7B linear stack")
    ap.add_argument("--layers", type=int, default=32, help="tp_decode: decoder blocks")
    ap.add_argument("--tp-pieces", action="store_true", help="tp_decode on one GPU: graphs between the all-reduce points, as several ranks run it")
    ap.add_argument("--no-graph", action="store_true", help="profiling aid: launch kernel by kernel instead of one CUDA graph per pass")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="profiling aid: skip the host-side reference timing")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    args.warmup = max(3, args.warmup)
    if args.workload == "tp_decode":
        run_tp_decode(args, rank, world, local)
        return

    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU path")
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local))
        dist = dist_mod
    abq = load_package()
    if args.shape:
        q, M, N, K = (int(v) for v in args.shape.split(":"))
        global SHAPES, WBITS, MS
        SHAPES, WBITS, MS = [(N, K)], [q], [M]
    gemms, status = build_workload(abq, torch, seed=20241 + rank)
    if args.only:
        pats = [tuple(int(v) for v in item.split(":")) for item in args.only.split(",")]
        gemms = [g for g in gemms if any(all(a == 0 or a == b for a, b in zip(pat, (g["q"], g["M"], g["N"], g["K"]))) for pat in pats)]
    n_gemm = len(gemms) // WEIGHT_COPIES
    bytes_per_step = sum(g["bytes"] for g in gemms if g["copy"] == 0)
    ops_per_step = sum(g["ops"] for g in gemms if g["copy"] == 0)

    sampler = ClockSampler(local)
    sampler.start()
    use_graph = not args.no_graph
    step_res = capture_passes(torch, abq, gemms, "resident") if use_graph else (lambda i: one_pass(abq, gemms, i % WEIGHT_COPIES, "resident"))
    step_e2e = capture_passes(torch, abq, gemms, "e2e") if use_graph else (lambda i: one_pass(abq, gemms, i % WEIGHT_COPIES, "e2e"))
    ms, wall_ms = timed(torch, dist, step_res, args.steps, args.warmup)
    clocks = sampler.stop()
    ms_e2e, _ = timed(torch, dist, step_e2e, args.steps, args.warmup)
    if int(status.item()) != 0:
        raise SystemExit(f"device status word {int(status.item())}: a bounded wait expired, the numbers are void")

    value = whole_job_rate(world, bytes_per_step, args.steps, ms) / 1e9
    e2e = whole_job_rate(world, bytes_per_step, args.steps, ms_e2e) / 1e9
    h2d = sum(g["host_x"].numel() * 4 for g in gemms if g["copy"] == 0)
    d2h = sum(g["out"].numel() * 2 for g in gemms if g["copy"] == 0)
    if args.only or args.shape:
        h2d, d2h = gemms[0]["e2e"]["x_host"].numel() * 4, gemms[0]["e2e"]["out_host"].numel() * 2  # the buffers travel whole
    peak, peak_kind = measured_peaks()
    per_gpu = bytes_per_step * args.steps / (ms * 1e-3) / 1e9
    line = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8",
        "data": "synthetic",
        "config": {"workload": WORKLOAD + f"; {n_gemm} GEMMs per step" + (f" (restricted by --only {args.only})" if args.only else ""),
                   "l2": f"two alternating copies of every weight, {bytes_per_step / 1e6:.0f} MB of distinct operands between reuses (> 126 MB L2)",
                   "replicas": world, "pdl": os.environ.get("ABQ_BENCH_PDL", "1") == "1", "cuda_graph_per_pass": use_graph},
        "effective_TOPS": whole_job_rate(world, ops_per_step, args.steps, ms) / 1e12,
        "e2e": {"value": e2e, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": n_gemm * args.steps,  # one decode_kernel per GEMM
        "clocks": clocks,
        "roofline": {"bound": "hbm", "kernel": "decode_kernel (36 launches per step, all shapes)", "achieved": per_gpu, "peak": peak,
                     "unit": "GB/s", "frac": per_gpu / peak, "peak_source": f"{peak_kind} (MEASURED_PEAKS.json hbm_gbs)",
                     "bytes_per_launch": bytes_per_step / max(1, n_gemm), "us_per_launch": ms * 1e3 / args.steps / max(1, n_gemm),
                     "traffic": DRAM_TRAFFIC_PER_ALGORITHMIC_BYTE * bytes_per_step / max(1, n_gemm),
                     "traffic_source": "ncu dram bytes of a single-shape capture, scaled by algorithmic bytes (mean launch of the sweep)"},
        "wall_ms_per_step": wall_ms / args.steps,
    }
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        base = cpu_baseline_sample("reference")
        line["cpu_baseline"] = {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")}
    if args.shape:
        line["config"]["workload"] = f"single GEMM --shape {args.shape} (profiling aid, not the sweep)"
    if rank == 0 and world == 1 and not args.no_prefill and not args.shape and not args.only:
        line["prefill"] = prefill_leg(torch, abq)
        line["routes"] = routes_leg(torch, abq)
        line["pack"] = pack_leg(torch, abq)
    if args.detail and rank == 0:
        line["detail"] = per_config_detail(torch, abq, gemms)
    if rank == 0:
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
