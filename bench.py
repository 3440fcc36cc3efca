#!/usr/bin/env python
"""Benchmark of the arbitrary-bit quantized GEMM path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload at every N (one replica per GPU, no data-path collective): the decode-shape sweep
W2A8, W3A8, W4A8 x M in {1, 4, 16} over the LLaMA-7B linear shapes (N, K) in {(4096, 4096),
(12288, 4096), (11008, 4096), (4096, 11008)}; weights unsigned uniform over their bit range with a
per-128-group fp16 scale ~U(0.001, 0.02) and an integer zero point, activations int8 ~N(0, 30)
clipped, fp16 dequantised output.  One pass = the 36 GEMMs once; one step = PASSES_PER_STEP passes
(one CUDA graph), so that the timed region is long enough for the clock sampler.  All data is synthetic
and seeded; it stands in for real checkpoints, which are not needed to time a GEMM.

Metric: algorithmic GB/s (weight bits + activation planes + scales + zero points + output, each
counted once per GEMM) summed over the sweep -- the decode path is HBM-bound, so this is the number
its roofline is stated in; per-WxAy figures (time, GB/s, fraction of the HBM peak, effective TOPS) are in
`detail`.  The weights are read in the library's prepared (load-time re-ordered) form, `planes` holds the
same sweep reading the reference's plane format directly.

The line also carries `e2e` (same metric through the C ABI with host buffers: activation planes are
copied from pinned host memory and the fp16 result is copied back inside the timed region),
`roofline` (dominant kernel against the measured HBM peak), `cpu_baseline` (the reference's CPU loop on
a bounded sample, rank 0, N=1 only), `config0` (the reference's own CPU-checkable case), `prefill`
(tensor-core route) and, on several GPUs, `tp_decode` (the tensor-parallel LLaMA-7B linear stack).
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
# Every weight exists once per token count and GEMM (q, M, N, K) reads copy MS.index(M): two reads of one buffer are a
# whole pass apart (the 36 GEMMs move 569 MB, 4.5 x the 126 MB L2), so no launch finds its weights in L2.
WEIGHT_COPIES = len(MS)
PASSES_PER_STEP = 200
METRIC = "quant_gemm_decode_sweep_algorithmic_GBps"
# dram__bytes_read + dram__bytes_write per algorithmic byte of the dominant kernel, from an ncu capture of a sweep-sized
# launch (stream_kernel: W2A8, M=1, 12288 x 4096, 14.25 MB against 13.79 MB; decode_kernel: W4A8, M=1, 32768 x 4096);
# traffic grows with the bytes, so it is scaled to the mean launch of the sweep
DRAM_TRAFFIC_PER_ALGORITHMIC_BYTE = {"stream_kernel": 1.033, "decode_kernel": 1.018}


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


def _params(abq, g, xbuf, obuf, kind, status):
    """abq_gemm_params of sweep GEMM `g` reading its weights as planes or in the prepared form."""
    B = abq.binding
    flags = abq.FLAG_PDL if os.environ.get("ABQ_BENCH_PDL", "1") == "1" else 0
    prepared = None
    if kind == "prepared":
        flags |= abq.FLAG_WEIGHTS_PREPARED
        prepared = g["prepared"]
    return B.make_params(g["M"], g["N"], g["K"], xbuf, g["planes"], obuf, x_bits=XBITS, w_bits=g["q"], x_signed=True, w_signed=False,
                         out_dtype=abq.OUT_FP16, scale_mode=abq.SCALE_GROUP, group_size=g.get("group", GROUP), w_scale=g["w_scale"], w_zero=g["w_zero"],
                         flags=flags, workspace=g["work"], status_word=status, w_prepared=prepared)


def build_workload(abq, torch, seed):
    """Seeded device-resident operands (packed by the library's own pack kernel), the prepared copy of every weight
    (made once here by abq_gemm_prepare_weights, as a model loader would) and the launch plans of every GEMM."""
    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed)

    def pack(codes, bits):
        rows, K = codes.shape
        planes = torch.empty((bits, rows, K // 32), dtype=torch.int32, device="cuda")
        abq.pack_int32(codes.contiguous(), planes, rows, K, bits)
        return planes

    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    acts = {}
    for M in MS:
        for K in sorted({k for _, k in SHAPES}):
            x = torch.clamp(torch.round(torch.randn((M, K), device="cuda", generator=gen) * 30.0), -128, 127).to(torch.int32)
            dev_x = pack(x, XBITS)
            host = torch.empty(dev_x.shape, dtype=torch.int32).pin_memory()
            host.copy_(dev_x)
            acts[(M, K)] = (host, dev_x)
    # e2e mode: the activation planes of a whole pass travel in ONE pinned host buffer -> one device buffer, the fp16
    # results of a pass in one device buffer -> one pinned host buffer; every GEMM works on its views of the two.
    # One token count after the other (a decode step runs all its GEMMs at one batch size), within it one bit width after the
    # other; ABQ_BENCH_ORDER=width puts the bit width outermost instead.
    order = [(q, M, N, K) for M in MS for q in WBITS for (N, K) in SHAPES]
    if os.environ.get("ABQ_BENCH_ORDER", "tokens") == "width":
        order = [(q, M, N, K) for q in WBITS for M in MS for (N, K) in SHAPES]
    x_words = sum(XBITS * M * (K // 32) for (_, M, _, K) in order)
    out_elems = sum(M * N for (_, M, N, _) in order)
    e2e = {"x_host": torch.empty(x_words, dtype=torch.int32).pin_memory(), "x_dev": torch.empty(x_words, dtype=torch.int32, device="cuda"),
           "out_dev": torch.empty(out_elems, dtype=torch.float16, device="cuda"), "out_host": torch.empty(out_elems, dtype=torch.float16).pin_memory()}
    gemms = []
    x_at = out_at = 0
    for (q, M, N, K) in order:
        codes = torch.randint(0, 1 << q, (N, K), dtype=torch.int32, device="cuda", generator=gen)
        g = dict(q=q, M=M, N=N, K=K, planes=pack(codes, q),
                 w_scale=(torch.rand((N, K // GROUP), device="cuda", generator=gen) * 0.019 + 0.001).to(torch.float16),
                 w_zero=torch.randint(0, 1 << q, (N, K // GROUP), dtype=torch.int32, device="cuda", generator=gen).to(torch.uint8),
                 work=torch.empty(max(256, abq.gemm_workspace_bytes(M, N, K, XBITS, q)), dtype=torch.uint8, device="cuda"),
                 out=torch.empty((M, N), dtype=torch.float16, device="cuda"), bytes=algorithmic_bytes(M, N, K, XBITS, q), ops=2 * M * N * K)
        del codes
        host_x, dev_x = acts[(M, K)]
        nx, no = XBITS * M * (K // 32), M * N
        e2e["x_host"][x_at:x_at + nx].copy_(host_x.view(-1))
        stage_x = e2e["x_dev"][x_at:x_at + nx].view(XBITS, M, K // 32)
        out_e2e = e2e["out_dev"][out_at:out_at + no].view(M, N)
        x_at, out_at = x_at + nx, out_at + no
        g["host_x"], g["dev_x"] = host_x, dev_x
        probe = _params(abq, g, dev_x, g["out"], "planes", status)
        nbytes = abq.gemm_prepared_weight_bytes(probe)
        g["prepared"] = torch.empty(nbytes, dtype=torch.uint8, device="cuda") if nbytes else None
        g["states"] = {"planes": abq.gemm_init(probe)}
        if nbytes:
            g["states"]["prepared"] = abq.gemm_init(_params(abq, g, dev_x, g["out"], "prepared", status))
            abq.gemm_prepare_weights(g["states"]["prepared"])
            g["states"]["e2e"] = abq.gemm_init(_params(abq, g, stage_x, out_e2e, "prepared", status))
        else:
            g["states"]["prepared"] = g["states"]["planes"]
            g["states"]["e2e"] = abq.gemm_init(_params(abq, g, stage_x, out_e2e, "planes", status))
        g["e2e"] = e2e
        gemms.append(g)
    torch.cuda.synchronize()
    return gemms, status


def one_pass(abq, gemms, mode):
    """One pass over the 36 GEMMs.  mode 'prepared' / 'planes': operands already in HBM, weights in the prepared form /
    as the reference's planes; mode 'e2e': the pass's activation planes come from pinned host memory in one copy and its
    results go back to pinned host memory in one copy, both inside the pass (weights prepared)."""
    if mode == "e2e" and gemms:
        gemms[0]["e2e"]["x_dev"].copy_(gemms[0]["e2e"]["x_host"], non_blocking=True)      # this pass's activation planes, host -> device
    for g in gemms:
        abq.gemm_exec(g["states"][mode])
    if mode == "e2e" and gemms:
        gemms[0]["e2e"]["out_host"].copy_(gemms[0]["e2e"]["out_dev"], non_blocking=True)  # this pass's results, device -> host


def capture_step(torch, abq, gemms, mode, passes):
    """One CUDA graph holding `passes` passes (36 kernels each, plus the two copies in e2e mode), so that the timed region
    measures the device and not the Python launch loop.  Returns a callable step(i)."""
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        one_pass(abq, gemms, mode)  # first launches outside capture: kernel attributes get set here
        side.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            for _ in range(passes):
                one_pass(abq, gemms, mode)
    torch.cuda.synchronize()
    return lambda i: g.replay()


def tune_in_pass(torch, abq, gemms, status, out_path):
    """The timed search with the whole pass as the yardstick.  A launch shape that wins when one GEMM is timed by itself
    (abq-llm_b200/tune.py) can lose between other GEMMs, where what counts is how it shares the SMs with its neighbours; so
    here every GEMM of the sweep in turn is re-planned a few ways (prepared-weights kernel as the heuristic shapes it, with
    sixteen warps in a CTA that fills the SM, the plane-reading kernel), the pass is timed with that one change, and the
    change is kept if the pass got faster.  Two rounds; the survivors are written as tuning-table lines."""
    names = ["ABQ_STREAM_MP", "ABQ_STREAM_CU", "ABQ_STREAM_RING", "ABQ_STREAM_WARPS", "ABQ_STREAM_FULL", "ABQ_STREAM_CTAS", "ABQ_STREAM_SLICES",
             "ABQ_STREAM_PREFILL", "ABQ_STREAM_PLANES", "ABQ_TUNE_IGNORE"]
    fields = ["mp", "cu", "ring", "warps", "full", "ctas", "slices", "prefill", "planes"]
    candidates = [dict(), dict(full=1, warps=16), dict(full=1, warps=8), dict(planes=1), dict(ctas=296), dict(cu=2), dict(cu=4), dict(cu=8),
                  dict(mp=2), dict(mp=4), dict(mp=8), dict(mp=8, cu=4), dict(mp=4, cu=4), dict(full=1, warps=16, cu=4), dict(full=1, warps=16, cu=8),
                  dict(full=1, warps=16, mp=8), dict(full=1, warps=8, cu=8),
                  # K split over CTAs small enough for two to share an SM (the only way 9..16 tokens get a neighbour on their SM)
                  dict(full=2, warps=8, slices=2, cu=2), dict(full=2, warps=8, slices=4, cu=2), dict(full=2, warps=8, slices=4, cu=1),
                  dict(full=2, warps=8, slices=8, cu=1), dict(full=1, warps=16, slices=2), dict(prefill=2), dict(prefill=4)]

    def plan(g, hints):
        saved = {n: os.environ.get(n) for n in names}
        for n in names:
            os.environ.pop(n, None)
        os.environ["ABQ_TUNE_IGNORE"] = "1"
        for k, v in hints.items():
            os.environ["ABQ_STREAM_" + k.upper()] = str(v)
        try:
            st = abq.gemm_init(_params(abq, g, g["dev_x"], g["out"], "prepared", status))
            if not hints.get("planes") and abq.state_kernel(st) != "stream_kernel":
                return None
            return st
        except abq.AbqError:
            return None
        finally:
            for n in names:
                os.environ.pop(n, None)
                if saved[n] is not None:
                    os.environ[n] = saved[n]

    def time_pass():
        step = capture_step(torch, abq, gemms, "prepared", 20)
        step(0)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(5):
            step(i)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / 100

    chosen = {}
    best = time_pass()
    print(f"in-pass search: {best:.1f} us per pass to start with", file=sys.stderr, flush=True)
    for rnd in range(2):
        for i, g in enumerate(gemms):
            if g["prepared"] is None:
                continue
            keep = g["states"]["prepared"]
            for h in candidates:
                if chosen.get(i) == h:
                    continue
                st = plan(g, h)
                if st is None:
                    continue
                g["states"]["prepared"] = st
                us = time_pass()
                if us < best * 0.997:  # more than the noise of the measurement
                    best, keep = us, st
                    chosen[i] = h
                    print(f"  round {rnd}: W{g['q']} M={g['M']} {g['N']}x{g['K']}: {h or 'heuristic'} -> {best:.1f} us per pass", file=sys.stderr, flush=True)
                else:
                    g["states"]["prepared"] = keep
            g["states"]["prepared"] = keep
    rows_class = lambda M: 1 if M == 1 else 2 if M == 2 else 4 if M <= 4 else 8 if M <= 8 else 16 if M <= 16 else 32
    lines = []
    for i, h in sorted(chosen.items()):
        g = gemms[i]
        lines.append(f"{g['q']} {XBITS} {rows_class(g['M'])} {g['N']} {g['K']} 1 {g.get('group', GROUP)} : " + " ".join(str(h.get(f, 0)) for f in fields) +
                     "   # chosen inside the sweep's pass")
    with open(out_path, "w") as f:
        f.write("\n".join(lines) + "\n")
    print(f"in-pass search: {best:.1f} us per pass, {len(lines)} lines -> {out_path} (an all-zero line means: the heuristic, whatever the table said)", file=sys.stderr)


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


def per_config_detail(torch, abq, gemms, status, peak, mode="prepared"):
    """Device time of every (WxAy, M, shape) GEMM by itself: a CUDA graph of back-to-back launches of that one GEMM, each
    on its own copy of the weights (enough copies that 260 MB of other weights pass between two reads of one buffer, so
    none is served from L2).  GB/s, fraction of the measured HBM peak and effective TOPS per config."""
    rows = []
    side = torch.cuda.Stream()
    for g in gemms:
        src = g["prepared"] if (mode == "prepared" and g["prepared"] is not None) else g["planes"]
        nbytes = src.numel() * src.element_size()
        copies = int(260e6 // nbytes) + 2
        clones = [src] + [src.clone() for _ in range(copies - 1)]
        states = []
        for c in clones:
            gg = dict(g)
            gg["prepared" if src is g["prepared"] else "planes"] = c
            states.append(abq.gemm_init(_params(abq, gg, g["dev_x"], g["out"], "prepared" if src is g["prepared"] else "planes", status)))
        with torch.cuda.stream(side):
            abq.gemm_exec(states[0])
            side.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for st in states:
                    abq.gemm_exec(st)
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 3
        e0.record()
        for _ in range(reps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (reps * copies)
        rows.append({"wxay": f"W{g['q']}A{XBITS}", "M": g["M"], "N": g["N"], "K": g["K"], "us": round(us, 3), "GBps": round(g["bytes"] / us / 1e3, 1),
                     "frac_of_hbm": round(g["bytes"] / us / 1e3 / peak, 3), "TOPS": round(g["ops"] / us / 1e6, 3)})
        del clones, states, graph
    return rows


# (w bits, x bits, M, N, K, scale group: 0 = per channel): every width pair of the prefill sweep at M = 2048 on one shape, the M
# sweep on W4A4 over two shapes, the four largest cases, and two with per-group scales + zero points
PREFILL_CASES = ([(x, x, 2048, 4096, 4096, 0) for x in (2, 3, 4, 5, 6, 7, 8)] + [(2, 4, 2048, 4096, 4096, 0), (2, 6, 2048, 4096, 4096, 0)] +
                 [(4, 4, M, N, K, 0) for M in (512, 4096) for (N, K) in ((4096, 4096), (12288, 4096))] + [(4, 4, 2048, 12288, 4096, 0)] +
                 [(4, 4, 4096, 11008, 4096, 0), (2, 8, 4096, 12288, 4096, 0), (8, 8, 4096, 4096, 11008, 0)] +
                 [(4, 8, 4096, 4096, 4096, 128), (2, 8, 2048, 11008, 4096, 128)])


def int8_library_rate(torch):
    """Dense int8 x int8 -> int32 8192^3 through the vendor library (torch._int_mm -> cuBLASLt), burst: the practical
    ceiling of the int8 tensor pipe next to the 2 x bf16 figure.  None if the call is not available."""
    try:
        n = 8192
        a = torch.randint(-128, 127, (n, n), dtype=torch.int8, device="cuda")
        b = torch.randint(-128, 127, (n, n), dtype=torch.int8, device="cuda").t()
        for _ in range(3):
            torch._int_mm(a, b)
        torch.cuda.synchronize()
        best = None
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch._int_mm(a, b)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            best = ms if best is None else min(best, ms)
        return 2.0 * n ** 3 / (best * 1e-3) / 1e12
    except Exception:  # noqa: BLE001 - a missing library kernel only removes a reported ceiling
        return None


def prefill_leg(torch, abq, reps=10):
    """Prefill shapes (M >= 512) on the tcgen05 kind::i8 route, per-channel or per-group fp16 scale: device time of the whole
    call (plane -> int8 expansion of both operands, the GEMM with its fused epilogue) per case with fp16 and with int32
    output, effective TOPS = 2*M*N*K / t, as a fraction of twice the measured dense bf16 rate (the int8 rate of the same
    pipe) and of the vendor library's int8 GEMM measured in this run; the same call with the weights expanded beforehand."""
    peak = None
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        peak = 2.0 * float(json.loads(f.read_text())["bf16_tflops"])
    lib_rate = int8_library_rate(torch)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(7)
    B = abq.binding
    rows = []

    def time_state(st):
        for _ in range(3):
            abq.gemm_exec(st)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            abq.gemm_exec(st)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / reps

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
        out32 = torch.empty((M, N), dtype=torch.int32, device="cuda")
        work = torch.empty(abq.gemm_workspace_bytes(M, N, K, p, q), dtype=torch.uint8, device="cuda")
        kw = dict(x_bits=p, w_bits=q, x_signed=bool(group), w_signed=False, workspace=work)
        kw16 = dict(kw, out_dtype=abq.OUT_FP16, scale_mode=abq.SCALE_GROUP if group else abq.SCALE_CHANNEL, group_size=group, w_scale=wsc, w_zero=wz)
        us = time_state(abq.gemm_init(B.make_params(M, N, K, xp, wp, out, **kw16)))
        us32 = None if group else time_state(abq.gemm_init(B.make_params(M, N, K, xp, wp, out32, **kw)))
        st2 = abq.gemm_init(B.make_params(M, N, K, xp, wp, out, flags=abq.FLAG_WEIGHTS_PREPARED, **kw16))
        abq.gemm_prepare_weights(st2)
        us2 = time_state(st2)
        ops = 2.0 * M * N * K
        row = {"wxay": f"W{q}A{p}", "scales": f"g{group} + zero" if group else "channel", "M": M, "N": N, "K": K, "us_fp16_out": round(us, 2),
               "TOPS": round(ops / us / 1e6, 1), "frac_of_2x_bf16": round(ops / us / 1e6 / peak, 3) if peak else None,
               "frac_of_library_int8": round(ops / us / 1e6 / lib_rate, 3) if lib_rate else None,
               "us_int32_out": None if us32 is None else round(us32, 2), "TOPS_int32_out": None if us32 is None else round(ops / us32 / 1e6, 1),
               "us_weights_prepared": round(us2, 2), "TOPS_weights_prepared": round(ops / us2 / 1e6, 1),
               "frac_weights_prepared": round(ops / us2 / 1e6 / peak, 3) if peak else None}
        rows.append(row)
        del xp, wp, out, out32, work
    return {"route": "tcgen05 kind::i8 (plane->int8 expansion included in the time)", "int8_peak_TOPS": peak,
            "peak_source": "2 x MEASURED_PEAKS.json bf16_tflops" if peak else None,
            "library_int8_TOPS": None if lib_rate is None else round(lib_rate, 1), "library_int8_source": "torch._int_mm 8192^3, best of 10, this run",
            "cases": rows}


def g64_leg(torch, abq, status, hbm_peak):
    """Scale groups of 64 (the W2A8 g64 configuration, LLaMA-2-13B shapes): decode GEMMs on prepared weights (64-feature
    units), timed like the rows of `detail`."""
    gen = torch.Generator(device="cuda")
    gen.manual_seed(64)
    q, group = 2, 64
    gemms = []
    for (M, N, K) in ((1, 5120, 5120), (1, 13824, 5120), (1, 5120, 13824), (16, 13824, 5120)):
        codes = torch.randint(0, 1 << q, (N, K), dtype=torch.int32, device="cuda", generator=gen)
        planes = torch.empty((q, N, K // 32), dtype=torch.int32, device="cuda")
        abq.pack_int32(codes, planes, N, K, q)
        x = torch.randint(-128, 128, (M, K), dtype=torch.int32, device="cuda", generator=gen)
        dev_x = torch.empty((XBITS, M, K // 32), dtype=torch.int32, device="cuda")
        abq.pack_int32(x, dev_x, M, K, XBITS)
        g = dict(q=q, M=M, N=N, K=K, group=group, planes=planes, dev_x=dev_x,
                 w_scale=(torch.rand((N, K // group), device="cuda", generator=gen) * 0.019 + 0.001).to(torch.float16),
                 w_zero=torch.randint(0, 1 << q, (N, K // group), dtype=torch.int32, device="cuda", generator=gen).to(torch.uint8),
                 work=torch.empty(max(256, abq.gemm_workspace_bytes(M, N, K, XBITS, q)), dtype=torch.uint8, device="cuda"),
                 out=torch.empty((M, N), dtype=torch.float16, device="cuda"), bytes=algorithmic_bytes(M, N, K, XBITS, q, group), ops=2 * M * N * K)
        nbytes = abq.gemm_prepared_weight_bytes(_params(abq, g, dev_x, g["out"], "planes", status))
        g["prepared"] = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
        abq.gemm_prepare_weights(abq.gemm_init(_params(abq, g, dev_x, g["out"], "prepared", status)))
        gemms.append(g)
    torch.cuda.synchronize()
    rows = per_config_detail(torch, abq, gemms, status, hbm_peak, "prepared")
    for r in rows:
        r["group_size"] = group
    return rows


def config0_leg(torch, abq, hbm_peak):
    """The reference's own CPU-checkable case (W4A4 unsigned, M=128, N=K=4096, int32 out): device time of the whole call
    on the route the planner picks, against both rooflines (it sits between the HBM-bound and the tensor-bound regime)."""
    gen = torch.Generator(device="cuda")
    gen.manual_seed(3)
    B = abq.binding
    M, N, K, p, q = 128, 4096, 4096, 4, 4

    def planes_of(rows_, bits):
        codes = torch.randint(0, 1 << bits, (rows_, K), dtype=torch.int32, device="cuda", generator=gen)
        out = torch.empty((bits, rows_, K // 32), dtype=torch.int32, device="cuda")
        abq.pack_int32(codes, out, rows_, K, bits)
        return out
    xp = planes_of(M, p)
    copies = 18  # 18 x 8.4 MB of planes between two reads of one buffer
    wps = [planes_of(N, q) for _ in range(copies)]
    out = torch.empty((M, N), dtype=torch.int32, device="cuda")
    work = torch.empty(abq.gemm_workspace_bytes(M, N, K, p, q), dtype=torch.uint8, device="cuda")
    states = [abq.gemm_init(B.make_params(M, N, K, xp, wp, out, x_bits=p, w_bits=q, x_signed=False, w_signed=False, workspace=work)) for wp in wps]
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        abq.gemm_exec(states[0])
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for st in states:
                abq.gemm_exec(st)
    torch.cuda.synchronize()
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(3):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (3 * copies)
    # the same with the weights expanded once beforehand (ABQ_FLAG_WEIGHTS_PREPARED: each plan keeps its expansion in a
    # workspace of its own; the call then expands the activations only)
    works = [torch.empty(abq.gemm_workspace_bytes(M, N, K, p, q), dtype=torch.uint8, device="cuda") for _ in wps]
    prepared = [abq.gemm_init(B.make_params(M, N, K, xp, wp, out, x_bits=p, w_bits=q, x_signed=False, w_signed=False, workspace=wk,
                                            flags=abq.FLAG_WEIGHTS_PREPARED)) for wp, wk in zip(wps, works)]
    for st in prepared:
        abq.gemm_prepare_weights(st)
    torch.cuda.synchronize()
    with torch.cuda.stream(side):
        abq.gemm_exec(prepared[0])
        side.synchronize()
        graph2 = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph2, stream=side):
            for st in prepared:
                abq.gemm_exec(st)
    torch.cuda.synchronize()
    graph2.replay()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(3):
        graph2.replay()
    e1.record()
    torch.cuda.synchronize()
    us_prepared = e0.elapsed_time(e1) * 1e3 / (3 * copies)
    nbytes = q * N * K // 8 + p * M * K // 8 + 4 * M * N
    peak = None
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        peak = 2.0 * float(json.loads(f.read_text())["bf16_tflops"])
    tops = 2.0 * M * N * K / us / 1e6
    return {"workload": "W4A4 unsigned, M=128, N=4096, K=4096, int32 out", "route": {2: "I8_MMA", 3: "I8_UMMA"}.get(states[0].route),
            "us": round(us, 2), "GBps": round(nbytes / us / 1e3, 1), "frac_of_hbm": round(nbytes / us / 1e3 / hbm_peak, 3), "TOPS": round(tops, 1),
            "frac_of_2x_bf16": round(tops / peak, 3) if peak else None, "us_weights_prepared": round(us_prepared, 2),
            "TOPS_weights_prepared": round(2.0 * M * N * K / us_prepared / 1e6, 1)}


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


WORKLOAD = ("decode sweep: W{2,3,4}A8 x M{1,4,16} x (N,K) in "
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


def tp_decode_measure(args, torch, dist, abq, rank, world):
    """`--workload tp_decode`: one decode step through the quantized linear layers of LLaMA-7B (32 blocks: fused QKV, O,
    fused gate+up, down; W4A4, per-channel scale + zero point, static activation scale), tensor parallel over the
    ranks: column-parallel QKV / gate+up, row-parallel O / down with an NCCL all-reduce after each.  Attention, norms,
    embedding and lm_head are outside the path (elementwise torch stand-ins keep the data flowing).  Strong scaling:
    the model is fixed, every rank holds 1/N of every weight."""
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
            for i, b in enumerate(blocks):  # a block writes its output where the next one reads its input
                h = b.forward(h, blocks[i + 1].input_buffer(M) if i + 1 < len(blocks) else None)
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
        n = args.tp_steps
        ms, _ = timed(torch, dist, fn, n, 3)
        kind = "none" if world == 1 else ({"auto": "fused" if M <= backend.fused_rows else "peer"}.get(backend.reduce_kind, backend.reduce_kind))
        results.append({"batch": M, "steps": n, "ms_per_step": ms / n, "tokens_per_s": M * n / (ms * 1e-3), "all_reduce": kind, "cuda_graph": "whole step" if graph is not None else ("between the all-reduces" if pieces else "no")})
    if int(backend.status.item()) != 0:
        raise SystemExit(f"tp_decode: device status word {int(backend.status.item())} (a bounded wait expired): the numbers are void")
    wbytes = layers * sum(sp.out_features * sp.in_features for sp in tp.llama_block_specs(hidden, ffn)) * q // 8
    del blocks
    return {"metric": "llama7b_w4a4_linear_stack_decode_tokens_per_s", "unit": "tokens/s", "tensor_parallel": world, "scaling": "strong",
            "workload": f"LLaMA-7B linear layers only, {layers} blocks, W4A4 per-channel + zero point, static activation scale; attention, "
                        "norms, embedding and lm_head are outside the path",
            "all_reduce": "none (one rank)" if world == 1 else (backend.reduce_kind if hasattr(backend, "reduce_kind") else
                                                                ("library peer all-reduce kernel" if backend.peer_reduce else "NCCL")),
            "weight_bytes_all_ranks": wbytes, "batches": results,
            "hbm_bound_tokens_per_s_batch1": world * measured_peaks()[0] * 1e9 / wbytes}


def reference_gpu_best():
    """The reference's "time every configuration, keep the best" on this GPU: a sample of 24 of its own decode-tile
    instantiations per width (W2A8, W3A8, W4A8; oracle/_ref/libabq_ref_gpu_sampled.so, compiled from its headers) on the four
    sweep shapes at M = 1, signed operands, int32 output, weight copies rotating so that no launch finds its planes in L2.
    A configuration counts only if its output equals this library's bit for bit; beside the best one: this library's time
    for the very same GEMM (int32 output, prepared weights)."""
    from oracle import oracle as O
    try:
        import torch
    except ImportError:
        return None
    if not (O.ref_sampled_available() and torch.cuda.is_available()):
        return None
    abq = load_package()
    B = abq.binding
    L = O.ref_sampled()
    configs = O.ref_sampled_configs()
    rng = np.random.default_rng(5)
    rows = []
    side = torch.cuda.Stream()

    def time_graph(launch, copies):
        with torch.cuda.stream(side):
            launch(0)
            side.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                for c in range(copies):
                    launch(c)
        torch.cuda.synchronize()
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / (2 * copies)

    for q in (2, 3, 4):
        for (N, K) in SHAPES:
            M, p = 1, 8
            x = rng.integers(-128, 128, size=(M, K), dtype=np.int32)
            w = rng.integers(-(1 << (q - 1)), 1 << (q - 1), size=(N, K), dtype=np.int32)
            xp = torch.from_numpy(O.pack(x, p).view(np.int32)).cuda()
            base = torch.from_numpy(O.pack(w, q).view(np.int32)).cuda()
            copies = int(260e6 // (q * N * K // 8)) + 2
            ws = [base] + [base.clone() for _ in range(copies - 1)]
            out = torch.zeros((M, N), dtype=torch.int32, device="cuda")
            ours = torch.zeros((M, N), dtype=torch.int32, device="cuda")
            work = torch.empty(max(256, abq.gemm_workspace_bytes(M, N, K, p, q)), dtype=torch.uint8, device="cuda")
            prm = B.make_params(M, N, K, xp, base, ours, x_bits=p, w_bits=q, x_signed=True, w_signed=True, route=abq.ROUTE_I8_MMA,
                                flags=abq.FLAG_PDL | abq.FLAG_WEIGHTS_PREPARED, workspace=work)
            preps = [torch.empty(abq.gemm_prepared_weight_bytes(prm), dtype=torch.uint8, device="cuda")]
            prm.w_prepared = preps[0].data_ptr()
            st0 = abq.gemm_init(prm)
            abq.gemm_prepare_weights(st0)
            torch.cuda.synchronize()
            preps += [preps[0].clone() for _ in range(copies - 1)]
            states = []
            for pr in preps:
                prm.w_prepared = pr.data_ptr()
                states.append(abq.gemm_init(prm))
            abq.gemm_exec(st0)
            torch.cuda.synchronize()
            us_ours = time_graph(lambda c: abq.gemm_exec(states[c], side), copies)
            best, passed, tried = None, 0, 0
            for (i, xb, wb, name) in configs:
                if wb != q:
                    continue
                tried += 1
                out.zero_()
                rc = L.abq_ref_sampled_gemm(i, xp.data_ptr(), base.data_ptr(), M, N, K, out.data_ptr(), 1, torch.cuda.current_stream().cuda_stream)
                torch.cuda.synchronize()
                if rc != 0 or not torch.equal(out, ours):
                    continue
                passed += 1
                us = time_graph(lambda c, i=i: L.abq_ref_sampled_gemm(i, xp.data_ptr(), ws[c].data_ptr(), M, N, K, out.data_ptr(), 1, side.cuda_stream), copies)
                if best is None or us < best[0]:
                    best = (us, name)
            rows.append({"wxay": f"W{q}A{p}", "M": M, "N": N, "K": K, "reference_best_us": None if best is None else round(best[0], 2),
                         "reference_best_config": None if best is None else best[1], "configs_tried": tried, "configs_passed": passed,
                         "this_library_us": round(us_ours, 2), "ratio": None if best is None else round(best[0] / us_ours, 2)})
            del ws, preps, states, base
    return rows


def run_tp_decode(args, rank, world, local):
    """`--workload tp_decode` by itself: the tensor-parallel linear stack as the headline of its own JSON line."""
    import torch
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local))
        dist = dist_mod
    abq = load_package()
    res = tp_decode_measure(args, torch, dist, abq, rank, world)
    if rank == 0:
        best = res["batches"][0]
        line = {"metric": res["metric"], "value": best["tokens_per_s"], "unit": "tokens/s", "n_gpus": world, "steps": best["steps"], "warmup": 3,
                "ms_per_step": best["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8",
                "data": "synthetic", "config": {"workload": res["workload"] + f"; tensor parallel {world}, batch 1 (value); batches 8 and 32 in `batches`"},
                "tp_decode": res}
        emit(line)
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
            "data": "synthetic", "config": {"workload": WORKLOAD + "; each step a bounded sample on the host cores, reference compute_ref",
                                           "sample": "one of the 36 timed GEMMs of the sweep: W2A8, M=16, N=4096, K=4096 (repeated); the other arm "
                                                     "reports its own time for this same GEMM as `reference_arm_gemm`"},
            "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    line["cpu_baseline"]["value"] = value
    gpu_rows = reference_gpu_kernels()  # context only: the arm's value stays the reference's CPU implementation
    if gpu_rows:
        line["reference_gpu_kernels"] = gpu_rows
    best_rows = reference_gpu_best()  # the reference's own search, on its own GPU kernels, on this GPU: context as well
    if best_rows:
        line["reference_gpu_best"] = best_rows
    emit(line)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--passes", type=int, default=PASSES_PER_STEP, help="passes over the 36 GEMMs per step (one CUDA graph)")
    ap.add_argument("--no-detail", action="store_true", help="skip the per-(WxAy, M, shape) timings")
    ap.add_argument("--only", default="", help="profiling aid: restrict the sweep to GEMMs 'q:M:N:K[,q:M:N:K...]' (0 = any)")
    ap.add_argument("--shape", default="", help="profiling aid: replace the sweep by the single GEMM 'q:M:N:K' (any size the route takes)")
    ap.add_argument("--weights", default="prepared", choices=["prepared", "planes"], help="profiling aid: which weight form the headline sweep reads")
    ap.add_argument("--no-prefill", action="store_true", help="skip the prefill / config0 / routes / pack legs")
    ap.add_argument("--workload", default="decode_sweep", choices=["decode_sweep", "tp_decode"],
                    help="decode_sweep (default, the headline metric) or tp_decode: tensor-parallel LLaMA-7B linear stack")
    ap.add_argument("--layers", type=int, default=32, help="tp_decode: decoder blocks")
    ap.add_argument("--tp-steps", type=int, default=40, help="tp_decode: timed decode steps per batch size")
    ap.add_argument("--no-tp", action="store_true", help="several GPUs: skip the tp_decode object")
    ap.add_argument("--tp-pieces", action="store_true", help="tp_decode on one GPU: graphs between the all-reduce points, as several ranks run it")
    ap.add_argument("--no-graph", action="store_true", help="profiling aid: launch kernel by kernel instead of one CUDA graph per step")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="profiling aid: skip the host-side reference timing")
    ap.add_argument("--tune-in-pass", default="", metavar="FILE", help="search launch shapes with the whole pass as the yardstick, write table lines to FILE, exit")
    args = ap.parse_args()
    # stdout carries the one JSON line and nothing else: whatever libraries print there meanwhile (NCCL's version banner) goes
    # to stderr; the descriptor is put back for the final print
    global REAL_STDOUT
    sys.stdout.flush()
    REAL_STDOUT = os.dup(1)
    os.dup2(2, 1)
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
    if args.tune_in_pass:
        tune_in_pass(torch, abq, gemms, status, args.tune_in_pass)
        return
    n_gemm = len(gemms)
    passes = 1 if args.no_graph else max(1, args.passes)
    bytes_per_pass = sum(g["bytes"] for g in gemms)
    ops_per_pass = sum(g["ops"] for g in gemms)
    bytes_per_step, ops_per_step = bytes_per_pass * passes, ops_per_pass * passes
    headline = args.weights
    other = "planes" if headline == "prepared" else "prepared"

    def stepper(mode):
        return capture_step(torch, abq, gemms, mode, passes) if not args.no_graph else (lambda i: one_pass(abq, gemms, mode))

    step_res, step_e2e, step_other = stepper(headline), stepper("e2e"), stepper(other)
    sampler = ClockSampler(local)
    sampler.start()
    ms, wall_ms = timed(torch, dist, step_res, args.steps, args.warmup)
    clocks = sampler.stop()
    ms_e2e, _ = timed(torch, dist, step_e2e, args.steps, args.warmup)
    ms_other, _ = timed(torch, dist, step_other, max(3, args.steps // 4), args.warmup)
    if int(status.item()) != 0:
        raise SystemExit(f"device status word {int(status.item())}: a bounded wait expired, the numbers are void")

    value = whole_job_rate(world, bytes_per_step, args.steps, ms) / 1e9
    e2e = whole_job_rate(world, bytes_per_step, args.steps, ms_e2e) / 1e9
    value_other = whole_job_rate(world, bytes_per_step, max(3, args.steps // 4), ms_other) / 1e9
    h2d = gemms[0]["e2e"]["x_host"].numel() * 4 * passes
    d2h = gemms[0]["e2e"]["out_host"].numel() * 2 * passes
    peak, peak_kind = measured_peaks()
    per_gpu = bytes_per_step * args.steps / (ms * 1e-3) / 1e9
    # which kernel each GEMM of the pass launches (the tuning table sends some shapes to the kernel that reads the planes);
    # the roofline object describes the one that takes the larger share of the launches
    kernels = [abq.state_kernel(g["states"][headline]) for g in gemms]
    counts = {k: kernels.count(k) for k in sorted(set(kernels))}
    kernel = max(counts, key=counts.get)
    ratio = DRAM_TRAFFIC_PER_ALGORITHMIC_BYTE.get(kernel)
    dom_bytes = sum(g["bytes"] for g, k in zip(gemms, kernels) if k == kernel) / counts[kernel]
    line = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8",
        "data": "synthetic",
        "config": {"workload": WORKLOAD + f"; {n_gemm} GEMMs per pass" + (f" (restricted by --only {args.only})" if args.only else ""),
                   "passes_per_step": passes, "ms_per_pass": ms / args.steps / passes,
                   "weights": ("prepared: the reference's bit-planes re-ordered once at load time by abq_gemm_prepare_weights (same bits, +64 B of "
                               "scale / zero point per 16 rows x 128 features); `planes` holds the sweep on the plane format itself")
                              if headline == "prepared" else "the reference's bit-plane format, read directly",
                   "l2": f"one copy of every weight per token count: {bytes_per_pass / 1e6:.0f} MB of other operands pass between two reads of a "
                         "buffer (> 4 x the 126 MB L2); inputs larger than L2, no flush needed",
                   "replicas": world, "pdl": os.environ.get("ABQ_BENCH_PDL", "1") == "1", "cuda_graph_per_step": not args.no_graph},
        "effective_TOPS": whole_job_rate(world, ops_per_step, args.steps, ms) / 1e12,
        "e2e": {"value": e2e, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "what": "per pass: one copy of all activation planes from pinned host memory, 36 GEMMs through the C ABI, one copy of all fp16 results back"},
        other: {"value": value_other, "unit": "GB/s", "ms_per_pass": ms_other / max(3, args.steps // 4) / passes,
                "frac_of_hbm": value_other / world / peak},
        "gpu_launches": n_gemm * passes * args.steps,  # one kernel of this library per GEMM
        "clocks": clocks,
        "roofline": {"bound": "hbm", "kernel": f"{kernel} ({counts[kernel]} of the {n_gemm} launches per pass; all: {counts})", "achieved": per_gpu, "peak": peak,
                     "unit": "GB/s", "frac": per_gpu / peak, "peak_source": f"{peak_kind} (MEASURED_PEAKS.json hbm_gbs)",
                     "bytes_per_launch": bytes_per_pass / max(1, n_gemm), "us_per_launch": ms * 1e3 / args.steps / passes / max(1, n_gemm),
                     "traffic": None if ratio is None else ratio * dom_bytes,
                     "traffic_source": f"ncu dram bytes of a sweep-sized single-shape capture of {kernel}, scaled by algorithmic bytes to its mean launch in the sweep"},
        "wall_ms_per_step": wall_ms / args.steps,
    }
    if args.shape:
        line["config"]["workload"] = f"single GEMM --shape {args.shape} (profiling aid, not the sweep)"
    extras = rank == 0 and world == 1 and not args.shape and not args.only
    if rank == 0 and not args.no_detail and world == 1:
        line["detail"] = per_config_detail(torch, abq, gemms, status, peak, headline)
        same = [r for r in line["detail"] if (r["wxay"], r["M"], r["N"], r["K"]) == ("W2A8", 16, 4096, 4096)]
        if same:  # the GEMM the reference arm samples, on this arm
            line["reference_arm_gemm"] = dict(same[0], note="the one sweep GEMM `--impl reference` times on the host cores")
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        base = cpu_baseline_sample("reference")
        line["cpu_baseline"] = {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")}
    if extras and not args.no_prefill:
        line["g64"] = g64_leg(torch, abq, status, peak)
        line["config0"] = config0_leg(torch, abq, peak)
        line["prefill"] = prefill_leg(torch, abq)
        line["routes"] = routes_leg(torch, abq)
        line["pack"] = pack_leg(torch, abq)
    if world > 1 and not args.no_tp and not args.shape and not args.only:
        del gemms, step_res, step_e2e, step_other
        torch.cuda.empty_cache()
        line["tp_decode"] = tp_decode_measure(args, torch, dist, abq, rank, world)  # every rank takes part; rank 0 reports
    if rank == 0:
        emit(line)
    if dist is not None:
        dist.destroy_process_group()


REAL_STDOUT = 1


def emit(line):
    """The JSON line, on the process's real stdout."""
    sys.stdout.flush()
    os.write(REAL_STDOUT, (json.dumps(line) + "\n").encode())


if __name__ == "__main__":
    main()
