"""Timed search over the launch shapes of the prepared-weights decode kernel, per problem; writes the table the planner loads.

The reference picks its tile configuration by timing every instantiated one on the target GPU and keeping the best per
shape (engine/test/test_mma/test_mma.h:33-46: `best_time`, `best_config`); its search space is a list of template
instantiations (engine/gen_kernel.cpp).  Here the search space is the planner's run-time parameters (token rows per column
block, units per chunk, ring depth, warps per CTA, one or two CTAs per SM, CTAs per launch), the timing is a CUDA graph of
back-to-back launches over rotating copies of the weights (none served from L2), and the winners go into
``abq_tune_table.txt`` (one line per problem; `build.py` puts it beside the shared library, where the planner finds it).
Problems without an entry keep the planner's heuristic.

    python abq-llm_b200/tune.py [--out abq-llm_b200/abq_tune_table.txt] [--problems sweep,tp] [--quick]

Needs a B200; there is no CPU path.
"""
from __future__ import annotations

import argparse
import itertools
import os
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
ENV = {"mp": "ABQ_STREAM_MP", "cu": "ABQ_STREAM_CU", "ring": "ABQ_STREAM_RING", "warps": "ABQ_STREAM_WARPS", "full": "ABQ_STREAM_FULL",
       "ctas": "ABQ_STREAM_CTAS", "slices": "ABQ_STREAM_SLICES", "prefill": "ABQ_STREAM_PREFILL", "planes": "ABQ_STREAM_PLANES"}
PLANE_ENV = {"warps": "ABQ_DECODE_WARPS", "slices": "ABQ_DECODE_SLICES", "ring": "ABQ_DECODE_RING", "cu": "ABQ_DECODE_SPLIT"}
FIELDS = ["mp", "cu", "ring", "warps", "full", "ctas", "slices", "prefill", "planes"]


def sweep_problems():
    """(w_bits, x_bits, M, N, K, group): the decode sweep (W{2,3,4}A8, M in {1, 4, 16}, LLaMA-7B shapes, g128)."""
    return [(q, 8, M, N, K, 128) for q in (2, 3, 4) for M in (1, 4, 16) for (N, K) in ((4096, 4096), (12288, 4096), (11008, 4096), (4096, 11008))]


def tp_problems():
    """The tensor-parallel LLaMA-7B linear stack (W4A4 per channel) at 1, 2, 4, 8 ranks and batch 1, 8, 32 (16 rows per launch)."""
    out = set()
    for tp in (1, 2, 4, 8):
        for M in (1, 8, 16):
            out.add((4, 4, M, 3 * 4096 // tp, 4096, 0))
            out.add((4, 4, M, 4096, 4096 // tp, 0))
            out.add((4, 4, M, 2 * 11008 // tp // 16 * 16, 4096, 0))
            out.add((4, 4, M, 4096, (11008 // 128 + tp - 1) // tp * 128, 0))
    return sorted(out)


def rows_class(M):
    return 1 if M == 1 else 2 if M == 2 else 4 if M <= 4 else 8 if M <= 8 else 16 if M <= 16 else 32


def candidates(M, group, quick, K=0):
    rc = rows_class(M)
    mps = [m for m in (1, 2, 4, 8) if m >= rc] if (group and rc <= 8) else [0]
    if quick:
        mps = mps[:2]
    # the kernel that reads the planes themselves: its heuristic shape, then warps x K slices x warps sharing a tile (in `cu`)
    yield dict(mp=0, cu=0, ring=0, warps=0, full=0, ctas=0, slices=0, prefill=0, planes=1)
    if not quick:
        for warps in (0, 8):
            for slices in (0, 2, 4):
                for split in (0, 1, 2, 4, 8, 16):
                    if (warps, slices, split) != (0, 0, 0) and split <= (warps or 16):
                        yield dict(mp=0, cu=split, ring=0, warps=warps, full=0, ctas=0, slices=slices, prefill=0, planes=1)
    for mp in mps:
        gs = 8 // mp if mp else 1
        for cu in sorted({gs, 2 * gs, 4 * gs} & set(range(1, 9))):
            for full, warps in ((0, 8), (1, 8), (1, 16)) + (((2, 8),) if rc == 16 else ()):
                for ctas in ((148, 296) if full != 1 else (148,)):
                    for slices in ((0, 2, 3, 4, 8) if rc == 16 else (0, 2, 4) if K >= 8192 else (0,)):
                        if full == 2 and slices == 0:
                            continue
                        yield dict(mp=mp, cu=cu, ring=0, warps=warps, full=full, ctas=ctas, slices=slices, prefill=0, planes=0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=str(PKG / "abq_tune_table.txt"))
    ap.add_argument("--problems", default="sweep,tp")
    ap.add_argument("--quick", action="store_true", help="fewer candidates per problem")
    ap.add_argument("--rows", type=int, default=0, help="only the problems with this many token rows")
    ap.add_argument("--min-k", type=int, default=0, help="only the problems with at least this many features")
    args = ap.parse_args()
    import torch
    if not torch.cuda.is_available():
        raise SystemExit("tune.py needs a CUDA device: there is no CPU path")
    sys.path.insert(0, str(PKG.parent))
    import importlib.util
    spec = importlib.util.spec_from_file_location("abq_llm_b200", PKG / "__init__.py", submodule_search_locations=[str(PKG)])
    abq = importlib.util.module_from_spec(spec)
    sys.modules["abq_llm_b200"] = abq
    spec.loader.exec_module(abq)
    B = abq.binding
    os.environ["ABQ_TUNE_IGNORE"] = "1"  # candidates are compared with the heuristic, not with an older table
    problems = []
    for name in args.problems.split(","):
        problems += {"sweep": sweep_problems, "tp": tp_problems}[name]()
    gen = torch.Generator(device="cuda")
    gen.manual_seed(1)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    lines = ["# w_bits x_bits rows_class N K grouped group_size : mp cu ring warps full ctas slices prefill planes   (us best, us heuristic)"]
    for (q, p, M, N, K, group) in problems:
        if (args.rows and M != args.rows) or K < args.min_k:
            continue
        codes = torch.randint(0, 1 << q, (N, K), dtype=torch.int32, device="cuda", generator=gen)
        planes = torch.empty((q, N, K // 32), dtype=torch.int32, device="cuda")
        abq.pack_int32(codes, planes, N, K, q)
        shape = (N, K // group) if group else (N,)
        ws = (torch.rand(shape, device="cuda", generator=gen) * 0.019 + 0.001).half()
        wz = torch.randint(0, 1 << q, shape, dtype=torch.int32, device="cuda", generator=gen).to(torch.uint8)
        x = torch.randint(-(1 << (p - 1)), 1 << (p - 1), (M, K), dtype=torch.int32, device="cuda", generator=gen)
        xp = torch.empty((p, M, K // 32), dtype=torch.int32, device="cuda")
        abq.pack_int32(x, xp, M, K, p)
        out = torch.empty((M, N), dtype=torch.float16, device="cuda")
        work = torch.empty(max(256, abq.gemm_workspace_bytes(M, N, K, p, q)), dtype=torch.uint8, device="cuda")

        def params(prep):
            return B.make_params(M, N, K, xp, planes, out, x_bits=p, w_bits=q, x_signed=True, w_signed=False, out_dtype=abq.OUT_FP16,
                                 scale_mode=abq.SCALE_GROUP if group else abq.SCALE_CHANNEL, group_size=group, w_scale=ws, w_zero=wz,
                                 route=abq.ROUTE_I8_MMA, flags=abq.FLAG_PDL | abq.FLAG_WEIGHTS_PREPARED, workspace=work, status_word=status, w_prepared=prep)
        nbytes = abq.gemm_prepared_weight_bytes(params(None))
        if not nbytes:
            continue
        prep = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
        abq.gemm_prepare_weights(abq.gemm_init(params(prep)))
        copies = int(260e6 // nbytes) + 2
        clones = [prep] + [prep.clone() for _ in range(copies - 1)]

        def time_plan(hints):
            names = list(ENV.values()) + list(PLANE_ENV.values())
            saved = {v: os.environ.get(v) for v in names}
            for v in names:
                os.environ.pop(v, None)
            if hints and hints.get("planes"):  # the plane-reading kernel takes its shape from its own variables
                os.environ[ENV["planes"]] = "1"
                for k, v in PLANE_ENV.items():
                    if hints.get(k):
                        os.environ[v] = str(hints[k])
            elif hints:
                for k, v in ENV.items():
                    if hints.get(k):
                        os.environ[v] = str(hints[k])
            try:
                states = [abq.gemm_init(params(c)) for c in clones]
                if hints and not hints.get("planes") and abq.state_kernel(states[0]) != "stream_kernel":
                    return None  # no launch shape with these hints: the plan fell back to the kernel that reads the planes
            except abq.AbqError:
                return None
            finally:
                for v in names:
                    os.environ.pop(v, None)
                    if saved[v] is not None:
                        os.environ[v] = saved[v]
            side = torch.cuda.Stream()
            with torch.cuda.stream(side):
                abq.gemm_exec(states[0])
                side.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    for st in states:
                        abq.gemm_exec(st)
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

        base = time_plan(None)
        best, best_h = base, None
        tried = planned = 0
        runner_up = (None, None)  # the best candidate on the prepared-weights kernel, whoever wins
        for h in candidates(M, group, args.quick, K):
            us = time_plan(h)
            tried += 1
            if us is None:
                continue
            planned += 1
            if not h["planes"] and (runner_up[0] is None or us < runner_up[0]):
                runner_up = (us, h)
            if us < best * 0.98:  # a candidate has to win by more than the noise to replace the heuristic
                best, best_h = us, h
        if int(status.item()) != 0:
            raise SystemExit(f"device status word {int(status.item())}: a bounded wait expired")
        print(f"W{q}A{p} M={M} {N}x{K} g{group}: heuristic {base:.2f} us, best {best:.2f} us {best_h}; {planned} of {tried} candidates planned, "
              f"best on prepared weights {runner_up[0] and round(runner_up[0], 2)} us {runner_up[1]}", file=sys.stderr, flush=True)
        if best_h is not None:
            lines.append(f"{q} {p} {rows_class(M)} {N} {K} {1 if group else 0} {group} : " + " ".join(str(best_h[f]) for f in FIELDS) + f"   # {best:.2f} {base:.2f}")
        del clones, prep, planes, codes
    Path(args.out).write_text("\n".join(lines) + "\n")
    print(f"{len(lines) - 1} entries -> {args.out}")


if __name__ == "__main__":
    main()
