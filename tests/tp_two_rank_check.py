"""Helper of test_gpu_tp_two_ranks.py, run under torch.distributed.run with two ranks (one GPU each): the block linears
with the all-reduce fused into the row-parallel GEMMs, and with the library's one-shot peer all-reduce kernel, against
the same block with torch.distributed (NCCL) all-reduces and against the unsharded block computed by the CPU oracle."""
import importlib.util
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from conftest import load_package
    abq = load_package()
    spec = importlib.util.spec_from_file_location("tp_linear_two_ranks", ROOT / "abq-llm_b200" / "tp_linear.py")
    tp = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = tp
    spec.loader.exec_module(tp)
    hidden, ffn, q = 1024, 2816, 4
    gen = torch.Generator(device="cuda")
    gen.manual_seed(5)
    weights = []
    for sp in tp.llama_block_specs(hidden, ffn):
        codes = torch.randint(0, 1 << q, (sp.out_features, sp.in_features), dtype=torch.int32, device="cuda", generator=gen)
        scale = (torch.rand((sp.out_features,), device="cuda", generator=gen) * 0.004 + 0.001).half()
        zero = torch.randint(0, 1 << q, (sp.out_features,), dtype=torch.int32, device="cuda", generator=gen).to(torch.uint8)
        weights.append((codes, scale, zero))
    outs = {}
    os.environ["ABQ_TP_FUSED_ROWS"] = "8"   # "auto" on two ranks would never pick the fused form by itself: make it mix the two
    for mode in ("fused", "peer", "nccl", "auto"):
        os.environ["ABQ_TP_REDUCE"] = mode
        be = tp.AbqBackend(abq, torch, dist, x_bits=8, x_scale=8.0, max_tokens=32)
        assert be.reduce_kind == mode and be.peer_reduce == (mode != "nccl")
        assert be.fused_rows == {"fused": 1 << 30, "auto": 8}.get(mode, 0)
        block = tp.TensorParallelBlockLinears(be, hidden, ffn, rank, world, weights, q, 0)
        for M in (1, 8, 32):
            gen.manual_seed(M)
            x = torch.randn((M, hidden), device="cuda", generator=gen).half()
            for _ in range(3):   # repeated calls: the call counters of the peer all-reduce advance
                y = block.forward(x)
            torch.cuda.synchronize()
            outs[(mode, M)] = y.clone()
        # one call site used back to back with data that changes from call to call: a rank that runs ahead must not
        # overwrite what its peer is still adding up
        gen.manual_seed(99)
        xs = [torch.randn((8, hidden), device="cuda", generator=gen).half() for _ in range(12)]
        ys = [block.forward(x).clone() for x in xs]   # no synchronisation between the calls
        torch.cuda.synchronize()
        outs[(mode, "chain")] = torch.stack(ys)
        assert int(be.status.item()) == 0
        del block, be
    keys = (1, 8, 32, "chain")
    ok = all(torch.equal(outs[("peer", M)], outs[("nccl", M)]) for M in keys)
    print(f"rank {rank} PEER_EQUALS_NCCL {ok}", flush=True)
    ok = all(torch.equal(outs[("fused", M)], outs[("nccl", M)]) for M in keys)
    print(f"rank {rank} FUSED_EQUALS_NCCL {ok}", flush=True)
    ok = all(torch.equal(outs[("auto", M)], outs[("nccl", M)]) for M in keys)
    print(f"rank {rank} AUTO_EQUALS_NCCL {ok}", flush=True)

    # ... and against the unsharded block computed by the CPU oracle (one rank, numpy stand-in for the GEMMs): what the
    # two ranks produce together is the model's result, not merely the same thing twice.  Tolerance: twice that of the
    # one-GPU test (chained GEMMs with fp16 intermediates, where one rounding difference moves a quantised code): here every
    # row-parallel output is in addition the fp16 sum of two fp16 partials.
    import numpy as np
    from test_tp_linear_gloo import NumpyBackend
    host_w = [(c.cpu().numpy(), s.cpu().numpy(), z.cpu().numpy()) for c, s, z in weights]
    whole = tp.TensorParallelBlockLinears(NumpyBackend(0, None, x_scale=8.0), hidden, ffn, 0, 1, host_w, q, 0)
    close = True
    for M in (1, 8, 32):
        gen.manual_seed(M)
        x = torch.randn((M, hidden), device="cuda", generator=gen).half()
        ref = whole.forward(x.cpu().numpy()).astype(np.float64)
        got = outs[("fused", M)].cpu().numpy().astype(np.float64)
        err = np.abs(got - ref)
        bound = 2.0 ** -5 * np.abs(ref) + 2.0 ** -6 * np.abs(ref).max()
        if rank == 0:
            print(f"M={M}: max |err| {err.max():.4g}, max |ref| {np.abs(ref).max():.4g}, worst err/bound {np.max(err / bound):.3f}", flush=True)
        close = close and bool(np.all(err <= bound))
    print(f"rank {rank} MATCHES_UNSHARDED_ORACLE {close}", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
