"""abq_peer_allreduce_half on one GPU: with a single rank the sum is the rank's own buffer; the call counter advances,
so that the same launch can be repeated (as a CUDA graph replay does).  Several ranks need several GPUs: that path is
exercised by `bench.py --workload tp_decode --gpus N`."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_single_rank_sum_is_the_buffer_and_the_counter_advances(abq, cuda):
    n = 8 * 1024 * 5 + 64   # several blocks, a ragged last one
    buf = torch.randn(n, device="cuda").to(torch.float16)
    pad = torch.zeros(64, dtype=torch.int32, device="cuda")
    bufs = torch.tensor([buf.data_ptr()], dtype=torch.int64, device="cuda")
    pads = torch.tensor([pad.data_ptr()], dtype=torch.int64, device="cuda")
    out = torch.zeros(n, dtype=torch.float16, device="cuda")
    counter = torch.zeros(2, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for call in range(1, 4):
        out.zero_()
        abq.peer_allreduce_half(bufs.data_ptr(), pads.data_ptr(), 0, 1, 8, out, n, counter, status)
        torch.cuda.synchronize()
        assert torch.equal(out, buf)
        assert counter.tolist() == [call, 0] and int(status.item()) == 0


def test_rejects_bad_arguments(abq, cuda):
    t = torch.zeros(16, dtype=torch.float16, device="cuda")
    p = torch.zeros(1, dtype=torch.int64, device="cuda")
    c = torch.zeros(2, dtype=torch.int32, device="cuda")
    with pytest.raises(abq.AbqError):
        abq.peer_allreduce_half(p.data_ptr(), p.data_ptr(), 0, 1, 0, t, 12, c)      # not a multiple of 8 values
    with pytest.raises(abq.AbqError):
        abq.peer_allreduce_half(p.data_ptr(), p.data_ptr(), 1, 1, 0, t, 16, c)      # rank outside the world
