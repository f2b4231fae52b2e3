"""Data-parallel exchange on real GPUs (needs at least two): the pattern of the reference's own distributed test
(test/cpp_unit/test_ddp_ops.cpp:64-218): every rank fills its delta tensors with rank + 1, exchanges, and expects the
mean or the sum; then a broadcast from rank 0. Ranks are child processes, one per GPU, joined through the rendezvous
file."""
import os
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, path, q):
    sys.path.insert(0, ROOT)
    import torch
    from cutagi_b200.comm import DeltaExchange
    torch.cuda.set_device(rank)
    sizes = [1000, 300000, 7, 4096 * 64, 11]
    ts = [torch.full((n,), float(rank + 1), device="cuda") for n in sizes]
    ex = DeltaExchange(ts, rank, world, rank, path, bucket_bytes=1 << 20, average=True, timeout_ms=60000)
    sp = torch.cuda.current_stream().cuda_stream
    ok = ex.num_buckets >= 2
    for step in range(3):                       # buckets re-arm after every wait
        for t in ts:
            t.fill_(float(rank + 1) * (step + 1))
        for i in reversed(range(len(ts))):      # any order of readiness works
            ex.ready(i, sp)
        ex.wait(sp)
        torch.cuda.synchronize()
        want = (step + 1) * (world + 1) / 2.0
        ok = ok and all(bool(torch.all(t == want)) for t in ts)
    b = torch.full((1234,), float(rank), device="cuda")
    ex.broadcast(b, 0, sp)
    torch.cuda.synchronize()
    ok = ok and bool(torch.all(b == 0.0))
    ex.check()
    ex.close()
    q.put((rank, ok))


def test_exchange_mean_and_broadcast(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    path = str(tmp_path / "nccl_id")
    procs = [ctx.Process(target=_worker, args=(r, 2, path, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok for _, ok in res)
