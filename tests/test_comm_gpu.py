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


def _train_worker(rank, world, path, q):
    """Two training steps of the small ResNet, each rank on its own batch, parameter deltas averaged through the exchange
    (launched from the layers' backward hooks), then the capped update."""
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import numpy as np
    import torch
    from cutagi_b200 import nn
    from cutagi_b200.comm import DeltaExchange
    from oracle_net import OracleNet, net_golden_problems
    torch.cuda.set_device(rank)
    spec, in_shape, batch, _ = net_golden_problems()["resnet"]
    net = nn.build(spec, in_shape)
    net.load_state_dict(OracleNet(None, spec, in_shape, seed=1).state_dict())   # identical replicas, the oracle's parameters
    upd = nn.OutputUpdater()
    deltas = net.pack_deltas()   # one buffer: the tensors of a bucket are merged into one collective
    ex = DeltaExchange(deltas, rank, world, rank, path, bucket_bytes=4 << 10, average=True, timeout_ms=60000)
    assert ex.num_collectives < len(deltas), (ex.num_collectives, len(deltas))
    sp = torch.cuda.current_stream().cuda_stream
    pos = {t.data_ptr(): i for i, t in enumerate(deltas)}
    for layer in net.named_layers().values():
        ids = [pos[t.data_ptr()] for t in layer.delta_tensors()]
        layer.on_ready = (lambda ids=ids: [ex.ready(i, sp) for i in ids])
    rng = np.random.default_rng(50 + rank)
    for step in range(2):
        x = rng.standard_normal((batch, int(np.prod(in_shape)))).astype(np.float32)
        obs = rng.standard_normal((batch, 11)).astype(np.float32)
        net(x)
        upd.update(net, obs, np.full((batch, 11), 0.5, np.float32))
        net.backward()
        ex.flush(sp)
        ex.wait(sp)
        net.step()
    torch.cuda.synchronize()
    ex.check()
    nb = ex.num_buckets
    ex.close()
    q.put((rank, nb, {k: (v[0], v[1]) for k, v in net.state_dict().items()}))


def test_data_parallel_training_matches_averaged_oracles(tmp_path, oracle):
    """The reference's data-parallel semantics (src/ddp.cpp:113-146: average the parameter deltas of all ranks, then every
    rank applies the capped update): two GPU ranks against two CPU oracles whose deltas are averaged on the host. The
    ranks must end bit-identical to each other."""
    import numpy as np
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    from oracle_net import OracleNet, net_golden_problems
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    path = str(tmp_path / "nccl_id_train")
    procs = [ctx.Process(target=_train_worker, args=(r, 2, path, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted((q.get(timeout=300) for _ in procs), key=lambda r: r[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert res[0][1] >= 2, "the deltas should span several buckets"
    spec, in_shape, batch, _ = net_golden_problems()["resnet"]
    cpus = [OracleNet(oracle, spec, in_shape, seed=1) for _ in range(2)]
    init = {k: {n: None if v is None else v.copy() for n, v in p.items()} for k, p in cpus[0].state_dict().items()}
    rngs = [np.random.default_rng(50 + r) for r in range(2)]
    for step in range(2):
        for net, rng in zip(cpus, rngs):
            x = rng.standard_normal((batch, int(np.prod(in_shape)))).astype(np.float32)
            obs = rng.standard_normal((batch, 11)).astype(np.float32)
            net.forward(x)
            net.update(obs, np.full((batch, 11), 0.5, np.float32))
            net.backward()
        la, lb = cpus[0].named_layers(), cpus[1].named_layers()
        for k in la:
            avg = tuple(None if a is None else ((a + b) * np.float32(0.5)).astype(np.float32) for a, b in zip(la[k].d, lb[k].d))
            la[k].d = lb[k].d = avg
        for net in cpus:
            net.step()
    ref = cpus[0].state_dict()
    worst = {}
    for k, (mw, vw) in res[0][2].items():
        assert np.array_equal(mw, res[1][2][k][0]) and np.array_equal(vw, res[1][2][k][1]), f"ranks differ in {k}"
        e_mu = np.abs(mw.reshape(ref[k]["mu_w"].shape) - ref[k]["mu_w"]).max() / np.abs(ref[k]["mu_w"]).max()
        e_var = np.abs(vw.reshape(ref[k]["var_w"].shape) - ref[k]["var_w"]).max() / np.abs(ref[k]["var_w"]).max()
        worst[k] = (float(e_mu), float(e_var))
        assert np.abs(ref[k]["mu_w"] - init[k]["mu_w"]).max() > 0, f"{k} was not updated"
    bad = {k: v for k, v in worst.items() if v[0] > 2e-3 or v[1] > 2e-3}
    assert not bad, bad
