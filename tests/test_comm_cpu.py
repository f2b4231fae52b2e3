"""Host-side logic of the data-parallel exchange, without a GPU: bucket plan, MPI-free rendezvous (including a rank 0
that never shows up), the exported symbols, and the N > 1 semantics on two gloo ranks: per-rank parameter deltas from the
CPU oracle, averaged, then the capped update, must leave every rank with identical parameters that equal the
single-process computation."""
import ctypes as C
import os
import re
import sys
import time

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_comm_library_exports_every_declared_symbol():
    from cutagi_b200 import build, comm
    if not os.path.exists(comm.LIB_PATH):
        build.build_comm()
    text = open(os.path.join(ROOT, "include", "tagi_b200_comm.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    syms = sorted(set(re.findall(r"\b(tagi_[a-z0-9_]+)\s*\(", text)))
    lib = C.CDLL(comm.LIB_PATH)
    assert not [s for s in syms if not hasattr(lib, s)]
    assert set(syms) <= set(comm._SIG) | {"tagi_comm_last_error_string"}


def test_bucket_plan():
    from cutagi_b200 import comm
    of, nb = comm.plan_buckets([10, 10, 10, 100, 5, 5], 100)   # 100-byte budget = 25 floats
    assert of == [0, 0, 1, 2, 3, 3] and nb == 4
    of, nb = comm.plan_buckets([1 << 20] * 4, 32 << 20)
    assert of == [0, 0, 0, 0] and nb == 1
    assert comm.plan_buckets([], 1024) == ([], 0)
    # ResNet-18-like: 41 tensors, last layer first; buckets never exceed the budget unless a single tensor does
    counts = [11 * 512] + [512 * 512 * 9] * 4 + [256 * 256 * 9] * 4 + [64 * 64 * 9] * 4
    of, nb = comm.plan_buckets(counts, 25 << 20)
    for b in range(nb):
        members = [c for c, o in zip(counts, of) if o == b]
        assert sum(members) * 4 <= (25 << 20) or len(members) == 1
    assert of == sorted(of)


def test_rendezvous_roundtrip_and_missing_publisher(tmp_path):
    from cutagi_b200 import comm
    from cutagi_b200.capi import TagiError
    path = str(tmp_path / "id")
    blob = bytes(range(128))
    comm.rendezvous_publish(path, blob)
    assert comm.rendezvous_fetch(path, 128, 1000) == blob
    t0 = time.time()
    with pytest.raises(TagiError) as e:
        comm.rendezvous_fetch(str(tmp_path / "never"), 128, 300)    # rank 0 never joined
    assert e.value.code == 4 and "rank 0" in str(e.value) and time.time() - t0 < 5


def test_id_rendezvous_skips_a_file_left_by_an_earlier_job(tmp_path):
    """The id file carries the world size and the time of writing: a leftover with another world size, or one older than
    the timeout, is not taken for this job's id."""
    import struct
    from cutagi_b200 import comm
    from cutagi_b200.capi import TagiError
    path = str(tmp_path / "id")
    ident = bytes(range(128))
    comm.rendezvous_publish_id(path, ident, 4)
    assert comm.rendezvous_fetch_id(path, 4, 1000) == ident
    with pytest.raises(TagiError) as e:            # same path, a job of another size
        comm.rendezvous_fetch_id(path, 2, 300)
    assert e.value.code == 4 and "no id of this job" in str(e.value)
    # a file written an hour ago: header = magic, world, pid, unix time in ms, then the id
    old = struct.pack("<8siiq", b"TAGIRDV1", 4, 1, int((time.time() - 3600) * 1000)) + bytes(128)
    comm.rendezvous_publish(path, old)
    with pytest.raises(TagiError):
        comm.rendezvous_fetch_id(path, 4, 300)
    comm.rendezvous_publish_id(path, ident, 4)     # rank 0 of this job replaces it
    assert comm.rendezvous_fetch_id(path, 4, 1000) == ident


def test_calls_without_communicator_fail_cleanly():
    from cutagi_b200 import comm
    from cutagi_b200.capi import TagiError
    with pytest.raises(TagiError) as e:
        comm._call("tagi_comm_flush", None, 1)
    assert e.value.code == 4 and "not initialised" in str(e.value)


def _ddp_worker(rank, world, port, tmpdir, q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    import torch.distributed as dist
    from cutagi_b200 import comm
    from oracle_lib import Oracle
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    o = Oracle()
    B, K, N = 6, 20, 12
    wr = np.random.default_rng(1)
    f32 = np.float32
    mw = (wr.standard_normal((N, K)) / np.sqrt(K)).astype(f32)
    vw = (wr.uniform(.5, 1.5, (N, K)) / K).astype(f32)
    mb, vb = np.zeros(N, f32), np.full(N, 1.0 / K, f32)
    # the id travels through the rendezvous file exactly as the NCCL id would
    path = os.path.join(tmpdir, "blob")
    if rank == 0:
        comm.rendezvous_publish(path, bytes([7] * 128))
    assert comm.rendezvous_fetch(path, 128, 20000) == bytes([7] * 128)
    r = np.random.default_rng(100 + rank)     # this rank's batch shard
    ma = r.standard_normal((B, K)).astype(f32)
    dm = (r.standard_normal((B, N)) * .1).astype(f32)
    dv = (-r.uniform(0, 1e-3, (B, N))).astype(f32)
    deltas = [torch.from_numpy(np.ascontiguousarray(x)) for x in o.linear_bwd_param(vw, vb, ma, dm, dv)]
    # bucket plan from the library, one allreduce per bucket (flattened), average
    of, nb = comm.plan_buckets([t.numel() for t in deltas], 1024)
    for b in range(nb):
        members = [t for t, x in zip(deltas, of) if x == b]
        flat = torch.cat([t.reshape(-1) for t in members])
        dist.all_reduce(flat)
        flat /= world
        off = 0
        for t in members:
            t.copy_(flat[off: off + t.numel()].reshape(t.shape))
            off += t.numel()
    dmw, dvw, dmb, dvb = [t.numpy() for t in deltas]
    o.param_update(B, mw, vw, dmw, dvw)
    o.param_update(B, mb, vb, dmb, dvb)
    q.put((rank, mw, vw, mb, vb))
    dist.destroy_process_group()


def test_two_gloo_ranks_average_then_update(tmp_path):
    import torch.multiprocessing as mp
    from oracle_lib import Oracle
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_ddp_worker, args=(r, 2, port, str(tmp_path), q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted([q.get(timeout=120) for _ in procs], key=lambda t: t[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for a, b in zip(res[0][1:], res[1][1:]):
        assert np.array_equal(a, b), "ranks diverged"
    # single-process expectation: average of the two shards' deltas, then the capped update
    o = Oracle()
    B, K, N = 6, 20, 12
    f32 = np.float32
    wr = np.random.default_rng(1)
    mw = (wr.standard_normal((N, K)) / np.sqrt(K)).astype(f32)
    vw = (wr.uniform(.5, 1.5, (N, K)) / K).astype(f32)
    mb, vb = np.zeros(N, f32), np.full(N, 1.0 / K, f32)
    acc = None
    for rank in range(2):
        r = np.random.default_rng(100 + rank)
        ma = r.standard_normal((B, K)).astype(f32)
        dm = (r.standard_normal((B, N)) * .1).astype(f32)
        dv = (-r.uniform(0, 1e-3, (B, N))).astype(f32)
        d = o.linear_bwd_param(vw, vb, ma, dm, dv)
        acc = [x.copy() for x in d] if acc is None else [a + x for a, x in zip(acc, d)]
    acc = [np.ascontiguousarray((a / f32(2)).astype(f32)) for a in acc]
    o.param_update(B, mw, vw, acc[0], acc[1])
    o.param_update(B, mb, vb, acc[2], acc[3])
    for got, want in zip(res[0][1:], (mw, vw, mb, vb)):
        assert np.array_equal(got, want)
