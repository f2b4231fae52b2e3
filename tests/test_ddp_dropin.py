"""cuTAGI's own data-parallel classes (cutagi.DDPConfig / cutagi.DDPSequential, include/ddp.h:84-145 of the cuTAGI tree)
implemented on this repository's exchange library (integration/ddp_b200.cpp in place of src/ddp.cpp).

* CPU: the order in which the shim enumerates parameterised layers through LayerBlock / ResNetBlock containers (the
  generic walk of integration/ddp_b200_walk.h, compiled here against a mock tree) is the order of the backward pass.
* One GPU: a DDPSequential with a single rank registers every parameter-delta tensor of the small ResNet, those inside
  the residual blocks included, and trains bit-identically to the plain Sequential.
* Two GPUs (skipped with fewer): two ranks train the small ResNet through cutagi.DDPSequential, each on its own batch;
  they end bit-identical and follow two CPU oracles whose parameter deltas are averaged on the host (src/ddp.cpp:113-146
  semantics, with the nested layers that the original skips).
The drop-in module is built where the cuTAGI sources are (make -C integration) and travels as a binary; the GPU tests are
skipped when it is absent.
"""
import glob
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BUILD = os.path.join(ROOT, "integration", "_build")

WALK_CHECK = r'''
#include <cstdio>
#include <string>
#include <vector>
#include "ddp_b200_walk.h"
// mock tree: kind 0 leaf, 1 sequence, 2 residual block (children: main block, shortcut)
struct Node { int kind; std::string name; std::vector<Node*> kids; };
int main() {
    std::vector<Node> pool; pool.reserve(64);
    auto leaf = [&](const char *n) { pool.push_back({0, n, {}}); return &pool.back(); };
    auto seq = [&](std::vector<Node*> k) { pool.push_back({1, "", k}); return &pool.back(); };
    auto res = [&](Node *m, Node *s) { pool.push_back({2, "", s ? std::vector<Node*>{m, s} : std::vector<Node*>{m}}); return &pool.back(); };
    // stem, identity block, projection block, head
    std::vector<Node*> top = {leaf("conv0"), leaf("bn0"),
        res(seq({leaf("b1.conv1"), leaf("b1.bn1"), leaf("b1.conv2"), leaf("b1.bn2")}), nullptr),
        res(seq({leaf("b2.conv1"), leaf("b2.bn1"), leaf("b2.conv2"), leaf("b2.bn2")}), seq({leaf("b2.sc.conv"), leaf("b2.sc.bn")})),
        leaf("fc")};
    ddp_b200_walk_backward(top, [](Node *n, std::vector<Node*> &out) { out = n->kids; return n->kind; },
                           [](Node *n) { std::printf("%s\n", n->name.c_str()); });
    return 0;
}
'''


def test_walk_visits_leaves_in_backward_order(tmp_path):
    src = tmp_path / "walk_check.cpp"
    src.write_text(WALK_CHECK)
    exe = tmp_path / "walk_check"
    subprocess.run(["g++", "-std=c++14", "-O1", "-I", os.path.join(ROOT, "integration"), str(src), "-o", str(exe)], check=True)
    got = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()
    assert got == ["fc",
                   "b2.bn2", "b2.conv2", "b2.bn1", "b2.conv1", "b2.sc.bn", "b2.sc.conv",     # main block, then shortcut
                   "b1.bn2", "b1.conv2", "b1.bn1", "b1.conv1",
                   "bn0", "conv0"]


@pytest.fixture(scope="module")
def cutagi():
    import torch   # first: a process has room for one NCCL, and the exchange library binds to the resident one
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    if not glob.glob(os.path.join(BUILD, "cutagi*.so")):
        pytest.skip("drop-in module not built (make -C integration needs the cuTAGI sources)")
    sys.path.insert(0, BUILD)
    import cutagi as m
    return m


def build_net(m, spec, in_shape, keep):
    """The spec of tests/oracle_net.py as cuTAGI layers (as tests/golden/make_net_golden.py builds it through pytagi)."""
    def layers(spec, first=False):
        out = []
        for item in spec:
            kind, a = item[0], item[1:]
            if kind == "conv":
                fi, fo, k, stride, pad, pad_type, bias = a
                wh = (in_shape[2], in_shape[1]) if first and not out else (0, 0)
                out.append(m.Conv2d(fi, fo, k, bias, stride, pad, pad_type, wh[0], wh[1]))
            elif kind == "linear":
                out.append(m.Linear(a[0], a[1], a[2]))
            elif kind == "relu":
                out.append(m.ReLU())
            elif kind == "bn":
                out.append(m.BatchNorm2d(a[0]))
            elif kind == "pool":
                out.append(m.AvgPool2d(a[0], a[1], a[2], a[3]))
            elif kind == "res":
                main = m.LayerBlock(layers(a[0]))
                if a[1]:
                    sc = m.LayerBlock(layers(a[1]))
                    keep.append(sc)
                    out.append(m.ResNetBlock(main, sc))
                else:
                    out.append(m.ResNetBlock(main))
                keep.append(main)
        keep.append(out)   # the module's containers do not own the Python objects
        return out
    return m.Sequential(layers(spec, first=True))


def load_oracle_parameters(net, cpu_net):
    """The oracle's seeded parameters into a cuTAGI network on the device (layer names carry a Cuda suffix there)."""
    sd = {k: (p["mu_w"].reshape(-1).tolist(), p["var_w"].reshape(-1).tolist(),
              [] if p["mu_b"] is None else p["mu_b"].tolist(), [] if p["var_b"] is None else p["var_b"].tolist())
          for k, p in cpu_net.state_dict().items()}
    keys = list(net.state_dict())
    assert {k.replace("Cuda", "") for k in keys} == set(sd), (sorted(keys), sorted(sd))
    net.load_state_dict({k: sd[k.replace("Cuda", "")] for k in keys})


def _train(m, model, stepper, xs, obs, batch, device):
    """stepper: the object whose forward / backward / step are called (a Sequential or a DDPSequential)."""
    upd = m.OutputUpdater(device)
    outs = []
    for x, o in zip(xs, obs):
        stepper.forward(x.reshape(-1), None)
        outs.append([np.asarray(v, np.float32) for v in stepper.get_outputs()])
        upd.update(model.output_z_buffer, o.reshape(-1), np.full(o.size, 0.5, np.float32), model.input_delta_z_buffer)
        stepper.backward()
        stepper.step()
    return outs


@pytest.mark.gpu
def test_single_rank_ddp_registers_nested_layers_and_trains_like_sequential(cutagi, tmp_path, monkeypatch):
    from cutagi_b200 import comm
    from oracle_net import OracleNet, net_golden_problems
    m = cutagi
    spec, in_shape, batch, _ = net_golden_problems()["resnet"]
    cpu_net = OracleNet(None, spec, in_shape, seed=1)
    rng = np.random.default_rng(3)
    n_in = int(np.prod(in_shape))
    xs = [rng.standard_normal((batch, n_in)).astype(np.float32) for _ in range(2)]
    obs = [rng.standard_normal((batch, 11)).astype(np.float32) for _ in range(2)]
    keep = []
    # plain Sequential
    plain = build_net(m, spec, in_shape, keep)
    plain.to_device("cuda:0")
    plain.preinit_layer()
    load_oracle_parameters(plain, cpu_net)
    ref_out = _train(m, plain, plain, xs, obs, batch, "cuda:0")
    ref_sd = plain.state_dict()
    # the same through DDPSequential with one rank
    monkeypatch.setenv("TAGI_B200_RENDEZVOUS", str(tmp_path / "id"))
    monkeypatch.setenv("TAGI_B200_BUCKET_MB", "1")
    model = build_net(m, spec, in_shape, keep)
    ddp = m.DDPSequential(model, m.DDPConfig([0], "nccl", 0, 1), True)
    load_oracle_parameters(model, cpu_net)
    n_tensors = sum(2 + 2 * (p["mu_b"] is not None) for p in cpu_net.state_dict().values())
    assert comm.load().tagi_comm_num_tensors() == n_tensors, "every parameter-delta tensor, nested layers included"
    out = _train(m, model, ddp, xs, obs, batch, ddp.get_device_with_index())
    ddp.barrier()
    for a, b in zip(out, ref_out):
        assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])
    sd = model.state_dict()
    for k in ref_sd:
        for u, v in zip(sd[k], ref_sd[k]):
            assert np.array_equal(np.asarray(u), np.asarray(v)), k
    del ddp


def _rank_worker(rank, world, path, q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    sys.path.insert(0, BUILD)
    os.environ["TAGI_B200_RENDEZVOUS"] = path
    os.environ["TAGI_B200_BUCKET_MB"] = "1"
    import torch  # noqa: F401  (its NCCL first)
    import cutagi as m
    from oracle_net import OracleNet, net_golden_problems
    from test_ddp_dropin import _train, build_net, load_oracle_parameters
    spec, in_shape, batch, _ = net_golden_problems()["resnet"]
    keep = []
    model = build_net(m, spec, in_shape, keep)
    ddp = m.DDPSequential(model, m.DDPConfig(list(range(world)), "nccl", rank, world), True)
    if rank == 0:   # the broadcast in the constructor has made every rank a copy of rank 0; now the oracle's parameters
        pass
    load_oracle_parameters(model, OracleNet(None, spec, in_shape, seed=1))
    rng = np.random.default_rng(50 + rank)
    n_in = int(np.prod(in_shape))
    xs, obs = [], []
    for _ in range(2):
        xs.append(rng.standard_normal((batch, n_in)).astype(np.float32))
        obs.append(rng.standard_normal((batch, 11)).astype(np.float32))
    _train(m, model, ddp, xs, obs, batch, ddp.get_device_with_index())
    ddp.barrier()
    sd = {k.replace("Cuda", ""): (np.asarray(v[0], np.float32), np.asarray(v[1], np.float32))
          for k, v in model.state_dict().items()}
    q.put((rank, sd))


@pytest.mark.gpu
def test_two_ranks_through_cutagi_ddpsequential(cutagi, tmp_path, oracle):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    from oracle_net import OracleNet, net_golden_problems
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank_worker, args=(r, 2, str(tmp_path / "id2"), q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted((q.get(timeout=300) for _ in procs), key=lambda r: r[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    spec, in_shape, batch, _ = net_golden_problems()["resnet"]
    cpus = [OracleNet(oracle, spec, in_shape, seed=1) for _ in range(2)]
    rngs = [np.random.default_rng(50 + r) for r in range(2)]
    n_in = int(np.prod(in_shape))
    for step in range(2):
        for net, rng in zip(cpus, rngs):
            x = rng.standard_normal((batch, n_in)).astype(np.float32)
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
    assert set(res[0][1]) == set(ref)
    for k, (mw, vw) in res[0][1].items():
        assert np.array_equal(mw, res[1][1][k][0]) and np.array_equal(vw, res[1][1][k][1]), f"ranks differ in {k}"
        e_mu = np.abs(mw.reshape(ref[k]["mu_w"].shape) - ref[k]["mu_w"]).max() / np.abs(ref[k]["mu_w"]).max()
        e_var = np.abs(vw.reshape(ref[k]["var_w"].shape) - ref[k]["var_w"]).max() / np.abs(ref[k]["var_w"]).max()
        assert e_mu < 2e-3 and e_var < 2e-3, (k, e_mu, e_var)
