"""Whole networks on the device (cutagi_b200.nn: Conv2d, BatchNorm2d, AvgPool2d, LayerBlock, ResNetBlock, Linear, ReLU on
the C ABI) against the oracle's network trainer, which reproduces the reference's own runs bit for bit
(tests/test_net_cpu.py), and against those runs themselves (tests/golden/net_golden.npz)."""
import os

import numpy as np
import pytest
from oracle_net import OracleNet, net_golden_problems, resnet_spec

pytestmark = pytest.mark.gpu
GOLD = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "net_golden.npz"))


def _rel(a, b):
    b = np.asarray(b, np.float64)
    return float(np.abs(np.asarray(a, np.float64).reshape(b.shape) - b).max() / max(np.abs(b).max(), 1e-300))


def _device_net(spec, in_shape, cpu):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from cutagi_b200 import nn
    net = nn.build(spec, in_shape)
    net.load_state_dict(cpu.state_dict())
    return net, nn.OutputUpdater()


@pytest.mark.parametrize("name", ["resnet", "cnn"])
def test_small_networks_follow_the_reference_run(oracle, name):
    spec, in_shape, batch, steps = net_golden_problems()[name]
    cpu = OracleNet(oracle, spec, in_shape, seed=1)
    net, upd = _device_net(spec, in_shape, cpu)
    xs, var_y = GOLD[f"{name}_x"], np.full(batch * 4, 1.0, np.float32)
    for s in range(steps):
        mu, var = net(xs[s])
        rmu, rvar = cpu.forward(xs[s])
        assert np.array_equal(rmu, GOLD[f"{name}_mu"][s])          # the oracle is on the reference's own run
        tol = (2e-5, 2e-4) if s == 0 else (1e-3, 1e-3)             # parameters drift apart slowly after updates
        assert _rel(mu.cpu().numpy(), rmu) < tol[0] and _rel(var.cpu().numpy(), rvar) < tol[1], (s, _rel(mu.cpu().numpy(), rmu))
        upd.update_using_indices(net, GOLD[f"{name}_obs"][s], var_y, GOLD[f"{name}_idx"][s])
        cpu.update_using_indices(GOLD[f"{name}_obs"][s], var_y, GOLD[f"{name}_idx"][s], 4)
        net.backward()
        cpu.backward()
        net.step()
        cpu.step()
    for k, (mw, vw, mb, vb) in net.state_dict().items():
        assert _rel(mw, GOLD[f"{name}_final_{k}_mu_w"]) < 1e-3 and _rel(vw, GOLD[f"{name}_final_{k}_var_w"]) < 1e-3, k


def test_resnet18_one_step_every_delta(oracle):
    """The reference's ResNet-18 (64/128/256/512 channels, two blocks per width, projection shortcuts) on 16 x 16 inputs,
    batch 4: one training step, predictions and every parameter-delta tensor against the oracle. The convolutions of
    this network run on the tensor-core path."""
    spec = resnet_spec(final_pool=2)
    in_shape, batch = (3, 16, 16), 4
    cpu = OracleNet(oracle, spec, in_shape, seed=5)
    net, upd = _device_net(spec, in_shape, cpu)
    rng = np.random.default_rng(2)
    x = rng.standard_normal((batch, 3 * 16 * 16)).astype(np.float32)
    mu, var = net(x)
    rmu, rvar = cpu.forward(x)
    assert _rel(mu.cpu().numpy(), rmu) < 1e-4 and _rel(var.cpu().numpy(), rvar) < 1e-3
    obs = rng.standard_normal((batch, 11)).astype(np.float32)
    var_obs = np.full((batch, 11), 0.5, np.float32)
    upd.update(net, obs, var_obs)
    cpu.update(obs, var_obs)
    net.backward()
    cpu.backward()
    named, cnamed = net.named_layers(), cpu.named_layers()
    assert set(named) == set(cnamed)
    worst = 0.0
    for k, layer in named.items():
        d = cnamed[k].d
        e1, e2 = _rel(layer.delta_mu_w.cpu().numpy(), d[0]), _rel(layer.delta_var_w.cpu().numpy(), d[1])
        worst = max(worst, e1, e2)
        assert e1 < 1e-3 and e2 < 1e-3, (k, e1, e2)
    # inference mode uses the running averages
    net.eval()
    mu_e, var_e = net(x)
    emu, evar = cpu.forward(x, train=False)
    assert _rel(mu_e.cpu().numpy(), emu) < 1e-4 and _rel(var_e.cpu().numpy(), evar) < 1e-3


def test_mixture_relu_resnet_one_step(oracle):
    """The MixtureReLU variant of the small ResNet (examples/tagi_resnet_model.py uses MixtureReLU): one step against the
    oracle."""
    spec, in_shape, batch, _ = net_golden_problems()["resnet"]
    spec = [tuple(("mrelu",) if it == ("relu",) else it) if it[0] != "res" else
            ("res", [("mrelu",) if x == ("relu",) else x for x in it[1]],
             None if it[2] is None else [("mrelu",) if x == ("relu",) else x for x in it[2]]) for it in spec]
    cpu = OracleNet(oracle, spec, in_shape, seed=3)
    net, upd = _device_net(spec, in_shape, cpu)
    rng = np.random.default_rng(4)
    x = rng.standard_normal((batch, int(np.prod(in_shape)))).astype(np.float32)
    mu, var = net(x)
    rmu, rvar = cpu.forward(x)
    assert _rel(mu.cpu().numpy(), rmu) < 1e-4 and _rel(var.cpu().numpy(), rvar) < 1e-3
    obs = rng.standard_normal((batch, 11)).astype(np.float32)
    upd.update(net, obs, np.full((batch, 11), 0.5, np.float32))
    cpu.update(obs, np.full((batch, 11), 0.5, np.float32))
    net.backward()
    cpu.backward()
    for k, layer in net.named_layers().items():
        d = cpu.named_layers()[k].d
        assert _rel(layer.delta_mu_w.cpu().numpy(), d[0]) < 1e-3 and _rel(layer.delta_var_w.cpu().numpy(), d[1]) < 1e-3, k


def test_shape_errors_are_raised():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from cutagi_b200 import nn
    with pytest.raises(RuntimeError):
        nn.build([("conv", 3, 4, 3, 1, 1, 1, True), ("relu",), ("bn", 5)], (3, 8, 8))
    with pytest.raises(RuntimeError):
        nn.build([("conv", 3, 4, 3, 2, 0, 0, True)], (3, 8, 8))   # (8 - 3) not divisible by the stride
    with pytest.raises(RuntimeError):
        nn.build([("res", [("conv", 3, 4, 3, 1, 1, 1, False)], None)], (3, 8, 8))   # identity shortcut, 3 != 4 channels


def test_packed_deltas_train_the_same_bits(oracle):
    """nn.Sequential.pack_deltas() moves every parameter-delta tensor into one buffer (what the data-parallel exchange
    wants: tensors of a bucket adjacent in memory travel as one collective). Two training steps of the small ResNet with
    and without packing must leave bit-identical parameters, the packed views must be adjacent and 16-byte aligned, and
    the padding between tensors must stay zero."""
    import torch
    spec, in_shape, batch, _ = net_golden_problems()["resnet"]
    cpu = OracleNet(oracle, spec, in_shape, seed=1)
    nets = [_device_net(spec, in_shape, cpu) for _ in range(2)]
    views = nets[1][0].pack_deltas()
    for a, b in zip(views[:-1], views[1:]):
        assert a.data_ptr() + 4 * a.numel() == b.data_ptr() and a.data_ptr() % 16 == 0
    assert [t.data_ptr() for t in views] == [t.data_ptr() for l in [nets[1][0]] for t in l.delta_tensors()]
    xs, var_y = GOLD["resnet_x"], np.full(batch * 4, 1.0, np.float32)
    for s in range(2):
        for net, upd in nets:
            net(xs[s])
            upd.update_using_indices(net, GOLD["resnet_obs"][s], var_y, GOLD["resnet_idx"][s])
            net.backward()
            net.step()
    plain, packed = nets[0][0].state_dict(), nets[1][0].state_dict()
    for k in plain:
        for a, b in zip(plain[k], packed[k]):
            assert (a is None and b is None) or np.array_equal(a, b), k
    # every delta tensor of the packed network is a view of the one buffer, and what lies between them is still zero
    flat = nets[1][0]._delta_flat
    used = torch.zeros_like(flat, dtype=torch.bool)
    for o, a in nets[1][0]._delta_slots():
        t = getattr(o, a)
        off = (t.data_ptr() - flat.data_ptr()) // 4
        assert 0 <= off and off + t.numel() <= flat.numel()
        used[off:off + t.numel()] = True
    assert bool((flat[~used] == 0).all())
