"""The drop-in build: cuTAGI's own `cutagi` extension module (its Sequential, state containers, activations, pooling,
output updater and bindings, compiled unchanged for sm_100a) with LinearCuda / Conv2dCuda implemented on libtagi_b200's
C ABI (integration/). The module is built where the cuTAGI sources are (make -C integration) and travels as a binary;
the test is skipped when it is absent. It drives the module exactly as the pytagi package does
(pytagi/nn/sequential.py:29-37, pytagi/nn/output_updater.py:45-81) and compares with the CPU oracle, whose training loop
is pinned on the reference's own run.
"""
import glob
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BUILD = os.path.join(ROOT, "integration", "_build")


@pytest.fixture(scope="module")
def cutagi():
    if not glob.glob(os.path.join(BUILD, "cutagi*.so")):
        pytest.skip("drop-in module not built (make -C integration needs the cuTAGI sources)")
    sys.path.insert(0, BUILD)
    import cutagi as m
    if not m.is_cuda_available():
        pytest.skip("no CUDA device")
    return m


def _rel(a, b):
    b = np.asarray(b, np.float64)
    return float(np.abs(np.asarray(a, np.float64).reshape(b.shape) - b).max() / max(np.abs(b).max(), 1e-300))


def test_mlp_training_through_cutagi_sequential(cutagi, oracle):
    """MNIST-shaped MLP, 20 steps: cuTAGI's Sequential on "cuda" (our Linear kernels inside) against the oracle."""
    from oracle_train import OracleMLP, cfg0_problem
    g = np.load(os.path.join(ROOT, "tests", "golden", "train_cfg0_golden.npz"))
    params, xs, labels = cfg0_problem(0)
    layers = [cutagi.Linear(784, 128, True), cutagi.ReLU(), cutagi.Linear(128, 128, True), cutagi.ReLU(),
              cutagi.Linear(128, 11, True)]   # kept alive: the module's Sequential does not own the Python objects
    net = cutagi.Sequential(layers)
    net.load_state_dict({f"Linear.{2 * i}": (p["mu_w"].reshape(-1).tolist(), p["var_w"].reshape(-1).tolist(),
                                            p["mu_b"].tolist(), p["var_b"].tolist()) for i, p in enumerate(params)})
    net.to_device("cuda")
    upd = cutagi.OutputUpdater(net.device)
    cpu = OracleMLP(oracle, params)
    var_y = np.full(32 * 4, 1.0, np.float32)
    for s in range(20):
        net.forward(xs[s].reshape(-1), None)
        mu, var = net.get_outputs()
        rmu, rvar = cpu.forward(xs[s])
        tol_mu, tol_var = (1e-5, 1e-4) if s == 0 else (1e-3, 1e-3)
        assert _rel(mu, rmu) < tol_mu and _rel(var, rvar) < tol_var, f"step {s}"
        assert _rel(mu, g["mu"][s]) < 1e-3, "against the reference's own CPU run"
        upd.update_using_indices(net.output_z_buffer, g["obs"][s].tolist(), var_y.tolist(), g["idx"][s].tolist(),
                                 net.input_delta_z_buffer)
        cpu.update_using_indices(g["obs"][s], var_y, g["idx"][s], 4)
        net.backward()
        cpu.backward()
        net.step()
        cpu.step(32)
    sd = net.state_dict()
    for i, p in enumerate(cpu.p):
        key = [k for k in sd if k.endswith(f".{2 * i}")][0]   # "LinearCuda.<index>" on the device
        mw, vw, mb, vb = sd[key]
        assert _rel(mw, p["mu_w"].reshape(-1)) < 1e-3 and _rel(vw, p["var_w"].reshape(-1)) < 1e-3


def test_input_size_mismatch_raises_like_the_reference(cutagi):
    """test/cpp_unit/test_mnist.cpp:496-502 asserts a std::runtime_error for a wrong input width."""
    layers = [cutagi.Linear(16, 8, True), cutagi.ReLU(), cutagi.Linear(9, 4, True)]
    net = cutagi.Sequential(layers)
    net.to_device("cuda")
    with pytest.raises(RuntimeError):
        net.forward(np.zeros(2 * 16, np.float32), None)


def test_cnn_forward_backward_through_cutagi(cutagi):
    """CIFAR-shaped CNN of the benchmark configurations at batch 8 (Conv3x3-ReLU-AvgPool2 x3, Linear 2048->256->11):
    cuTAGI's CPU classes against the drop-in CUDA build, same parameters, two training steps."""
    keep = []

    def build():
        layers = [cutagi.Conv2d(3, 32, 3, True, 1, 1, 1, 32, 32), cutagi.ReLU(), cutagi.AvgPool2d(2, 2),
                  cutagi.Conv2d(32, 64, 3, True, 1, 1, 1), cutagi.ReLU(), cutagi.AvgPool2d(2, 2),
                  cutagi.Conv2d(64, 128, 3, True, 1, 1, 1), cutagi.ReLU(), cutagi.AvgPool2d(2, 2),
                  cutagi.Linear(2048, 256, True), cutagi.ReLU(), cutagi.Linear(256, 11, True)]
        keep.append(layers)   # the module's Sequential does not own the Python objects
        return cutagi.Sequential(layers)
    cutagi.manual_seed(7)
    rng = np.random.default_rng(0)
    B = 8
    x0 = rng.random(B * 3 * 32 * 32, dtype=np.float32)
    cpu = build()
    cpu.forward(x0, None)                    # conv layers create their parameters in their first forward
    gpu = build()
    gpu.to_device("cuda")
    gpu.forward(x0, None)
    cpu_sd = cpu.state_dict()
    gpu.load_state_dict({k: cpu_sd[k.replace("Cuda", "")] for k in gpu.state_dict()})
    ucpu, ugpu = cutagi.OutputUpdater(cpu.device), cutagi.OutputUpdater(gpu.device)
    hrc = cutagi.Utils()
    for s in range(2):
        x = rng.random(B * 3 * 32 * 32, dtype=np.float32)
        labels = rng.integers(0, 10, B).astype(np.int32)
        obs, idx, _ = hrc.label_to_obs_wrapper(labels, 10)
        var_y = [1.0] * (B * 4)
        outs = []
        for net, upd in ((cpu, ucpu), (gpu, ugpu)):
            net.forward(x, None)
            outs.append(net.get_outputs())
            upd.update_using_indices(net.output_z_buffer, [float(v) for v in obs], var_y, [int(v) for v in idx],
                                     net.input_delta_z_buffer)
            net.backward()
            net.step()
        tol = (1e-5, 1e-4) if s == 0 else (1e-3, 1e-3)
        assert _rel(outs[1][0], outs[0][0]) < tol[0] * 10 and _rel(outs[1][1], outs[0][1]) < tol[1] * 10, s


def test_small_resnet_through_cutagi_sequential(cutagi, oracle):
    """The block structure of the reference's ResNet-18 at reduced size (conv stem, identity block, projection block with
    stride 2, global pooling, Linear head) trained through cuTAGI's own Sequential / LayerBlock / ResNetBlock on "cuda",
    where Linear, Conv2d, BatchNorm2d, AvgPool2d, ReLU and the capped update run on this library (integration/), against
    the CPU oracle, whose runs of this network are pinned bit for bit on the reference's CPU classes."""
    from oracle_net import OracleNet, net_golden_problems
    from test_ddp_dropin import build_net, load_oracle_parameters
    m = cutagi
    spec, in_shape, batch, _ = net_golden_problems()["resnet"]
    cpu = OracleNet(oracle, spec, in_shape, seed=1)
    keep = []
    net = build_net(m, spec, in_shape, keep)
    net.to_device("cuda")
    net.preinit_layer()
    load_oracle_parameters(net, cpu)
    upd = m.OutputUpdater(net.device)
    rng = np.random.default_rng(11)
    n_in = int(np.prod(in_shape))
    for s in range(3):
        x = rng.standard_normal((batch, n_in)).astype(np.float32)
        obs = rng.standard_normal((batch, 11)).astype(np.float32)
        var_obs = np.full((batch, 11), 0.5, np.float32)
        net.forward(x.reshape(-1), None)
        mu, var = net.get_outputs()
        rmu, rvar = cpu.forward(x)
        tol = (2e-5, 2e-4) if s == 0 else (1e-3, 1e-3)
        assert _rel(mu, rmu) < tol[0] and _rel(var, rvar) < tol[1], (s, _rel(mu, rmu), _rel(var, rvar))
        upd.update(net.output_z_buffer, obs.reshape(-1), var_obs.reshape(-1), net.input_delta_z_buffer)
        cpu.update(obs, var_obs)
        net.backward()
        cpu.backward()
        net.step()
        cpu.step()
    ref = cpu.state_dict()
    for k, v in net.state_dict().items():
        r = ref[k.replace("Cuda", "")]
        assert _rel(v[0], r["mu_w"].reshape(-1)) < 1e-3 and _rel(v[1], r["var_w"].reshape(-1)) < 1e-3, k
