"""Whole training steps on the GPU (forward, output innovation, backward, capped update, all through the C ABI) against
the CPU oracle, whose training loop is pinned bit-for-bit on the reference's own 100 steps (tests/test_train_cpu.py).

Tolerances. One step from identical parameters: the per-layer bar (1e-5 on means, 1e-4 on variances). After N steps
rounding differences feed back through the updates (and through ReLU's switch at zero), so the N-step comparison uses
1e-3 on the predictive means and variances and on the parameters, relative to each tensor's largest magnitude.
"""
import os

import numpy as np
import pytest
from oracle_train import OracleMLP, cfg0_problem

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _gpu_net(params):
    from cutagi_b200 import nn
    layers = []
    for i, p in enumerate(params):
        n, k = p["mu_w"].shape
        lin = nn.Linear(k, n)
        lin.load(p)
        layers.append(lin)
        if i < len(params) - 1:
            layers.append(nn.ReLU())
    return nn.Sequential(*layers)


def _rel(a, b):
    b = np.asarray(b, np.float64)
    return float(np.abs(np.asarray(a, np.float64) - b).max() / max(np.abs(b).max(), 1e-300))


def test_mnist_shaped_mlp_100_steps(oracle):
    """Configuration 0: MLP 784-128-128-11, batch 32, hierarchical-softmax targets (4 observed outputs per sample),
    observation variance 1; predictions compared after every step, parameters at the end, also against the golden
    file produced by the reference itself."""
    import gpu_util as G
    from cutagi_b200 import nn
    g = np.load(os.path.join(ROOT, "tests", "golden", "train_cfg0_golden.npz"))
    params, xs, labels = cfg0_problem(0)
    cpu = OracleMLP(oracle, params)
    gpu = _gpu_net(params)
    upd = nn.OutputUpdater()
    var_y = np.full(32 * 4, 1.0, np.float32)
    worst_mu = worst_var = 0.0
    for s in range(100):
        mu, var = gpu(xs[s])
        mu, var = mu.cpu().numpy(), var.cpu().numpy()
        rmu, rvar = cpu.forward(xs[s])
        if s == 0:
            G.check("mu step 0", mu, rmu, G.RTOL_MU)
            G.check("var step 0", var, rvar, G.RTOL_VAR)
        worst_mu, worst_var = max(worst_mu, _rel(mu, rmu)), max(worst_var, _rel(var, rvar))
        assert _rel(mu, g["mu"][s]) < 1e-3 and _rel(var, g["var"][s]) < 1e-3, f"step {s} vs the reference's own run"
        upd.update_using_indices(gpu, g["obs"][s], var_y, g["idx"][s])
        cpu.update_using_indices(g["obs"][s], var_y, g["idx"][s], 4)
        gpu.backward()
        cpu.backward()
        gpu.step()
        cpu.step(32)
    assert worst_mu < 1e-3 and worst_var < 1e-3, (worst_mu, worst_var)
    lin = [l for l in gpu.layers if isinstance(l, nn.Linear)]
    for i, (l, p) in enumerate(zip(lin, cpu.p)):
        for k in ("mu_w", "var_w", "mu_b", "var_b"):
            assert _rel(getattr(l, k).cpu().numpy().reshape(p[k].shape), p[k]) < 1e-3, (i, k)
            assert _rel(getattr(l, k).cpu().numpy().reshape(-1), g[f"{k}{i}"]) < 1e-3, (i, k, "golden")


def test_one_step_every_tensor_at_the_per_layer_bar(oracle):
    """One full step from identical parameters: every intermediate delta and every updated parameter within the
    per-layer tolerance."""
    import gpu_util as G
    from cutagi_b200 import nn
    params, xs, labels = cfg0_problem(3, sizes=(64, 256, 128, 11), batch=48, steps=1)
    rng = np.random.default_rng(9)
    y = rng.standard_normal((48, 11)).astype(np.float32)
    var_y = np.full((48, 11), 0.25, np.float32)
    cpu, gpu, upd = OracleMLP(oracle, params), _gpu_net(params), nn.OutputUpdater()
    mu, var = gpu(xs[0])
    rmu, rvar = cpu.forward(xs[0])
    G.check("mu", mu.cpu().numpy(), rmu, G.RTOL_MU)
    G.check("var", var.cpu().numpy(), rvar, G.RTOL_VAR)
    upd.update(gpu, y, var_y)
    cpu.update(y, var_y)
    G.check("out dmu", gpu.delta[0].cpu().numpy(), cpu.delta[0], G.RTOL_MU)
    G.check("out dvar", gpu.delta[1].cpu().numpy(), cpu.delta[1], G.RTOL_VAR)
    gpu.backward()
    cpu.backward()
    lin = [l for l in gpu.layers if isinstance(l, nn.Linear)]
    for i, (l, d) in enumerate(zip(lin, cpu.dparams)):
        G.check(f"dmu_w{i}", l.delta_mu_w.cpu().numpy(), d[0], G.RTOL_MU)
        G.check(f"dvar_w{i}", l.delta_var_w.cpu().numpy(), d[1], G.RTOL_VAR)
        G.check(f"dmu_b{i}", l.delta_mu_b.cpu().numpy(), d[2], G.RTOL_MU)
        G.check(f"dvar_b{i}", l.delta_var_b.cpu().numpy(), d[3], G.RTOL_VAR)
    gpu.step()
    cpu.step(48)
    for i, (l, p) in enumerate(zip(lin, cpu.p)):
        G.check(f"mu_w{i}", l.mu_w.cpu().numpy(), p["mu_w"], G.RTOL_MU)
        G.check(f"var_w{i}", l.var_w.cpu().numpy(), p["var_w"], G.RTOL_VAR)


def test_deep_regression_mlp_steps(oracle):
    """Configuration 2 at reduced width (1 -> 512 -> 512 -> 512 -> 1, batch 256: the full 4096-wide network costs the CPU
    oracle minutes per step): x ~ U[-5, 5], y = x^3 + eps, eps ~ N(0, 9), observation variance 9; the hidden layers run
    on the tensor-core kernels, the 1-wide layers on the FFMA kernels."""
    from cutagi_b200 import nn
    params, _, _ = cfg0_problem(5, sizes=(1, 512, 512, 512, 1), batch=256, steps=1)
    rng = np.random.default_rng(6)
    cpu, gpu, upd = OracleMLP(oracle, params), _gpu_net(params), nn.OutputUpdater()
    var_y = np.full((256, 1), 9.0, np.float32)
    for s in range(5):
        x = rng.uniform(-5, 5, (256, 1)).astype(np.float32)
        y = (x ** 3 + rng.standard_normal((256, 1)) * 3).astype(np.float32)
        mu, var = gpu(x)
        rmu, rvar = cpu.forward(x)
        assert _rel(mu.cpu().numpy(), rmu) < 1e-3 and _rel(var.cpu().numpy(), rvar) < 1e-3, s
        upd.update(gpu, y, var_y)
        cpu.update(y, var_y)
        gpu.backward()
        cpu.backward()
        gpu.step()
        cpu.step(256)
    from cutagi_b200 import capi
    assert capi.tc_status() == 0
