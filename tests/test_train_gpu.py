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


def test_deep_regression_mlp_full_width_one_step_sampled(oracle):
    """Configuration 2 at its full size (1 -> 4096 -> 4096 -> 4096 -> 1, batch 2048), one training step. The CPU oracle
    needs minutes for one such step, so every layer is checked on a sample, given the GPU's own inputs of that layer:
    forward and state pass on six batch rows (they depend on that row only), parameter deltas and the capped update on
    six output features (they depend on that feature's delta column only)."""
    import torch
    import gpu_util as G
    from cutagi_b200 import capi, nn
    sizes, B = (1, 4096, 4096, 4096, 1), 2048
    params, _, _ = cfg0_problem(7, sizes=sizes, batch=B, steps=1)
    rng = np.random.default_rng(8)
    x = rng.uniform(-5, 5, (B, 1)).astype(np.float32)
    y = (x ** 3 + rng.standard_normal((B, 1)) * 3).astype(np.float32)
    rows = np.sort(rng.choice(B, 6, replace=False))
    h = lambda t: t.detach().cpu().numpy()
    lin = []
    for p in params:
        n, k = p["mu_w"].shape
        layer = nn.Linear(k, n)
        layer.load(p)
        lin.append(layer)
    capi.tc_status()
    # forward, layer by layer, keeping every layer's input
    mu, var, jcb = torch.from_numpy(x).cuda(), torch.zeros(B, 1, device="cuda"), None
    inputs = []
    for i, (layer, p) in enumerate(zip(lin, params)):
        inputs.append((mu, var, jcb))
        last = i == len(lin) - 1
        out = layer.forward(mu, var, jcb, act=0 if last else capi.ACT_RELU)
        rmu, rvar = oracle.linear_fwd(p["mu_w"], p["var_w"], p["mu_b"], p["var_b"],
                                      np.ascontiguousarray(h(mu)[rows]), np.ascontiguousarray(h(var)[rows]))
        if not last:
            rmu, rvar, rj = G.relu_of(rmu, rvar)
            assert np.array_equal(h(out[2])[rows], rj), f"layer {i}: ReLU Jacobian"
        G.check(f"layer {i} mu", h(out[0])[rows], rmu, G.RTOL_MU)
        G.check(f"layer {i} var", h(out[1])[rows], rvar, G.RTOL_VAR)
        mu, var, jcb = out
    # output innovation (observation variance 9), then backward layer by layer
    rd = oracle.output_delta(h(mu), h(var), np.ones((B, 1), np.float32), y, np.full((B, 1), 9.0, np.float32))
    dmu, dvar = torch.from_numpy(rd[0]).cuda(), torch.from_numpy(rd[1]).cuda()
    for i in reversed(range(len(lin))):
        layer, p = lin[i], params[i]
        mu_a, _, j = inputs[i]
        N = sizes[i + 1]
        feats = np.sort(rng.choice(N, min(6, N), replace=False))
        nxt = layer.backward(dmu, dvar, state_update=i > 0)
        col = lambda t: np.ascontiguousarray(h(t)[:, feats])
        r = oracle.linear_bwd_param(np.ascontiguousarray(p["var_w"][feats]), np.ascontiguousarray(p["var_b"][feats]),
                                    h(mu_a), col(dmu), col(dvar))
        got = [h(layer.delta_mu_w)[feats], h(layer.delta_var_w)[feats], h(layer.delta_mu_b)[feats],
               h(layer.delta_var_b)[feats]]
        for name, a, b, tol in zip(("dmu_w", "dvar_w", "dmu_b", "dvar_b"), got, r, (1e-5, 1e-4, 1e-5, 1e-4)):
            G.check(f"layer {i} {name}", a, b, tol)
        if i > 0:
            rs = oracle.linear_bwd_state(p["mu_w"], np.ascontiguousarray(h(j)[rows]), np.ascontiguousarray(h(dmu)[rows]),
                                         np.ascontiguousarray(h(dvar)[rows]))
            G.check(f"layer {i} dmu_a", h(nxt[0])[rows], rs[0], G.RTOL_MU)
            G.check(f"layer {i} dvar_a", h(nxt[1])[rows], rs[1], G.RTOL_VAR)
            dmu, dvar = nxt
        # capped update of the sampled features, from the GPU's own deltas
        mw, vw = np.ascontiguousarray(p["mu_w"][feats]), np.ascontiguousarray(p["var_w"][feats])
        oracle.param_update(B, mw, vw, np.ascontiguousarray(got[0]), np.ascontiguousarray(got[1]))
        layer.step(B)
        G.check(f"layer {i} mu_w after step", h(layer.mu_w)[feats], mw, G.RTOL_MU)
        G.check(f"layer {i} var_w after step", h(layer.var_w)[feats], vw, G.RTOL_VAR)
    assert capi.tc_status() == 0


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
