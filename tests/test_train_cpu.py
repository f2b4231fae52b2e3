"""Pins the oracle's whole-step restatement (forward, output innovation, backward, capped update) on 100 training
steps of the reference itself (tests/golden/train_cfg0_golden.npz, made by tests/golden/make_train_golden.py from the
reference's CPU build): MNIST-shaped MLP 784-128-128-11, batch 32, hierarchical-softmax targets."""
import os

import numpy as np
from oracle_train import OracleMLP, cfg0_problem

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_oracle_training_reproduces_reference_bit_for_bit(oracle):
    g = np.load(os.path.join(ROOT, "tests", "golden", "train_cfg0_golden.npz"))
    params, xs, labels = cfg0_problem(0)
    assert float(xs.astype(np.float64).sum()) == g["input_checksum"][0], "numpy generator drifted"
    assert float(labels.sum()) == g["input_checksum"][1]
    net = OracleMLP(oracle, params)
    var_y = np.full(32 * 4, 1.0, np.float32)
    for s in range(100):
        mu, var = net.forward(xs[s])
        assert np.array_equal(mu, g["mu"][s]) and np.array_equal(var, g["var"][s]), f"step {s}"
        net.update_using_indices(g["obs"][s], var_y, g["idx"][s], 4)
        net.backward()
        net.step(32)
    for i, p in enumerate(net.p):
        for k in ("mu_w", "var_w", "mu_b", "var_b"):
            assert np.array_equal(p[k].reshape(-1), g[f"{k}{i}"]), (i, k)
