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


def test_label_to_obs_matches_the_reference():
    """Hierarchical-softmax encoding of the device-side mirror (cutagi_b200.nn.Utils, host-only code) against the
    observations and indices the reference derived from the same labels (tests/golden/train_cfg0_golden.npz)."""
    import importlib.util
    import os
    import sys
    import types
    from oracle_train import cfg0_problem
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    g = np.load(os.path.join(root, "tests", "golden", "train_cfg0_golden.npz"))
    _, _, labels = cfg0_problem(0)
    # the package imports the CUDA library on import; the encoder itself is plain numpy, so load the class alone
    src = open(os.path.join(root, "cutagi_b200", "nn.py")).read()
    body = "import math\nimport numpy as np\n" + src[src.index("class Utils:"):]
    mod = types.ModuleType("nn_utils_only")
    exec(compile(body, "nn_utils_only", "exec"), mod.__dict__)
    u = mod.Utils()
    for s in range(labels.shape[0]):
        obs, idx, n = u.label_to_obs(labels[s], 10)
        assert n == 4 and np.array_equal(obs, g["obs"][s]) and np.array_equal(idx, g["idx"][s])
