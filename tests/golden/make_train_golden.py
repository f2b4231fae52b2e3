"""Generates tests/golden/train_cfg0_golden.npz by training the MNIST-shaped MLP (784-128-128-11, batch 32, 100 steps,
observation variance 1, hierarchical-softmax targets) with the reference itself: its CPU-only pybind11 module
(make -C oracle refmodule) driven through the reference's own `pytagi` package.

    make -C oracle refmodule && python tests/golden/make_train_golden.py

Stored: the hierarchical-softmax observations and indices the reference derived from the labels, the predictions
(mu, var) after every step, and the final parameters. Inputs and initial parameters come from tests/oracle_train.py's
seeded generator; a checksum guards against a drift of numpy's generator.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "oracle", "_ref"))
sys.path.insert(0, os.environ.get("CUTAGI_SRC", "/root/reference"))   # the cuTAGI source tree (its pytagi package)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from oracle_train import cfg0_problem  # noqa: E402


def main():
    import pytagi  # noqa: F401
    from pytagi import Utils
    from pytagi.nn import Linear, OutputUpdater, ReLU, Sequential
    sizes, batch, steps = (784, 128, 128, 11), 32, 100
    params, xs, labels = cfg0_problem(0, sizes, batch, steps)
    net = Sequential(Linear(784, 128), ReLU(), Linear(128, 128), ReLU(), Linear(128, 11))
    net.set_threads(4)
    net.load_state_dict({f"Linear.{2 * i}": (p["mu_w"].reshape(-1).tolist(), p["var_w"].reshape(-1).tolist(),
                                            p["mu_b"].tolist(), p["var_b"].tolist()) for i, p in enumerate(params)})
    upd = OutputUpdater(net.device)
    utils = Utils()
    n_enc = 4
    var_y = np.full(batch * n_enc, 1.0, np.float32)
    out = {"obs": [], "idx": [], "mu": [], "var": []}
    for s in range(steps):
        obs, idx, _ = utils.label_to_obs(labels=labels[s], num_classes=10)
        m, v = net(xs[s].reshape(-1))
        upd.update_using_indices(output_states=net.output_z_buffer, mu_obs=obs, var_obs=var_y, selected_idx=idx,
                                 delta_states=net.input_delta_z_buffer)
        net.backward()
        net.step()
        out["obs"].append(np.asarray(obs, np.float32))
        out["idx"].append(np.asarray(idx, np.int32))
        out["mu"].append(np.asarray(m, np.float32).reshape(batch, 11))
        out["var"].append(np.asarray(v, np.float32).reshape(batch, 11))
    sd = net.state_dict()
    final = {}
    for i in range(3):
        mw, vw, mb, vb = sd[f"Linear.{2 * i}"]
        final[f"mu_w{i}"], final[f"var_w{i}"] = np.asarray(mw, np.float32), np.asarray(vw, np.float32)
        final[f"mu_b{i}"], final[f"var_b{i}"] = np.asarray(mb, np.float32), np.asarray(vb, np.float32)
    path = os.path.join(HERE, "train_cfg0_golden.npz")
    np.savez_compressed(path, obs=np.stack(out["obs"]), idx=np.stack(out["idx"]), mu=np.stack(out["mu"]),
                        var=np.stack(out["var"]), input_checksum=np.array([float(xs.astype(np.float64).sum()),
                                                                           float(labels.sum())]), **final)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
