"""The oracle's network trainer (tests/oracle_net.py: Conv2d, BatchNorm2d, AvgPool2d, LayerBlock, ResNetBlock, Linear,
ReLU composed like the reference's containers) against the reference's own training runs of a small ResNet and a small
CNN (tests/golden/net_golden.npz, produced by the reference's CPU module through pytagi). Every op of the oracle is
bit-identical to the reference's, and so is the composition: predictions of every step and the final parameters match
exactly."""
import os

import numpy as np
import pytest
from oracle_net import OracleNet, net_golden_problems

GOLD = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "net_golden.npz"))


@pytest.mark.parametrize("name", ["resnet", "cnn"])
def test_oracle_net_reproduces_the_reference_run(oracle, name):
    spec, in_shape, batch, steps = net_golden_problems()[name]
    net = OracleNet(oracle, spec, in_shape, seed=1)
    checksum = float(sum(np.abs(p["mu_w"]).astype(np.float64).sum() for p in net.state_dict().values()))
    assert checksum == float(GOLD[f"{name}_checksum"][0]), "numpy generator drift: regenerate the fixture"
    xs, var_y = GOLD[f"{name}_x"], np.full(batch * 4, 1.0, np.float32)
    for s in range(steps):
        mu, var = net.forward(xs[s])
        assert np.array_equal(mu, GOLD[f"{name}_mu"][s]), f"step {s}: max diff {np.abs(mu - GOLD[f'{name}_mu'][s]).max()}"
        assert np.array_equal(var, GOLD[f"{name}_var"][s]), f"step {s}"
        net.update_using_indices(GOLD[f"{name}_obs"][s], var_y, GOLD[f"{name}_idx"][s], 4)
        net.backward()
        net.step()
    for k, p in net.state_dict().items():
        assert np.array_equal(p["mu_w"].reshape(-1), GOLD[f"{name}_final_{k}_mu_w"]), k
        assert np.array_equal(p["var_w"].reshape(-1), GOLD[f"{name}_final_{k}_var_w"]), k
        if p["mu_b"] is not None:
            assert np.array_equal(p["mu_b"], GOLD[f"{name}_final_{k}_mu_b"]), k
            assert np.array_equal(p["var_b"], GOLD[f"{name}_final_{k}_var_b"]), k


def test_full_resnet18_spec_shapes(oracle):
    """The 224 x 224 ResNet-18 of the benchmark configuration: layer and parameter counts only (no arithmetic)."""
    from oracle_net import resnet_spec
    spec = resnet_spec(stem=("conv", 3, 64, 6, 2, 2, 1, False), stem_pool=("pool", 3, 2, 1, 2), final_pool=7)
    net = OracleNet(oracle, spec, (3, 224, 224))
    assert net.out_shape == (11,)
    sd = net.state_dict()
    assert sum(k.startswith("Conv2d") for k in sd) == 20 and sum(k.startswith("BatchNorm2d") for k in sd) == 20
    n = sum(p["mu_w"].size + (0 if p["mu_b"] is None else p["mu_b"].size) for p in sd.values())
    assert n == 11_680_512 + 2 * 4800 + 512 * 11 + 11   # conv weights, BatchNorm scales and shifts, classifier
