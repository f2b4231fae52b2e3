"""CPU trainer for TAGI MLPs built from the oracle's per-op restatements (test infrastructure).

Mirrors what the reference's `Sequential` does for a stack of Linear / ReLU layers (src/sequential.cpp:279-335,
387-411, 440-448): forward with the input Jacobian set to one, innovation at the output, backward in reverse order with
the first layer computing parameter deltas only, then the capped update of every layer.
"""
import numpy as np

F32 = np.float32


def cfg0_problem(seed=0, sizes=(784, 128, 128, 11), batch=32, steps=100):
    """Seeded synthetic stand-in for the MNIST configuration: He-style parameters, U[0,1] inputs, uniform labels."""
    rng = np.random.default_rng(seed)
    params = []
    for k, n in zip(sizes[:-1], sizes[1:]):
        params.append(dict(
            mu_w=(rng.standard_normal((n, k)) * np.sqrt(1.0 / k)).astype(F32),
            var_w=np.full((n, k), 1.0 / k, F32),
            mu_b=np.zeros(n, F32),
            var_b=np.full(n, 1.0 / k, F32)))
    xs = rng.random((steps, batch, sizes[0]), dtype=np.float32)
    labels = rng.integers(0, 10, (steps, batch)).astype(np.int32)
    return params, xs, labels


class OracleMLP:
    def __init__(self, oracle, params):
        self.o = oracle
        self.p = [{k: v.copy() for k, v in layer.items()} for layer in params]

    def forward(self, x, var_x=None):
        o = self.o
        mu, var = np.ascontiguousarray(x, F32), (np.zeros_like(x, F32) if var_x is None else var_x)
        jcb = np.ones_like(mu)
        self.saved = []
        for i, p in enumerate(self.p):
            self.saved.append((mu, jcb))
            mu, var = o.linear_fwd(p["mu_w"], p["var_w"], p["mu_b"], p["var_b"], mu, var)
            jcb = np.ones_like(mu)
            if i < len(self.p) - 1:
                mu, var, jcb = o.relu(mu, var)
        self.out = (mu, var, jcb)
        return mu, var

    def update_using_indices(self, obs, var_obs, idx, n_enc):
        mu, var, jcb = self.out
        self.delta = self.o.output_delta_selected(mu, var, jcb, obs, var_obs, idx, n_enc)

    def update(self, obs, var_obs):
        mu, var, jcb = self.out
        self.delta = self.o.output_delta(mu, var, jcb, np.ascontiguousarray(obs, F32).reshape(mu.shape),
                                         np.ascontiguousarray(var_obs, F32).reshape(mu.shape))

    def backward(self):
        o = self.o
        dmu, dvar = self.delta
        self.dparams = [None] * len(self.p)
        for i in reversed(range(len(self.p))):
            p = self.p[i]
            mu_a, jcb = self.saved[i]
            self.dparams[i] = o.linear_bwd_param(p["var_w"], p["var_b"], mu_a, dmu, dvar)
            if i > 0:
                dmu, dvar = o.linear_bwd_state(p["mu_w"], jcb, dmu, dvar)

    def step(self, batch):
        for p, d in zip(self.p, self.dparams):
            self.o.param_update(batch, p["mu_w"], p["var_w"], d[0], d[1])
            self.o.param_update(batch, p["mu_b"], p["var_b"], d[2], d[3])
