"""Generates tests/golden/layers_golden.npz from the reference's own CPU classes `BatchNorm2d` and `AvgPool2d` and its
MixtureReLU kernel.

Run in the build container, where the reference sources exist:
    make -C oracle ref && python tests/golden/make_layers_golden.py
Each case stores its seeded inputs and what the reference's forward (training mode: batch statistics, running
averages) and backward produced for them, so that the oracle port can be pinned where the reference is absent.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
from oracle_lib import ConvGeom, RefLib  # noqa: E402

EPS, MOMENTUM = 1e-5, 0.9
BN_CASES = [  # (B, C, hi, wi, bias, first_batch)
    (4, 8, 6, 6, 1, 1), (3, 5, 7, 5, 0, 0), (2, 64, 4, 4, 1, 0), (1, 3, 2, 2, 1, 1), (8, 16, 8, 8, 0, 1),
]
POOL_CASES = [  # AvgPool2d(2, 2), global pooling, the ResNet stem's overlapping 3x3 stride-2 pool, other overlaps
    dict(B=2, fi=3, hi=8, wi=8, fo=3, k=2, stride=2, pad=0, pad_type=0),
    dict(B=2, fi=4, hi=4, wi=4, fo=4, k=4, stride=4, pad=0, pad_type=0),
    dict(B=2, fi=3, hi=8, wi=8, fo=3, k=3, stride=2, pad=1, pad_type=2),
    dict(B=2, fi=3, hi=9, wi=9, fo=3, k=3, stride=2, pad=1, pad_type=1),
    dict(B=1, fi=2, hi=7, wi=7, fo=2, k=3, stride=1, pad=1, pad_type=1),
    dict(B=2, fi=2, hi=12, wi=12, fo=2, k=3, stride=1, pad=0, pad_type=0),
]


def main():
    ref = RefLib()
    f = np.float32
    out = {}
    for i, (B, C, hi, wi, bias, first) in enumerate(BN_CASES):
        rng = np.random.default_rng(4000 + i)
        n = hi * wi
        ma, va = rng.standard_normal((B, C, n)).astype(f), rng.uniform(0.01, 0.5, (B, C, n)).astype(f)
        mw, vw = rng.standard_normal(C).astype(f), rng.uniform(0.01, 0.2, C).astype(f)
        mb, vb = (rng.standard_normal(C).astype(f), rng.uniform(0.01, 0.2, C).astype(f)) if bias else (None, None)
        mra, vra = rng.standard_normal(C).astype(f), rng.uniform(0.5, 1.5, C).astype(f)
        j = rng.uniform(0, 1, (B, C, n)).astype(f)
        dmo, dvo = rng.standard_normal((B, C, n)).astype(f) * f(0.1), -rng.uniform(0, 1e-3, (B, C, n)).astype(f)
        ra_m, ra_v = mra.copy(), vra.copy()
        mz, vz, mean, var = ref.bn2d_forward(EPS, MOMENTUM, mw, vw, mb, vb, ma, va, ra_m, ra_v, hi, wi, True, bool(first))
        dm, dv, dmw, dvw, dmb, dvb = ref.bn2d_backward(EPS, mw, vw, vb, ma, j, mean, var, dmo, dvo, hi, wi)
        p = f"bn{i}_"
        out.update({p + "shape": np.array([B, C, hi, wi, bias, first]), p + "mu_a": ma, p + "var_a": va, p + "mu_w": mw,
                    p + "var_w": vw, p + "mu_ra_in": mra, p + "var_ra_in": vra, p + "jcb": j, p + "dmu_o": dmo,
                    p + "dvar_o": dvo, p + "mu_z": mz, p + "var_z": vz, p + "mean": mean, p + "var": var,
                    p + "mu_ra": ra_m, p + "var_ra": ra_v, p + "dmu": dm, p + "dvar": dv, p + "dmu_w": dmw,
                    p + "dvar_w": dvw})
        if bias:
            out.update({p + "mu_b": mb, p + "var_b": vb, p + "dmu_b": dmb, p + "dvar_b": dvb})
    for i, kw in enumerate(POOL_CASES):
        g = ConvGeom(**kw)
        rng = np.random.default_rng(5000 + i)
        ma, va = rng.standard_normal((g.B, g.n_in)).astype(f), rng.uniform(0.01, 0.5, (g.B, g.n_in)).astype(f)
        j = rng.uniform(0, 1, (g.B, g.n_in)).astype(f)
        dmo, dvo = rng.standard_normal((g.B, g.n_out)).astype(f), -rng.uniform(0, 1e-3, (g.B, g.n_out)).astype(f)
        mz, vz, dm, dv, wo, ho = ref.avgpool2d(g, ma, va, j, dmo, dvo)
        assert (wo, ho) == (g.wo, g.ho)
        p = f"pool{i}_"
        out.update({p + "geom": np.array([g.B, g.fi, g.hi, g.wi, g.k, g.stride, g.pad, g.pad_type, g.ho, g.wo]),
                    p + "mu_a": ma, p + "var_a": va, p + "jcb": j, p + "dmu_o": dmo, p + "dvar_o": dvo, p + "mu_z": mz,
                    p + "var_z": vz, p + "dmu": dm, p + "dvar": dv})
    # MixtureReLU moments (src/activation.cpp:152-178): means on both sides of zero, small and large variances
    rng = np.random.default_rng(6000)
    mz = np.concatenate([rng.standard_normal(4000) * 2, np.linspace(-12, 12, 97)]).astype(f)
    vz = np.concatenate([rng.uniform(1e-4, 3, 4000), np.full(97, 0.5)]).astype(f)
    ma, va, j = ref.mixture_relu(mz, vz)
    out.update({"mrelu_mu_z": mz, "mrelu_var_z": vz, "mrelu_mu_a": ma, "mrelu_var_a": va, "mrelu_jcb": j})
    out["n_bn"], out["n_pool"] = np.array(len(BN_CASES)), np.array(len(POOL_CASES))
    out["eps_momentum"] = np.array([EPS, MOMENTUM], np.float32)
    path = os.path.join(HERE, "layers_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
