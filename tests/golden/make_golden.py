"""Generates tests/golden/ops_golden.npz from the reference's own CPU classes.

Run in the build container, where the reference sources exist:
    make -C oracle ref && python tests/golden/make_golden.py
Each case stores its seeded inputs and the outputs that the reference's `Linear` / `Conv2d`
(forward, backward) and `BaseLayer::update_weights/update_biases` produced for them, so that the
oracle port can be pinned on machines where the reference is absent.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
from oracle_lib import ConvGeom, RefLib  # noqa: E402

LINEAR_CASES = [  # (B, K, N, bias)
    (1, 1, 1, 1), (3, 1, 17, 1), (17, 129, 1, 0), (5, 7, 3, 1), (4, 64, 64, 1), (32, 128, 11, 1),
    (9, 65, 63, 0), (16, 100, 36, 1),
]
CONV_CASES = [  # cfg3 / ResNet-18 geometries at toy extents plus the odd ones
    dict(B=2, fi=3, hi=8, wi=8, fo=4, k=3, stride=1, pad=1, pad_type=1, has_bias=1),
    dict(B=2, fi=3, hi=8, wi=8, fo=4, k=3, stride=2, pad=1, pad_type=2, has_bias=0),
    dict(B=3, fi=2, hi=12, wi=12, fo=5, k=6, stride=2, pad=2, pad_type=1, has_bias=0),
    dict(B=2, fi=4, hi=6, wi=6, fo=3, k=2, stride=2, pad=0, pad_type=0, has_bias=0),
    dict(B=2, fi=2, hi=9, wi=9, fo=3, k=5, stride=1, pad=2, pad_type=1, has_bias=1),
    dict(B=1, fi=2, hi=7, wi=7, fo=3, k=3, stride=2, pad=2, pad_type=2, has_bias=1),
    dict(B=1, fi=1, hi=5, wi=5, fo=1, k=1, stride=1, pad=0, pad_type=0, has_bias=1),
    dict(B=2, fi=5, hi=4, wi=4, fo=7, k=3, stride=1, pad=0, pad_type=0, has_bias=1),
]


def draw(rng, *shape, lo=None, hi=None):
    if lo is None:
        return rng.standard_normal(shape).astype(np.float32)
    return rng.uniform(lo, hi, shape).astype(np.float32)


def main():
    ref = RefLib()
    out = {}
    for i, (B, K, N, bias) in enumerate(LINEAR_CASES):
        rng = np.random.default_rng(1000 + i)
        mw, vw = draw(rng, N, K) / np.float32(np.sqrt(K)), draw(rng, N, K, lo=0.5, hi=1.5) / np.float32(K)
        mb, vb = (draw(rng, N) * np.float32(0.1), draw(rng, N, lo=1e-3, hi=1e-2)) if bias else (None, None)
        ma, va, j = draw(rng, B, K), draw(rng, B, K, lo=1e-3, hi=1e-1), draw(rng, B, K, lo=0, hi=1)
        dm, dv = draw(rng, B, N) * np.float32(0.1), -draw(rng, B, N, lo=0, hi=1e-3)
        mz, vz = ref.linear_forward(mw, vw, mb, vb, ma, va)
        dma, dva, dmw, dvw, dmb, dvb = ref.linear_backward(mw, vw, vb, ma, j, dm, dv)
        p = f"lin{i}_"
        out.update({p + "shape": np.array([B, K, N, bias]), p + "mu_w": mw, p + "var_w": vw, p + "mu_a": ma,
                    p + "var_a": va, p + "jcb": j, p + "dmu_z": dm, p + "dvar_z": dv, p + "mu_z": mz, p + "var_z": vz,
                    p + "dmu_a": dma, p + "dvar_a": dva, p + "dmu_w": dmw, p + "dvar_w": dvw})
        if bias:
            out.update({p + "mu_b": mb, p + "var_b": vb, p + "dmu_b": dmb, p + "dvar_b": dvb})
    for i, kw in enumerate(CONV_CASES):
        g = ConvGeom(**kw)
        rng = np.random.default_rng(2000 + i)
        mw, vw = draw(rng, g.fo, g.Kc) / np.float32(np.sqrt(g.Kc)), draw(rng, g.fo, g.Kc, lo=0.5, hi=1.5) / np.float32(g.Kc)
        mb, vb = (draw(rng, g.fo) * np.float32(0.1), draw(rng, g.fo, lo=1e-3, hi=1e-2)) if g.has_bias else (None, None)
        ma, va = draw(rng, g.B, g.n_in), draw(rng, g.B, g.n_in, lo=1e-3, hi=1e-1)
        j = draw(rng, g.B, g.n_in, lo=0, hi=1)
        dm, dv = draw(rng, g.B, g.n_out) * np.float32(0.1), -draw(rng, g.B, g.n_out, lo=0, hi=1e-3)
        mz, vz = ref.conv2d_forward(g, mw, vw, mb, vb, ma, va)
        dma, dva, dmw, dvw, dmb, dvb = ref.conv2d_backward(g, mw, vw, vb, ma, j, dm, dv)
        p = f"conv{i}_"
        out.update({p + "geom": np.array([g.B, g.fi, g.hi, g.wi, g.fo, g.k, g.stride, g.pad, g.pad_type, g.has_bias,
                                          g.ho, g.wo]),
                    p + "mu_w": mw, p + "var_w": vw, p + "mu_a": ma, p + "var_a": va, p + "jcb": j, p + "dmu_z": dm,
                    p + "dvar_z": dv, p + "mu_z": mz, p + "var_z": vz, p + "dmu_a": dma, p + "dvar_a": dva,
                    p + "dmu_w": dmw, p + "dvar_w": dvw})
        if g.has_bias:
            out.update({p + "mu_b": mb, p + "var_b": vb, p + "dmu_b": dmb, p + "dvar_b": dvb})
    # capped update: batch sizes on each side of the cap-factor thresholds, with deltas large enough to hit
    # the cap and to drive some variances negative
    for i, bs in enumerate([1, 2, 255, 256]):
        rng = np.random.default_rng(3000 + i)
        n, nb = 257, 13
        mw, vw = draw(rng, n), draw(rng, n, lo=1e-4, hi=1e-2)
        mb, vb = draw(rng, nb), draw(rng, nb, lo=1e-4, hi=1e-2)
        dmw, dvw = draw(rng, n) * np.float32(0.05), draw(rng, n) * np.float32(0.01)
        dmb, dvb = draw(rng, nb) * np.float32(0.05), draw(rng, nb) * np.float32(0.01)
        p = f"upd{i}_"
        out.update({p + "batch": np.array([bs]), p + "mu_w0": mw.copy(), p + "var_w0": vw.copy(),
                    p + "mu_b0": mb.copy(), p + "var_b0": vb.copy(), p + "dmu_w": dmw, p + "dvar_w": dvw,
                    p + "dmu_b": dmb, p + "dvar_b": dvb})
        neg = ref.param_update(bs, mw, vw, mb, vb, dmw, dvw, dmb, dvb)
        out.update({p + "mu_w1": mw, p + "var_w1": vw, p + "mu_b1": mb, p + "var_b1": vb, p + "neg": np.array([neg])})
    path = os.path.join(HERE, "ops_golden.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes", len(out), "arrays")


if __name__ == "__main__":
    main()
