"""Pins the CPU restatement (oracle/) on the reference's own outputs.

The reference has no golden vectors for Linear / Conv2d; tests/golden/ops_golden.npz holds outputs of its CPU
classes for seeded inputs (tests/golden/make_golden.py). The port reproduces the reference's summation order, so
the comparison is bit-exact. Where the compiled reference classes are present (oracle/_ref), they are also
compared live on fresh random shapes.
"""
import numpy as np
import pytest
from oracle_lib import ConvGeom, RefLib

N_LIN, N_CONV, N_UPD = 8, 8, 4


def _opt(g, key):
    return np.ascontiguousarray(g[key]) if key in g.files else None


@pytest.mark.parametrize("i", range(N_LIN))
def test_linear_matches_golden(oracle, golden, i):
    p = f"lin{i}_"
    g = {k[len(p):]: np.ascontiguousarray(golden[k]) for k in golden.files if k.startswith(p)}
    mz, vz = oracle.linear_fwd(g["mu_w"], g["var_w"], g.get("mu_b"), g.get("var_b"), g["mu_a"], g["var_a"])
    assert np.array_equal(mz, g["mu_z"]) and np.array_equal(vz, g["var_z"])
    dma, dva = oracle.linear_bwd_state(g["mu_w"], g["jcb"], g["dmu_z"], g["dvar_z"])
    assert np.array_equal(dma, g["dmu_a"]) and np.array_equal(dva, g["dvar_a"])
    dmw, dvw, dmb, dvb = oracle.linear_bwd_param(g["var_w"], g.get("var_b"), g["mu_a"], g["dmu_z"], g["dvar_z"])
    assert np.array_equal(dmw, g["dmu_w"]) and np.array_equal(dvw, g["dvar_w"])
    if "var_b" in g:
        assert np.array_equal(dmb, g["dmu_b"]) and np.array_equal(dvb, g["dvar_b"])


@pytest.mark.parametrize("i", range(N_CONV))
def test_conv_matches_golden(oracle, golden, i):
    p = f"conv{i}_"
    g = {k[len(p):]: np.ascontiguousarray(golden[k]) for k in golden.files if k.startswith(p)}
    B, fi, hi, wi, fo, k, stride, pad, pad_type, has_bias, ho, wo = [int(v) for v in g["geom"]]
    geom = ConvGeom(B=B, fi=fi, hi=hi, wi=wi, fo=fo, k=k, stride=stride, pad=pad, pad_type=pad_type,
                    has_bias=has_bias)
    assert (geom.ho, geom.wo) == (ho, wo)
    mz, vz = oracle.conv2d_fwd(geom, g["mu_w"], g["var_w"], g.get("mu_b"), g.get("var_b"), g["mu_a"], g["var_a"])
    assert np.array_equal(mz, g["mu_z"]) and np.array_equal(vz, g["var_z"])
    dma, dva = oracle.conv2d_bwd_state(geom, g["mu_w"], g["jcb"], g["dmu_z"], g["dvar_z"])
    assert np.array_equal(dma, g["dmu_a"]) and np.array_equal(dva, g["dvar_a"])
    dmw, dvw, dmb, dvb = oracle.conv2d_bwd_param(geom, g["var_w"], g.get("var_b"), g["mu_a"], g["dmu_z"],
                                                 g["dvar_z"])
    assert np.array_equal(dmw, g["dmu_w"]) and np.array_equal(dvw, g["dvar_w"])
    if has_bias:
        assert np.array_equal(dmb, g["dmu_b"]) and np.array_equal(dvb, g["dvar_b"])


@pytest.mark.parametrize("i", range(N_UPD))
def test_param_update_matches_golden(oracle, golden, i):
    p = f"upd{i}_"
    g = {k[len(p):]: np.ascontiguousarray(golden[k]) for k in golden.files if k.startswith(p)}
    bs = int(g["batch"][0])
    mw, vw, mb, vb = g["mu_w0"].copy(), g["var_w0"].copy(), g["mu_b0"].copy(), g["var_b0"].copy()
    neg = oracle.param_update(bs, mw, vw, g["dmu_w"], g["dvar_w"])
    oracle.param_update(bs, mb, vb, g["dmu_b"], g["dvar_b"])
    assert neg == int(g["neg"][0])
    for a, b in ((mw, "mu_w1"), (vw, "var_w1"), (mb, "mu_b1"), (vb, "var_b1")):
        assert np.array_equal(a, g[b])


def test_f64_variant_agrees_with_f32(oracle, golden):
    g = {k[5:]: np.ascontiguousarray(golden[k]) for k in golden.files if k.startswith("lin5_")}
    m32, v32 = oracle.linear_fwd(g["mu_w"], g["var_w"], g.get("mu_b"), g.get("var_b"), g["mu_a"], g["var_a"])
    m64, v64 = oracle.linear_fwd(g["mu_w"], g["var_w"], g.get("mu_b"), g.get("var_b"), g["mu_a"], g["var_a"], f64=True)
    assert np.abs(m32 - m64).max() <= 1e-5 * np.abs(m64).max()
    assert np.abs(v32 - v64).max() <= 1e-5 * np.abs(v64).max()


@pytest.mark.skipif(not RefLib.available(), reason="compiled reference classes (oracle/_ref) not present")
def test_live_reference_random_shapes(oracle):
    ref = RefLib()
    rng = np.random.default_rng(7)

    def f(*s, lo=None, hi=None):
        return (rng.standard_normal(s) if lo is None else rng.uniform(lo, hi, s)).astype(np.float32)

    for _ in range(6):
        B, K, N = (int(v) for v in rng.integers(1, 40, 3))
        mw, vw, mb, vb = f(N, K), f(N, K, lo=.1, hi=1), f(N), f(N, lo=.1, hi=1)
        ma, va, j = f(B, K), f(B, K, lo=.01, hi=.1), f(B, K, lo=0, hi=1)
        dm, dv = f(B, N), -f(B, N, lo=0, hi=1e-3)
        for a, b in zip(oracle.linear_fwd(mw, vw, mb, vb, ma, va), ref.linear_forward(mw, vw, mb, vb, ma, va)):
            assert np.array_equal(a, b)
        got = oracle.linear_bwd_state(mw, j, dm, dv) + oracle.linear_bwd_param(vw, vb, ma, dm, dv)
        for a, b in zip(got, ref.linear_backward(mw, vw, vb, ma, j, dm, dv)):
            assert np.array_equal(a, b)
    for kw in (dict(B=2, fi=3, hi=10, wi=10, fo=4, k=3, stride=1, pad=1, pad_type=1),
               dict(B=1, fi=2, hi=11, wi=11, fo=3, k=3, stride=2, pad=1, pad_type=1),
               dict(B=2, fi=2, hi=8, wi=8, fo=2, k=4, stride=2, pad=2, pad_type=2)):
        g = ConvGeom(**kw)
        mw, vw, mb, vb = f(g.fo, g.Kc), f(g.fo, g.Kc, lo=.1, hi=1), f(g.fo), f(g.fo, lo=.1, hi=1)
        ma, va, j = f(g.B, g.n_in), f(g.B, g.n_in, lo=.01, hi=.1), f(g.B, g.n_in, lo=0, hi=1)
        dm, dv = f(g.B, g.n_out), -f(g.B, g.n_out, lo=0, hi=1e-3)
        for a, b in zip(oracle.conv2d_fwd(g, mw, vw, mb, vb, ma, va), ref.conv2d_forward(g, mw, vw, mb, vb, ma, va)):
            assert np.array_equal(a, b)
        got = oracle.conv2d_bwd_state(g, mw, j, dm, dv) + oracle.conv2d_bwd_param(g, vw, vb, ma, dm, dv)
        for a, b in zip(got, ref.conv2d_backward(g, mw, vw, vb, ma, j, dm, dv)):
            assert np.array_equal(a, b)


def test_conv_out_size_rule(oracle):
    from oracle_lib import conv_out_size
    assert conv_out_size(3, 1, 32, 32, 1, 1) == (32, 32)
    assert conv_out_size(6, 2, 224, 224, 2, 1) == (112, 112)
    assert conv_out_size(3, 2, 56, 56, 1, 2) == (28, 28)
    assert conv_out_size(2, 2, 56, 56, 0, 0) == (28, 28)
    with pytest.raises(ValueError):
        conv_out_size(3, 2, 8, 8, 0, 0)
