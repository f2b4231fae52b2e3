"""Pins the oracle's BatchNorm2d / AvgPool2d / residual-add restatement on the reference's own CPU classes:
tests/golden/layers_golden.npz holds their outputs for seeded inputs (tests/golden/make_layers_golden.py). The port keeps
the reference's summation order, so the comparison is bit-exact. Where the compiled reference classes are present
(oracle/_ref) fresh random cases are compared live as well."""
import os

import numpy as np
import pytest
from oracle_lib import ConvGeom, RefLib

GOLD = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "layers_golden.npz"))
EPS, MOM = (float(v) for v in GOLD["eps_momentum"])


def _case(prefix):
    return {k[len(prefix):]: np.ascontiguousarray(GOLD[k]) for k in GOLD.files if k.startswith(prefix)}


@pytest.mark.parametrize("i", range(int(GOLD["n_bn"])))
def test_batchnorm2d_matches_golden(oracle, i):
    g = _case(f"bn{i}_")
    B, C, hi, wi, bias, first = (int(v) for v in g["shape"])
    mean, var = oracle.bn2d_stats(g["mu_a"], g["var_a"])
    assert np.array_equal(mean, g["mean"]) and np.array_equal(var, g["var"])
    mra, vra = g["mu_ra_in"].copy(), g["var_ra_in"].copy()
    oracle.bn2d_running(0.0 if first else MOM, mean, var, mra, vra)   # first training batch: momentum 0
    assert np.array_equal(mra, g["mu_ra"]) and np.array_equal(vra, g["var_ra"])
    mz, vz = oracle.bn2d_fwd(EPS, g["mu_w"], g["var_w"], g.get("mu_b"), g.get("var_b"), g["mu_a"], g["var_a"], mean, var)
    assert np.array_equal(mz, g["mu_z"]) and np.array_equal(vz, g["var_z"])
    dm, dv = oracle.bn2d_bwd_state(EPS, g["mu_w"], g["jcb"], var, g["dmu_o"], g["dvar_o"])
    assert np.array_equal(dm, g["dmu"]) and np.array_equal(dv, g["dvar"])
    dmw, dvw, dmb, dvb = oracle.bn2d_bwd_param(EPS, g["var_w"], g.get("var_b"), g["mu_a"], mean, var, g["dmu_o"],
                                               g["dvar_o"])
    assert np.array_equal(dmw, g["dmu_w"]) and np.array_equal(dvw, g["dvar_w"])
    if bias:
        assert np.array_equal(dmb, g["dmu_b"]) and np.array_equal(dvb, g["dvar_b"])


@pytest.mark.parametrize("i", range(int(GOLD["n_pool"])))
def test_avgpool2d_matches_golden(oracle, i):
    g = _case(f"pool{i}_")
    B, C, hi, wi, k, stride, pad, pad_type, ho, wo = (int(v) for v in g["geom"])
    geom = ConvGeom(B=B, fi=C, hi=hi, wi=wi, fo=C, k=k, stride=stride, pad=pad, pad_type=pad_type)
    assert (geom.ho, geom.wo) == (ho, wo)
    mz, vz = oracle.avgpool2d_fwd(geom, g["mu_a"], g["var_a"])
    assert np.array_equal(mz, g["mu_z"]) and np.array_equal(vz, g["var_z"])
    dm, dv = oracle.avgpool2d_bwd_state(geom, g["jcb"], g["dmu_o"], g["dvar_o"])
    assert np.array_equal(dm, g["dmu"]) and np.array_equal(dv, g["dvar"])


def test_mixture_relu_matches_golden(oracle):
    ma, va, j = oracle.mixture_relu(np.ascontiguousarray(GOLD["mrelu_mu_z"]), np.ascontiguousarray(GOLD["mrelu_var_z"]))
    assert np.array_equal(ma, GOLD["mrelu_mu_a"]) and np.array_equal(va, GOLD["mrelu_var_a"])
    assert np.array_equal(j, GOLD["mrelu_jcb"])


def test_add_shortcut(oracle):
    """src/resnet_block.cpp:8-31."""
    rng = np.random.default_rng(3)
    a, va, s, vs, j = (rng.standard_normal(257).astype(np.float32) for _ in range(5))
    x, vx = a.copy(), va.copy()
    oracle.add_shortcut(s, vs, None, x, vx)
    assert np.array_equal(x, a + s) and np.array_equal(vx, va + vs)
    x, vx = a.copy(), va.copy()
    oracle.add_shortcut(s, vs, j, x, vx)
    assert np.array_equal(x, a + s * j) and np.array_equal(vx, va + vs * j * j)


@pytest.mark.skipif(not RefLib.available(), reason="compiled reference classes (oracle/_ref) not present")
def test_live_reference_random_cases(oracle):
    ref = RefLib()
    rng = np.random.default_rng(11)
    f = np.float32
    for _ in range(4):
        B, C, hi, wi = (int(v) for v in rng.integers(2, 9, 4))
        n = hi * wi
        ma, va = rng.standard_normal((B, C, n)).astype(f), rng.uniform(0.01, 0.5, (B, C, n)).astype(f)
        mw, vw, mb, vb = (rng.uniform(0.1, 1, C).astype(f) for _ in range(4))
        j, dmo = rng.uniform(0, 1, (B, C, n)).astype(f), rng.standard_normal((B, C, n)).astype(f)
        dvo = -rng.uniform(0, 1e-3, (B, C, n)).astype(f)
        for threads in (1, 3):
            mra, vra = np.zeros(C, f), np.ones(C, f)
            mz, vz, mean, var = ref.bn2d_forward(EPS, MOM, mw, vw, mb, vb, ma, va, mra, vra, hi, wi, True, False, threads)
            om, ov = oracle.bn2d_stats(ma, va)
            assert np.array_equal(om, mean) and np.array_equal(ov, var)
            for a, b in zip(oracle.bn2d_fwd(EPS, mw, vw, mb, vb, ma, va, om, ov), (mz, vz)):
                assert np.array_equal(a, b)
            got = oracle.bn2d_bwd_state(EPS, mw, j, ov, dmo, dvo) + oracle.bn2d_bwd_param(EPS, vw, vb, ma, om, ov, dmo, dvo)
            for a, b in zip(got, ref.bn2d_backward(EPS, mw, vw, vb, ma, j, mean, var, dmo, dvo, hi, wi, threads)):
                assert np.array_equal(a, b)
    # inference mode normalises with the running averages
    mra, vra = rng.standard_normal(C).astype(f), rng.uniform(0.5, 2, C).astype(f)
    mz, vz, _, _ = ref.bn2d_forward(EPS, MOM, mw, vw, mb, vb, ma, va, mra.copy(), vra.copy(), hi, wi, False, False)
    for a, b in zip(oracle.bn2d_fwd(EPS, mw, vw, mb, vb, ma, va, mra, vra), (mz, vz)):
        assert np.array_equal(a, b)
    for kw in (dict(B=2, fi=3, hi=10, wi=10, fo=3, k=2, stride=2, pad=0, pad_type=0),
               dict(B=1, fi=2, hi=11, wi=11, fo=2, k=3, stride=2, pad=1, pad_type=1),
               dict(B=2, fi=2, hi=7, wi=7, fo=2, k=7, stride=7, pad=0, pad_type=0)):
        g = ConvGeom(**kw)
        ma, va = rng.standard_normal((g.B, g.n_in)).astype(f), rng.uniform(0.01, 0.5, (g.B, g.n_in)).astype(f)
        j, dmo = rng.uniform(0, 1, (g.B, g.n_in)).astype(f), rng.standard_normal((g.B, g.n_out)).astype(f)
        dvo = -rng.uniform(0, 1e-3, (g.B, g.n_out)).astype(f)
        mz, vz, dm, dv, wo, ho = ref.avgpool2d(g, ma, va, j, dmo, dvo)
        got = oracle.avgpool2d_fwd(g, ma, va) + oracle.avgpool2d_bwd_state(g, j, dmo, dvo)
        for a, b in zip(got, (mz, vz, dm, dv)):
            assert np.array_equal(a, b)
