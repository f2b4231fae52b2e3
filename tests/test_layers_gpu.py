"""BatchNorm2d, AvgPool2d and the residual add through the C ABI against the CPU oracle (bit-identical to the
reference's CPU classes on the cases of tests/golden/layers_golden.npz). Tolerance as for the hot path: 1e-5 on means and
mean deltas, 1e-4 on variances and variance deltas, relative to the largest reference entry of the tensor."""
import ctypes as C
import os

import numpy as np
import pytest
from oracle_lib import ConvGeom

pytestmark = pytest.mark.gpu
GOLD = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "layers_golden.npz"))
EPS, MOM = (float(v) for v in GOLD["eps_momentum"])
f32 = np.float32


@pytest.fixture(scope="module")
def G():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import gpu_util
    return gpu_util


def _case(prefix):
    return {k[len(prefix):]: np.ascontiguousarray(GOLD[k]) for k in GOLD.files if k.startswith(prefix)}


def _bn_forward(G, B, Cn, wihi, training, momentum, mw, vw, mb, vb, ma, va, mra, vra, misalign=0):
    from cutagi_b200.capi import lib
    d = [G.dev(x, misalign) for x in (mw, vw, mb, vb, ma, va)]
    ra_m, ra_v = G.dev(mra.copy()), G.dev(vra.copy())
    mean, var = G.Out(Cn), G.Out(Cn)
    mz, vz = G.Out(B * Cn * wihi, misalign), G.Out(B * Cn * wihi, misalign)
    lib.tagi_bn2d_fwd(B, Cn, wihi, int(mb is not None), int(training), C.c_float(EPS), C.c_float(momentum), G.p(d[0]),
                      G.p(d[1]), G.p(d[2]), G.p(d[3]), G.p(d[4]), G.p(d[5]), G.p(ra_m), G.p(ra_v), mean.ptr(), var.ptr(),
                      mz.ptr(), vz.ptr(), None)
    shape = (B, Cn, wihi)
    stats = (mean.get(), var.get()) if training else (None, None)
    return mz.get(shape), vz.get(shape), stats[0], stats[1], ra_m.cpu().numpy(), ra_v.cpu().numpy()


def _bn_backward(G, B, Cn, wihi, mw, vw, vb, ma, jcb, mean, var, dmo, dvo, state_update=True):
    from cutagi_b200.capi import lib
    d = [G.dev(x) for x in (mw, vw, vb, ma, jcb, mean, var, dmo, dvo)]
    dm, dv = G.Out(B * Cn * wihi), G.Out(B * Cn * wihi)
    o = [G.Out(Cn) for _ in range(4)]
    lib.tagi_bn2d_bwd(B, Cn, wihi, int(vb is not None), int(state_update), C.c_float(EPS), *[G.p(x) for x in d], dm.ptr(),
                      dv.ptr(), o[0].ptr(), o[1].ptr(), o[2].ptr(), o[3].ptr(), None)
    import torch
    torch.cuda.synchronize()
    shape = (B, Cn, wihi)
    outs = [dm.get(shape), dv.get(shape)] if state_update else [None, None]
    outs += [o[0].get(), o[1].get()]
    outs += [o[2].get(), o[3].get()] if vb is not None else [None, None]
    return outs


def _check_bn(G, oracle, B, Cn, wihi, bias, first, rng=None, g=None, misalign=0):
    if g is None:
        g = dict(mu_a=rng.standard_normal((B, Cn, wihi)).astype(f32) + f32(0.5),
                 var_a=rng.uniform(0.01, 0.5, (B, Cn, wihi)).astype(f32), mu_w=rng.standard_normal(Cn).astype(f32),
                 var_w=rng.uniform(0.01, 0.2, Cn).astype(f32), mu_ra_in=rng.standard_normal(Cn).astype(f32),
                 var_ra_in=rng.uniform(0.5, 1.5, Cn).astype(f32), jcb=rng.uniform(0, 1, (B, Cn, wihi)).astype(f32),
                 dmu_o=rng.standard_normal((B, Cn, wihi)).astype(f32) * f32(0.1),
                 dvar_o=-rng.uniform(0, 1e-3, (B, Cn, wihi)).astype(f32))
        if bias:
            g["mu_b"], g["var_b"] = rng.standard_normal(Cn).astype(f32), rng.uniform(0.01, 0.2, Cn).astype(f32)
    mom = 0.0 if first else MOM
    mean, var = oracle.bn2d_stats(g["mu_a"], g["var_a"])
    mra, vra = g["mu_ra_in"].copy(), g["var_ra_in"].copy()
    oracle.bn2d_running(mom, mean, var, mra, vra)
    rz = oracle.bn2d_fwd(EPS, g["mu_w"], g["var_w"], g.get("mu_b"), g.get("var_b"), g["mu_a"], g["var_a"], mean, var)
    mz, vz, gm, gv, gra_m, gra_v = _bn_forward(G, B, Cn, wihi, True, mom, g["mu_w"], g["var_w"], g.get("mu_b"),
                                               g.get("var_b"), g["mu_a"], g["var_a"], g["mu_ra_in"], g["var_ra_in"],
                                               misalign)
    G.check("batch mean", gm, mean, G.RTOL_MU)
    G.check("batch var", gv, var, G.RTOL_VAR)
    G.check("mu_ra", gra_m, mra, G.RTOL_MU)
    G.check("var_ra", gra_v, vra, G.RTOL_VAR)
    G.check("mu_z", mz, rz[0], G.RTOL_MU)
    G.check("var_z", vz, rz[1], G.RTOL_VAR)
    # inference: running averages as given
    ez = oracle.bn2d_fwd(EPS, g["mu_w"], g["var_w"], g.get("mu_b"), g.get("var_b"), g["mu_a"], g["var_a"], g["mu_ra_in"],
                         g["var_ra_in"])
    mz, vz, _, _, ra_m, ra_v = _bn_forward(G, B, Cn, wihi, False, MOM, g["mu_w"], g["var_w"], g.get("mu_b"), g.get("var_b"),
                                           g["mu_a"], g["var_a"], g["mu_ra_in"], g["var_ra_in"])
    G.check("mu_z eval", mz, ez[0], G.RTOL_MU)
    G.check("var_z eval", vz, ez[1], G.RTOL_VAR)
    assert np.array_equal(ra_m, g["mu_ra_in"]) and np.array_equal(ra_v, g["var_ra_in"])
    # backward with the oracle's statistics
    rs = oracle.bn2d_bwd_state(EPS, g["mu_w"], g["jcb"], var, g["dmu_o"], g["dvar_o"])
    rp = oracle.bn2d_bwd_param(EPS, g["var_w"], g.get("var_b"), g["mu_a"], mean, var, g["dmu_o"], g["dvar_o"])
    got = _bn_backward(G, B, Cn, wihi, g["mu_w"], g["var_w"], g.get("var_b"), g["mu_a"], g["jcb"], mean, var, g["dmu_o"],
                       g["dvar_o"])
    G.check("dmu", got[0], rs[0], G.RTOL_MU)
    G.check("dvar", got[1], rs[1], G.RTOL_VAR)
    G.check("dmu_w", got[2], rp[0], G.RTOL_MU)
    G.check("dvar_w", got[3], rp[1], G.RTOL_VAR)
    if bias:
        G.check("dmu_b", got[4], rp[2], G.RTOL_MU)
        G.check("dvar_b", got[5], rp[3], G.RTOL_VAR)
    return g, mean, var, rp


@pytest.mark.parametrize("i", range(int(GOLD["n_bn"])))
def test_batchnorm2d_golden(G, oracle, i):
    g = _case(f"bn{i}_")
    B, Cn, hi, wi, bias, first = (int(v) for v in g["shape"])
    _check_bn(G, oracle, B, Cn, hi * wi, bias, first, g=g)


@pytest.mark.parametrize("B,Cn,wihi,bias,first", [
    (64, 16, 28 * 28, 1, 0),     # 12 slices per channel
    (8, 512, 49, 0, 0),          # 7x7 planes: H*W not a multiple of 4
    (5, 7, 4097, 1, 1),          # slice boundary inside an image, ragged last slice
    (2, 3, 1, 1, 0),             # one pixel per plane
    (16, 64, 56 * 56, 0, 0),     # ResNet-18 layer1 plane at batch 16
])
def test_batchnorm2d_shapes(G, oracle, B, Cn, wihi, bias, first):
    _check_bn(G, oracle, B, Cn, wihi, bias, first, rng=np.random.default_rng(B * 131 + Cn))


def test_batchnorm2d_misaligned_and_param_only(G, oracle):
    rng = np.random.default_rng(5)
    g, mean, var, rp = _check_bn(G, oracle, 3, 6, 20, 1, 0, rng=rng, misalign=1)
    got = _bn_backward(G, 3, 6, 20, g["mu_w"], g["var_w"], g["var_b"], g["mu_a"], g["jcb"], mean, var, g["dmu_o"],
                       g["dvar_o"], state_update=False)
    G.check("dmu_w", got[2], rp[0], G.RTOL_MU)
    G.check("dvar_w", got[3], rp[1], G.RTOL_VAR)


def _pool(G, g, ma, va, jcb, dmo, dvo):
    from cutagi_b200.capi import lib
    d = [G.dev(x) for x in (ma, va, jcb, dmo, dvo)]
    mz, vz, dm, dv = G.Out(g.B * g.n_out), G.Out(g.B * g.n_out), G.Out(g.B * g.n_in), G.Out(g.B * g.n_in)
    cg = G.cgeom(g)
    lib.tagi_avgpool2d_fwd(C.byref(cg), G.p(d[0]), G.p(d[1]), mz.ptr(), vz.ptr(), None)
    lib.tagi_avgpool2d_bwd_state(C.byref(cg), G.p(d[2]), G.p(d[3]), G.p(d[4]), dm.ptr(), dv.ptr(), None)
    return mz.get((g.B, g.n_out)), vz.get((g.B, g.n_out)), dm.get((g.B, g.n_in)), dv.get((g.B, g.n_in))


POOLS = [dict(B=128, fi=32, hi=32, wi=32, fo=32, k=2, stride=2, pad=0, pad_type=0),    # CNN pools
         dict(B=4, fi=64, hi=112, wi=112, fo=64, k=3, stride=2, pad=1, pad_type=2),    # ResNet-18 stem pool
         dict(B=16, fi=512, hi=7, wi=7, fo=512, k=7, stride=7, pad=0, pad_type=0),     # global pooling
         dict(B=3, fi=5, hi=9, wi=9, fo=5, k=3, stride=2, pad=1, pad_type=1),
         dict(B=2, fi=3, hi=11, wi=11, fo=3, k=3, stride=1, pad=1, pad_type=1)]


@pytest.mark.parametrize("kw", POOLS, ids=lambda k: "c{fi}_h{hi}_k{k}_s{stride}_p{pad}t{pad_type}".format(**k))
def test_avgpool2d_shapes(G, oracle, kw):
    g = ConvGeom(**kw)
    rng = np.random.default_rng(g.fi + g.k)
    ma, va = rng.standard_normal((g.B, g.n_in)).astype(f32), rng.uniform(0.01, 0.5, (g.B, g.n_in)).astype(f32)
    j = rng.uniform(0, 1, (g.B, g.n_in)).astype(f32)
    dmo, dvo = rng.standard_normal((g.B, g.n_out)).astype(f32), -rng.uniform(0, 1e-3, (g.B, g.n_out)).astype(f32)
    ref = oracle.avgpool2d_fwd(g, ma, va) + oracle.avgpool2d_bwd_state(g, j, dmo, dvo)
    got = _pool(G, g, ma, va, j, dmo, dvo)
    for name, a, b, tol in zip(("mu_z", "var_z", "dmu", "dvar"), got, ref, (G.RTOL_MU, G.RTOL_VAR) * 2):
        G.check(name, a, b, tol)


@pytest.mark.parametrize("i", range(int(GOLD["n_pool"])))
def test_avgpool2d_golden(G, i):
    g = _case(f"pool{i}_")
    B, Cn, hi, wi, k, stride, pad, pad_type, ho, wo = (int(v) for v in g["geom"])
    geom = ConvGeom(B=B, fi=Cn, hi=hi, wi=wi, fo=Cn, k=k, stride=stride, pad=pad, pad_type=pad_type)
    got = _pool(G, geom, g["mu_a"], g["var_a"], g["jcb"], g["dmu_o"], g["dvar_o"])
    for name, a, key, tol in zip(("mu_z", "var_z", "dmu", "dvar"), got, ("mu_z", "var_z", "dmu", "dvar"),
                                 (G.RTOL_MU, G.RTOL_VAR) * 2):
        G.check(name, a, g[key], tol)


def test_avgpool2d_geometry_error(G):
    from cutagi_b200 import capi
    g = ConvGeom(B=1, fi=2, hi=8, wi=8, fo=2, k=2, stride=2, pad=0, pad_type=0)
    cg = G.cgeom(g)
    cg.wo = 5
    x = G.dev(np.zeros(g.n_in, f32))
    o = G.Out(g.n_out)
    with pytest.raises(capi.TagiError):
        capi.lib.tagi_avgpool2d_fwd(C.byref(cg), G.p(x), G.p(x), o.ptr(), o.ptr(), None)


def test_add_shortcut(G, oracle):
    from cutagi_b200.capi import lib
    rng = np.random.default_rng(9)
    n = 100003
    a, va, s, vs, j = (rng.standard_normal(n).astype(f32) for _ in range(5))
    for jcb in (None, j):
        ra, rva = a.copy(), va.copy()
        oracle.add_shortcut(s, vs, jcb, ra, rva)
        da, dva, ds, dvs, dj = (G.dev(x) for x in (a.copy(), va.copy(), s, vs, jcb))
        lib.tagi_add_shortcut(G.p(ds), G.p(dvs), G.p(dj), n, G.p(da), G.p(dva), None)
        G.check("mu", da.cpu().numpy(), ra, G.RTOL_MU)
        G.check("var", dva.cpu().numpy(), rva, G.RTOL_VAR)


def test_mixture_relu(G, oracle):
    """tagi_mixture_relu_fwd against the reference's outputs (golden) and, on a larger tensor, against the oracle."""
    from cutagi_b200.capi import lib
    rng = np.random.default_rng(12)
    big_m, big_v = (rng.standard_normal(300001) * 3).astype(f32), rng.uniform(1e-4, 4, 300001).astype(f32)
    for mz, vz, ref in ((np.ascontiguousarray(GOLD["mrelu_mu_z"]), np.ascontiguousarray(GOLD["mrelu_var_z"]),
                         (GOLD["mrelu_mu_a"], GOLD["mrelu_var_a"], GOLD["mrelu_jcb"])),
                        (big_m, big_v, oracle.mixture_relu(big_m, big_v)),
                        (big_m[:300000], big_v[:300000], oracle.mixture_relu(big_m[:300000], big_v[:300000]))):  # 16-byte path
        dm, dv = G.dev(mz), G.dev(vz)
        o = [G.Out(mz.size) for _ in range(3)]
        lib.tagi_mixture_relu_fwd(G.p(dm), G.p(dv), mz.size, o[0].ptr(), o[1].ptr(), o[2].ptr(), None)
        G.check("mu_a", o[0].get(), ref[0], G.RTOL_MU)
        G.check("var_a", o[1].get(), ref[1], G.RTOL_VAR)
        G.check("jcb", o[2].get(), ref[2], G.RTOL_MU)


@pytest.mark.parametrize("i", range(4))
def test_param_update_single_and_multi(G, golden, i):
    """tagi_param_update and tagi_param_update_multi against the reference's BaseLayer::update_weights / update_biases
    (tests/golden/ops_golden.npz: batch sizes on both sides of the cap-factor thresholds, deltas that hit the cap and that
    drive variances negative). The weight variance reset counter is the reference's neg_var_w_counter."""
    import torch
    from cutagi_b200.capi import lib
    g = {k[len(f"upd{i}_"):]: np.ascontiguousarray(golden[k]) for k in golden.files if k.startswith(f"upd{i}_")}
    bs = int(g["batch"][0])
    for multi in (False, True):
        t = {k: G.dev(g[k]) for k in ("mu_w0", "var_w0", "mu_b0", "var_b0", "dmu_w", "dvar_w", "dmu_b", "dvar_b")}
        neg = torch.zeros(1, dtype=torch.int32, device="cuda")
        if multi:
            table = torch.tensor([[t["mu_w0"].data_ptr(), t["var_w0"].data_ptr(), t["dmu_w"].data_ptr(),
                                   t["dvar_w"].data_ptr(), t["mu_w0"].numel()]], dtype=torch.int64, device="cuda")
            lib.tagi_param_update_multi(bs, 1, table.data_ptr(), neg.data_ptr(), None)
            table_b = torch.tensor([[t["mu_b0"].data_ptr(), t["var_b0"].data_ptr(), t["dmu_b"].data_ptr(),
                                     t["dvar_b"].data_ptr(), t["mu_b0"].numel()]], dtype=torch.int64, device="cuda")
            lib.tagi_param_update_multi(bs, 1, table_b.data_ptr(), None, None)
        else:
            lib.tagi_param_update(bs, t["mu_w0"].numel(), G.p(t["mu_w0"]), G.p(t["var_w0"]), G.p(t["dmu_w"]), G.p(t["dvar_w"]),
                                  neg.data_ptr(), None)
            lib.tagi_param_update(bs, t["mu_b0"].numel(), G.p(t["mu_b0"]), G.p(t["var_b0"]), G.p(t["dmu_b"]), G.p(t["dvar_b"]),
                                  None, None)
        torch.cuda.synchronize()
        for a, b in (("mu_w0", "mu_w1"), ("var_w0", "var_w1"), ("mu_b0", "mu_b1"), ("var_b0", "var_b1")):
            G.check(b, t[a].cpu().numpy(), g[b], 1e-6)
        assert int(neg.item()) == int(g["neg"][0])


@pytest.mark.parametrize("n", [1000003, 1 << 20])
def test_activations_in_place(G, oracle, n):
    """tagi_relu_fwd and tagi_mixture_relu_fwd with mu_a = mu_z and var_a = var_z (how tagi_*_fwd_act runs them after a
    forward pass that could not fold the activation in): same results as the out-of-place call, bit for bit, on the
    scalar (odd n) and the 16-byte (n a multiple of 4) kernels."""
    import torch
    from cutagi_b200.capi import lib
    rng = np.random.default_rng(n)
    mz = rng.standard_normal(n).astype(np.float32)
    vz = rng.uniform(1e-3, 1.0, n).astype(np.float32)
    for fn, ref in ((lib.tagi_relu_fwd, oracle.relu(mz, vz)), (lib.tagi_mixture_relu_fwd, None)):
        m, v = torch.from_numpy(mz).cuda(), torch.from_numpy(vz).cuda()
        om, ov, oj, j = torch.empty_like(m), torch.empty_like(m), torch.empty_like(m), torch.empty_like(m)
        fn(m.data_ptr(), v.data_ptr(), n, om.data_ptr(), ov.data_ptr(), oj.data_ptr(), None)
        fn(m.data_ptr(), v.data_ptr(), n, m.data_ptr(), v.data_ptr(), j.data_ptr(), None)
        torch.cuda.synchronize()
        assert torch.equal(m, om) and torch.equal(v, ov) and torch.equal(j, oj)
        if ref is not None:
            for a, b in zip((m, v, j), ref):
                assert np.array_equal(a.cpu().numpy(), b)
