"""GPU parity of the Conv2d entry points (through the C ABI) against the CPU oracle and the golden fixtures."""
import ctypes as C

import numpy as np
import pytest
from oracle_lib import ConvGeom

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def G():
    import gpu_util
    return gpu_util


def _run_all(G, oracle, g, x):
    mz, vz = G.conv_fwd(g, x["mu_w"], x["var_w"], x["mu_b"], x["var_b"], x["mu_a"], x["var_a"])
    rmz, rvz = oracle.conv2d_fwd(g, x["mu_w"], x["var_w"], x["mu_b"], x["var_b"], x["mu_a"], x["var_a"])
    G.check("mu_z", mz, rmz, G.RTOL_MU)
    G.check("var_z", vz, rvz, G.RTOL_VAR)
    da, dv = G.conv_bwd_state(g, x["mu_w"], x["jcb"], x["dmu_z"], x["dvar_z"])
    rda, rdv = oracle.conv2d_bwd_state(g, x["mu_w"], x["jcb"], x["dmu_z"], x["dvar_z"])
    G.check("dmu_a", da, rda, G.RTOL_MU)
    G.check("dvar_a", dv, rdv, G.RTOL_VAR)
    dmw, dvw, dmb, dvb = G.conv_bwd_param(g, x["var_w"], x["var_b"], x["mu_a"], x["dmu_z"], x["dvar_z"])
    r = oracle.conv2d_bwd_param(g, x["var_w"], x["var_b"], x["mu_a"], x["dmu_z"], x["dvar_z"])
    G.check("dmu_w", dmw, r[0], G.RTOL_MU)
    G.check("dvar_w", dvw, r[1], G.RTOL_VAR)
    if g.has_bias:
        G.check("dmu_b", dmb, r[2], G.RTOL_MU)
        G.check("dvar_b", dvb, r[3], G.RTOL_VAR)


@pytest.mark.parametrize("i", range(8))
def test_golden_cases(G, golden, i):
    p = f"conv{i}_"
    x = {k[len(p):]: np.ascontiguousarray(golden[k]) for k in golden.files if k.startswith(p)}
    B, fi, hi, wi, fo, k, stride, pad, pad_type, has_bias, ho, wo = [int(v) for v in x["geom"]]
    g = ConvGeom(B=B, fi=fi, hi=hi, wi=wi, fo=fo, k=k, stride=stride, pad=pad, pad_type=pad_type, has_bias=has_bias)
    mz, vz = G.conv_fwd(g, x["mu_w"], x["var_w"], x.get("mu_b"), x.get("var_b"), x["mu_a"], x["var_a"])
    G.check("mu_z", mz, x["mu_z"], G.RTOL_MU)
    G.check("var_z", vz, x["var_z"], G.RTOL_VAR)
    da, dv = G.conv_bwd_state(g, x["mu_w"], x["jcb"], x["dmu_z"], x["dvar_z"])
    G.check("dmu_a", da, x["dmu_a"], G.RTOL_MU)
    G.check("dvar_a", dv, x["dvar_a"], G.RTOL_VAR)
    dmw, dvw, dmb, dvb = G.conv_bwd_param(g, x["var_w"], x.get("var_b"), x["mu_a"], x["dmu_z"], x["dvar_z"])
    G.check("dmu_w", dmw, x["dmu_w"], G.RTOL_MU)
    G.check("dvar_w", dvw, x["dvar_w"], G.RTOL_VAR)
    if has_bias:
        G.check("dmu_b", dmb, x["dmu_b"], G.RTOL_MU)
        G.check("dvar_b", dvb, x["dvar_b"], G.RTOL_VAR)


# the layer geometries of the CIFAR-shaped CNN and of ResNet-18 at reduced batch / image extent, plus odd ones
GEOMS = [
    dict(B=4, fi=3, hi=32, wi=32, fo=32, k=3, stride=1, pad=1, pad_type=1, has_bias=1),     # CNN conv1
    dict(B=4, fi=32, hi=16, wi=16, fo=64, k=3, stride=1, pad=1, pad_type=1, has_bias=1),    # CNN conv2
    dict(B=4, fi=64, hi=8, wi=8, fo=128, k=3, stride=1, pad=1, pad_type=1, has_bias=1),     # CNN conv3
    dict(B=2, fi=3, hi=32, wi=32, fo=64, k=6, stride=2, pad=2, pad_type=1, has_bias=0),     # ResNet stem (k6 s2 p2)
    dict(B=2, fi=64, hi=14, wi=14, fo=64, k=3, stride=1, pad=1, pad_type=1, has_bias=0),    # layer1 block conv
    dict(B=2, fi=64, hi=14, wi=14, fo=128, k=3, stride=2, pad=1, pad_type=2, has_bias=0),   # down-sampling conv
    dict(B=2, fi=64, hi=14, wi=14, fo=128, k=2, stride=2, pad=0, pad_type=0, has_bias=0),   # projection shortcut
    dict(B=3, fi=128, hi=7, wi=7, fo=256, k=3, stride=1, pad=1, pad_type=1, has_bias=0),
    dict(B=1, fi=5, hi=9, wi=9, fo=7, k=5, stride=2, pad=2, pad_type=1, has_bias=1),
    dict(B=2, fi=1, hi=5, wi=5, fo=1, k=1, stride=1, pad=0, pad_type=0, has_bias=1),
    dict(B=5, fi=2, hi=6, wi=6, fo=130, k=3, stride=1, pad=0, pad_type=0, has_bias=1),
]


@pytest.mark.parametrize("kw", GEOMS, ids=lambda k: "fi{fi}_fo{fo}_h{hi}_k{k}_s{stride}_p{pad}t{pad_type}".format(**k))
def test_layer_geometries(G, oracle, kw):
    g = ConvGeom(**kw)
    rng = np.random.default_rng(g.fi * 131 + g.fo * 7 + g.hi)
    _run_all(G, oracle, g, G.conv_inputs(rng, g))


def test_split_contraction_parameter_pass(G, oracle):
    """Long contraction (B*ho*wo) with a small weight tensor: the parameter pass slices the contraction and sums
    the slices in a fixed order; check parity and run-to-run bit equality."""
    g = ConvGeom(B=16, fi=16, hi=28, wi=28, fo=32, k=3, stride=1, pad=1, pad_type=1, has_bias=1)
    rng = np.random.default_rng(17)
    x = G.conv_inputs(rng, g)
    a = G.conv_bwd_param(g, x["var_w"], x["var_b"], x["mu_a"], x["dmu_z"], x["dvar_z"])
    b = G.conv_bwd_param(g, x["var_w"], x["var_b"], x["mu_a"], x["dmu_z"], x["dvar_z"])
    r = oracle.conv2d_bwd_param(g, x["var_w"], x["var_b"], x["mu_a"], x["dmu_z"], x["dvar_z"])
    for name, u, v, w, tol in zip(("dmu_w", "dvar_w", "dmu_b", "dvar_b"), a, b, r,
                                  (G.RTOL_MU, G.RTOL_VAR, G.RTOL_MU, G.RTOL_VAR)):
        assert np.array_equal(u, v)
        G.check(name, u, w, tol)


def test_geometry_errors(G):
    from cutagi_b200.capi import ConvGeom as CG, TagiError, conv_out_size, lib
    assert conv_out_size(6, 2, 224, 224, 2, 1) == (112, 112)
    assert conv_out_size(3, 2, 56, 56, 1, 2) == (28, 28)
    with pytest.raises(TagiError) as e:
        conv_out_size(3, 2, 8, 8, 0, 0)   # the reference raises for a stride that does not divide
    assert e.value.code == 1 and "invalid hyperparameters" in str(e.value).lower()
    import torch
    q = torch.zeros(4096, device="cuda").data_ptr()
    bad = CG(1, 1, 8, 8, 1, 5, 5, 3, 1, 0, 0, 0)   # ho / wo inconsistent (should be 6)
    with pytest.raises(TagiError):
        lib.tagi_conv2d_fwd(C.byref(bad), q, q, q, q, q, q, q, q, None)


# ------------------------------------------------------------------------------------------------------------------
# Conv2d on the tensor-core kernels (gather pass + the Linear tcgen05 kernels), forced, and the FFMA path, forced
# ------------------------------------------------------------------------------------------------------------------
TC_GEOMS = [
    dict(B=4, fi=32, hi=16, wi=16, fo=64, k=3, stride=1, pad=1, pad_type=1, has_bias=1),    # CNN conv2
    dict(B=4, fi=64, hi=8, wi=8, fo=128, k=3, stride=1, pad=1, pad_type=1, has_bias=1),     # CNN conv3
    dict(B=4, fi=64, hi=14, wi=14, fo=64, k=3, stride=1, pad=1, pad_type=1, has_bias=0),    # ResNet layer1 block conv
    dict(B=4, fi=64, hi=14, wi=14, fo=128, k=3, stride=2, pad=1, pad_type=2, has_bias=0),   # down-sampling conv
    dict(B=4, fi=64, hi=14, wi=14, fo=128, k=2, stride=2, pad=0, pad_type=0, has_bias=0),   # projection shortcut
    dict(B=8, fi=128, hi=7, wi=7, fo=256, k=3, stride=1, pad=1, pad_type=1, has_bias=0),    # 7x7 images: 49 pixels
    dict(B=4, fi=4, hi=10, wi=10, fo=8, k=5, stride=1, pad=2, pad_type=1, has_bias=1),      # tiny channels
    dict(B=2, fi=16, hi=12, wi=12, fo=260, k=1, stride=1, pad=0, pad_type=0, has_bias=1),   # 1x1, ragged fo tile
    dict(B=16, fi=32, hi=32, wi=32, fo=64, k=3, stride=1, pad=1, pad_type=1, has_bias=1),   # parameter pass in 16 slices
    dict(B=6, fi=16, hi=30, wi=30, fo=32, k=3, stride=1, pad=1, pad_type=1, has_bias=0),    # ragged last slice
    dict(B=4, fi=16, hi=15, wi=15, fo=32, k=3, stride=2, pad=1, pad_type=1, has_bias=1),    # stride 2, odd image
    dict(B=4, fi=8, hi=19, wi=19, fo=16, k=5, stride=3, pad=2, pad_type=1, has_bias=0),     # stride 3, 5x5
    dict(B=4, fi=3, hi=32, wi=32, fo=64, k=6, stride=2, pad=2, pad_type=1, has_bias=0),     # ResNet stem: 3 channels, 6x6
    # outputs wider than one tile take the gather pass through scratch, narrower ones gather inside the kernel:
    dict(B=4, fi=192, hi=10, wi=10, fo=32, k=3, stride=1, pad=1, pad_type=1, has_bias=1),   # state pass explicit, forward implicit
    dict(B=4, fi=32, hi=10, wi=10, fo=192, k=3, stride=1, pad=1, pad_type=1, has_bias=1),   # forward explicit, state pass implicit
    dict(B=5, fi=16, hi=13, wi=11, fo=32, k=3, stride=1, pad=1, pad_type=1, has_bias=0),    # 715 rows: ragged last row tile
    # image rows that are no 16-byte multiples while the planes are: the implicit parameter pass treats a plane as one row
    dict(B=8, fi=32, hi=14, wi=14, fo=48, k=3, stride=1, pad=1, pad_type=1, has_bias=1),    # 14 x 14, as ResNet layer3
    dict(B=12, fi=20, hi=10, wi=10, fo=24, k=5, stride=1, pad=2, pad_type=1, has_bias=0),   # 10 x 10, 5 x 5 taps
    dict(B=24, fi=8, hi=6, wi=6, fo=160, k=3, stride=1, pad=1, pad_type=1, has_bias=0),     # 6 x 6 planes, two column tiles
]


@pytest.mark.parametrize("kw", TC_GEOMS, ids=lambda k: "fi{fi}_fo{fo}_h{hi}_k{k}_s{stride}_p{pad}t{pad_type}".format(**k))
def test_conv_tensor_core_path(G, oracle, kw):
    from cutagi_b200 import capi
    from cutagi_b200.capi import lib
    g = ConvGeom(**kw)
    rng = np.random.default_rng(g.fi * 31 + g.fo)
    lib.tagi_set_impl(capi.IMPL_TF32X3)
    try:
        capi.tc_status()
        _run_all(G, oracle, g, G.conv_inputs(rng, g))
        assert capi.tc_status() == 0
    finally:
        lib.tagi_set_impl(capi.IMPL_AUTO)


def test_conv_ffma_path_forced(G, oracle):
    from cutagi_b200 import capi
    from cutagi_b200.capi import lib
    g = ConvGeom(B=4, fi=32, hi=16, wi=16, fo=64, k=3, stride=1, pad=1, pad_type=1, has_bias=1)
    lib.tagi_set_impl(capi.IMPL_FFMA)
    try:
        _run_all(G, oracle, g, G.conv_inputs(np.random.default_rng(2), g))
    finally:
        lib.tagi_set_impl(capi.IMPL_AUTO)


def test_conv_tensor_core_rejects_odd_channels(G):
    import torch
    from cutagi_b200 import capi
    from cutagi_b200.capi import ConvGeom as CG, TagiError, lib
    q = torch.zeros(1 << 16, device="cuda").data_ptr()
    g = CG(2, 3, 8, 8, 8, 8, 8, 3, 1, 1, 1, 0)   # fi = 3
    lib.tagi_set_impl(capi.IMPL_TF32X3)
    try:
        with pytest.raises(TagiError) as e:
            lib.tagi_conv2d_fwd(C.byref(g), q, q, q, q, q, q, q, q, None)
        assert e.value.code == 3
    finally:
        lib.tagi_set_impl(capi.IMPL_AUTO)
    lib.tagi_conv2d_fwd(C.byref(g), q, q, q, q, q, q, q, q, None)   # AUTO: FFMA kernels
    torch.cuda.synchronize()


@pytest.mark.parametrize("kw", TC_GEOMS[:6] + TC_GEOMS[12:], ids=lambda k: "fi{fi}_fo{fo}_h{hi}_k{k}_s{stride}".format(**k))
@pytest.mark.parametrize("impl", ["auto", "ffma"])
def test_conv_forward_with_fused_relu(G, kw, impl):
    """tagi_conv2d_fwd_relu = tagi_conv2d_fwd followed by the ReLU moments, bit for bit: in the epilogue of the CTA-pair
    kernel (256 or more output rows, implicit and explicit gathers) and as two steps elsewhere."""
    from cutagi_b200 import capi
    from cutagi_b200.capi import lib
    g = ConvGeom(**kw)
    x = G.conv_inputs(np.random.default_rng(g.fi * 7 + g.fo), g)
    lib.tagi_set_impl(capi.IMPL_FFMA if impl == "ffma" else capi.IMPL_AUTO)
    try:
        capi.tc_status()
        args = (g, x["mu_w"], x["var_w"], x["mu_b"], x["var_b"], x["mu_a"], x["var_a"])
        mz, vz = G.conv_fwd(*args)
        got = G.conv_fwd_relu(*args)
        assert capi.tc_status() == 0
    finally:
        lib.tagi_set_impl(capi.IMPL_AUTO)
    assert (mz < 0).any() and (mz > 0).any()
    for name, a, b in zip(("mu_a", "var_a", "jcb"), got, G.relu_of(mz, vz)):
        np.testing.assert_array_equal(a, b, err_msg=name)


@pytest.mark.parametrize("kw", [TC_GEOMS[0], TC_GEOMS[3], TC_GEOMS[5], TC_GEOMS[6], TC_GEOMS[13]],
                         ids=lambda k: "fi{fi}_fo{fo}_h{hi}_k{k}_s{stride}".format(**k))
@pytest.mark.parametrize("impl", ["auto", "ffma"])
def test_conv_state_pass_with_null_jacobian(G, kw, impl):
    """jcb = NULL stands for a Jacobian of ones: same bits as the pass given a tensor of ones (implicit and explicit
    gathers, the col2im pass of strided layers, the FFMA kernels)."""
    from cutagi_b200 import capi
    from cutagi_b200.capi import lib
    g = ConvGeom(**kw)
    x = G.conv_inputs(np.random.default_rng(g.fi * 3 + g.fo), g)
    ones = np.ones_like(x["jcb"])
    lib.tagi_set_impl(capi.IMPL_FFMA if impl == "ffma" else capi.IMPL_AUTO)
    try:
        ref = G.conv_bwd_state(g, x["mu_w"], ones, x["dmu_z"], x["dvar_z"])
        got = G.conv_bwd_state(g, x["mu_w"], None, x["dmu_z"], x["dvar_z"])
    finally:
        lib.tagi_set_impl(capi.IMPL_AUTO)
    for name, a, b in zip(("dmu_a", "dvar_a"), got, ref):
        np.testing.assert_array_equal(a, b, err_msg=name)


@pytest.mark.parametrize("kw", [TC_GEOMS[0], TC_GEOMS[3], TC_GEOMS[14], TC_GEOMS[6]],
                         ids=lambda k: "fi{fi}_fo{fo}_h{hi}_k{k}_s{stride}".format(**k))
def test_conv_forward_with_fused_mixture_relu(G, kw):
    """tagi_conv2d_fwd_act(TAGI_ACT_MIXTURE_RELU) against tagi_conv2d_fwd followed by tagi_mixture_relu_fwd."""
    from cutagi_b200 import capi
    g = ConvGeom(**kw)
    x = G.conv_inputs(np.random.default_rng(g.fi * 11 + g.fo), g)
    args = (g, x["mu_w"], x["var_w"], x["mu_b"], x["var_b"], x["mu_a"], x["var_a"])
    ref = G.mixture_relu(*G.conv_fwd(*args))
    got = G.conv_fwd_relu(*args, act=capi.ACT_MIXTURE_RELU)
    assert capi.tc_status() == 0
    for name, a, b, tol in zip(("mu_a", "var_a", "jcb"), got, ref, (G.RTOL_MU, G.RTOL_VAR, G.RTOL_MU)):
        G.check(name, a, b, tol)


# ------------------------------------------------------------------------------------------------------------------
# The layer shapes of the CIFAR-shaped CNN (batch 128) and of ResNet-18 (batch 64, 224 x 224) at full size
# ------------------------------------------------------------------------------------------------------------------
def _bench_layers():
    import os
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    if root not in sys.path:
        sys.path.insert(0, root)
    import bench
    return bench.CONV_LAYERS


@pytest.mark.parametrize("name,kw", _bench_layers(), ids=lambda v: v.replace(" ", "_") if isinstance(v, str) else "")
def test_configuration_layer_shapes_sampled(G, oracle, name, kw):
    """Every Conv2d layer shape of the CNN and ResNet-18 configurations at its full batch and image size: the planner
    picks other tile widths, slice counts and gather variants here than at the reduced sizes above. The GPU runs the
    whole layer; the CPU oracle runs a sample. Forward and state-pass outputs of an image depend on that image only
    (two images are checked); parameter deltas of an output channel depend on that channel's deltas only (three
    channels are checked, over the whole batch)."""
    from cutagi_b200 import capi
    g = ConvGeom(**kw)
    rng = np.random.default_rng(g.fi * 977 + g.fo * 13 + g.hi)
    x = G.conv_inputs(rng, g)
    imgs = np.sort(rng.choice(g.B, 2, replace=False))
    chans = np.sort(rng.choice(g.fo, 3, replace=False))
    gi = ConvGeom(**{**kw, "B": 2})
    sub = lambda a: np.ascontiguousarray(a[imgs])
    capi.tc_status()

    mz, vz = G.conv_fwd(g, x["mu_w"], x["var_w"], x["mu_b"], x["var_b"], x["mu_a"], x["var_a"])
    rmz, rvz = oracle.conv2d_fwd(gi, x["mu_w"], x["var_w"], x["mu_b"], x["var_b"], sub(x["mu_a"]), sub(x["var_a"]))
    G.check("mu_z", mz[imgs], rmz, G.RTOL_MU)
    G.check("var_z", vz[imgs], rvz, G.RTOL_VAR)
    assert vz.min() > 0
    del mz, vz

    da, dv = G.conv_bwd_state(g, x["mu_w"], x["jcb"], x["dmu_z"], x["dvar_z"])
    rda, rdv = oracle.conv2d_bwd_state(gi, x["mu_w"], sub(x["jcb"]), sub(x["dmu_z"]), sub(x["dvar_z"]))
    G.check("dmu_a", da[imgs], rda, G.RTOL_MU)
    G.check("dvar_a", dv[imgs], rdv, G.RTOL_VAR)
    assert dv.max() <= 0
    del da, dv

    dmw, dvw, dmb, dvb = G.conv_bwd_param(g, x["var_w"], x["var_b"], x["mu_a"], x["dmu_z"], x["dvar_z"])
    gc = ConvGeom(**{**kw, "fo": len(chans)})
    woho = g.ho * g.wo
    pick = lambda a: np.ascontiguousarray(a.reshape(g.B, g.fo, woho)[:, chans, :]).reshape(g.B, -1)
    args = (gc, np.ascontiguousarray(x["var_w"][chans]),
            None if x["var_b"] is None else np.ascontiguousarray(x["var_b"][chans]), x["mu_a"], pick(x["dmu_z"]),
            pick(x["dvar_z"]))
    r = oracle.conv2d_bwd_param(*args)
    r64 = oracle.conv2d_bwd_param(*args, f64=True)
    # The contraction of this pass runs over B * ho * wo terms (802 816 for the ResNet-18 stem). The reference sums them
    # one after the other in FP32, and that sum's own rounding error, measured here against the FP64 restatement,
    # reaches 3e-5 (means) / 5e-4 (variances, all terms of one sign) at these sizes: more than the tolerance. So the
    # GPU result must be within the tolerance of the exactly rounded result, and within the tolerance plus the
    # reference's own measured deviation of the reference.
    names = ("dmu_w", "dvar_w", "dmu_b", "dvar_b")
    got = (dmw[chans], dvw[chans], dmb[chans] if g.has_bias else None, dvb[chans] if g.has_bias else None)
    for i, tol in enumerate((G.RTOL_MU, G.RTOL_VAR, G.RTOL_MU, G.RTOL_VAR)):
        if got[i] is None:
            continue
        a, b32, b64 = (np.asarray(v, np.float64).reshape(got[i].shape) for v in (got[i], r[i], r64[i]))
        G.check(f"{names[i]} vs FP64", a, b64, tol)
        noise = np.abs(b32 - b64).max()
        err = np.abs(a - b32).max()
        assert err <= tol * np.abs(b32).max() + noise, \
            f"{names[i]}: max err {err:.3e} vs the FP32 reference, whose own deviation from FP64 is {noise:.3e}"
    assert dvw.max() <= 0
    assert capi.tc_status() == 0, "a bounded device-side wait ran out"


def test_reserved_scratch_covers_all_three_passes(G):
    """tagi_conv2d_workspace_bytes + tagi_reserve_scratch: once the library's scratch block has been sized for a layer,
    none of its passes makes the block grow or allocates device memory (free memory as the driver reports it stays the
    same), whichever kernels the planner picks. Layers of three kinds: patch kernels, gather through scratch (7 x 7 images), strided."""
    import torch
    from cutagi_b200.capi import lib
    P = lambda t: t.data_ptr()
    for kw in (dict(B=16, fi=64, hi=28, wi=28, fo=64, k=3, stride=1, pad=1, pad_type=1, has_bias=1),
               dict(B=32, fi=128, hi=7, wi=7, fo=256, k=3, stride=1, pad=1, pad_type=1, has_bias=0),
               dict(B=16, fi=32, hi=28, wi=28, fo=64, k=3, stride=2, pad=1, pad_type=2, has_bias=0)):
        g = ConvGeom(**kw)
        cg = G.cgeom(g)
        need = lib.tagi_conv2d_workspace_bytes(C.byref(cg))
        assert need > 0
        lib.tagi_reserve_scratch(need)
        t = lambda n: torch.rand(n, device="cuda") * 0.1 + 0.01
        n_in, n_out, nw = g.B * g.n_in, g.B * g.n_out, g.fo * g.Kc
        mw, vw, mb, vb, ma, va, j, dm, dv = t(nw), t(nw), t(g.fo), t(g.fo), t(n_in), t(n_in), t(n_in), t(n_out), t(n_out)
        mz, vz, da, dva, dw, dvw, db, dvb = t(n_out), t(n_out), t(n_in), t(n_in), t(nw), t(nw), t(g.fo), t(g.fo)
        cap0 = lib.tagi_scratch_bytes()
        assert cap0 >= need
        for attempt in range(2):   # the first round may load kernel code; the second must not change free memory at all
            torch.cuda.synchronize()
            free0, _ = torch.cuda.mem_get_info()
            lib.tagi_conv2d_fwd(C.byref(cg), P(mw), P(vw), P(mb), P(vb), P(ma), P(va), P(mz), P(vz), None)
            lib.tagi_conv2d_bwd_param(C.byref(cg), P(vw), P(vb), P(ma), P(dm), P(dv), P(dw), P(dvw), P(db), P(dvb), None)
            lib.tagi_conv2d_bwd_state(C.byref(cg), P(mw), P(j), P(dm), P(dv), P(da), P(dva), None)
            torch.cuda.synchronize()
            free1, _ = torch.cuda.mem_get_info()
            assert lib.tagi_scratch_bytes() == cap0, "the scratch block grew although it had been reserved"
        assert free1 == free0, (kw, free0 - free1)
