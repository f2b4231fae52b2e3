"""GPU parity of the Linear entry points (through the C ABI) against the CPU oracle and the golden fixtures."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def G():
    import gpu_util
    return gpu_util


def _run_all(G, oracle, x, misalign=0, tag=""):
    mz, vz = G.linear_fwd(x["mu_w"], x["var_w"], x["mu_b"], x["var_b"], x["mu_a"], x["var_a"], misalign)
    rmz, rvz = oracle.linear_fwd(x["mu_w"], x["var_w"], x["mu_b"], x["var_b"], x["mu_a"], x["var_a"])
    G.check(tag + "mu_z", mz, rmz, G.RTOL_MU)
    G.check(tag + "var_z", vz, rvz, G.RTOL_VAR)
    da, dv = G.linear_bwd_state(x["mu_w"], x["jcb"], x["dmu_z"], x["dvar_z"], misalign)
    rda, rdv = oracle.linear_bwd_state(x["mu_w"], x["jcb"], x["dmu_z"], x["dvar_z"])
    G.check(tag + "dmu_a", da, rda, G.RTOL_MU)
    G.check(tag + "dvar_a", dv, rdv, G.RTOL_VAR)
    dmw, dvw, dmb, dvb = G.linear_bwd_param(x["var_w"], x["var_b"], x["mu_a"], x["dmu_z"], x["dvar_z"], misalign)
    r = oracle.linear_bwd_param(x["var_w"], x["var_b"], x["mu_a"], x["dmu_z"], x["dvar_z"])
    G.check(tag + "dmu_w", dmw, r[0], G.RTOL_MU)
    G.check(tag + "dvar_w", dvw, r[1], G.RTOL_VAR)
    if x["var_b"] is not None:
        G.check(tag + "dmu_b", dmb, r[2], G.RTOL_MU)
        G.check(tag + "dvar_b", dvb, r[3], G.RTOL_VAR)


@pytest.mark.parametrize("i", range(8))
def test_golden_cases(G, golden, i):
    p = f"lin{i}_"
    g = {k[len(p):]: np.ascontiguousarray(golden[k]) for k in golden.files if k.startswith(p)}
    mz, vz = G.linear_fwd(g["mu_w"], g["var_w"], g.get("mu_b"), g.get("var_b"), g["mu_a"], g["var_a"])
    G.check("mu_z", mz, g["mu_z"], G.RTOL_MU)
    G.check("var_z", vz, g["var_z"], G.RTOL_VAR)
    da, dv = G.linear_bwd_state(g["mu_w"], g["jcb"], g["dmu_z"], g["dvar_z"])
    G.check("dmu_a", da, g["dmu_a"], G.RTOL_MU)
    G.check("dvar_a", dv, g["dvar_a"], G.RTOL_VAR)
    dmw, dvw, dmb, dvb = G.linear_bwd_param(g["var_w"], g.get("var_b"), g["mu_a"], g["dmu_z"], g["dvar_z"])
    G.check("dmu_w", dmw, g["dmu_w"], G.RTOL_MU)
    G.check("dvar_w", dvw, g["dvar_w"], G.RTOL_VAR)
    if "var_b" in g:
        G.check("dmu_b", dmb, g["dmu_b"], G.RTOL_MU)
        G.check("dvar_b", dvb, g["dvar_b"], G.RTOL_VAR)


# every tile-edge residue of the 64- and 128-wide tiles, vector and scalar load paths, with and without bias
EDGE = [(1, 1, 1), (3, 5, 11), (4, 4, 4), (5, 3, 1), (11, 63, 65), (63, 64, 127), (64, 65, 128), (65, 127, 129),
        (127, 128, 64), (128, 129, 63), (129, 11, 5), (32, 784, 128), (32, 128, 11), (16, 785, 6), (130, 260, 132),
        (256, 8, 256), (7, 1, 300), (300, 300, 1)]


@pytest.mark.parametrize("B,K,N", EDGE)
@pytest.mark.parametrize("bias", [True, False])
def test_edge_shapes(G, oracle, B, K, N, bias):
    rng = np.random.default_rng(B * 1000003 + K * 1009 + N)
    _run_all(G, oracle, G.linear_inputs(rng, B, K, N, bias))


@pytest.mark.parametrize("B,K,N", [(8, 64, 64), (33, 128, 96), (130, 256, 132)])
def test_misaligned_pointers(G, oracle, B, K, N):
    """Buffers that start 4 bytes past a 16-byte boundary must take the scalar paths and still be exact."""
    rng = np.random.default_rng(99 + B)
    _run_all(G, oracle, G.linear_inputs(rng, B, K, N), misalign=1)


@pytest.mark.parametrize("B,K,N", [(256, 1024, 1024), (1024, 512, 1536), (2048, 256, 1280)])
def test_large_tile_path(G, oracle, B, K, N):
    rng = np.random.default_rng(5 + B)
    _run_all(G, oracle, G.linear_inputs(rng, B, K, N))


def test_benchmark_shape_sampled(G, oracle):
    """B=1024, 4096 -> 4096: the CPU oracle on this shape takes minutes, so rows are sampled. Forward and state
    backward outputs of a batch row depend on that row only; parameter deltas of an output feature depend on that
    feature's delta column only."""
    rng = np.random.default_rng(2024)
    B, K, N = 1024, 4096, 4096
    x = G.linear_inputs(rng, B, K, N)
    rows = np.sort(rng.choice(B, 6, replace=False))
    feats = np.sort(rng.choice(N, 6, replace=False))
    mz, vz = G.linear_fwd(x["mu_w"], x["var_w"], x["mu_b"], x["var_b"], x["mu_a"], x["var_a"])
    rmz, rvz = oracle.linear_fwd(x["mu_w"], x["var_w"], x["mu_b"], x["var_b"],
                                 np.ascontiguousarray(x["mu_a"][rows]), np.ascontiguousarray(x["var_a"][rows]))
    G.check("mu_z", mz[rows], rmz, G.RTOL_MU)
    G.check("var_z", vz[rows], rvz, G.RTOL_VAR)
    da, dv = G.linear_bwd_state(x["mu_w"], x["jcb"], x["dmu_z"], x["dvar_z"])
    rda, rdv = oracle.linear_bwd_state(x["mu_w"], np.ascontiguousarray(x["jcb"][rows]),
                                       np.ascontiguousarray(x["dmu_z"][rows]), np.ascontiguousarray(x["dvar_z"][rows]))
    G.check("dmu_a", da[rows], rda, G.RTOL_MU)
    G.check("dvar_a", dv[rows], rdv, G.RTOL_VAR)
    dmw, dvw, dmb, dvb = G.linear_bwd_param(x["var_w"], x["var_b"], x["mu_a"], x["dmu_z"], x["dvar_z"])
    r = oracle.linear_bwd_param(np.ascontiguousarray(x["var_w"][feats]), np.ascontiguousarray(x["var_b"][feats]),
                                x["mu_a"], np.ascontiguousarray(x["dmu_z"][:, feats]),
                                np.ascontiguousarray(x["dvar_z"][:, feats]))
    G.check("dmu_w", dmw[feats], r[0], G.RTOL_MU)
    G.check("dvar_w", dvw[feats], r[1], G.RTOL_VAR)
    G.check("dmu_b", dmb[feats], r[2], G.RTOL_MU)
    G.check("dvar_b", dvb[feats], r[3], G.RTOL_VAR)
    # size-independent properties: variances are positive, variance deltas non-positive
    assert vz.min() > 0 and dv.max() <= 0 and dvw.max() <= 0


def test_forward_closer_to_exact_than_tolerance(G, oracle):
    """Arbitration against FP64: the GPU result is within the stated tolerance of the exactly-rounded value too."""
    rng = np.random.default_rng(11)
    x = G.linear_inputs(rng, 64, 2048, 192)
    mz, vz = G.linear_fwd(x["mu_w"], x["var_w"], x["mu_b"], x["var_b"], x["mu_a"], x["var_a"])
    m64, v64 = oracle.linear_fwd(x["mu_w"], x["var_w"], x["mu_b"], x["var_b"], x["mu_a"], x["var_a"], f64=True)
    G.check("mu_z vs f64", mz, m64, G.RTOL_MU)
    G.check("var_z vs f64", vz, v64, G.RTOL_VAR)


def test_error_statuses(G):
    import torch
    from cutagi_b200.capi import TagiError, lib
    t = torch.zeros(64, device="cuda")
    q = t.data_ptr()
    with pytest.raises(TagiError) as e:
        lib.tagi_linear_fwd(q, q, q, q, q, q, 0, 4, 4, 1, q, q, None)
    assert e.value.code == 1 and "positive" in str(e.value)
    with pytest.raises(TagiError) as e:
        lib.tagi_linear_fwd(None, q, q, q, q, q, 2, 4, 4, 1, q, q, None)
    assert e.value.code == 1 and "mu_w" in str(e.value)
    with pytest.raises(TagiError):
        lib.tagi_linear_bwd_param(q, None, q, q, q, 2, 4, 4, 1, q, q, q, q, None)
    # a failed call leaves the context usable
    lib.tagi_linear_fwd(q, q, q, q, q, q, 2, 4, 4, 1, q, q, None)
    torch.cuda.synchronize()


def test_deterministic(G):
    rng = np.random.default_rng(3)
    x = G.linear_inputs(rng, 96, 320, 200)
    a = G.linear_bwd_param(x["var_w"], x["var_b"], x["mu_a"], x["dmu_z"], x["dvar_z"])
    b = G.linear_bwd_param(x["var_w"], x["var_b"], x["mu_a"], x["dmu_z"], x["dvar_z"])
    for u, v in zip(a, b):
        assert np.array_equal(u, v)


# ------------------------------------------------------------------------------------------------------------------
# The same parity bar for each implementation explicitly (FFMA on the CUDA cores, 3xTF32 on the tensor cores)
# ------------------------------------------------------------------------------------------------------------------
@pytest.fixture
def force_impl():
    from cutagi_b200.capi import lib
    yield lambda i: lib.tagi_set_impl(i)
    lib.tagi_set_impl(0)


TC_SHAPES = [(128, 64, 128), (4, 8, 12), (132, 200, 260), (256, 256, 384), (512, 2048, 512), (384, 1024, 640),
             (260, 516, 132), (64, 4096, 128)]


@pytest.mark.parametrize("B,K,N", TC_SHAPES)
def test_tensor_core_path(G, oracle, force_impl, B, K, N):
    """TF32X3 forced: every shape with 16-byte aligned rows runs on tcgen05, including ragged tile edges."""
    from cutagi_b200 import capi
    force_impl(capi.IMPL_TF32X3)
    capi.tc_status()
    rng = np.random.default_rng(B * 7 + K * 3 + N)
    _run_all(G, oracle, G.linear_inputs(rng, B, K, N), tag="tc ")
    assert capi.tc_status() == 0, "a bounded device-side wait ran out"


@pytest.mark.parametrize("B,K,N", [(512, 2048, 512), (130, 260, 132)])
def test_ffma_path(G, oracle, force_impl, B, K, N):
    from cutagi_b200 import capi
    force_impl(capi.IMPL_FFMA)
    rng = np.random.default_rng(B + K + N)
    _run_all(G, oracle, G.linear_inputs(rng, B, K, N), tag="ffma ")


PAIR_SHAPES = [(256, 64, 128), (260, 200, 260), (512, 2048, 512), (300, 516, 1000), (1024, 256, 112), (256, 4096, 256)]


@pytest.mark.parametrize("B,K,N", PAIR_SHAPES)
def test_tensor_core_cta_pair_variant(G, oracle, force_impl, B, K, N):
    """tagi_tc_set_variant(3): the same kernels on CTA pairs (tcgen05 cta_group::2, 256-row tiles, each CTA staging
    half of the B rows). Passes that have fewer than 256 output rows fall back to the one-CTA kernel."""
    from cutagi_b200 import capi
    from cutagi_b200.capi import lib
    force_impl(capi.IMPL_TF32X3)
    lib.tagi_tc_set_variant(3)
    try:
        capi.tc_status()
        rng = np.random.default_rng(B * 5 + K * 3 + N)
        _run_all(G, oracle, G.linear_inputs(rng, B, K, N), tag="pair ")
        assert capi.tc_status() == 0, "a bounded device-side wait ran out"
    finally:
        lib.tagi_tc_set_variant(3)


@pytest.mark.parametrize("variant", [1])
def test_tensor_core_one_cta_variants(G, oracle, force_impl, variant):
    """The one-CTA kernel at shapes where the default would use CTA pairs."""
    from cutagi_b200 import capi
    from cutagi_b200.capi import lib
    force_impl(capi.IMPL_TF32X3)
    lib.tagi_tc_set_variant(variant)
    try:
        rng = np.random.default_rng(21)
        _run_all(G, oracle, G.linear_inputs(rng, 260, 516, 132), tag="one-cta ")
        _run_all(G, oracle, G.linear_inputs(rng, 512, 1024, 384), tag="one-cta ")
        assert capi.tc_status() == 0
    finally:
        lib.tagi_tc_set_variant(3)


@pytest.mark.parametrize("sms", [132, 64])
def test_tensor_core_sm_budget_only_changes_the_tiling(G, oracle, force_impl, sms):
    """tagi_tc_set_sm_budget: tiles planned for fewer SMs (the exchange's kernels hold the rest); same results."""
    from cutagi_b200 import capi
    from cutagi_b200.capi import lib
    force_impl(capi.IMPL_TF32X3)
    lib.tagi_tc_set_sm_budget(sms)
    try:
        rng = np.random.default_rng(23)
        _run_all(G, oracle, G.linear_inputs(rng, 512, 1024, 1536), tag=f"budget {sms} ")
        assert capi.tc_status() == 0
        with pytest.raises(capi.TagiError):
            lib.tagi_tc_set_sm_budget(1)
    finally:
        lib.tagi_tc_set_sm_budget(0)


@pytest.mark.parametrize("B,K,N,cuts", [(256, 512, 768, (0, 256, 512, 768)), (64, 100, 37, (0, 5, 36, 37)),
                                         (128, 256, 384, (0, 128, 384))])
def test_parameter_pass_by_row_ranges(G, oracle, B, K, N, cuts):
    """tagi_linear_bwd_param_rows over a partition of the output features gives the whole pass (tensor-core ranges where
    aligned, FFMA otherwise); rows outside a range are left alone."""
    import torch
    from cutagi_b200.capi import lib
    x = G.linear_inputs(np.random.default_rng(B + N), B, K, N)
    ref = oracle.linear_bwd_param(x["var_w"], x["var_b"], x["mu_a"], x["dmu_z"], x["dvar_z"])
    d = {k: G.dev(x[k]) for k in ("var_w", "var_b", "mu_a", "dmu_z", "dvar_z")}
    ow, ov, obm, obv = G.Out(N * K), G.Out(N * K), G.Out(N), G.Out(N)
    for n0, n1 in zip(cuts[:-1], cuts[1:]):
        lib.tagi_linear_bwd_param_rows(G.p(d["var_w"]), G.p(d["var_b"]), G.p(d["mu_a"]), G.p(d["dmu_z"]), G.p(d["dvar_z"]),
                                       B, K, N, n0, n1, 1, ow.ptr(), ov.ptr(), obm.ptr(), obv.ptr(), None)
    G.check("dmu_w", ow.get((N, K)), ref[0], G.RTOL_MU)
    G.check("dvar_w", ov.get((N, K)), ref[1], G.RTOL_VAR)
    G.check("dmu_b", obm.get(), ref[2], G.RTOL_MU)
    G.check("dvar_b", obv.get(), ref[3], G.RTOL_VAR)
    # a single range leaves the other rows untouched
    keep = torch.full((N * K,), 7.0, device="cuda")
    keep2, kb, kb2 = keep.clone(), torch.full((N,), 7.0, device="cuda"), torch.full((N,), 7.0, device="cuda")
    lib.tagi_linear_bwd_param_rows(G.p(d["var_w"]), G.p(d["var_b"]), G.p(d["mu_a"]), G.p(d["dmu_z"]), G.p(d["dvar_z"]), B, K,
                                   N, cuts[1], cuts[2], 1, G.p(keep), G.p(keep2), G.p(kb), G.p(kb2), None)
    h = keep.cpu().numpy().reshape(N, K)
    assert np.all(h[: cuts[1]] == 7.0) and np.all(h[cuts[2]:] == 7.0) and not np.any(h[cuts[1]:cuts[2]] == 7.0)
    hb = kb.cpu().numpy()
    assert np.all(hb[: cuts[1]] == 7.0) and np.all(hb[cuts[2]:] == 7.0)


def test_tensor_core_rejects_unaligned(G, force_impl):
    import torch
    from cutagi_b200 import capi
    from cutagi_b200.capi import TagiError, lib
    force_impl(capi.IMPL_TF32X3)
    q = torch.zeros(1 << 16, device="cuda").data_ptr()
    with pytest.raises(TagiError) as e:
        lib.tagi_linear_fwd(q, q, q, q, q, q, 8, 6, 8, 1, q, q, None)   # K not a multiple of 4
    assert e.value.code == 3
    with pytest.raises(TagiError):
        lib.tagi_linear_fwd(q + 4, q, q, q, q, q, 8, 8, 8, 1, q, q, None)   # misaligned pointer
    force_impl(capi.IMPL_AUTO)
    lib.tagi_linear_fwd(q, q, q, q, q, q, 8, 6, 8, 1, q, q, None)   # AUTO falls back to FFMA
    torch.cuda.synchronize()


def test_tensor_core_constant_variance_weights(G, oracle, force_impl):
    """TAGI's initialisation gives every weight the same variance (1 / fan_in): operand rounding errors do not
    average out for such inputs, which is what a single-TF32 product would fail on."""
    from cutagi_b200 import capi
    force_impl(capi.IMPL_TF32X3)
    rng = np.random.default_rng(42)
    B, K, N = 256, 1536, 256
    x = G.linear_inputs(rng, B, K, N)
    x["var_w"] = np.full((N, K), 1.0 / K, np.float32)
    x["var_a"] = np.full((B, K), 0.0123, np.float32)
    x["mu_a"] = np.abs(x["mu_a"])
    _run_all(G, oracle, x, tag="tc const ")
    assert capi.tc_status() == 0


def test_benchmark_shape_is_tensor_core_and_in_tolerance_vs_f64(G, oracle, force_impl):
    from cutagi_b200 import capi
    force_impl(capi.IMPL_TF32X3)
    rng = np.random.default_rng(77)
    B, K, N = 1024, 4096, 4096
    x = G.linear_inputs(rng, B, K, N)
    rows = np.sort(rng.choice(B, 4, replace=False))
    mz, vz = G.linear_fwd(x["mu_w"], x["var_w"], x["mu_b"], x["var_b"], x["mu_a"], x["var_a"])
    m64, v64 = oracle.linear_fwd(x["mu_w"], x["var_w"], x["mu_b"], x["var_b"],
                                 np.ascontiguousarray(x["mu_a"][rows]), np.ascontiguousarray(x["var_a"][rows]), f64=True)
    G.check("mu_z vs f64", mz[rows], m64, G.RTOL_MU)
    G.check("var_z vs f64", vz[rows], v64, G.RTOL_VAR)
    assert capi.tc_status() == 0


@pytest.mark.parametrize("B,K,N", [(256, 1024, 1024), (1024, 512, 1536), (300, 260, 132), (130, 256, 132), (32, 784, 128),
                                   (3, 5, 11)])
@pytest.mark.parametrize("bias", [True, False])
def test_forward_with_fused_relu(G, B, K, N, bias):
    """tagi_linear_fwd_relu = tagi_linear_fwd followed by the ReLU moments, bit for bit: in the epilogue of the CTA-pair
    kernel (256 or more rows) and as two steps on the other kernels."""
    from cutagi_b200 import capi
    x = G.linear_inputs(np.random.default_rng(B + K + N), B, K, N, bias)
    capi.tc_status()
    args = (x["mu_w"], x["var_w"], x["mu_b"], x["var_b"], x["mu_a"], x["var_a"])
    mz, vz = G.linear_fwd(*args)
    got = G.linear_fwd_relu(*args)
    assert capi.tc_status() == 0
    assert (mz < 0).any() and (mz > 0).any()
    for name, a, b in zip(("mu_a", "var_a", "jcb"), got, G.relu_of(mz, vz)):
        np.testing.assert_array_equal(a, b, err_msg=name)


def test_fused_relu_rejects_null_jacobian(G):
    import torch
    from cutagi_b200.capi import TagiError, lib
    q = torch.zeros(1 << 12, device="cuda").data_ptr()
    with pytest.raises(TagiError):
        lib.tagi_linear_fwd_relu(q, q, q, q, q, q, 4, 8, 8, 1, q, q, None, None)


@pytest.mark.parametrize("B,K,N,impl", [(256, 1024, 512, "auto"), (300, 260, 132, "tc"), (130, 256, 132, "auto"),
                                        (33, 65, 17, "auto"), (512, 256, 384, "ffma")])
def test_state_pass_with_null_jacobian(G, force_impl, B, K, N, impl):
    """jcb = NULL stands for a Jacobian of ones: same bits as the pass given a tensor of ones, on every kernel."""
    from cutagi_b200 import capi
    if impl != "auto":
        force_impl(capi.IMPL_TF32X3 if impl == "tc" else capi.IMPL_FFMA)
    x = G.linear_inputs(np.random.default_rng(B + N), B, K, N)
    ones = np.ones((B, K), np.float32)
    ref = G.linear_bwd_state(x["mu_w"], ones, x["dmu_z"], x["dvar_z"])
    got = G.linear_bwd_state(x["mu_w"], None, x["dmu_z"], x["dvar_z"])
    for name, a, b in zip(("dmu_a", "dvar_a"), got, ref):
        np.testing.assert_array_equal(a, b, err_msg=name)


@pytest.mark.parametrize("B,K,N", [(256, 1024, 1024), (300, 260, 132), (130, 256, 132), (3, 5, 11)])
def test_forward_with_fused_mixture_relu(G, B, K, N):
    """tagi_linear_fwd_act(TAGI_ACT_MIXTURE_RELU) against tagi_linear_fwd followed by tagi_mixture_relu_fwd, and with
    TAGI_ACT_RELU bit for bit against tagi_linear_fwd_relu; unknown activation ids are refused."""
    from cutagi_b200 import capi
    x = G.linear_inputs(np.random.default_rng(B + K + N + 1), B, K, N, True)
    args = (x["mu_w"], x["var_w"], x["mu_b"], x["var_b"], x["mu_a"], x["var_a"])
    ref = G.mixture_relu(*G.linear_fwd(*args))
    got = G.linear_fwd_relu(*args, act=capi.ACT_MIXTURE_RELU)
    for name, a, b, tol in zip(("mu_a", "var_a", "jcb"), got, ref, (G.RTOL_MU, G.RTOL_VAR, G.RTOL_MU)):
        G.check(name, a, b, tol)
    for a, b in zip(G.linear_fwd_relu(*args, act=capi.ACT_RELU), G.linear_fwd_relu(*args)):
        np.testing.assert_array_equal(a, b)
    with pytest.raises(capi.TagiError):
        G.linear_fwd_relu(*args, act=7)
