"""tagi_conv2d_bwd_param_noalloc: the parameter-delta pass for callers that may not allocate device memory.

Trainers that hand the whole GPU to their own pool at start-up, services with a fixed memory budget, and code that runs
while another thread captures a stream in the global mode cannot let a library call cudaMalloc. This entry point keeps its
split-contraction scratch in an array inside the library image instead. The test calls it through the C ABI twice in a
row (the second call finds the first call's leftovers in the shared array) and compares with tagi_conv2d_bwd_param on the
same inputs, within the tolerances every other GPU test uses (1e-5 on mean deltas, 1e-4 on variance deltas). The file is
collected last so that a run which stops at the first failure has already run every other test; it needs nothing from
them and also passes alone in a fresh process.
"""
import ctypes as C

import numpy as np
import pytest
from oracle_lib import ConvGeom

pytestmark = pytest.mark.gpu


def _call(entry, g, x):
    import torch
    import gpu_util as G
    d = [G.dev(x[k]) for k in ("var_w", "var_b", "mu_a", "dmu_z", "dvar_z")]
    ow, ov, obm, obv = G.Out(g.fo * g.Kc), G.Out(g.fo * g.Kc), G.Out(g.fo), G.Out(g.fo)
    cg = G.cgeom(g)
    entry(C.byref(cg), G.p(d[0]), G.p(d[1]), G.p(d[2]), G.p(d[3]), G.p(d[4]), ow.ptr(), ov.ptr(), obm.ptr(), obv.ptr(),
          None)
    torch.cuda.synchronize()
    return ow.get((g.fo, g.Kc)), ov.get((g.fo, g.Kc)), obm.get(), obv.get()


@pytest.mark.parametrize("kw", [
    # long contraction, small weight tensor: the contraction is cut into slices that go through the static scratch
    dict(B=16, fi=16, hi=28, wi=28, fo=32, k=3, stride=1, pad=1, pad_type=1, has_bias=1),
    # 147456 weights: fewer slices fit the static scratch than the allocating entry point would use
    dict(B=20, fi=128, hi=14, wi=14, fo=128, k=3, stride=1, pad=1, pad_type=1, has_bias=1),
])
def test_matches_allocating_entry_point_on_two_calls_in_a_row(kw):
    import gpu_util as G
    from cutagi_b200.capi import lib
    g = ConvGeom(**kw)
    x = G.conv_inputs(np.random.default_rng(5), g)
    ref = _call(lib.tagi_conv2d_bwd_param, g, x)
    for attempt in range(2):
        got = _call(lib.tagi_conv2d_bwd_param_noalloc, g, x)
        for name, a, b, tol in zip(("dmu_w", "dvar_w", "dmu_b", "dvar_b"), got, ref,
                                   (G.RTOL_MU, G.RTOL_VAR, G.RTOL_MU, G.RTOL_VAR)):
            G.check(f"{name} (call {attempt + 1})", a, b, tol)
    # a different layer right after: the array still holds the previous layer's partial sums
    g2 = ConvGeom(B=4, fi=8, hi=20, wi=20, fo=24, k=5, stride=1, pad=2, pad_type=1, has_bias=1)
    x2 = G.conv_inputs(np.random.default_rng(6), g2)
    for a, b, tol in zip(_call(lib.tagi_conv2d_bwd_param_noalloc, g2, x2), _call(lib.tagi_conv2d_bwd_param, g2, x2),
                         (G.RTOL_MU, G.RTOL_VAR, G.RTOL_MU, G.RTOL_VAR)):
        G.check("second layer", a, b, tol)


def test_rejects_layers_beyond_the_static_limit():
    import torch
    from cutagi_b200.capi import ConvGeom as CG, TagiError, lib
    q = torch.zeros(16, device="cuda").data_ptr()
    big = CG(1, 512, 7, 7, 512, 7, 7, 3, 1, 1, 1, 0)   # 512 * 512 * 9 = 2359296 weights > 1048576
    with pytest.raises(TagiError) as e:
        lib.tagi_conv2d_bwd_param_noalloc(C.byref(big), q, q, q, q, q, q, q, q, q, None)
    assert e.value.code == 3 and "exceeds the limit" in str(e.value)
