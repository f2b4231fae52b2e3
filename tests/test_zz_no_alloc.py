"""tagi_conv2d_bwd_param_noalloc: the parameter-delta pass for callers that may not allocate device memory.

Trainers that hand the whole GPU to their own pool at start-up, services with a fixed memory budget, and code that runs
while another thread captures a stream in the global mode cannot let a library call cudaMalloc. This entry point keeps its
split-contraction scratch in an array inside the library image instead. The test calls it through the C ABI twice in a
row (the second call finds the first call's leftovers in the shared array) and compares with tagi_conv2d_bwd_param on the
same inputs and with the CPU oracle, within the tolerances every other GPU test uses (1e-5 on mean deltas, 1e-4 on
variance deltas), and checks the property the entry point exists for: after the first call on a device (which loads the
library's device code and looks the array up) further calls leave the device's free memory unchanged. The file is
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
def test_matches_allocating_entry_point_on_two_calls_in_a_row(kw, oracle):
    import gpu_util as G
    from cutagi_b200.capi import lib
    g = ConvGeom(**kw)
    x = G.conv_inputs(np.random.default_rng(5), g)
    ref = _call(lib.tagi_conv2d_bwd_param, g, x)
    cpu = oracle.conv2d_bwd_param(g, x["var_w"], x["var_b"], x["mu_a"], x["dmu_z"], x["dvar_z"])
    for attempt in range(2):
        got = _call(lib.tagi_conv2d_bwd_param_noalloc, g, x)
        for name, a, b, c, tol in zip(("dmu_w", "dvar_w", "dmu_b", "dvar_b"), got, ref, cpu,
                                      (G.RTOL_MU, G.RTOL_VAR, G.RTOL_MU, G.RTOL_VAR)):
            G.check(f"{name} (call {attempt + 1})", a, b, tol)
            G.check(f"{name} vs the CPU oracle (call {attempt + 1})", a, np.asarray(c).reshape(a.shape), tol)
    # a different layer right after: the array still holds the previous layer's partial sums
    g2 = ConvGeom(B=4, fi=8, hi=20, wi=20, fo=24, k=5, stride=1, pad=2, pad_type=1, has_bias=1)
    x2 = G.conv_inputs(np.random.default_rng(6), g2)
    for a, b, tol in zip(_call(lib.tagi_conv2d_bwd_param_noalloc, g2, x2), _call(lib.tagi_conv2d_bwd_param, g2, x2),
                         (G.RTOL_MU, G.RTOL_VAR, G.RTOL_MU, G.RTOL_VAR)):
        G.check("second layer", a, b, tol)


def test_calls_after_the_first_leave_free_device_memory_unchanged():
    """What the entry point is for: once the first call on the device has been made, a call takes no device memory.
    Inputs and outputs are allocated before the measurement; free memory as the driver reports it (cudaMemGetInfo) is
    the same before and after two further calls on different layer shapes."""
    import torch
    import gpu_util as G
    from cutagi_b200.capi import lib
    shapes = [dict(B=16, fi=16, hi=28, wi=28, fo=32, k=3, stride=1, pad=1, pad_type=1, has_bias=1),
              dict(B=8, fi=64, hi=14, wi=14, fo=64, k=3, stride=1, pad=1, pad_type=1, has_bias=0)]
    calls = []
    for kw in shapes:
        g = ConvGeom(**kw)
        x = G.conv_inputs(np.random.default_rng(9), g)
        d = [G.dev(x[k]) for k in ("var_w", "var_b", "mu_a", "dmu_z", "dvar_z")]
        out = [torch.empty(g.fo * g.Kc, device="cuda"), torch.empty(g.fo * g.Kc, device="cuda"),
               torch.empty(g.fo, device="cuda"), torch.empty(g.fo, device="cuda")]
        calls.append((G.cgeom(g), d, out))

    def run(i):
        cg, d, out = calls[i]
        lib.tagi_conv2d_bwd_param_noalloc(C.byref(cg), G.p(d[0]), G.p(d[1]), G.p(d[2]), G.p(d[3]), G.p(d[4]),
                                          out[0].data_ptr(), out[1].data_ptr(), out[2].data_ptr(), out[3].data_ptr(), None)
        torch.cuda.synchronize()
    run(0)                                   # first call on the device: module load + symbol look-up
    run(1)
    free0, _ = torch.cuda.mem_get_info()
    run(0)
    run(1)
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0, f"device memory changed by {free0 - free1} bytes across calls of the no-allocation entry point"


def test_rejects_layers_beyond_the_static_limit():
    import torch
    from cutagi_b200.capi import ConvGeom as CG, TagiError, lib
    q = torch.zeros(16, device="cuda").data_ptr()
    big = CG(1, 512, 7, 7, 512, 7, 7, 3, 1, 1, 1, 0)   # 512 * 512 * 9 = 2359296 weights > 1048576
    with pytest.raises(TagiError) as e:
        lib.tagi_conv2d_bwd_param_noalloc(C.byref(big), q, q, q, q, q, q, q, q, q, None)
    assert e.value.code == 3 and "exceeds the limit" in str(e.value)
