"""Helpers for the GPU parity tests: device buffers with guard bands, calls through the C ABI, tolerances.

Tolerance (stated by the task for this path): per output tensor
    max|x - ref| <= RTOL_MU  * max|ref|   for means / mean deltas      (1e-5)
    max|x - ref| <= RTOL_VAR * max|ref|   for variances / var deltas   (1e-4)
`ref` is the CPU oracle (bit-identical to the reference's CPU classes on the pinned cases).
"""
import ctypes as C

import numpy as np
import torch

from cutagi_b200 import capi
from cutagi_b200.capi import lib

RTOL_MU = 1e-5
RTOL_VAR = 1e-4
GUARD = 64
SENTINEL = -777.25


def dev(a, misalign=0):
    """numpy float32 -> CUDA tensor; `misalign` floats of offset from the 256-byte allocation boundary."""
    if a is None:
        return None
    t = torch.empty(a.size + misalign, dtype=torch.float32, device="cuda")
    v = t[misalign:]
    v.copy_(torch.from_numpy(np.ascontiguousarray(a).reshape(-1)))
    return v


class Out:
    """Output buffer of n floats with sentinel guard bands on both sides."""

    def __init__(self, n, misalign=0):
        self.n = n
        self.buf = torch.full((n + 2 * GUARD + misalign,), SENTINEL, dtype=torch.float32, device="cuda")
        self.view = self.buf[GUARD + misalign: GUARD + misalign + n]
        self.lo = GUARD + misalign

    def ptr(self):
        return self.view.data_ptr()

    def get(self, shape=None):
        torch.cuda.synchronize()
        h = self.buf.cpu().numpy()
        assert np.all(h[: self.lo] == SENTINEL) and np.all(h[self.lo + self.n:] == SENTINEL), "guard band overwritten"
        out = h[self.lo: self.lo + self.n].copy()
        assert not np.any(out == SENTINEL), "output not fully written"
        return out.reshape(shape) if shape is not None else out


def p(t):
    return None if t is None else t.data_ptr()


def check(name, got, ref, rtol):
    ref = np.asarray(ref, dtype=np.float64)
    got = np.asarray(got, dtype=np.float64)
    assert got.shape == ref.shape, (name, got.shape, ref.shape)
    assert np.all(np.isfinite(got)), f"{name}: non-finite values"
    scale = np.abs(ref).max()
    err = np.abs(got - ref).max()
    assert err <= rtol * scale + 1e-37, f"{name}: max err {err:.3e} > {rtol:g} * max|ref| {scale:.3e}"
    return err / max(scale, 1e-300)


def linear_fwd(mw, vw, mb, vb, ma, va, misalign=0):
    B, K = ma.shape
    N = mw.shape[0]
    d = [dev(x, misalign) for x in (mw, vw, mb, vb, ma, va)]
    mz, vz = Out(B * N, misalign), Out(B * N, misalign)
    lib.tagi_linear_fwd(p(d[0]), p(d[1]), p(d[2]), p(d[3]), p(d[4]), p(d[5]), B, K, N, int(mb is not None),
                        mz.ptr(), vz.ptr(), None)
    return mz.get((B, N)), vz.get((B, N))


def linear_fwd_relu(mw, vw, mb, vb, ma, va, misalign=0, act=None):
    """act None: tagi_linear_fwd_relu; else tagi_linear_fwd_act with that activation id."""
    B, K = ma.shape
    N = mw.shape[0]
    d = [dev(x, misalign) for x in (mw, vw, mb, vb, ma, va)]
    o = [Out(B * N, misalign) for _ in range(3)]
    if act is None:
        lib.tagi_linear_fwd_relu(p(d[0]), p(d[1]), p(d[2]), p(d[3]), p(d[4]), p(d[5]), B, K, N, int(mb is not None),
                                 o[0].ptr(), o[1].ptr(), o[2].ptr(), None)
    else:
        lib.tagi_linear_fwd_act(p(d[0]), p(d[1]), p(d[2]), p(d[3]), p(d[4]), p(d[5]), B, K, N, int(mb is not None), act,
                                o[0].ptr(), o[1].ptr(), o[2].ptr(), None)
    return tuple(x.get((B, N)) for x in o)


def mixture_relu(mz, vz):
    """tagi_mixture_relu_fwd on forward outputs."""
    d = [dev(x) for x in (mz, vz)]
    o = [Out(mz.size) for _ in range(3)]
    lib.tagi_mixture_relu_fwd(p(d[0]), p(d[1]), mz.size, o[0].ptr(), o[1].ptr(), o[2].ptr(), None)
    return tuple(x.get(mz.shape) for x in o)


def relu_of(mz, vz):
    """The ReLU moments (src/activation.cpp:7-29) of forward outputs, on the host."""
    ma = np.maximum(mz, np.float32(0))
    off = ma == 0
    return ma, np.where(off, np.float32(0), vz), np.where(off, np.float32(0), np.float32(1))


def linear_bwd_state(mw, jcb, dm, dv, misalign=0):
    """jcb None: the NULL Jacobian (ones)."""
    B = dm.shape[0]
    N, K = mw.shape
    d = [dev(x, misalign) for x in (mw, jcb, dm, dv)]
    oa, ob = Out(B * K, misalign), Out(B * K, misalign)
    lib.tagi_linear_bwd_state(p(d[0]), p(d[1]), p(d[2]), p(d[3]), B, K, N, oa.ptr(), ob.ptr(), None)
    return oa.get((B, K)), ob.get((B, K))


def linear_bwd_param(vw, vb, ma, dm, dv, misalign=0):
    B, K = ma.shape
    N = vw.shape[0]
    d = [dev(x, misalign) for x in (vw, vb, ma, dm, dv)]
    ow, ov, obm, obv = Out(N * K, misalign), Out(N * K, misalign), Out(N, misalign), Out(N, misalign)
    lib.tagi_linear_bwd_param(p(d[0]), p(d[1]), p(d[2]), p(d[3]), p(d[4]), B, K, N, int(vb is not None),
                              ow.ptr(), ov.ptr(), obm.ptr(), obv.ptr(), None)
    if vb is None:
        torch.cuda.synchronize()
        return ow.get((N, K)), ov.get((N, K)), None, None
    return ow.get((N, K)), ov.get((N, K)), obm.get(), obv.get()


def cgeom(g):
    return capi.ConvGeom(g.B, g.fi, g.hi, g.wi, g.fo, g.ho, g.wo, g.k, g.stride, g.pad, g.pad_type, g.has_bias)


def conv_fwd(g, mw, vw, mb, vb, ma, va):
    d = [dev(x) for x in (mw, vw, mb, vb, ma, va)]
    mz, vz = Out(g.B * g.n_out), Out(g.B * g.n_out)
    cg = cgeom(g)
    lib.tagi_conv2d_fwd(C.byref(cg), p(d[0]), p(d[1]), p(d[2]), p(d[3]), p(d[4]), p(d[5]), mz.ptr(), vz.ptr(), None)
    return mz.get((g.B, g.n_out)), vz.get((g.B, g.n_out))


def conv_fwd_relu(g, mw, vw, mb, vb, ma, va, act=None):
    d = [dev(x) for x in (mw, vw, mb, vb, ma, va)]
    o = [Out(g.B * g.n_out) for _ in range(3)]
    cg = cgeom(g)
    if act is None:
        lib.tagi_conv2d_fwd_relu(C.byref(cg), p(d[0]), p(d[1]), p(d[2]), p(d[3]), p(d[4]), p(d[5]), o[0].ptr(), o[1].ptr(),
                                 o[2].ptr(), None)
    else:
        lib.tagi_conv2d_fwd_act(C.byref(cg), p(d[0]), p(d[1]), p(d[2]), p(d[3]), p(d[4]), p(d[5]), act, o[0].ptr(),
                                o[1].ptr(), o[2].ptr(), None)
    return tuple(x.get((g.B, g.n_out)) for x in o)


def conv_bwd_state(g, mw, jcb, dm, dv):
    d = [dev(x) for x in (mw, jcb, dm, dv)]
    oa, ob = Out(g.B * g.n_in), Out(g.B * g.n_in)
    cg = cgeom(g)
    lib.tagi_conv2d_bwd_state(C.byref(cg), p(d[0]), p(d[1]), p(d[2]), p(d[3]), oa.ptr(), ob.ptr(), None)
    return oa.get((g.B, g.n_in)), ob.get((g.B, g.n_in))


def conv_bwd_param(g, vw, vb, ma, dm, dv):
    d = [dev(x) for x in (vw, vb, ma, dm, dv)]
    ow, ov, obm, obv = Out(g.fo * g.Kc), Out(g.fo * g.Kc), Out(g.fo), Out(g.fo)
    cg = cgeom(g)
    lib.tagi_conv2d_bwd_param(C.byref(cg), p(d[0]), p(d[1]), p(d[2]), p(d[3]), p(d[4]), ow.ptr(), ov.ptr(),
                              obm.ptr(), obv.ptr(), None)
    if not g.has_bias:
        torch.cuda.synchronize()
        return ow.get((g.fo, g.Kc)), ov.get((g.fo, g.Kc)), None, None
    return ow.get((g.fo, g.Kc)), ov.get((g.fo, g.Kc)), obm.get(), obv.get()


def linear_inputs(rng, B, K, N, bias=True):
    """Value distributions of the Linear micro-benchmark configuration, at any shape."""
    f32 = np.float32
    mw = (rng.standard_normal((N, K)) / np.sqrt(K)).astype(f32)
    vw = (rng.uniform(0.5, 1.5, (N, K)) / K).astype(f32)
    mb = (rng.standard_normal(N) * 0.1).astype(f32) if bias else None
    vb = np.full(N, 1e-3, f32) if bias else None
    ma = rng.standard_normal((B, K)).astype(f32)
    va = rng.uniform(1e-3, 1e-1, (B, K)).astype(f32)
    jcb = rng.uniform(0, 1, (B, K)).astype(f32)
    dm = (rng.standard_normal((B, N)) * 0.1).astype(f32)
    dv = (-rng.uniform(0, 1e-3, (B, N))).astype(f32)
    return dict(mu_w=mw, var_w=vw, mu_b=mb, var_b=vb, mu_a=ma, var_a=va, jcb=jcb, dmu_z=dm, dvar_z=dv)


def conv_inputs(rng, g):
    f32 = np.float32
    mw = (rng.standard_normal((g.fo, g.Kc)) / np.sqrt(g.Kc)).astype(f32)
    vw = (rng.uniform(0.5, 1.5, (g.fo, g.Kc)) / g.Kc).astype(f32)
    mb = (rng.standard_normal(g.fo) * 0.1).astype(f32) if g.has_bias else None
    vb = np.full(g.fo, 1e-3, f32) if g.has_bias else None
    ma = rng.standard_normal((g.B, g.n_in)).astype(f32)
    va = rng.uniform(1e-3, 1e-1, (g.B, g.n_in)).astype(f32)
    jcb = rng.uniform(0, 1, (g.B, g.n_in)).astype(f32)
    dm = (rng.standard_normal((g.B, g.n_out)) * 0.1).astype(f32)
    dv = (-rng.uniform(0, 1e-3, (g.B, g.n_out))).astype(f32)
    return dict(mu_w=mw, var_w=vw, mu_b=mb, var_b=vb, mu_a=ma, var_a=va, jcb=jcb, dmu_z=dm, dvar_z=dv)
