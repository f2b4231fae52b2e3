"""ctypes access to the checker libraries (test infrastructure).

`Oracle`  : oracle/libtagi_oracle.so, the plain-C restatement (built on demand with `make -C oracle port`).
`RefLib`  : oracle/_ref/libtagi_ref.so, the reference's own CPU classes behind a C ABI; only present where
            the reference sources were available at build time.
Both take and return numpy float32 arrays (float64 for the `_f64` arbitration variants).
"""
import ctypes as C
import os
import subprocess
from dataclasses import dataclass

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")

_fp = C.POINTER(C.c_float)
_dp = C.POINTER(C.c_double)


def _f(a):
    if a is None:
        return None
    assert a.dtype == np.float32 and a.flags.c_contiguous
    return a.ctypes.data_as(_fp)


def _d(a):
    assert a.dtype == np.float64 and a.flags.c_contiguous
    return a.ctypes.data_as(_dp)


class ConvGeomC(C.Structure):
    _fields_ = [(n, C.c_int) for n in
                ("B", "fi", "hi", "wi", "fo", "ho", "wo", "k", "stride", "pad", "pad_type", "has_bias")]


@dataclass
class ConvGeom:
    B: int
    fi: int
    hi: int
    wi: int
    fo: int
    k: int
    stride: int = 1
    pad: int = 0
    pad_type: int = 1
    has_bias: int = 1
    ho: int = 0
    wo: int = 0

    def __post_init__(self):
        if self.ho == 0 or self.wo == 0:
            self.wo, self.ho = conv_out_size(self.k, self.stride, self.wi, self.hi, self.pad, self.pad_type)

    @property
    def Kc(self):
        return self.k * self.k * self.fi

    @property
    def n_in(self):
        return self.fi * self.hi * self.wi

    @property
    def n_out(self):
        return self.fo * self.ho * self.wo

    def c(self):
        return ConvGeomC(self.B, self.fi, self.hi, self.wi, self.fo, self.ho, self.wo, self.k, self.stride,
                         self.pad, self.pad_type, self.has_bias)


def conv_out_size(k, stride, wi, hi, pad, pad_type):
    """(wo, ho) by the reference's rule; ValueError where the reference raises."""
    if pad_type == 1:
        nw, nh = wi - k + 2 * pad, hi - k + 2 * pad
    elif pad_type == 2:
        nw, nh = wi - k + pad, hi - k + pad
    else:
        nw, nh = wi - k, hi - k
    if nw % stride or nh % stride or nw < 0 or nh < 0:
        raise ValueError("invalid conv hyper-parameters")
    return nw // stride + 1, nh // stride + 1


def build_oracle():
    so = os.path.join(ORACLE_DIR, "libtagi_oracle.so")
    srcs = [os.path.join(ORACLE_DIR, f) for f in ("tagi_oracle.c", "tagi_oracle.h", "tagi_oracle_body.inc")]
    if not os.path.exists(so) or any(os.path.getmtime(s) > os.path.getmtime(so) for s in srcs):
        subprocess.run(["make", "-C", ORACLE_DIR, "port"], check=True, capture_output=True)
    return so


class Oracle:
    def __init__(self):
        self.lib = C.CDLL(build_oracle())
        self.lib.tagi_oracle_param_update.restype = C.c_int
        self.lib.tagi_oracle_param_update.argtypes = [C.c_int, C.c_size_t, _fp, _fp, _fp, _fp]

    # ---- Linear -------------------------------------------------------------------------------
    def linear_fwd(self, mu_w, var_w, mu_b, var_b, mu_a, var_a, f64=False):
        B, K = mu_a.shape
        N = mu_w.shape[0]
        dt, p, sfx = (np.float64, _d, "_f64") if f64 else (np.float32, _f, "_f32")
        mz, vz = np.empty((B, N), dt), np.empty((B, N), dt)
        getattr(self.lib, "tagi_oracle_linear_fwd" + sfx)(
            B, K, N, int(mu_b is not None), _f(mu_w), _f(var_w), _f(mu_b), _f(var_b), _f(mu_a), _f(var_a),
            p(mz), p(vz))
        return mz, vz

    def linear_bwd_state(self, mu_w, jcb, dmu_z, dvar_z, f64=False):
        B, K = jcb.shape
        N = mu_w.shape[0]
        dt, p, sfx = (np.float64, _d, "_f64") if f64 else (np.float32, _f, "_f32")
        dm, dv = np.empty((B, K), dt), np.empty((B, K), dt)
        getattr(self.lib, "tagi_oracle_linear_bwd_state" + sfx)(
            B, K, N, _f(mu_w), _f(jcb), _f(dmu_z), _f(dvar_z), p(dm), p(dv))
        return dm, dv

    def linear_bwd_param(self, var_w, var_b, mu_a, dmu_z, dvar_z, f64=False):
        B, K = mu_a.shape
        N = var_w.shape[0]
        dt, p, sfx = (np.float64, _d, "_f64") if f64 else (np.float32, _f, "_f32")
        dmw, dvw = np.empty((N, K), dt), np.empty((N, K), dt)
        dmb, dvb = np.zeros(N, dt), np.zeros(N, dt)
        getattr(self.lib, "tagi_oracle_linear_bwd_param" + sfx)(
            B, K, N, int(var_b is not None), _f(var_w), _f(var_b), _f(mu_a), _f(dmu_z), _f(dvar_z),
            p(dmw), p(dvw), p(dmb), p(dvb))
        return dmw, dvw, dmb, dvb

    # ---- Conv2d -------------------------------------------------------------------------------
    def conv2d_fwd(self, g, mu_w, var_w, mu_b, var_b, mu_a, var_a, f64=False):
        dt, p, sfx = (np.float64, _d, "_f64") if f64 else (np.float32, _f, "_f32")
        mz, vz = np.empty((g.B, g.n_out), dt), np.empty((g.B, g.n_out), dt)
        gc = g.c()
        getattr(self.lib, "tagi_oracle_conv2d_fwd" + sfx)(
            C.byref(gc), _f(mu_w), _f(var_w), _f(mu_b), _f(var_b), _f(mu_a), _f(var_a), p(mz), p(vz))
        return mz, vz

    def conv2d_bwd_state(self, g, mu_w, jcb, dmu_z, dvar_z, f64=False):
        dt, p, sfx = (np.float64, _d, "_f64") if f64 else (np.float32, _f, "_f32")
        dm, dv = np.empty((g.B, g.n_in), dt), np.empty((g.B, g.n_in), dt)
        gc = g.c()
        getattr(self.lib, "tagi_oracle_conv2d_bwd_state" + sfx)(
            C.byref(gc), _f(mu_w), _f(jcb), _f(dmu_z), _f(dvar_z), p(dm), p(dv))
        return dm, dv

    def conv2d_bwd_param(self, g, var_w, var_b, mu_a, dmu_z, dvar_z, f64=False):
        dt, p, sfx = (np.float64, _d, "_f64") if f64 else (np.float32, _f, "_f32")
        dmw, dvw = np.empty((g.fo, g.Kc), dt), np.empty((g.fo, g.Kc), dt)
        dmb, dvb = np.zeros(g.fo, dt), np.zeros(g.fo, dt)
        gc = g.c()
        getattr(self.lib, "tagi_oracle_conv2d_bwd_param" + sfx)(
            C.byref(gc), _f(var_w), _f(var_b), _f(mu_a), _f(dmu_z), _f(dvar_z), p(dmw), p(dvw), p(dmb), p(dvb))
        return dmw, dvw, dmb, dvb

    # ---- neighbours ---------------------------------------------------------------------------
    def relu(self, mu_z, var_z):
        ma, va, j = np.empty_like(mu_z), np.empty_like(mu_z), np.empty_like(mu_z)
        self.lib.tagi_oracle_relu(C.c_size_t(mu_z.size), _f(mu_z), _f(var_z), _f(ma), _f(va), _f(j))
        return ma, va, j

    def mixture_relu(self, mu_z, var_z):
        ma, va, j = np.empty_like(mu_z), np.empty_like(mu_z), np.empty_like(mu_z)
        self.lib.tagi_oracle_mixture_relu(C.c_size_t(mu_z.size), _f(mu_z), _f(var_z), _f(ma), _f(va), _f(j))
        return ma, va, j

    def output_delta(self, mu_a, var_a, jcb, obs, var_obs):
        dm, dv = np.empty_like(mu_a), np.empty_like(mu_a)
        self.lib.tagi_oracle_output_delta(C.c_size_t(mu_a.size), _f(mu_a), _f(var_a), _f(jcb), _f(obs), _f(var_obs),
                                          _f(dm), _f(dv))
        return dm, dv

    def output_delta_selected(self, mu_a, var_a, jcb, obs, var_obs, idx, n_enc):
        B, n_out = mu_a.shape
        dm, dv = np.empty_like(mu_a), np.empty_like(mu_a)
        idx = np.ascontiguousarray(idx, np.int32)
        self.lib.tagi_oracle_output_delta_selected(
            B, n_out, n_enc, _f(mu_a), _f(var_a), _f(jcb), _f(obs), _f(var_obs),
            idx.ctypes.data_as(C.POINTER(C.c_int)), _f(dm), _f(dv))
        return dm, dv

    def param_update(self, batch_size, mu, var, dmu, dvar):
        """In place on mu, var; returns the number of variances that were reset."""
        return self.lib.tagi_oracle_param_update(batch_size, mu.size, _f(mu), _f(var), _f(dmu), _f(dvar))

    # ---- BatchNorm2d / AvgPool2d / residual add (activations [B][C][H*W]) ---------------------------------
    def bn2d_stats(self, mu_a, var_a):
        B, C_, wihi = mu_a.shape
        mean, var = np.empty(C_, np.float32), np.empty(C_, np.float32)
        self.lib.tagi_oracle_bn2d_stats(B, C_, wihi, _f(mu_a), _f(var_a), _f(mean), _f(var))
        return mean, var

    def bn2d_running(self, momentum, mean, var, mu_ra, var_ra):
        """In place on mu_ra, var_ra."""
        self.lib.tagi_oracle_bn2d_running(mean.size, C.c_float(momentum), _f(mean), _f(var), _f(mu_ra), _f(var_ra))

    def bn2d_fwd(self, eps, mu_w, var_w, mu_b, var_b, mu_a, var_a, mean, var):
        B, C_, wihi = mu_a.shape
        mz, vz = np.empty_like(mu_a), np.empty_like(mu_a)
        self.lib.tagi_oracle_bn2d_fwd(B, C_, wihi, int(mu_b is not None), C.c_float(eps), _f(mu_w), _f(var_w), _f(mu_b),
                                      _f(var_b), _f(mu_a), _f(var_a), _f(mean), _f(var), _f(mz), _f(vz))
        return mz, vz

    def bn2d_bwd_state(self, eps, mu_w, jcb, var, dmu_o, dvar_o):
        B, C_, wihi = jcb.shape
        dm, dv = np.empty_like(jcb), np.empty_like(jcb)
        self.lib.tagi_oracle_bn2d_bwd_state(B, C_, wihi, C.c_float(eps), _f(mu_w), _f(jcb), _f(var), _f(dmu_o), _f(dvar_o),
                                            _f(dm), _f(dv))
        return dm, dv

    def bn2d_bwd_param(self, eps, var_w, var_b, mu_a, mean, var, dmu_o, dvar_o):
        B, C_, wihi = mu_a.shape
        dmw, dvw, dmb, dvb = (np.zeros(C_, np.float32) for _ in range(4))
        self.lib.tagi_oracle_bn2d_bwd_param(B, C_, wihi, int(var_b is not None), C.c_float(eps), _f(var_w), _f(var_b),
                                            _f(mu_a), _f(mean), _f(var), _f(dmu_o), _f(dvar_o), _f(dmw), _f(dvw),
                                            _f(dmb), _f(dvb))
        return dmw, dvw, dmb, dvb

    def avgpool2d_fwd(self, g, mu_a, var_a):
        mz, vz = np.empty((g.B, g.n_out), np.float32), np.empty((g.B, g.n_out), np.float32)
        gc = g.c()
        self.lib.tagi_oracle_avgpool2d_fwd(C.byref(gc), _f(mu_a), _f(var_a), _f(mz), _f(vz))
        return mz, vz

    def avgpool2d_bwd_state(self, g, jcb, dmu_o, dvar_o):
        dm, dv = np.empty((g.B, g.n_in), np.float32), np.empty((g.B, g.n_in), np.float32)
        gc = g.c()
        self.lib.tagi_oracle_avgpool2d_bwd_state(C.byref(gc), _f(jcb), _f(dmu_o), _f(dvar_o), _f(dm), _f(dv))
        return dm, dv

    def add_shortcut(self, mu_s, var_s, jcb, mu_a, var_a):
        """In place on mu_a, var_a; jcb None for a plain sum."""
        self.lib.tagi_oracle_add_shortcut(C.c_size_t(mu_a.size), _f(mu_s), _f(var_s), _f(jcb), _f(mu_a), _f(var_a))


class RefLib:
    """The reference's CPU classes (Linear, Conv2d, BaseLayer update) through oracle/ref_shim.cpp."""

    PATH = os.path.join(ORACLE_DIR, "_ref", "libtagi_ref.so")

    @classmethod
    def available(cls):
        return os.path.exists(cls.PATH)

    def __init__(self):
        self.lib = C.CDLL(self.PATH)
        self.lib.tagi_ref_last_error.restype = C.c_char_p

    def _chk(self, rc):
        if rc != 0:
            raise RuntimeError(self.lib.tagi_ref_last_error().decode())

    def linear_forward(self, mu_w, var_w, mu_b, var_b, mu_a, var_a, threads=4):
        B, K = mu_a.shape
        N = mu_w.shape[0]
        mz, vz = np.empty((B, N), np.float32), np.empty((B, N), np.float32)
        self._chk(self.lib.tagi_ref_linear_forward(B, K, N, int(mu_b is not None), threads, _f(mu_w), _f(var_w),
                                                   _f(mu_b), _f(var_b), _f(mu_a), _f(var_a), _f(mz), _f(vz)))
        return mz, vz

    def linear_backward(self, mu_w, var_w, var_b, mu_a, jcb, dmu_z, dvar_z, threads=4, state_update=True):
        B, K = mu_a.shape
        N = mu_w.shape[0]
        dma, dva = np.zeros((B, K), np.float32), np.zeros((B, K), np.float32)
        dmw, dvw = np.empty((N, K), np.float32), np.empty((N, K), np.float32)
        dmb, dvb = np.zeros(N, np.float32), np.zeros(N, np.float32)
        self._chk(self.lib.tagi_ref_linear_backward(
            B, K, N, int(var_b is not None), threads, int(state_update), _f(mu_w), _f(var_w), _f(var_b), _f(mu_a),
            _f(jcb), _f(dmu_z), _f(dvar_z), _f(dma), _f(dva), _f(dmw), _f(dvw), _f(dmb), _f(dvb)))
        return dma, dva, dmw, dvw, dmb, dvb

    def conv2d_out_size(self, k, stride, wi, hi, pad, pad_type):
        wo, ho = C.c_int(0), C.c_int(0)
        self._chk(self.lib.tagi_ref_conv2d_out_size(k, stride, wi, hi, pad, pad_type, C.byref(wo), C.byref(ho)))
        return wo.value, ho.value

    def conv2d_forward(self, g, mu_w, var_w, mu_b, var_b, mu_a, var_a, threads=4):
        mz, vz = np.empty((g.B, g.n_out), np.float32), np.empty((g.B, g.n_out), np.float32)
        self._chk(self.lib.tagi_ref_conv2d_forward(
            g.B, g.fi, g.hi, g.wi, g.fo, g.k, g.stride, g.pad, g.pad_type, g.has_bias, threads, _f(mu_w), _f(var_w),
            _f(mu_b), _f(var_b), _f(mu_a), _f(var_a), _f(mz), _f(vz)))
        return mz, vz

    def conv2d_backward(self, g, mu_w, var_w, var_b, mu_a, jcb, dmu_z, dvar_z, threads=4, state_update=True):
        dma, dva = np.zeros((g.B, g.n_in), np.float32), np.zeros((g.B, g.n_in), np.float32)
        dmw, dvw = np.empty((g.fo, g.Kc), np.float32), np.empty((g.fo, g.Kc), np.float32)
        dmb, dvb = np.zeros(g.fo, np.float32), np.zeros(g.fo, np.float32)
        self._chk(self.lib.tagi_ref_conv2d_backward(
            g.B, g.fi, g.hi, g.wi, g.fo, g.k, g.stride, g.pad, g.pad_type, g.has_bias, threads, int(state_update),
            _f(mu_w), _f(var_w), _f(var_b), _f(mu_a), _f(jcb), _f(dmu_z), _f(dvar_z), _f(dma), _f(dva), _f(dmw),
            _f(dvw), _f(dmb), _f(dvb)))
        return dma, dva, dmw, dvw, dmb, dvb

    def param_update(self, batch_size, mu_w, var_w, mu_b, var_b, dmu_w, dvar_w, dmu_b, dvar_b):
        neg = C.c_int(0)
        nb = 0 if mu_b is None else mu_b.size
        self._chk(self.lib.tagi_ref_param_update(
            batch_size, C.c_size_t(mu_w.size), C.c_size_t(nb), _f(mu_w), _f(var_w), _f(mu_b), _f(var_b), _f(dmu_w),
            _f(dvar_w), _f(dmu_b), _f(dvar_b), C.byref(neg)))
        return neg.value

    def bn2d_forward(self, eps, momentum, mu_w, var_w, mu_b, var_b, mu_a, var_a, mu_ra, var_ra, hi, wi, training=True,
                     first_batch=True, threads=1):
        """Returns mu_z, var_z, batch mean, batch variance; mu_ra / var_ra are updated in place."""
        B, C_, wihi = mu_a.shape
        mz, vz = np.empty_like(mu_a), np.empty_like(mu_a)
        mb, vb = np.zeros(C_, np.float32), np.zeros(C_, np.float32)
        self._chk(self.lib.tagi_ref_bn2d_forward(
            B, C_, hi, wi, int(mu_b is not None), threads, int(training), int(first_batch), C.c_float(eps),
            C.c_float(momentum), _f(mu_w), _f(var_w), _f(mu_b), _f(var_b), _f(mu_a), _f(var_a), _f(mu_ra), _f(var_ra),
            _f(mb), _f(vb), _f(mz), _f(vz)))
        return mz, vz, mb, vb

    def bn2d_backward(self, eps, mu_w, var_w, var_b, mu_a, jcb, mean, var, dmu_o, dvar_o, hi, wi, threads=1):
        B, C_, wihi = mu_a.shape
        dm, dv = np.empty_like(mu_a), np.empty_like(mu_a)
        dmw, dvw, dmb, dvb = (np.zeros(C_, np.float32) for _ in range(4))
        self._chk(self.lib.tagi_ref_bn2d_backward(
            B, C_, hi, wi, int(var_b is not None), threads, C.c_float(eps), _f(mu_w), _f(var_w), _f(var_b), _f(mu_a),
            _f(jcb), _f(mean), _f(var), _f(dmu_o), _f(dvar_o), _f(dm), _f(dv), _f(dmw), _f(dvw), _f(dmb), _f(dvb)))
        return dm, dv, dmw, dvw, dmb, dvb

    def avgpool2d(self, g, mu_a, var_a, jcb=None, dmu_o=None, dvar_o=None, threads=1):
        """Forward, and backward when deltas are given. g.fi channels; returns (mu_z, var_z, dmu, dvar, wo, ho)."""
        wo, ho = C.c_int(0), C.c_int(0)
        mz, vz = np.empty((g.B, g.n_out), np.float32), np.empty((g.B, g.n_out), np.float32)
        dm, dv = np.zeros((g.B, g.n_in), np.float32), np.zeros((g.B, g.n_in), np.float32)
        self._chk(self.lib.tagi_ref_avgpool2d(
            g.B, g.fi, g.hi, g.wi, g.k, g.stride, g.pad, g.pad_type, threads, _f(mu_a), _f(var_a), _f(jcb), _f(dmu_o),
            _f(dvar_o), C.byref(wo), C.byref(ho), _f(mz), _f(vz), _f(dm), _f(dv)))
        return mz, vz, dm, dv, wo.value, ho.value

    def mixture_relu(self, mu_z, var_z):
        ma, va, j = np.empty_like(mu_z), np.empty_like(mu_z), np.empty_like(mu_z)
        self._chk(self.lib.tagi_ref_mixture_relu(C.c_size_t(mu_z.size), _f(mu_z), _f(var_z), _f(ma), _f(va), _f(j)))
        return ma, va, j
