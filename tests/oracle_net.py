"""CPU trainer for TAGI networks built from the oracle's per-op restatements (test infrastructure): Linear, Conv2d,
ReLU, BatchNorm2d, AvgPool2d, LayerBlock and ResNetBlock composed the way the reference's containers compose them
(src/sequential.cpp:279-335,387-411,440-448, src/layer_block.cpp:151-220, src/resnet_block.cpp:183-269).

A network is described by a spec, a list of tuples, from which both this CPU trainer and the device-side mirror
(cutagi_b200.nn.build) are constructed:
    ("conv", fi, fo, k, stride, pad, pad_type, bias)   ("linear", K, N, bias)   ("relu",)   ("mrelu",)
    ("bn", C)   ("pool", k, stride, pad, pad_type)   ("res", [main spec], [shortcut spec] or None)
Parameter names follow the reference's state_dict ("Conv2d.0", "BatchNorm2d.main.3.2", "Linear.6", ...).
"""
import numpy as np
from oracle_lib import ConvGeom

F32 = np.float32
BN_EPS, BN_MOMENTUM = 1e-5, 0.9


def ones_like(a):
    return np.ones_like(a, F32)


class OLinear:
    kind = "Linear"

    def __init__(self, o, K, N, bias=True):
        self.o, self.K, self.N, self.bias = o, K, N, bias

    def init(self, shape, rng):
        assert int(np.prod(shape)) == self.K, (shape, self.K)
        s = np.sqrt(1.0 / self.K)
        self.p = dict(mu_w=(rng.standard_normal((self.N, self.K)) * s).astype(F32), var_w=np.full((self.N, self.K), s * s, F32),
                      mu_b=(rng.standard_normal(self.N) * s).astype(F32) if self.bias else None,
                      var_b=np.full(self.N, s * s, F32) if self.bias else None)
        return (self.N,)

    def forward(self, mu, var, jcb, train=True):
        self.saved = (mu, jcb)
        p = self.p
        mz, vz = self.o.linear_fwd(p["mu_w"], p["var_w"], p["mu_b"], p["var_b"], mu, var)
        return mz, vz, ones_like(mz)

    def backward(self, dmu, dvar, state_update=True):
        mu_a, jcb = self.saved
        self.d = self.o.linear_bwd_param(self.p["var_w"], self.p["var_b"], mu_a, dmu, dvar)
        return self.o.linear_bwd_state(self.p["mu_w"], jcb, dmu, dvar) if state_update else (None, None)

    def step(self, batch):
        self.o.param_update(batch, self.p["mu_w"], self.p["var_w"], self.d[0], self.d[1])
        if self.bias:
            self.o.param_update(batch, self.p["mu_b"], self.p["var_b"], self.d[2], self.d[3])

    def named(self, prefix, idx):
        return {f"{self.kind}.{prefix}{idx}": self}


class OConv(OLinear):
    kind = "Conv2d"

    def __init__(self, o, fi, fo, k, stride=1, pad=0, pad_type=1, bias=True):
        self.o, self.a, self.bias = o, (fi, fo, k, stride, pad, pad_type), bias

    def init(self, shape, rng):
        fi, fo, k, stride, pad, pad_type = self.a
        C, H, W = shape
        assert C == fi, (shape, fi)
        self.g1 = ConvGeom(B=1, fi=fi, hi=H, wi=W, fo=fo, k=k, stride=stride, pad=pad, pad_type=pad_type, has_bias=int(self.bias))
        s = np.sqrt(1.0 / (k * k * fi))
        self.p = dict(mu_w=(rng.standard_normal((fo, k * k * fi)) * s).astype(F32), var_w=np.full((fo, k * k * fi), s * s, F32),
                      mu_b=(rng.standard_normal(fo) * s).astype(F32) if self.bias else None,
                      var_b=np.full(fo, s * s, F32) if self.bias else None)
        return (fo, self.g1.ho, self.g1.wo)

    def _g(self, B):
        g = self.g1
        return ConvGeom(B=B, fi=g.fi, hi=g.hi, wi=g.wi, fo=g.fo, k=g.k, stride=g.stride, pad=g.pad, pad_type=g.pad_type,
                        has_bias=g.has_bias)

    def forward(self, mu, var, jcb, train=True):
        self.saved = (mu, jcb)
        p = self.p
        mz, vz = self.o.conv2d_fwd(self._g(mu.shape[0]), p["mu_w"], p["var_w"], p["mu_b"], p["var_b"], mu, var)
        return mz, vz, ones_like(mz)

    def backward(self, dmu, dvar, state_update=True):
        mu_a, jcb = self.saved
        g = self._g(mu_a.shape[0])
        self.d = self.o.conv2d_bwd_param(g, self.p["var_w"], self.p["var_b"], mu_a, dmu, dvar)
        return self.o.conv2d_bwd_state(g, self.p["mu_w"], jcb, dmu, dvar) if state_update else (None, None)


class OReLU:
    def __init__(self, o):
        self.o = o

    def init(self, shape, rng):
        return shape

    def forward(self, mu, var, jcb, train=True):
        return self.o.relu(mu, var)

    def backward(self, dmu, dvar, state_update=True):
        return dmu, dvar

    def step(self, batch):
        pass

    def named(self, prefix, idx):
        return {}


class OMixtureReLU(OReLU):
    def forward(self, mu, var, jcb, train=True):
        return self.o.mixture_relu(mu, var)


class OBatchNorm2d:
    kind = "BatchNorm2d"

    def __init__(self, o, C, bias=True):
        self.o, self.C, self.bias, self.first = o, C, bias, True

    def init(self, shape, rng):
        C = self.C
        assert shape[0] == C
        self.wihi = shape[1] * shape[2]
        # init_weight_bias_norm (src/param_init.cpp): mu_w = 1, var_w = 2 / (2 * C), mu_b = 0, var_b as var_w
        self.p = dict(mu_w=np.ones(C, F32), var_w=np.full(C, 1.0 / C, F32), mu_b=np.zeros(C, F32) if self.bias else None,
                      var_b=np.full(C, 1.0 / C, F32) if self.bias else None)
        self.mu_ra, self.var_ra = np.zeros(C, F32), np.ones(C, F32)
        return shape

    def forward(self, mu, var, jcb, train=True):
        B = mu.shape[0]
        a, va = mu.reshape(B, self.C, self.wihi), var.reshape(B, self.C, self.wihi)
        p = self.p
        if train:
            self.mean, self.var = self.o.bn2d_stats(a, va)
            self.o.bn2d_running(0.0 if self.first else BN_MOMENTUM, self.mean, self.var, self.mu_ra, self.var_ra)
            self.first = False
            mean, v = self.mean, self.var
        else:
            mean, v = self.mu_ra, self.var_ra
        self.saved = (a, jcb.reshape(a.shape))
        mz, vz = self.o.bn2d_fwd(BN_EPS, p["mu_w"], p["var_w"], p["mu_b"], p["var_b"], a, va, mean, v)
        mz, vz = mz.reshape(B, -1), vz.reshape(B, -1)
        return mz, vz, ones_like(mz)

    def backward(self, dmu, dvar, state_update=True):
        a, jcb = self.saved
        d, dv = dmu.reshape(a.shape), dvar.reshape(a.shape)
        self.d = self.o.bn2d_bwd_param(BN_EPS, self.p["var_w"], self.p["var_b"], a, self.mean, self.var, d, dv)
        if not state_update:
            return None, None
        dm, dvv = self.o.bn2d_bwd_state(BN_EPS, self.p["mu_w"], jcb, self.var, d, dv)
        return dm.reshape(a.shape[0], -1), dvv.reshape(a.shape[0], -1)

    step = OLinear.step
    named = OLinear.named


class OAvgPool2d:
    def __init__(self, o, k, stride=-1, pad=0, pad_type=0):
        self.o, self.a = o, (k, stride, pad, pad_type)

    def init(self, shape, rng):
        k, stride, pad, pad_type = self.a
        C, H, W = shape
        if stride < 0:   # pytagi's default: only meaningful for global pooling
            assert k == W == H
            stride = k
        self.g1 = ConvGeom(B=1, fi=C, hi=H, wi=W, fo=C, k=k, stride=stride, pad=pad, pad_type=pad_type)
        return (C, self.g1.ho, self.g1.wo)

    def _g(self, B):
        g = self.g1
        return ConvGeom(B=B, fi=g.fi, hi=g.hi, wi=g.wi, fo=g.fo, k=g.k, stride=g.stride, pad=g.pad, pad_type=g.pad_type)

    def forward(self, mu, var, jcb, train=True):
        self.saved = jcb
        mz, vz = self.o.avgpool2d_fwd(self._g(mu.shape[0]), mu, var)
        return mz, vz, ones_like(mz)

    def backward(self, dmu, dvar, state_update=True):
        if not state_update:
            return None, None
        return self.o.avgpool2d_bwd_state(self._g(dmu.shape[0]), self.saved, dmu, dvar)

    def step(self, batch):
        pass

    def named(self, prefix, idx):
        return {}


class OLayerBlock:
    def __init__(self, layers):
        self.layers = layers

    def init(self, shape, rng):
        for layer in self.layers:
            shape = layer.init(shape, rng)
        return shape

    def forward(self, mu, var, jcb, train=True):
        for layer in self.layers:
            mu, var, jcb = layer.forward(mu, var, jcb, train)
        return mu, var, jcb

    def backward(self, dmu, dvar, state_update=True):
        # src/layer_block.cpp:189-220: the block's first layer runs only when the block is asked for state deltas
        for layer in reversed(self.layers[1:]):
            dmu, dvar = layer.backward(dmu, dvar, True)
        if state_update and len(self.layers) > 1:
            dmu, dvar = self.layers[0].backward(dmu, dvar, True)
        return dmu, dvar

    def step(self, batch):
        for layer in self.layers:
            layer.step(batch)

    def named(self, prefix, idx):
        out = {}
        for i, layer in enumerate(self.layers):
            out.update(layer.named(f"{prefix}{idx}.", i))
        return out


class OResNetBlock:
    def __init__(self, o, main, shortcut=None):
        self.o, self.main, self.shortcut = o, main, shortcut

    def init(self, shape, rng):
        out = self.main.init(shape, rng)
        if self.shortcut is not None:
            assert self.shortcut.init(shape, rng) == out
        else:
            assert out == shape
        return out

    def forward(self, mu, var, jcb, train=True):
        self.jcb_in = jcb
        mz, vz, _ = self.main.forward(mu, var, jcb, train)
        if self.shortcut is not None:
            ms, vs, _ = self.shortcut.forward(mu, var, jcb, train)
        else:
            ms, vs = mu, var
        mz, vz = mz.copy(), vz.copy()
        self.o.add_shortcut(ms, vs, None, mz, vz)
        return mz, vz, ones_like(mz)

    def backward(self, dmu, dvar, state_update=True):
        dm, dv = self.main.backward(dmu, dvar, state_update)
        dm, dv = dm.copy(), dv.copy()
        if self.shortcut is not None:
            sm, sv = self.shortcut.backward(dmu, dvar, state_update)
            self.o.add_shortcut(sm, sv, None, dm, dv)
        else:
            self.o.add_shortcut(dmu, dvar, self.jcb_in, dm, dv)
        return dm, dv

    def step(self, batch):
        self.main.step(batch)
        if self.shortcut is not None:
            self.shortcut.step(batch)

    def named(self, prefix, idx):
        out = self.main.named(f"{prefix}main.", idx)
        if self.shortcut is not None:
            out.update(self.shortcut.named(f"{prefix}shortcut.", idx))
        return out


def build_layers(o, spec):
    out = []
    for item in spec:
        kind, a = item[0], item[1:]
        if kind == "conv":
            out.append(OConv(o, *a))
        elif kind == "linear":
            out.append(OLinear(o, *a))
        elif kind == "relu":
            out.append(OReLU(o))
        elif kind == "mrelu":
            out.append(OMixtureReLU(o))
        elif kind == "bn":
            out.append(OBatchNorm2d(o, *a))
        elif kind == "pool":
            out.append(OAvgPool2d(o, *a))
        elif kind == "res":
            out.append(OResNetBlock(o, OLayerBlock(build_layers(o, a[0])), OLayerBlock(build_layers(o, a[1])) if a[1] else None))
        else:
            raise ValueError(kind)
    return out


class OracleNet:
    """forward / update / backward / step of the reference's Sequential for the layers above."""

    def __init__(self, oracle, spec, in_shape, seed=0):
        self.o, self.layers, self.in_shape = oracle, build_layers(oracle, spec), tuple(in_shape)
        shape, rng = self.in_shape, np.random.default_rng(seed)
        for layer in self.layers:
            shape = layer.init(shape, rng)
        self.out_shape = shape
        self.input_state_update = False

    def named_layers(self):
        out = {}
        for i, layer in enumerate(self.layers):
            if isinstance(layer, OResNetBlock):
                out.update(layer.named("", i))
            elif isinstance(layer, OLayerBlock):
                out.update(layer.named("", i))
            else:
                out.update(layer.named("", i))
        return out

    def state_dict(self):
        return {k: layer.p for k, layer in self.named_layers().items()}

    def load_state_dict(self, sd):
        """sd: name -> (mu_w, var_w, mu_b, var_b) flat sequences, as the reference's state_dict returns them."""
        named = self.named_layers()
        assert set(sd) == set(named), (sorted(sd), sorted(named))
        for k, (mw, vw, mb, vb) in sd.items():
            p = named[k].p
            p["mu_w"] = np.asarray(mw, F32).reshape(p["mu_w"].shape).copy()
            p["var_w"] = np.asarray(vw, F32).reshape(p["var_w"].shape).copy()
            if p["mu_b"] is not None:
                p["mu_b"], p["var_b"] = np.asarray(mb, F32).copy(), np.asarray(vb, F32).copy()

    def forward(self, x, var_x=None, train=True):
        mu = np.ascontiguousarray(x, F32).reshape(-1, int(np.prod(self.in_shape)))
        var = np.zeros_like(mu) if var_x is None else np.ascontiguousarray(var_x, F32).reshape(mu.shape)
        jcb = ones_like(mu)
        self.batch = mu.shape[0]
        for layer in self.layers:
            mu, var, jcb = layer.forward(mu, var, jcb, train)
        self.out = (mu, var, jcb)
        return mu, var

    def update_using_indices(self, obs, var_obs, idx, n_enc):
        mu, var, jcb = self.out
        self.delta = self.o.output_delta_selected(mu, var, jcb, np.ascontiguousarray(obs, F32),
                                                  np.ascontiguousarray(var_obs, F32), idx, n_enc)

    def update(self, obs, var_obs):
        mu, var, jcb = self.out
        self.delta = self.o.output_delta(mu, var, jcb, np.ascontiguousarray(obs, F32).reshape(mu.shape),
                                         np.ascontiguousarray(var_obs, F32).reshape(mu.shape))

    def backward(self):
        dmu, dvar = self.delta
        for i in reversed(range(len(self.layers))):
            dmu, dvar = self.layers[i].backward(dmu, dvar, i > 0 or self.input_state_update)

    def step(self):
        for layer in self.layers:
            layer.step(self.batch)


def resnet_spec(widths=(64, 128, 256, 512), in_ch=3, stem=("conv", 3, 64, 3, 1, 1, 1, False), stem_pool=None,
                final_pool=4, n_out=11):
    """ResNet-18 of the reference (test/cpp_unit/test_resnet.cpp:84-110,228-263 with ReLU; the 224 x 224 variant of
    examples/tagi_resnet_model.py:146-268 uses the 6 x 6 stride-2 stem, the overlapping 3 x 3 stem pool and a 7 x 7
    final pool): two blocks per width, the first block of each later width strided with a projection shortcut."""
    def block(i, o, stride=1, pt=1):
        return [("conv", i, o, 3, stride, 1, pt, False), ("relu",), ("bn", o), ("conv", o, o, 3, 1, 1, 1, False), ("relu",),
                ("bn", o)]
    spec = [stem, ("relu",), ("bn", stem[2])]
    if stem_pool:
        spec.append(stem_pool)
    prev = stem[2]
    for w in widths:
        if w == prev:
            spec.append(("res", block(prev, w), None))
        else:
            spec.append(("res", block(prev, w, 2, 2), [("conv", prev, w, 2, 2, 0, 1, False), ("relu",), ("bn", w)]))
        spec.append(("res", block(w, w), None))
        prev = w
    spec += [("pool", final_pool, -1, 0, 0), ("linear", prev, n_out, True)]
    return spec


def net_golden_problems():
    """name -> (spec, input shape, batch, steps) of the networks behind tests/golden/net_golden.npz."""
    resnet = resnet_spec(widths=(4, 8), stem=("conv", 3, 4, 3, 1, 1, 1, False), final_pool=4)
    cnn = [("conv", 3, 4, 3, 1, 1, 1, True), ("relu",), ("pool", 2, 2, 0, 0), ("conv", 4, 8, 3, 1, 1, 1, True), ("relu",),
           ("pool", 2, 2, 0, 0), ("linear", 32, 16, True), ("relu",), ("linear", 16, 11, True)]
    return {"resnet": (resnet, (3, 8, 8), 4, 4), "cnn": (cnn, (3, 8, 8), 4, 4)}
