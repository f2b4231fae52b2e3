"""Device-side mirror of the part of the pytagi API that surrounds the hot path (Linear, Conv2d, ReLU, BatchNorm2d,
AvgPool2d, LayerBlock, ResNetBlock, Sequential, OutputUpdater), with the same names and argument meaning, so that whole
TAGI training steps run through the C ABI.

Every arithmetic step is a call into libtagi_b200.so; torch is used for device memory only. The mirror exists for
parity tests and measurements. Inside cuTAGI the same entry points are reached through the reference's own classes
(the shims under integration/); this module is not meant to replace them.
"""
import ctypes
import math

import numpy as np
import torch

from . import capi
from .capi import lib


def _p(t):
    return None if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


class Linear:
    """cutagi.Linear(ip_size, op_size, bias, gain_weight, gain_bias, method) (src/bindings/linear_layer_bindings.cpp:8-22).
    He initialisation as in src/param_init.cpp:5-22,158-187: mu ~ N(0, gain/sqrt(fan_in)), var = gain^2 / fan_in."""

    # called right after the parameter deltas of this layer have been launched (the data-parallel exchange hooks in here,
    # so that it overlaps the state pass and the backward of the earlier layers)
    on_ready = None

    def __init__(self, input_size, output_size, bias=True, gain_weight=1.0, gain_bias=1.0, init_method="He", seed=None):
        self.input_size, self.output_size, self.bias = input_size, output_size, bias
        rng = np.random.default_rng(seed)
        scale = math.sqrt(1.0 / input_size)
        self.load(dict(mu_w=(rng.standard_normal((output_size, input_size)) * gain_weight * scale).astype(np.float32),
                       var_w=np.full((output_size, input_size), (gain_weight * scale) ** 2, np.float32),
                       mu_b=(rng.standard_normal(output_size) * gain_bias * scale).astype(np.float32),
                       var_b=np.full(output_size, (gain_bias * scale) ** 2, np.float32)))

    def init_shape(self, shape):
        if int(np.prod(shape)) != self.input_size:
            raise RuntimeError(f"Input size mismatch: {self.input_size} vs {int(np.prod(shape))}")
        return (self.output_size,)

    def named(self, prefix, idx):
        return {f"{type(self).__name__}.{prefix}{idx}": self}

    def load(self, p):
        dev = torch.device("cuda")
        self.mu_w = torch.from_numpy(np.ascontiguousarray(p["mu_w"], np.float32)).to(dev).reshape(self.output_size, -1)
        self.var_w = torch.from_numpy(np.ascontiguousarray(p["var_w"], np.float32)).to(dev).reshape(self.output_size, -1)
        self.mu_b = torch.from_numpy(np.ascontiguousarray(p["mu_b"], np.float32)).to(dev) if self.bias else None
        self.var_b = torch.from_numpy(np.ascontiguousarray(p["var_b"], np.float32)).to(dev) if self.bias else None
        self.delta_mu_w, self.delta_var_w = torch.zeros_like(self.mu_w), torch.zeros_like(self.var_w)
        self.delta_mu_b = torch.zeros_like(self.mu_b) if self.bias else None
        self.delta_var_b = torch.zeros_like(self.var_b) if self.bias else None
        self.neg_var = torch.zeros(1, dtype=torch.int32, device=dev)

    def forward(self, mu_a, var_a, jcb, train=True, act=0):
        """act = capi.ACT_RELU / ACT_MIXTURE_RELU: the activation layer that follows is folded into the call
        (tagi_linear_fwd_act) and the moments after it and its Jacobian are returned."""
        B = mu_a.shape[0]
        if mu_a.shape[1] != self.input_size:
            raise RuntimeError(f"Input size mismatch: {self.input_size} vs {mu_a.shape[1]}")
        self.saved = (mu_a, jcb)   # what the reference copies into bwd_states (src/base_layer.cpp:212-228)
        mu_z = torch.empty(B, self.output_size, device=mu_a.device)
        var_z = torch.empty_like(mu_z)
        if act:
            j = torch.empty_like(mu_z)
            lib.tagi_linear_fwd_act(_p(self.mu_w), _p(self.var_w), _p(self.mu_b), _p(self.var_b), _p(mu_a), _p(var_a), B,
                                    self.input_size, self.output_size, int(self.bias), act, _p(mu_z), _p(var_z), _p(j),
                                    _stream())
            return mu_z, var_z, j
        lib.tagi_linear_fwd(_p(self.mu_w), _p(self.var_w), _p(self.mu_b), _p(self.var_b), _p(mu_a), _p(var_a), B,
                            self.input_size, self.output_size, int(self.bias), _p(mu_z), _p(var_z), _stream())
        return mu_z, var_z, None   # Jacobian of a Linear output is one

    def backward(self, dmu, dvar, state_update=True):
        mu_a, jcb = self.saved
        B = mu_a.shape[0]
        lib.tagi_linear_bwd_param(_p(self.var_w), _p(self.var_b), _p(mu_a), _p(dmu), _p(dvar), B, self.input_size,
                                  self.output_size, int(self.bias), _p(self.delta_mu_w), _p(self.delta_var_w),
                                  _p(self.delta_mu_b), _p(self.delta_var_b), _stream())
        if self.on_ready is not None:
            self.on_ready()
        if not state_update:
            return None, None
        dmu_a, dvar_a = torch.empty_like(mu_a), torch.empty_like(mu_a)
        lib.tagi_linear_bwd_state(_p(self.mu_w), _p(jcb), _p(dmu), _p(dvar), B, self.input_size, self.output_size,
                                  _p(dmu_a), _p(dvar_a), _stream())
        return dmu_a, dvar_a

    def step(self, batch_size):
        lib.tagi_param_update(batch_size, self.mu_w.numel(), _p(self.mu_w), _p(self.var_w), _p(self.delta_mu_w),
                              _p(self.delta_var_w), _p(self.neg_var), _stream())
        if self.bias:
            lib.tagi_param_update(batch_size, self.mu_b.numel(), _p(self.mu_b), _p(self.var_b), _p(self.delta_mu_b),
                                  _p(self.delta_var_b), None, _stream())

    def _delta_slots(self):
        """(object, attribute) of every parameter-delta tensor, in the order the backward pass produces them."""
        return [(self, a) for a in ("delta_mu_w", "delta_var_w", "delta_mu_b", "delta_var_b")
                if getattr(self, a) is not None]

    def delta_tensors(self):
        """Parameter-delta tensors in the order the backward pass produces them (for the data-parallel exchange)."""
        return [getattr(o, a) for o, a in self._delta_slots()]


class _NoParams:
    def init_shape(self, shape):
        return shape

    def named(self, prefix, idx):
        return {}

    def step(self, batch_size):
        pass

    def _delta_slots(self):
        return []

    def delta_tensors(self):
        return []


class ReLU(_NoParams):
    def forward(self, mu_z, var_z, jcb, train=True):
        mu_a, var_a, j = torch.empty_like(mu_z), torch.empty_like(mu_z), torch.empty_like(mu_z)
        lib.tagi_relu_fwd(_p(mu_z), _p(var_z), mu_z.numel(), _p(mu_a), _p(var_a), _p(j), _stream())
        return mu_a, var_a, j

    def backward(self, dmu, dvar, state_update=True):   # its Jacobian was saved by the next layer
        return dmu, dvar


class MixtureReLU(ReLU):
    """cutagi.MixtureReLU(): rectified-Gaussian moments instead of the ReLU's linearisation (src/activation.cpp:152-178)."""

    def forward(self, mu_z, var_z, jcb, train=True):
        mu_a, var_a, j = torch.empty_like(mu_z), torch.empty_like(mu_z), torch.empty_like(mu_z)
        lib.tagi_mixture_relu_fwd(_p(mu_z), _p(var_z), mu_z.numel(), _p(mu_a), _p(var_a), _p(j), _stream())
        return mu_a, var_a, j


def _geom(B, fi, hi, wi, fo, k, stride, pad, pad_type, has_bias):
    wo, ho = capi.conv_out_size(k, stride, wi, hi, pad, pad_type)
    return capi.ConvGeom(B, fi, hi, wi, fo, ho, wo, k, stride, pad, pad_type, int(has_bias))


class Conv2d(Linear):
    """cutagi.Conv2d(in_channels, out_channels, kernel_size, bias, stride, padding, padding_type, in_width, in_height,
    gain_weight, gain_bias, init_method) (src/bindings/conv2d_layer_bindings.cpp). He initialisation with
    fan_in = kernel_size^2 * in_channels (src/param_init.cpp). Activations [B][C*H*W], weights [fo][fi*k*k]."""

    def __init__(self, in_channels, out_channels, kernel_size, bias=True, stride=1, padding=0, padding_type=1, in_width=0,
                 in_height=0, gain_weight=1.0, gain_bias=1.0, init_method="He", seed=None):
        self.fi, self.fo, self.k, self.bias = in_channels, out_channels, kernel_size, bias
        self.stride, self.pad, self.pad_type, self.wi, self.hi = stride, padding, padding_type, in_width, in_height
        self.output_size = out_channels   # rows of the weight matrix (load() reshapes by it)
        fan_in = kernel_size * kernel_size * in_channels
        rng = np.random.default_rng(seed)
        scale = math.sqrt(1.0 / fan_in)
        self.load(dict(mu_w=(rng.standard_normal((out_channels, fan_in)) * gain_weight * scale).astype(np.float32),
                       var_w=np.full((out_channels, fan_in), (gain_weight * scale) ** 2, np.float32),
                       mu_b=(rng.standard_normal(out_channels) * gain_bias * scale).astype(np.float32),
                       var_b=np.full(out_channels, (gain_bias * scale) ** 2, np.float32)))

    def init_shape(self, shape):
        C, H, W = shape
        if C != self.fi:
            raise RuntimeError(f"Input channel mismatch: {self.fi} vs {C}")
        self.hi, self.wi = H, W
        self.wo, self.ho = capi.conv_out_size(self.k, self.stride, W, H, self.pad, self.pad_type)
        self.input_size = C * H * W
        return (self.fo, self.ho, self.wo)

    def _g(self, B):
        return _geom(B, self.fi, self.hi, self.wi, self.fo, self.k, self.stride, self.pad, self.pad_type, self.bias)

    def forward(self, mu_a, var_a, jcb, train=True, act=0):
        B = mu_a.shape[0]
        if mu_a.shape[1] != self.input_size:
            raise RuntimeError(f"Input size mismatch: {self.input_size} vs {mu_a.shape[1]}")
        self.saved = (mu_a, jcb)
        mu_z = torch.empty(B, self.fo * self.ho * self.wo, device=mu_a.device)
        var_z = torch.empty_like(mu_z)
        g = self._g(B)
        if train and getattr(self, "_reserved_for", None) != B:
            # size the library's scratch pool for all three passes of this layer before the first of them runs, so that no
            # pass has to grow the pool in the middle of a step (or of a stream capture)
            lib.tagi_reserve_scratch(lib.tagi_conv2d_workspace_bytes(ctypes.byref(g)))
            self._reserved_for = B
        if act:
            j = torch.empty_like(mu_z)
            lib.tagi_conv2d_fwd_act(ctypes.byref(g), _p(self.mu_w), _p(self.var_w), _p(self.mu_b), _p(self.var_b),
                                    _p(mu_a), _p(var_a), act, _p(mu_z), _p(var_z), _p(j), _stream())
            return mu_z, var_z, j
        lib.tagi_conv2d_fwd(ctypes.byref(g), _p(self.mu_w), _p(self.var_w), _p(self.mu_b), _p(self.var_b), _p(mu_a),
                            _p(var_a), _p(mu_z), _p(var_z), _stream())
        return mu_z, var_z, None

    def backward(self, dmu, dvar, state_update=True):
        mu_a, jcb = self.saved
        g = self._g(mu_a.shape[0])
        lib.tagi_conv2d_bwd_param(ctypes.byref(g), _p(self.var_w), _p(self.var_b), _p(mu_a), _p(dmu), _p(dvar),
                                  _p(self.delta_mu_w), _p(self.delta_var_w), _p(self.delta_mu_b), _p(self.delta_var_b),
                                  _stream())
        if self.on_ready is not None:
            self.on_ready()
        if not state_update:
            return None, None
        dmu_a, dvar_a = torch.empty_like(mu_a), torch.empty_like(mu_a)
        lib.tagi_conv2d_bwd_state(ctypes.byref(g), _p(self.mu_w), _p(jcb), _p(dmu), _p(dvar), _p(dmu_a), _p(dvar_a),
                                  _stream())
        return dmu_a, dvar_a


class BatchNorm2d(Linear):
    """cutagi.BatchNorm2d(num_features, eps, momentum, bias, gain_weight, gain_bias)
    (src/bindings/batchnorm_layer_bindings.cpp); parameters as init_weight_bias_norm (src/param_init.cpp) sets them:
    mu_w = 1, var_w = 1 / num_features, mu_b = 0, var_b = 1 / num_features; running averages 0 and 1. The first training
    batch replaces the running averages (momentum 0), as BatchNorm2d::forward does (src/batchnorm_layer.cpp:862-868)."""

    def __init__(self, num_features, eps=1e-5, momentum=0.9, bias=True, gain_weight=1.0, gain_bias=1.0):
        C = num_features
        self.C, self.eps, self.momentum, self.bias, self.first_batch = C, eps, momentum, bias, True
        self.output_size = C
        self.load(dict(mu_w=np.ones(C, np.float32), var_w=np.full(C, gain_weight * gain_weight / C, np.float32),
                       mu_b=np.zeros(C, np.float32), var_b=np.full(C, gain_bias * gain_bias / C, np.float32)))
        dev = torch.device("cuda")
        self.mu_ra, self.var_ra = torch.zeros(C, device=dev), torch.ones(C, device=dev)
        self.mu_batch, self.var_batch = torch.zeros(C, device=dev), torch.zeros(C, device=dev)

    def load(self, p):
        super().load(p)
        self.mu_w, self.var_w = self.mu_w.reshape(-1), self.var_w.reshape(-1)
        self.delta_mu_w, self.delta_var_w = self.delta_mu_w.reshape(-1), self.delta_var_w.reshape(-1)

    def init_shape(self, shape):
        if shape[0] != self.C:
            raise RuntimeError(f"Input channel mismatch: {self.C} vs {shape[0]}")
        self.wihi = shape[1] * shape[2]
        return shape

    def forward(self, mu_a, var_a, jcb, train=True):
        B = mu_a.shape[0]
        self.saved = (mu_a, jcb)
        mu_z, var_z = torch.empty_like(mu_a), torch.empty_like(mu_a)
        momentum = 0.0 if (train and self.first_batch) else self.momentum
        if train:
            self.first_batch = False
        lib.tagi_bn2d_fwd(B, self.C, self.wihi, int(self.bias), int(train), ctypes.c_float(self.eps),
                          ctypes.c_float(momentum), _p(self.mu_w), _p(self.var_w), _p(self.mu_b), _p(self.var_b), _p(mu_a),
                          _p(var_a), _p(self.mu_ra), _p(self.var_ra), _p(self.mu_batch), _p(self.var_batch), _p(mu_z),
                          _p(var_z), _stream())
        return mu_z, var_z, None

    def backward(self, dmu, dvar, state_update=True):
        mu_a, jcb = self.saved
        dmu_a = torch.empty_like(mu_a) if state_update else None
        dvar_a = torch.empty_like(mu_a) if state_update else None
        lib.tagi_bn2d_bwd(mu_a.shape[0], self.C, self.wihi, int(self.bias), int(state_update), ctypes.c_float(self.eps),
                          _p(self.mu_w), _p(self.var_w), _p(self.var_b), _p(mu_a), _p(jcb), _p(self.mu_batch),
                          _p(self.var_batch), _p(dmu), _p(dvar), _p(dmu_a), _p(dvar_a), _p(self.delta_mu_w),
                          _p(self.delta_var_w), _p(self.delta_mu_b), _p(self.delta_var_b), _stream())
        if self.on_ready is not None:
            self.on_ready()
        return dmu_a, dvar_a


class AvgPool2d(_NoParams):
    """cutagi.AvgPool2d(kernel_size, stride=-1, padding=0, padding_type=0) (src/bindings/pooling_layer_bindings.cpp).
    stride -1 is accepted for global pooling (kernel = image extent), where the reference's size rule yields 1 x 1."""

    def __init__(self, kernel_size, stride=-1, padding=0, padding_type=0):
        self.k, self.stride, self.pad, self.pad_type = kernel_size, stride, padding, padding_type

    def init_shape(self, shape):
        self.C, self.hi, self.wi = shape
        if self.stride < 0:
            if not (self.k == self.hi == self.wi):
                raise RuntimeError("Invalid hyperparameters for pooling layer: stride -1 needs kernel_size = image extent")
            self.stride = self.k
        self.wo, self.ho = capi.conv_out_size(self.k, self.stride, self.wi, self.hi, self.pad, self.pad_type)
        return (self.C, self.ho, self.wo)

    def _g(self, B):
        return _geom(B, self.C, self.hi, self.wi, self.C, self.k, self.stride, self.pad, self.pad_type, 0)

    def forward(self, mu_a, var_a, jcb, train=True):
        B = mu_a.shape[0]
        self.saved = (B, jcb)
        mu_z = torch.empty(B, self.C * self.ho * self.wo, device=mu_a.device)
        var_z = torch.empty_like(mu_z)
        g = self._g(B)
        lib.tagi_avgpool2d_fwd(ctypes.byref(g), _p(mu_a), _p(var_a), _p(mu_z), _p(var_z), _stream())
        return mu_z, var_z, None

    def backward(self, dmu, dvar, state_update=True):
        if not state_update:
            return None, None
        B, jcb = self.saved
        dmu_a = torch.empty(B, self.C * self.hi * self.wi, device=dmu.device)
        dvar_a = torch.empty_like(dmu_a)
        g = self._g(B)
        lib.tagi_avgpool2d_bwd_state(ctypes.byref(g), _p(jcb), _p(dmu), _p(dvar), _p(dmu_a), _p(dvar_a), _stream())
        return dmu_a, dvar_a


fuse_relu = True   # run a Linear / Conv2d layer and the ReLU layer directly behind it as one call


def _forward_layers(layers, mu, var, jcb, train):
    """The layers in order. A Linear / Conv2d layer directly followed by a ReLU layer runs as one fused call
    (tagi_linear_fwd_act / tagi_conv2d_fwd_act): same results, the moments before the activation are never stored.
    (A MixtureReLU stays a pass of its own: inside the forward kernel it was measured slower.)"""
    fusable = {ReLU: capi.ACT_RELU}
    i = 0
    while i < len(layers):
        layer = layers[i]
        if fuse_relu and type(layer) in (Linear, Conv2d) and i + 1 < len(layers) and type(layers[i + 1]) in fusable:
            mu, var, jcb = layer.forward(mu, var, jcb, train, act=fusable[type(layers[i + 1])])
            i += 2
        else:
            mu, var, jcb = layer.forward(mu, var, jcb, train)
            i += 1
    return mu, var, jcb


class LayerBlock:
    """cutagi.LayerBlock(*layers) (src/layer_block.cpp:151-220): the layers in order; in the backward pass the block's
    first layer runs only when the block is asked for state deltas."""

    def __init__(self, *layers):
        self.layers = list(layers)

    def init_shape(self, shape):
        for layer in self.layers:
            shape = layer.init_shape(shape)
        return shape

    def forward(self, mu, var, jcb, train=True):
        return _forward_layers(self.layers, mu, var, jcb, train)

    def backward(self, dmu, dvar, state_update=True):
        for layer in reversed(self.layers[1:]):
            dmu, dvar = layer.backward(dmu, dvar, True)
        if state_update and len(self.layers) > 1:
            dmu, dvar = self.layers[0].backward(dmu, dvar, True)
        return dmu, dvar

    def step(self, batch_size):
        for layer in self.layers:
            layer.step(batch_size)

    def named(self, prefix, idx):
        out = {}
        for i, layer in enumerate(self.layers):
            out.update(layer.named(f"{prefix}{idx}.", i))
        return out

    def _delta_slots(self):
        return [s for layer in reversed(self.layers) for s in layer._delta_slots()]

    def delta_tensors(self):
        return [t for layer in reversed(self.layers) for t in layer.delta_tensors()]


class ResNetBlock:
    """cutagi.ResNetBlock(main_block, shortcut=None) (src/resnet_block.cpp:183-269): output = main(x) + shortcut(x) (or x),
    output Jacobian one; deltas = main's + shortcut's (projection) or + incoming deltas times the input Jacobian (identity)."""

    def __init__(self, main_block, shortcut=None):
        self.main, self.shortcut = main_block, shortcut

    def init_shape(self, shape):
        out = self.main.init_shape(shape)
        other = self.shortcut.init_shape(shape) if self.shortcut is not None else shape
        if tuple(other) != tuple(out):
            raise RuntimeError(f"ResNetBlock: main block output {out} does not match the shortcut's {other}")
        return out

    def forward(self, mu, var, jcb, train=True):
        self.jcb_in = jcb
        mu_z, var_z, _ = self.main.forward(mu, var, jcb, train)
        mu_s, var_s = (mu, var) if self.shortcut is None else self.shortcut.forward(mu, var, jcb, train)[:2]
        lib.tagi_add_shortcut(_p(mu_s), _p(var_s), None, mu_z.numel(), _p(mu_z), _p(var_z), _stream())
        return mu_z, var_z, None

    def backward(self, dmu, dvar, state_update=True):
        dmu_a, dvar_a = self.main.backward(dmu, dvar, state_update)
        if self.shortcut is not None:
            dmu_s, dvar_s = self.shortcut.backward(dmu, dvar, state_update)
            lib.tagi_add_shortcut(_p(dmu_s), _p(dvar_s), None, dmu_a.numel(), _p(dmu_a), _p(dvar_a), _stream())
        else:
            lib.tagi_add_shortcut(_p(dmu), _p(dvar), _p(self.jcb_in), dmu_a.numel(), _p(dmu_a), _p(dvar_a), _stream())
        return dmu_a, dvar_a

    def step(self, batch_size):
        self.main.step(batch_size)
        if self.shortcut is not None:
            self.shortcut.step(batch_size)

    def named(self, prefix, idx):
        out = self.main.named(f"{prefix}main.", idx)
        if self.shortcut is not None:
            out.update(self.shortcut.named(f"{prefix}shortcut.", idx))
        return out

    def _delta_slots(self):
        # backward order: main block first, then the shortcut
        return self.main._delta_slots() + (self.shortcut._delta_slots() if self.shortcut is not None else [])

    def delta_tensors(self):
        return self.main.delta_tensors() + (self.shortcut.delta_tensors() if self.shortcut is not None else [])


class Sequential:
    """forward / backward / step of cutagi.Sequential (src/sequential.cpp:279-335, 387-411, 440-448) for Linear / ReLU
    stacks. `input_state_update` as in include/sequential.h:45 (default: the first layer computes parameter deltas only)."""

    def __init__(self, *layers, in_shape=None):
        self.layers = list(layers)
        self.input_state_update = False
        first = self.layers[0]
        if in_shape is None:   # as the reference: the first layer knows its input extent
            in_shape = (first.fi, first.hi, first.wi) if isinstance(first, Conv2d) else (first.input_size,)
        shape = self.in_shape = tuple(in_shape)
        for layer in self.layers:
            shape = layer.init_shape(shape)
        self.out_shape = shape
        self.training = True

    def train(self):
        self.training = True

    def eval(self):
        self.training = False

    def named_layers(self):
        out = {}
        for i, layer in enumerate(self.layers):
            out.update(layer.named("", i))
        return out

    def state_dict(self):
        """name -> (mu_w, var_w, mu_b, var_b) as numpy arrays, with the reference's names (src/sequential.cpp:630-700)."""
        def h(t):
            return None if t is None else t.detach().cpu().numpy()
        self.check_kernels()
        return {k: (h(l.mu_w), h(l.var_w), h(l.mu_b), h(l.var_b)) for k, l in self.named_layers().items()}

    def load_state_dict(self, sd):
        named = self.named_layers()
        if set(sd) != set(named):
            raise RuntimeError(f"state_dict keys do not match the network: {sorted(set(sd) ^ set(named))}")
        for k, v in sd.items():
            if isinstance(v, dict):
                v = (v["mu_w"], v["var_w"], v["mu_b"], v["var_b"])
            named[k].load(dict(mu_w=np.asarray(v[0], np.float32), var_w=np.asarray(v[1], np.float32),
                               mu_b=None if v[2] is None else np.asarray(v[2], np.float32),
                               var_b=None if v[3] is None else np.asarray(v[3], np.float32)))
        self._ptable = None   # the tensors were replaced: the update table is rebuilt on the next step
        self._delta_views = None

    def _delta_slots(self):
        return [s for layer in reversed(self.layers) for s in layer._delta_slots()]

    def delta_tensors(self):
        """All parameter-delta tensors in the order the backward pass produces them (after pack_deltas(): the padded
        views of the one buffer that holds them)."""
        if getattr(self, "_delta_views", None) is not None:
            return list(self._delta_views)
        return [t for layer in reversed(self.layers) for t in layer.delta_tensors()]

    def pack_deltas(self):
        """Moves every layer's parameter-delta tensors into one buffer, back to back in the order the backward pass
        produces them, each padded to a multiple of four floats (every tensor stays 16-byte aligned; the padding is
        zero and stays zero). The data-parallel exchange then moves the tensors of a bucket as one collective instead
        of one per tensor (tagi_comm_finalize_buckets merges tensors that are adjacent in memory). Returns the padded
        1-D views in that order; a layer's own delta attributes are views of the same memory. load_state_dict()
        undoes the packing."""
        slots = self._delta_slots()
        sizes = [getattr(o, a).numel() for o, a in slots]
        padded = [(n + 3) // 4 * 4 for n in sizes]
        flat = torch.zeros(sum(padded), device="cuda")
        views, off = [], 0
        for (o, a), n, m in zip(slots, sizes, padded):
            old = getattr(o, a)
            new = flat[off:off + n].view(old.shape)
            new.copy_(old)
            setattr(o, a, new)
            views.append(flat[off:off + m])
            off += m
        self._delta_flat, self._delta_views = flat, views
        self._ptable = None   # the update table holds the old addresses
        return list(views)

    def __call__(self, mu_x, var_x=None):
        return self.forward(mu_x, var_x)

    def forward(self, mu_x, var_x=None):
        mu = torch.as_tensor(mu_x, dtype=torch.float32, device="cuda")
        mu = mu.reshape(-1, int(np.prod(self.in_shape))).contiguous()
        var = torch.zeros_like(mu) if var_x is None else torch.as_tensor(var_x, dtype=torch.float32,
                                                                         device="cuda").reshape(mu.shape).contiguous()
        jcb = None
        self.batch = mu.shape[0]
        mu, var, jcb = _forward_layers(self.layers, mu, var, jcb, self.training)
        self.output = (mu, var, jcb)
        self.delta = (torch.zeros_like(mu), torch.zeros_like(mu))   # input_delta_z_buffer
        return mu, var

    def forward_staged(self, io, slot):
        """Forward pass on the batch staged in slot `slot` of a hostio.HostPipeline: the upload runs on the pipeline's
        stream and the kernels wait for it on the device. Returns (mu, var) and the slot's device observations and
        indices for the output updater."""
        io.upload(slot, _stream())
        x, obs, idx = io.device_tensors(slot)
        mu, var = self.forward(x)
        return mu, var, obs, idx

    def check_kernels(self):
        """Raises when a bounded device-side wait of the tensor-core kernels ran out since the last check (the launch
        that it belonged to left its outputs incomplete). Synchronises with the device; state_dict() calls it."""
        status = capi.tc_status()
        if status != 0:
            raise capi.TagiError(capi.TAGI_OK, f"a bounded wait of the tensor-core kernels ran out (status {status})")

    def backward(self):
        dmu, dvar = self.delta
        for i in reversed(range(len(self.layers))):
            dmu, dvar = self.layers[i].backward(dmu, dvar, state_update=(i > 0 or self.input_state_update))
        self.input_delta = (dmu, dvar)

    def step(self):
        """Capped update of every parameter tensor of the network in one launch (tagi_param_update_multi)."""
        if getattr(self, "_ptable", None) is None:
            rows = []
            for layer in self.named_layers().values():
                rows.append((layer.mu_w, layer.var_w, layer.delta_mu_w, layer.delta_var_w))
                if layer.mu_b is not None:
                    rows.append((layer.mu_b, layer.var_b, layer.delta_mu_b, layer.delta_var_b))
            table = [[t[0].data_ptr(), t[1].data_ptr(), t[2].data_ptr(), t[3].data_ptr(), t[0].numel()] for t in rows]
            self._ptable = torch.tensor(table, dtype=torch.int64, device="cuda")   # five 8-byte fields per descriptor
            self._ptable_rows = rows                                                # keeps the tensors alive
            self.neg_var = torch.zeros(1, dtype=torch.int32, device="cuda")
        lib.tagi_param_update_multi(self.batch, self._ptable.shape[0], _p(self._ptable), _p(self.neg_var), _stream())


class OutputUpdater:
    """cutagi.OutputUpdater.update / update_using_indices (src/base_output_updater.cpp:352-386)."""

    def update(self, model, mu_obs, var_obs):
        mu, var, jcb = model.output
        if jcb is None:
            jcb = torch.ones_like(mu)
        obs = torch.as_tensor(mu_obs, dtype=torch.float32, device="cuda").reshape(mu.shape).contiguous()
        vobs = torch.as_tensor(var_obs, dtype=torch.float32, device="cuda").reshape(mu.shape).contiguous()
        lib.tagi_output_delta(_p(mu), _p(var), _p(jcb), _p(obs), _p(vobs), mu.numel(), _p(model.delta[0]),
                              _p(model.delta[1]), _stream())

    def update_using_indices(self, model, mu_obs, var_obs, selected_idx):
        mu, var, jcb = model.output
        if jcb is None:
            jcb = torch.ones_like(mu)
        B, n_out = mu.shape
        obs = torch.as_tensor(mu_obs, dtype=torch.float32, device="cuda").contiguous()
        vobs = torch.as_tensor(var_obs, dtype=torch.float32, device="cuda").contiguous()
        idx = torch.as_tensor(selected_idx, dtype=torch.int32, device="cuda").contiguous()
        n_enc = idx.numel() // B
        lib.tagi_output_delta_selected(_p(mu), _p(var), _p(jcb), _p(obs), _p(vobs), _p(idx), B, n_out, n_enc,
                                       _p(model.delta[0]), _p(model.delta[1]), _stream())


def build(spec, in_shape, seed=None):
    """Sequential from a spec (list of tuples): ("conv", fi, fo, k, stride, pad, pad_type, bias), ("linear", K, N, bias),
    ("relu",), ("bn", C), ("pool", k, stride, pad, pad_type), ("res", [main spec], [shortcut spec] or None)."""
    count = [0]

    def next_seed():   # one seed per parameterised layer, so that equally shaped layers do not start identical
        count[0] += 1
        return None if seed is None else seed + count[0]

    def layers(spec):
        out = []
        for item in spec:
            kind, a = item[0], item[1:]
            if kind == "conv":
                fi, fo, k, stride, pad, pad_type, bias = a
                out.append(Conv2d(fi, fo, k, bias=bias, stride=stride, padding=pad, padding_type=pad_type, seed=next_seed()))
            elif kind == "linear":
                out.append(Linear(a[0], a[1], bias=a[2], seed=next_seed()))
            elif kind == "relu":
                out.append(ReLU())
            elif kind == "mrelu":
                out.append(MixtureReLU())
            elif kind == "bn":
                out.append(BatchNorm2d(a[0]))
            elif kind == "pool":
                out.append(AvgPool2d(*a))
            elif kind == "res":
                out.append(ResNetBlock(LayerBlock(*layers(a[0])), LayerBlock(*layers(a[1])) if a[1] else None))
            else:
                raise ValueError(kind)
        return out
    return Sequential(*layers(spec), in_shape=in_shape)


def resnet18_spec(image=224, n_out=11, act="relu"):
    """The reference's ResNet-18 (examples/tagi_resnet_model.py:146-268 for 224 x 224 inputs, :56-143 /
    test/cpp_unit/test_resnet.cpp:84-110,228-263 for 32 x 32); act = "relu" as in the C++ test or "mrelu" (MixtureReLU) as in
    the Python example."""
    def block(i, o, stride=1, pt=1):
        return [("conv", i, o, 3, stride, 1, pt, False), (act,), ("bn", o), ("conv", o, o, 3, 1, 1, 1, False), (act,),
                ("bn", o)]
    if image == 224:
        spec = [("conv", 3, 64, 6, 2, 2, 1, False), (act,), ("bn", 64), ("pool", 3, 2, 1, 2)]
        final_pool = 7
    else:
        spec = [("conv", 3, 64, 3, 1, 1, 1, False), (act,), ("bn", 64)]
        final_pool = image // 8
    prev = 64
    for w in (64, 128, 256, 512):
        if w == prev:
            spec.append(("res", block(prev, w), None))
        else:
            spec.append(("res", block(prev, w, 2, 2), [("conv", prev, w, 2, 2, 0, 1, False), (act,), ("bn", w)]))
        spec.append(("res", block(w, w), None))
        prev = w
    return spec + [("pool", final_pool, -1, 0, 0), ("linear", 512, n_out, True)]


class Utils:
    """pytagi.Utils.label_to_obs (pytagi/tagi_utils.py:24-48): class labels -> hierarchical-softmax observations."""

    @staticmethod
    def class_to_obs(num_classes):
        """Per class: L = ceil(log2(num_classes)) observations (+1 for a 0 bit, -1 for a 1 bit, most significant bit
        first) and the one-based output unit that carries each of them: the root for the first bit, then the node reached
        by the bits read so far, nodes numbered level by level (src/cost.cpp:76-139)."""
        L = max(1, math.ceil(math.log2(num_classes)))
        level = [0] * (L + 1)
        level[L] = num_classes
        for i in range(L - 1, -1, -1):
            level[i] = math.ceil(level[i + 1] / 2.0)
        first = np.cumsum(level) + 1   # one-based index of the first node below each level
        obs = np.empty((num_classes, L), np.float32)
        idx = np.ones((num_classes, L), np.int32)
        for r in range(num_classes):
            bits = [(r >> (L - 1 - c)) & 1 for c in range(L)]
            obs[r] = [(-1.0) ** b for b in bits]
            for c in range(L - 1):
                prefix = int("".join(str(b) for b in bits[: c + 1]), 2)
                idx[r, c + 1] = prefix + first[c]
        return obs, idx, L, int(idx.max())

    def label_to_obs(self, labels, num_classes):
        """Returns (obs, obs_idx, num_obs): flat float32 / int32 arrays of len(labels) * L entries."""
        obs, idx, L, _ = self.class_to_obs(num_classes)
        labels = np.asarray(labels, np.int64).reshape(-1)
        return obs[labels].reshape(-1), idx[labels].reshape(-1), L
