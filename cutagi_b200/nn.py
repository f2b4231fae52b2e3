"""Device-side mirror of the part of the pytagi API that surrounds the hot path (Linear, ReLU, Sequential,
OutputUpdater), with the same names and argument meaning, so that whole TAGI training steps run through the C ABI.

Every arithmetic step is a call into libtagi_b200.so; torch is used for device memory only. The mirror exists for
parity tests and measurements. Inside cuTAGI the same entry points are reached through the reference's own classes
(see INTEGRATION.md); this module is not meant to replace them.
"""
import math

import numpy as np
import torch

from .capi import lib


def _p(t):
    return None if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


class Linear:
    """cutagi.Linear(ip_size, op_size, bias, gain_weight, gain_bias, method) (src/bindings/linear_layer_bindings.cpp:8-22).
    He initialisation as in src/param_init.cpp:5-22,158-187: mu ~ N(0, gain/sqrt(fan_in)), var = gain^2 / fan_in."""

    def __init__(self, input_size, output_size, bias=True, gain_weight=1.0, gain_bias=1.0, init_method="He", seed=None):
        self.input_size, self.output_size, self.bias = input_size, output_size, bias
        rng = np.random.default_rng(seed)
        scale = math.sqrt(1.0 / input_size)
        self.load(dict(mu_w=(rng.standard_normal((output_size, input_size)) * gain_weight * scale).astype(np.float32),
                       var_w=np.full((output_size, input_size), (gain_weight * scale) ** 2, np.float32),
                       mu_b=(rng.standard_normal(output_size) * gain_bias * scale).astype(np.float32),
                       var_b=np.full(output_size, (gain_bias * scale) ** 2, np.float32)))

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

    def forward(self, mu_a, var_a, jcb):
        B = mu_a.shape[0]
        if mu_a.shape[1] != self.input_size:
            raise RuntimeError(f"Input size mismatch: {self.input_size} vs {mu_a.shape[1]}")
        self.saved = (mu_a, jcb)   # what the reference copies into bwd_states (src/base_layer.cpp:212-228)
        mu_z = torch.empty(B, self.output_size, device=mu_a.device)
        var_z = torch.empty_like(mu_z)
        lib.tagi_linear_fwd(_p(self.mu_w), _p(self.var_w), _p(self.mu_b), _p(self.var_b), _p(mu_a), _p(var_a), B,
                            self.input_size, self.output_size, int(self.bias), _p(mu_z), _p(var_z), _stream())
        return mu_z, var_z, None   # Jacobian of a Linear output is one

    def backward(self, dmu, dvar, state_update=True):
        mu_a, jcb = self.saved
        B = mu_a.shape[0]
        lib.tagi_linear_bwd_param(_p(self.var_w), _p(self.var_b), _p(mu_a), _p(dmu), _p(dvar), B, self.input_size,
                                  self.output_size, int(self.bias), _p(self.delta_mu_w), _p(self.delta_var_w),
                                  _p(self.delta_mu_b), _p(self.delta_var_b), _stream())
        if not state_update:
            return None, None
        if jcb is None:
            jcb = torch.ones_like(mu_a)
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

    def delta_tensors(self):
        """Parameter-delta tensors in the order the backward pass produces them (for the data-parallel exchange)."""
        return [t for t in (self.delta_mu_w, self.delta_var_w, self.delta_mu_b, self.delta_var_b) if t is not None]


class ReLU:
    def forward(self, mu_z, var_z, jcb):
        mu_a, var_a, j = torch.empty_like(mu_z), torch.empty_like(mu_z), torch.empty_like(mu_z)
        lib.tagi_relu_fwd(_p(mu_z), _p(var_z), mu_z.numel(), _p(mu_a), _p(var_a), _p(j), _stream())
        return mu_a, var_a, j

    def backward(self, dmu, dvar, state_update=True):   # its Jacobian was saved by the next layer
        return dmu, dvar

    def step(self, batch_size):
        pass


class Sequential:
    """forward / backward / step of cutagi.Sequential (src/sequential.cpp:279-335, 387-411, 440-448) for Linear / ReLU
    stacks. `input_state_update` as in include/sequential.h:45 (default: the first layer computes parameter deltas only)."""

    def __init__(self, *layers):
        self.layers = list(layers)
        self.input_state_update = False

    def __call__(self, mu_x, var_x=None):
        return self.forward(mu_x, var_x)

    def forward(self, mu_x, var_x=None):
        mu = torch.as_tensor(mu_x, dtype=torch.float32, device="cuda")
        first = self.layers[0]
        mu = mu.reshape(-1, first.input_size).contiguous()
        var = torch.zeros_like(mu) if var_x is None else torch.as_tensor(var_x, dtype=torch.float32,
                                                                         device="cuda").reshape(mu.shape).contiguous()
        jcb = None
        self.batch = mu.shape[0]
        for layer in self.layers:
            mu, var, jcb = layer.forward(mu, var, jcb)
        self.output = (mu, var, jcb)
        self.delta = (torch.zeros_like(mu), torch.zeros_like(mu))   # input_delta_z_buffer
        return mu, var

    def backward(self):
        dmu, dvar = self.delta
        for i in reversed(range(len(self.layers))):
            dmu, dvar = self.layers[i].backward(dmu, dvar, state_update=(i > 0 or self.input_state_update))
        self.input_delta = (dmu, dvar)

    def step(self):
        for layer in self.layers:
            layer.step(self.batch)


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
