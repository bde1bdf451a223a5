"""Recurrent mixers: a state of fixed size per request, carried from token to token in 32-bit.

Each mixer declares its state (`StateNeeds`, by name) and gets it per slot in the cache view; a step's kernels walk
every request's rows in order from that state and leave the new one behind, so a request may be cut into steps
anywhere. Projections run in the compute dtype with 32-bit results; whatever enters a recurrence (gates, decays,
step sizes) is computed in 32-bit from them.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import CacheNeeds, Mixer, StateNeeds, TensorNeed, register_mixer


@register_mixer("mingru")
class MinGRU(Mixer):
    """A gated recurrence whose gates read only the current token:
        z = sigmoid(W_z h + b_z), u = W_x h + b_x, c = u + 1/2 (u >= 0) or sigmoid(u) (u < 0),
        S_t = (1 - z) S_(t-1) + z c (element by element), out = W_o (S_t * silu(W_g h)).
    params: width (the model's), inner (the recurrence's). tensors: z, z_bias, x, x_bias, g, o."""

    graph_safe = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.width = int(spec.params["width"])
        self.inner = int(spec.params["inner"])
        self.w_zxg = self.b_zxg = self.w_o = None

    def cache_needs(self):
        return CacheNeeds(state={"mingru": StateNeeds((self.inner,))})

    def tensors(self):
        t, W, E = self.spec.tensors, self.inner, self.width
        return {t["z"]: TensorNeed((W, E)), t["z_bias"]: TensorNeed((W,)), t["x"]: TensorNeed((W, E)),
                t["x_bias"]: TensorNeed((W,)), t["g"]: TensorNeed((W, E)), t["o"]: TensorNeed((E, W))}

    def load(self, get):
        t = self.spec.tensors
        self.w_zxg = torch.cat([get(t["z"]), get(t["x"]), get(t["g"])], dim=0).contiguous()
        bz, bx = get(t["z_bias"]), get(t["x_bias"])
        self.b_zxg = torch.cat([bz, bx, torch.zeros_like(bz)]).contiguous()
        self.w_o = get(t["o"])

    def weight_bytes(self):
        return sum(w.numel() * w.element_size() for w in (self.w_zxg, self.b_zxg, self.w_o))

    def forward(self, h, stream, step, cache) -> None:
        zxg = self.rt.linear(h, self.w_zxg, bias=self.b_zxg, out_dtype=torch.float32)
        out = self.rt.empty(h.shape[0], self.inner)
        ops.mingru_scan(zxg, cache.state["mingru"], out, step)
        self.rt.stream(stream).add_linear(out, self.w_o)


@register_mixer("mamba2")
class Mamba2(Mixer):
    """A selective state space with one scalar decay per head. W_in h = [z | x | B | C | dt] (inner, inner, G N,
    G N, heads; inner = heads * vdim); x, B, C pass a causal convolution per channel (bias, silu);
    dt = softplus(dt + dt_bias); per head (group = head // (heads / G)), with S of N x vdim,
        S_t = exp(-exp(A_log) dt) S_(t-1) + dt B_t x_t^T,   y_t = S_t^T C_t + D x_t;
    y * silu(z) is RMS-normed in `norm_groups` equal parts, times `norm`, then W_o.
    The state is S and the convolution's last taps - 1 inputs.
    params: width, heads, vdim, state, groups, conv (taps), norm_groups, eps.
    tensors: in, conv, conv_bias, dt_bias, A_log, D, norm, o."""

    graph_safe = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.width = int(p["width"])
        self.heads, self.vdim, self.n_state = int(p["heads"]), int(p["vdim"]), int(p["state"])
        self.groups, self.taps, self.norm_groups = int(p["groups"]), int(p["conv"]), int(p["norm_groups"])
        self.eps = float(p["eps"])
        self.inner = self.heads * self.vdim
        self.channels = self.inner + 2 * self.groups * self.n_state
        if self.heads % self.groups:
            raise ValueError(f"mamba2: {self.groups} groups must divide {self.heads} heads")
        if self.inner % self.norm_groups:
            raise ValueError(f"mamba2: {self.norm_groups} norm groups must divide the inner size {self.inner}")
        if self.taps < 1:
            raise ValueError("mamba2: the convolution needs at least one tap")
        self.w_in = self.conv_w = self.conv_b = self.dt_bias = self.a_log = self.d = self.norm_w = self.w_o = None

    def cache_needs(self):
        return CacheNeeds(state={"conv": StateNeeds((self.taps - 1, self.channels)),
                                 "ssm": StateNeeds((self.heads, self.vdim, self.n_state))})

    def tensors(self):
        t = self.spec.tensors
        H = self.heads
        return {t["in"]: TensorNeed((self.inner + self.channels + H, self.width)),
                t["conv"]: TensorNeed((self.channels, self.taps)), t["conv_bias"]: TensorNeed((self.channels,)),
                t["dt_bias"]: TensorNeed((H,), keep_fp32=True), t["A_log"]: TensorNeed((H,), keep_fp32=True),
                t["D"]: TensorNeed((H,), keep_fp32=True),
                t["norm"]: TensorNeed((self.inner,), keep_fp32=True, init="ones"),
                t["o"]: TensorNeed((self.width, self.inner))}

    def load(self, get):
        t = self.spec.tensors
        self.w_in, self.conv_w, self.conv_b = get(t["in"]), get(t["conv"]), get(t["conv_bias"])
        self.dt_bias, self.a_log, self.d = get(t["dt_bias"]), get(t["A_log"]), get(t["D"])
        self.norm_w, self.w_o = get(t["norm"]), get(t["o"])

    def weight_bytes(self):
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.conv_w, self.conv_b, self.dt_bias,
                                                          self.a_log, self.d, self.norm_w, self.w_o))

    def forward(self, h, stream, step, cache) -> None:
        rt, rows = self.rt, h.shape[0]
        proj = rt.linear(h, self.w_in, out_dtype=torch.float32)  # [z | x B C | dt]
        xbc = rt.empty(rows, self.channels, dtype=torch.float32)
        ops.causal_conv(proj, self.inner, self.conv_w, self.conv_b, cache.state["conv"], xbc, step)
        y = rt.empty(rows, self.inner, dtype=torch.float32)
        ops.ssm_scan(xbc, proj, self.inner + self.channels, self.dt_bias, self.a_log, self.d, cache.state["ssm"], y,
                     step, self.heads, self.vdim, self.n_state, self.groups)
        out = rt.empty(rows, self.inner)
        ops.gated_group_norm(y, proj, self.norm_w, out, self.norm_groups, self.eps)
        rt.stream(stream).add_linear(out, self.w_o)
