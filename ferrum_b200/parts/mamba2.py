"""A selective state-space mixer with one scalar decay per head (the Mamba-2 recurrence).

With inner = heads * P, N the state size per element and G groups that share B and C, the input
product gives per token [z: inner | x: inner | B: G N | C: G N | dt: heads].  x, B and C pass a
causal convolution of `taps` taps per channel and silu; per head h (group h / (heads / G)):

    dt = softplus(dt + dt_bias_h)
    S <- exp(-exp(A_log_h) dt) S + dt B x^T            (S: N x P, float32, zero before the first token)
    y = S^T C + D_h x

then y * silu(z) is RMS-normed in `norm_groups` equal parts, multiplied by a weight, and projected
back.  A request's state row keeps S and the convolution's last taps - 1 inputs, both float32; the
walk over a portion's tokens is sequential, so a token's result does not depend on how the sequence
was cut into steps.  The reference has no recurrent mixer (crates/model/src/llama.rs:185-257 is its
only one).
"""
from __future__ import annotations

import math

import torch

from ..ops import lib as ops
from .base import CacheNeed, Mixer, ParamSpec, StateNeed
from .linear import RESIDUAL, STORE_F32, linear, linear_deferred


def _draw_a_log(shape, g, device, std):
    """ln of a decay rate drawn from U(1, 16): the usual start of such a layer."""
    return torch.log(1.0 + 15.0 * torch.rand(shape, generator=g, device=device, dtype=torch.float32))


def _draw_dt_bias(shape, g, device, std):
    """The inverse softplus of a step size drawn log-uniformly from [0.001, 0.1]."""
    dt = torch.exp(torch.rand(shape, generator=g, device=device, dtype=torch.float32) * math.log(100.0) + math.log(0.001))
    return dt + torch.log(-torch.expm1(-dt))


class Mamba2Mixer(Mixer):
    graph_safe = True

    def __init__(self, width, heads, head_dim, state, groups, norm_groups, taps, eps, dtype):
        if heads % groups:
            raise ValueError("groups does not divide heads")
        self.width, self.H, self.P, self.N, self.G = width, int(heads), int(head_dim), int(state), int(groups)
        self.norm_groups, self.taps, self.eps, self.dtype = int(norm_groups), int(taps), float(eps), dtype
        self.inner = self.H * self.P
        self.channels = self.inner + 2 * self.G * self.N
        if self.inner % self.norm_groups:
            raise ValueError("norm_groups does not divide heads * head_dim")
        for n in ("in_weight", "conv_weight", "conv_bias", "dt_bias", "A_log", "D", "norm_weight", "o_weight"):
            setattr(self, "w_" + n, None)

    def param_specs(self):
        E, H = self.width, self.H
        return {"in.weight": ParamSpec((2 * self.inner + 2 * self.G * self.N + H, E)),
                "conv.weight": ParamSpec((self.channels, self.taps), kind="vector", init="normal"),
                "conv.bias": ParamSpec((self.channels,), kind="vector", init="normal"),
                "dt_bias": ParamSpec((H,), kind="vector", init=_draw_dt_bias),
                "A_log": ParamSpec((H,), kind="vector", init=_draw_a_log),
                "D": ParamSpec((H,), kind="vector", init="ones_normal"),
                "norm.weight": ParamSpec((self.inner,), kind="vector", init="ones_normal"),
                "o.weight": ParamSpec((E, self.inner))}

    def cache_need(self):
        return CacheNeed(state=StateNeed((self.inner * self.N + (self.taps - 1) * self.channels,), torch.float32))

    def forward(self, x, ctx, cache, residual, accumulate=True, defer=False):
        T, cap = ctx.n_tokens, ctx.token_capacity
        proj = ctx.buf("ssm_proj", (cap, self.w_in_weight.shape[0]), torch.float32)
        linear(x, self.w_in_weight, proj, STORE_F32, ctx, M=T)
        xbc = ctx.buf("ssm_xbc", (cap, self.channels), torch.float32)
        y = ctx.buf("ssm_y", (cap, self.inner), torch.float32)
        out = ctx.buf("ssm_out", (cap, self.inner), self.dtype)
        ops.mamba2_mix(proj, T, ctx, self.w_conv_weight, self.w_conv_bias, self.w_dt_bias, self.w_A_log, self.w_D,
                       self.w_norm_weight, self.H, self.P, self.N, self.G, self.norm_groups, self.eps, cache.state, xbc, y, out)
        if defer and not accumulate:
            part = linear_deferred(out, self.w_o_weight, ctx, T)
            if part is not None:
                return part
        linear(out, self.w_o_weight, residual, RESIDUAL if accumulate else STORE_F32, ctx, M=T)
        return None
