"""Dense gated feed-forward: down(act(gate(x)) * up(x)), added to the residual stream.

crates/model/src/llama.rs:261-285; silu(g) = g / (1 + exp(-g)) (crates/kernels/src/math.rs:8-10).
Gate and up are stored as one matrix [2F, E] so that one kernel reads x once; on the
tensor-core path that kernel also applies the activation (two accumulators, one epilogue).

`bias=True` gives every projection a bias vector (the reference refuses biases,
crates/model/src/weights.rs:165-167): gate and up then leave their product in float32, one
kernel adds the biases and applies the activation, and the down bias is either added by a block
that sums the sublayer's result itself (`accumulate=False`; it reads `down_bias`) or, when the
part adds into the residual stream, is not supported.  `act` names the activation of the gate
("silu" or "gelu_tanh").  `extra_rows` appends further weight rows to the gate/up matrix: a
block that needs another product of the same input gets it from the same launch
(`forward(..., extra_out=...)` returns a view of those columns).
"""
from __future__ import annotations

import torch

from ..ops import lib as ops
from .base import FeedForward, ParamSpec
from .linear import RESIDUAL, STORE, STORE_F32, linear, linear_deferred, linear_swiglu


class SwiGLU(FeedForward):
    graph_safe = True

    def __init__(self, width, hidden, dtype, bias=False, act="silu", wide_products=False):
        """wide_products: where gate and up do not run on the fused tensor-core kernel (rows that are no
        16-byte multiples), they stay float32 until the activation has been applied, so that the
        activation's input is rounded nowhere; without it that path stores them in the compute type."""
        if act not in ops.GLU_ACTS:
            raise ValueError(f"unknown activation {act!r}")
        if act != "silu" and not bias:
            raise ValueError("the fused gate/up kernels apply silu; another activation runs on the biased path")
        self.width, self.hidden, self.dtype, self.bias, self.act = width, hidden, dtype, bool(bias), act
        self.wide_products = bool(wide_products)
        self.w_gate_weight = self.w_up_weight = self.w_down_weight = None
        self.w_gate_bias = self.w_up_bias = self.w_down_bias = None
        self.w_gate_up = None
        self.extra_rows = None          # set by a block before finalize: [n, width] rows appended to gate/up
        self.extra_out = None           # float32 [T, n] view of the extra product of the last forward

    def param_specs(self):
        out = {"gate.weight": ParamSpec((self.hidden, self.width)),
               "up.weight": ParamSpec((self.hidden, self.width)),
               "down.weight": ParamSpec((self.width, self.hidden))}
        if self.bias:
            out.update({"gate.bias": ParamSpec((self.hidden,), kind="vector", init="normal"),
                        "up.bias": ParamSpec((self.hidden,), kind="vector", init="normal"),
                        "down.bias": ParamSpec((self.width,), kind="vector", init="normal")})
        return out

    @property
    def down_bias(self):
        return self.w_down_bias

    def finalize(self):
        rows = [self.w_gate_weight, self.w_up_weight]
        if self.extra_rows is not None:
            if not self.bias:
                raise ValueError("extra rows ride on the float32 gate/up product of the biased path")
            rows.append(self.extra_rows)
        self.w_gate_up = torch.cat(rows, dim=0).contiguous()
        self.w_gate_weight = self.w_up_weight = self.extra_rows = None

    def forward(self, x, ctx, residual, accumulate=True, defer=False):
        F, T = self.hidden, ctx.n_tokens
        act = ctx.buf("ffn_act", (ctx.token_capacity, F), self.dtype)
        if self.bias:
            if accumulate:
                raise ValueError("a biased feed-forward hands its result to a block that adds the down bias")
            n = self.w_gate_up.shape[0]
            # a few tokens: the product stays in partials and the activation kernel sums them
            part = linear_deferred(x, self.w_gate_up, ctx, T) if ctx.defer_swiglu else None
            if part is not None:
                self.extra_out = ctx.buf("ffn_extra", (ctx.token_capacity, n - 2 * F), torch.float32) if n > 2 * F else None
                ops.bias_glu_reduce(part, self.w_gate_bias, self.w_up_bias, act, T, F, self.act, extra=self.extra_out)
            else:
                gu = ctx.buf("ffn_gate_up_f32", (ctx.token_capacity, n), torch.float32)
                linear(x, self.w_gate_up, gu, STORE_F32, ctx, M=T)
                self.extra_out = gu[:, 2 * F:] if n > 2 * F else None
                ops.bias_glu(gu, self.w_gate_bias, self.w_up_bias, act, T, F, self.act)
        elif ops.gemm_tc_supported(x, self.w_gate_up):
            linear_swiglu(x, self.w_gate_up, act, F, ctx, M=T)
        elif self.wide_products and self.dtype != torch.float32:
            gu = ctx.buf("ffn_gate_up_f32", (ctx.token_capacity, 2 * F), torch.float32)
            linear(x, self.w_gate_up, gu, STORE_F32, ctx, M=T)
            ops.bias_glu(gu, None, None, act, T, F, self.act)
        else:
            gu = ctx.buf("ffn_gate_up", (ctx.token_capacity, 2 * F), self.dtype)
            linear(x, self.w_gate_up, gu, STORE, ctx, M=T)
            ops.swiglu(gu, act, T, F)
        if defer and not accumulate:
            part = linear_deferred(act, self.w_down_weight, ctx, T)
            if part is not None:
                return part
        linear(act, self.w_down_weight, residual, RESIDUAL if accumulate else STORE_F32, ctx, M=T)
        return None
