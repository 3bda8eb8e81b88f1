"""A pre-norm block: h += mixer(norm1(h)); h += ffn(norm2(h)).

The reference's order (crates/model/src/llama.rs:183-285; docs/ARCHITECTURE.md "Forward
pass").  The two residual sums happen inside the parts' last kernels, in float32.
"""
from __future__ import annotations

import torch

from ..ops import lib as ops
from .base import CacheNeed, FeedForward, Mixer, Norm, ParamSpec, Part, StateNeed
from .linear import STORE_F32, linear


class PreNormBlock(Part):
    graph_safe = True

    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Norm, ffn: FeedForward,
                 names=("attn_norm.", "attn_", "ffn_norm.", "ffn_")):
        self.norm1, self.mixer, self.norm2, self.ffn = norm1, mixer, norm2, ffn
        self._names = names

    def children(self):
        return list(zip(self._names, (self.norm1, self.mixer, self.norm2, self.ffn)))

    def forward(self, h, ctx, cache):
        x = self.norm1.forward(h, ctx)
        ctx.flush_residual()            # no-op when the norm took the pending sum itself
        self.mixer.forward(x, ctx, cache, h)
        x = self.norm2.forward(h, ctx)
        ctx.flush_residual()
        self.ffn.forward(x, ctx, h)


# Up to this many tokens in a step the block's second chain (gates, feed-forward) runs on a second stream.
OVERLAP_MAX_TOKENS = 64


class ParallelGatedBlock(Part):
    """Both sublayers read norms of the SAME residual row and their gated results are added together:

        n = groupnorm(h);  a = n * w1;  b = n * w2
        m = a + (a of the request's previous token - a) * shift        (token shift; zeros before the first token)
        h += mixer(m) * sigmoid(G1 a + c1) + ffn(b) * sigmoid(G2 b + c2)

    One normalisation serves both weight vectors.  The previous token's `a` is part of a request's
    state (one float32 row per request and run of the block), so the block, not its mixer, asks
    the cache for it (`cache_need`).  `ffn` may be None (a layer without a feed-forward has neither
    a second norm weight nor a second gate); `token_shift=False` leaves m = a.  The sublayers hand
    their results over in float32 buffers (`accumulate=False`); a biased feed-forward's down bias
    is added in the same final kernel.  The reference has no such arrangement (its block is
    `PreNormBlock`'s)."""
    graph_safe = True

    def __init__(self, width, eps, groups, dtype, mixer: Mixer, ffn: FeedForward = None, token_shift=True,
                 names=("mix.", "mlp.")):
        if groups < 1 or width % groups:
            raise ValueError(f"{groups} groups do not divide a width of {width}")
        self.width, self.eps, self.groups, self.dtype = width, float(eps), int(groups), dtype
        self.mixer, self.ffn, self.token_shift = mixer, ffn, bool(token_shift)
        self._names = names
        self.w_norm1_weight = self.w_norm2_weight = self.w_shift_weight = None
        self.w_rg1_weight = self.w_rg1_bias = self.w_rg2_weight = self.w_rg2_bias = None
        self._rg2_fused = False

    def param_specs(self):
        E = self.width
        out = {"norm1.weight": ParamSpec((E,), kind="vector", init="ones_normal"),
               "rg1.weight": ParamSpec((E, E)), "rg1.bias": ParamSpec((E,), kind="vector")}
        if self.token_shift:
            out["shift.weight"] = ParamSpec((E,), kind="vector", init="uniform")
        if self.ffn is not None:
            out.update({"norm2.weight": ParamSpec((E,), kind="vector", init="ones_normal"),
                        "rg2.weight": ParamSpec((E, E)), "rg2.bias": ParamSpec((E,), kind="vector")})
        return out

    def children(self):
        out = [(self._names[0], self.mixer)]
        if self.ffn is not None:
            out.append((self._names[1], self.ffn))
        return out

    def cache_need(self):
        need = self.mixer.cache_need()
        if not self.token_shift:
            return need
        if need.state is not None:
            raise ValueError("the block's token shift and its mixer both want the run's state")
        return CacheNeed(paged=need.paged, state=StateNeed((self.width,), torch.float32))

    def finalize(self):
        # the second gate's product reads the same rows as the feed-forward's gate/up product: one launch
        if self.ffn is not None and getattr(self.ffn, "bias", False) and hasattr(self.ffn, "extra_rows"):
            self.ffn.extra_rows = self.w_rg2_weight
            self._rg2_fused = True
        super().finalize()
        if self._rg2_fused:
            self.w_rg2_weight = None

    def forward(self, h, ctx, cache):
        ctx.flush_residual()
        T, E, cap = ctx.n_tokens, self.width, ctx.token_capacity
        a = ctx.buf("pgb_a", (cap, E), self.dtype)
        m = ctx.buf("pgb_m", (cap, E), self.dtype)
        b = ctx.buf("pgb_b", (cap, E), self.dtype) if self.ffn is not None else None
        stage = ctx.buf("pgb_stage", (ctx.max_requests, E), torch.float32) if self.token_shift else None
        state = cache.state if self.token_shift else None
        ops.norm_pair_shift(h, self.w_norm1_weight, self.w_norm2_weight if b is not None else None,
                            self.w_shift_weight if self.token_shift else None, a, m, b, T, ctx, state, stage, self.groups,
                            self.eps)
        y1 = ctx.buf("pgb_y1", (cap, E), torch.float32)
        g1 = ctx.buf("pgb_g1", (cap, E), torch.float32)
        y2 = ctx.buf("pgb_y2", (cap, E), torch.float32) if self.ffn is not None else None
        g2 = ctx.buf("pgb_g2", (cap, E), torch.float32) if self.ffn is not None and not self._rg2_fused else None

        p1 = p2 = None

        def gates_and_ffn(defer):
            """The second chain; the feed-forward's last product may stay in partials (`defer`), so it runs last."""
            nonlocal g2, p2
            linear(a, self.w_rg1_weight, g1, STORE_F32, ctx, M=T)
            if self.ffn is not None:
                if not self._rg2_fused:
                    linear(b, self.w_rg2_weight, g2, STORE_F32, ctx, M=T)
                p2 = self.ffn.forward(b, ctx, y2, accumulate=False, defer=defer)
                ctx.flush_residual()
                if self._rg2_fused:
                    g2 = self.ffn.extra_out

        # The mixer reads m; the gates and the feed-forward read a and b: two chains that meet only in
        # the final sum.  In steps of a few tokens every kernel of a chain waits for the one before it
        # far longer than it computes, so the second chain runs on a second stream beside the first.
        if T <= OVERLAP_MAX_TOKENS and not ops.profiling() and str(ctx.device) != "cpu":
            side, fork, join = ctx.side_stream()
            main = torch.cuda.current_stream()
            fork.record(main)
            side.wait_event(fork)
            ctx.lane = 1
            try:
                with torch.cuda.stream(side):
                    gates_and_ffn(True)
                    join.record(side)
            finally:
                ctx.lane = 0
            # (each chain's last product may stay in partials of its own lane's workspace: the final kernel sums both)
            p1 = self.mixer.forward(m, ctx, cache, y1, accumulate=False, defer=True)
            main.wait_event(join)
        else:
            self.mixer.forward(m, ctx, cache, y1, accumulate=False)
            gates_and_ffn(False)
        c2 = getattr(self.ffn, "down_bias", None) if self.ffn is not None else None
        ops.gated_residual(h, T, y1 if p1 is None else None, g1, self.w_rg1_bias, y2 if p2 is None else None, c2, g2,
                           self.w_rg2_bias if y2 is not None else None,
                           ctx=ctx, stage=stage, state=state, p1=p1, p2=p2)
