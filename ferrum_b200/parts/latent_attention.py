"""Attention whose keys and values are expanded from a small cached latent.

Per token the cache keeps one row: a normalised latent c (`kv_rank` elements), from which every
head's unrotated key part (U_k c) and value (U_v c) follow, and one rotated key part (`rot_dim`
elements) that all heads share.  Queries go through a latent of their own (`q_rank`), are laid
out per head as [`dim` unrotated | `rot_dim` rotated], and the score of head h for key j is
(q_plain . U_k,h c_j + q_rot . k_rot,j) * scale.  The key map is folded into the query
(q' = [U_k,h^T q_plain | q_rot]) and the value map applied after the weighted sum, so attention
runs on the cached rows themselves: one shared row of kv_rank + rot_dim key elements whose first
kv_rank elements are the values, for all heads.  An output gate sigmoid(W_g x)_h scales head h
before the output projection.  `window` > 0: a query at p sees keys p - window + 1 .. p.

A mixer built with `own_latent=False` has no down-projection for keys and values: it runs as a
schedule entry with `cache_of`, reads the rows another run cached, and expands them with its own
U_k, U_v (and may look back over a window of its own).

The reference has no such mixer (its attention caches whole keys and values:
crates/model/src/llama.rs:185-257).
"""
from __future__ import annotations

import torch

from ..ops import lib as ops
from . import attention_plan
from .base import CacheNeed, Mixer, PagedKVNeed, ParamSpec
from .linear import RESIDUAL, STORE, STORE_F32, linear, linear_deferred


# Steps of single tokens cut every token's keys among CTAs while they bring fewer rows than this per SM.
SPLIT_BELOW = 4
MAX_SPLITS = 1024       # what the merge kernel folds per (token, head)


class LatentAttention(Mixer):
    graph_safe = True

    def __init__(self, width, heads, dim, rot_dim, vdim, kv_rank, q_rank, eps, scale, dtype, rotary=None, window=0,
                 own_latent=True):
        """rotary: a `RotaryEmbedding` over the rot_dim part (its rope_dim leading elements turn,
        "half" pairing), or None for no rotation."""
        self.width, self.H, self.Dn, self.Rr, self.Dv = width, int(heads), int(dim), int(rot_dim), int(vdim)
        self.R, self.Rq = int(kv_rank), int(q_rank)
        self.eps, self.scale, self.dtype = float(eps), float(scale), dtype
        self.rotary, self.window, self.own_latent = rotary, int(window), bool(own_latent)
        if rotary is not None and (rotary.rope_dim > self.Rr or rotary.pairing != 1):
            raise ValueError("the rotary table must cover at most rot_dim elements, paired (i, i + dims/2)")
        self.Dk = self.R + self.Rr
        for name in ("dq_weight", "dq_norm_weight", "uq_weight", "dkv_weight", "dkv_norm_weight", "uk_weight", "uv_weight",
                     "g_weight", "o_weight"):
            setattr(self, "w_" + name, None)
        self.w_in = self.w_uk_t = self.w_uv_h = None

    def param_specs(self):
        E, H = self.width, self.H
        out = {"dq.weight": ParamSpec((self.Rq, E)), "dq_norm.weight": ParamSpec((self.Rq,), kind="vector", init="ones_normal"),
               "uq.weight": ParamSpec((H * (self.Dn + self.Rr), self.Rq)),
               "uk.weight": ParamSpec((H * self.Dn, self.R)), "uv.weight": ParamSpec((H * self.Dv, self.R)),
               "g.weight": ParamSpec((H, E)), "o.weight": ParamSpec((E, H * self.Dv))}
        if self.own_latent:
            out["dkv.weight"] = ParamSpec((self.R + self.Rr, E))
            out["dkv_norm.weight"] = ParamSpec((self.R,), kind="vector", init="ones_normal")
        return out

    def finalize(self):
        # one product for everything that reads the mixer's input: query latent | key/value latent | gate logits
        rows = [self.w_dq_weight] + ([self.w_dkv_weight] if self.own_latent else []) + [self.w_g_weight]
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.w_dq_weight = self.w_dkv_weight = self.w_g_weight = None
        # per head: U_k,h^T as [kv_rank, dim] (a linear map from the head's plain query part) and U_v,h as [vdim, kv_rank]
        self.w_uk_t = self.w_uk_weight.view(self.H, self.Dn, self.R).transpose(1, 2).contiguous()
        self.w_uv_h = self.w_uv_weight.view(self.H, self.Dv, self.R)     # (a view: contiguous [H, vdim, kv_rank])
        self.w_uk_weight = None

    def cache_need(self):
        return CacheNeed(paged=PagedKVNeed(1, self.Dk, self.window, parts=1))

    def forward(self, x, ctx, cache, residual, accumulate=True, defer=False):
        T, H, Dn, Rr, Dv, R, Rq, Dk = ctx.n_tokens, self.H, self.Dn, self.Rr, self.Dv, self.R, self.Rq, self.Dk
        cap = ctx.token_capacity
        writes = self.own_latent
        if writes != cache.writes:
            raise ValueError("a latent mixer without a key/value projection runs as a reader of another run's cache "
                             "(and one with it as a writer)")
        # a few tokens: the product stays in partials and the next kernel sums them while it reads
        part = linear_deferred(x, self.w_in, ctx, T) if ctx.defer_residuals else None
        proj = None
        if part is None:
            proj = ctx.buf("lat_proj", (cap, self.w_in.shape[0]), torch.float32)
            linear(x, self.w_in, proj, STORE_F32, ctx, M=T)
        cq = ctx.buf("lat_cq", (cap, Rq), self.dtype)
        gate = ctx.buf("lat_gate", (cap, H), torch.float32)
        table = ctx.block_tables[cache.group]
        off_gate = Rq + (Dk if writes else 0)
        ops.latent_prep(proj, T, 0, Rq, self.w_dq_norm_weight, Rq if writes else -1, R, Rr,
                        self.w_dkv_norm_weight if writes else None, off_gate, H, ctx, table, self.rotary, cache.plane,
                        cache.page_stride, cache.page_size, cq, gate, self.eps, partials=part)
        q = ctx.buf("lat_q", (cap, H * (Dn + Rr)), self.dtype)
        linear(cq, self.w_uq_weight, q, STORE, ctx, M=T)
        qf = ctx.buf("lat_qf", (cap, H * Dk), self.dtype)
        few = T <= ops.head_linear_max_tokens()      # every head's product in one launch: a few tokens on the CUDA cores ...
        if few or ops.head_linear_mma_supported(q, Dn + Rr, self.w_uk_t, qf, Dk):     # ... many on the tensor cores
            ops.head_linear(q, Dn + Rr, self.w_uk_t, qf, Dk, T)
        else:
            for h in range(H):
                linear(q[:, h * (Dn + Rr):h * (Dn + Rr) + Dn], self.w_uk_t[h], qf[:, h * Dk:h * Dk + R], STORE, ctx, M=T)
        ops.latent_q_rope(q, qf, T, ctx.positions, self.rotary, H, Dn, Rr, R, ctx.err)
        o = ctx.buf("lat_o", (cap, H * R), self.dtype)
        single = ctx.max_q_len == 1
        part, slots = None, 0
        if single and T * -(-H // 8) < SPLIT_BELOW * attention_plan.sm_count():
            # few single tokens: their key ranges are cut among CTAs.  The number of slots depends on the
            # batch's sizes alone while a CUDA graph is captured or replayed (the longest context the table holds).
            split = ops.attention_latent_split()
            longest = table.shape[1] * cache.page_size if ctx.fixed_shapes else ctx.max_kv_len
            if self.window > 0:
                longest = min(longest, self.window + split)
            slots = longest // split + 2
            if slots <= MAX_SPLITS:
                part = ctx.buf("lat_part", (T * H * slots * (R + 2),), torch.float32)
            else:
                slots = 0
        ops.attention_latent(qf, o, gate, T, ctx, table, cache.plane, cache.page_stride, cache.page_size, H, Dk, R,
                             self.scale, self.window, single_tokens=single, part=part, split_slots=slots)
        ov = ctx.buf("lat_ov", (cap, H * Dv), self.dtype)
        if few or ops.head_linear_mma_supported(o, R, self.w_uv_h, ov, Dv):
            ops.head_linear(o, R, self.w_uv_h, ov, Dv, T)
        else:
            for h in range(H):
                linear(o[:, h * R:(h + 1) * R], self.w_uv_h[h], ov[:, h * Dv:(h + 1) * Dv], STORE, ctx, M=T)
        if defer and not accumulate:
            part = linear_deferred(ov, self.w_o_weight, ctx, T)
            if part is not None:
                return part
        linear(ov, self.w_o_weight, residual, RESIDUAL if accumulate else STORE_F32, ctx, M=T)
        return None
