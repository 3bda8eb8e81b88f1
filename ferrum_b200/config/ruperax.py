"""Typed configuration of the Ruperax decoder.

Its config.json is nested: `architecture`, `vocab`, `width`, `max_positions`, `embedding.scale`,
`norm.{eps, groups}` and `layers`, a list whose entries give the layer's `type` (which mixer), the
mixer's sizes under `mixer` and its feed-forward under `mlp` (null: none).  Every size and every
constant that can differ between two models of the design is read here and nowhere else.

Mixer `latent_attention`: heads, dim (unrotated query/key elements per head), rot_dim (rotated
elements, one key part shared by all heads), vdim, kv_rank, q_rank, scale, mask.size (how many
keys a query looks back over, itself included), rot.{base, dims}, and optionally kv_from (the
layer whose cached rows this layer reads instead of making its own).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional, Tuple

from ..errors import ConfigError


@dataclass(frozen=True)
class LatentAttentionSpec:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    window: int                 # mask.size: a query at p sees keys p - window + 1 .. p
    rot_base: float
    rot_dims: int
    kv_from: Optional[int] = None


@dataclass(frozen=True)
class DenseMlpSpec:
    ff: int
    kind: str = "dense"


@dataclass(frozen=True)
class LayerSpec:
    type: str
    mixer: LatentAttentionSpec
    mlp: Optional[DenseMlpSpec]


@dataclass(frozen=True)
class RuperaxConfig:
    architecture: str
    n_vocab: int
    n_embd: int
    n_ctx_train: int            # max_positions: rows of the learned position table
    embedding_scale: float
    norm_eps: float
    norm_groups: int
    layers: Tuple[LayerSpec, ...]
    eos_token_ids: Tuple[int, ...] = ()
    stored_dtype: str = "bfloat16"
    extra: dict = field(default_factory=dict, compare=False)

    @property
    def n_layer(self):
        return len(self.layers)

    def __post_init__(self):
        for k in ("n_vocab", "n_embd", "n_ctx_train", "norm_groups"):
            v = getattr(self, k)
            if not isinstance(v, int) or v <= 0:
                raise ConfigError(f"ruperax: {k} must be a positive integer, found {v!r}")
        if self.n_embd % self.norm_groups:
            raise ConfigError("ruperax: norm.groups does not divide width")
        if not (math.isfinite(self.norm_eps) and self.norm_eps > 0.0):
            raise ConfigError("ruperax: invalid norm.eps")
        if not self.layers:
            raise ConfigError("ruperax: no layers")
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            for k in ("heads", "dim", "vdim", "kv_rank", "q_rank", "window"):
                if getattr(m, k) <= 0:
                    raise ConfigError(f"ruperax: layer {i}: {k} must be positive")
            if m.rot_dim < 0 or m.rot_dims < 0 or m.rot_dims % 2 or m.rot_dims > m.rot_dim:
                raise ConfigError(f"ruperax: layer {i}: rot.dims must be even and at most rot_dim")
            if m.rot_dims and not (math.isfinite(m.rot_base) and m.rot_base > 0):
                raise ConfigError(f"ruperax: layer {i}: invalid rot.base")
            if m.kv_from is not None:
                if not 0 <= m.kv_from < i:
                    raise ConfigError(f"ruperax: layer {i}: kv_from must name an earlier layer")
                src = self.layers[m.kv_from].mixer
                if src.kv_from is not None:
                    raise ConfigError(f"ruperax: layer {i}: kv_from names a layer that keeps no rows of its own")
                if (src.kv_rank, src.rot_dim, src.rot_dims, src.rot_base) != (m.kv_rank, m.rot_dim, m.rot_dims, m.rot_base):
                    raise ConfigError(f"ruperax: layer {i}: kv_rank, rot_dim and rotation must equal those of layer {m.kv_from}")

    @staticmethod
    def from_dict(d: dict) -> "RuperaxConfig":
        def need(obj, key, where=""):
            if not isinstance(obj, dict) or key not in obj or obj[key] is None:
                raise ConfigError(f"config.json: missing required key {where}{key!r}")
            return obj[key]

        layers = []
        for i, L in enumerate(need(d, "layers")):
            where = f"layers[{i}]."
            kind = need(L, "type", where)
            if kind != "latent_attention":
                raise ConfigError(f"config.json: {where}type {kind!r} is not a mixer of this design")
            m = need(L, "mixer", where)
            rot = m.get("rot") or {}
            rot_dim = int(m.get("rot_dim", 0))
            spec = LatentAttentionSpec(
                heads=int(need(m, "heads", where)), dim=int(need(m, "dim", where)), rot_dim=rot_dim,
                vdim=int(need(m, "vdim", where)), kv_rank=int(need(m, "kv_rank", where)), q_rank=int(need(m, "q_rank", where)),
                scale=float(need(m, "scale", where)), window=int(need(need(m, "mask", where), "size", where + "mask.")),
                rot_base=float(rot.get("base", 10000.0)), rot_dims=int(rot.get("dims", rot_dim)),
                kv_from=None if m.get("kv_from") is None else int(m["kv_from"]))
            mlp = L.get("mlp")
            if mlp is not None:
                if need(mlp, "kind", where + "mlp.") != "dense":
                    raise ConfigError(f"config.json: {where}mlp.kind {mlp['kind']!r} is not a feed-forward of this design")
                mlp = DenseMlpSpec(ff=int(need(mlp, "ff", where + "mlp.")))
            layers.append(LayerSpec(kind, spec, mlp))
        norm = need(d, "norm")
        return RuperaxConfig(
            architecture=str(d.get("architecture") or (d.get("architectures") or ["Ruperax"])[0]),
            n_vocab=int(need(d, "vocab")), n_embd=int(need(d, "width")), n_ctx_train=int(need(d, "max_positions")),
            embedding_scale=float((d.get("embedding") or {}).get("scale", 1.0)),
            norm_eps=float(need(norm, "eps", "norm.")), norm_groups=int(norm.get("groups", 1)), layers=tuple(layers),
            stored_dtype=str(d.get("torch_dtype", "bfloat16")), extra={})
