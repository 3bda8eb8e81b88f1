"""Typed configuration of the Vikupel decoder.

Its config.json is nested: `architecture`, `vocab`, `width`, `norm.eps`, `residual_mult`,
`token_side.dim` (the per-layer slice of a second embedding table; absent: no such input), `loop`
(`start`, `stop`, `times`: layers start .. stop-1 run `times` times in a row) and `layers`, a list
whose entries give the layer's `type` (which mixer), the mixer's sizes under `mixer` and its
feed-forward under `mlp` (null: none).  Every size and every constant that can differ between two
models of the design is read here and nowhere else.

Mixers:
  `attention`    heads, kv_heads, dim, vdim, scale, mask.size (a query sees itself and the
                 mask.size - 1 keys before it; no `mask`: every earlier key); a distance penalty and
                 an output gate (their numbers are tensors).
  `attention_2`  heads, kv_heads, dim, vdim, scale, rot.{base, dims, scaling.{factor, low, high,
                 original}} (the scaling block may be absent); causal (or `mask.size` as above), unit-norm
                 queries and keys, values turned by position.  `rot.value_layout` ("halves", the default, or
                 "interleaved") names how a value's elements pair up.
  `mamba2`       heads, vdim, state, groups, norm_groups, conv (taps).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional, Tuple, Union

from ..errors import ConfigError
from .llama import RopeScaling


@dataclass(frozen=True)
class AttentionSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int = 0                         # 0: every earlier key
    distance_penalty: bool = False
    gate: bool = False
    rot_base: float = 0.0
    rot_dims: int = 0                       # 0: no rotation
    rot_scaling: Optional[RopeScaling] = None
    unit_norm: bool = False
    rotate_values: bool = False
    value_layout: str = "halves"


@dataclass(frozen=True)
class Mamba2Spec:
    heads: int
    vdim: int
    state: int
    groups: int
    norm_groups: int
    conv: int


@dataclass(frozen=True)
class DenseMlpSpec:
    ff: int
    kind: str = "dense"


@dataclass(frozen=True)
class LayerSpec:
    type: str
    mixer: Union[AttentionSpec, Mamba2Spec]
    mlp: Optional[DenseMlpSpec]


@dataclass(frozen=True)
class LoopSpec:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class VikupelConfig:
    architecture: str
    n_vocab: int
    n_embd: int
    norm_eps: float
    residual_mult: float
    side_dim: int                           # 0: no per-layer token input
    layers: Tuple[LayerSpec, ...]
    loop: Optional[LoopSpec] = None
    n_ctx_train: int = 8192                 # positions the rotary tables cover unless the caller asks for more or fewer
    eos_token_ids: Tuple[int, ...] = ()
    stored_dtype: str = "bfloat16"
    extra: dict = field(default_factory=dict, compare=False)

    @property
    def n_layer(self):
        return len(self.layers)

    def run_order(self):
        """Layer indices in the order they run (a looped range is listed once per pass)."""
        n = len(self.layers)
        if self.loop is None:
            return list(range(n))
        a, b, k = self.loop.start, self.loop.stop, self.loop.times
        return list(range(a)) + list(range(a, b)) * k + list(range(b, n))

    def __post_init__(self):
        for k in ("n_vocab", "n_embd"):
            v = getattr(self, k)
            if not isinstance(v, int) or v <= 0:
                raise ConfigError(f"vikupel: {k} must be a positive integer, found {v!r}")
        if not (math.isfinite(self.norm_eps) and self.norm_eps > 0.0):
            raise ConfigError("vikupel: invalid norm.eps")
        if not math.isfinite(self.residual_mult):
            raise ConfigError("vikupel: invalid residual_mult")
        if self.side_dim < 0:
            raise ConfigError("vikupel: token_side.dim must not be negative")
        if not self.layers:
            raise ConfigError("vikupel: no layers")
        if self.loop is not None:
            lp = self.loop
            if not (0 <= lp.start <= lp.stop <= len(self.layers)) or lp.times < 1:
                raise ConfigError(f"vikupel: loop {lp.start}..{lp.stop} x {lp.times} does not fit {len(self.layers)} layers")
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            if isinstance(m, AttentionSpec):
                for k in ("heads", "kv_heads", "dim", "vdim"):
                    if getattr(m, k) <= 0:
                        raise ConfigError(f"vikupel: layer {i}: {k} must be positive")
                if m.heads % m.kv_heads:
                    raise ConfigError(f"vikupel: layer {i}: kv_heads does not divide heads")
                if m.window < 0:
                    raise ConfigError(f"vikupel: layer {i}: mask.size must be positive")
                if m.rot_dims % 2 or m.rot_dims > m.dim or m.rot_dims < 0:
                    raise ConfigError(f"vikupel: layer {i}: rot.dims must be even and at most dim")
                if m.rot_dims and not (math.isfinite(m.rot_base) and m.rot_base > 0):
                    raise ConfigError(f"vikupel: layer {i}: invalid rot.base")
                if m.rotate_values and (m.vdim % 2 or not (math.isfinite(m.rot_base) and m.rot_base > 0)):
                    raise ConfigError(f"vikupel: layer {i}: rotated values need an even vdim and a rot.base")
                if m.value_layout not in ("halves", "interleaved"):
                    raise ConfigError(f"vikupel: layer {i}: unknown value layout {m.value_layout!r}")
            else:
                for k in ("heads", "vdim", "state", "groups", "norm_groups", "conv"):
                    if getattr(m, k) <= 0:
                        raise ConfigError(f"vikupel: layer {i}: {k} must be positive")
                if m.heads % m.groups:
                    raise ConfigError(f"vikupel: layer {i}: groups does not divide heads")
                if (m.heads * m.vdim) % m.norm_groups:
                    raise ConfigError(f"vikupel: layer {i}: norm_groups does not divide heads * vdim")

    @staticmethod
    def from_dict(d: dict) -> "VikupelConfig":
        def need(obj, key, where=""):
            if not isinstance(obj, dict) or key not in obj or obj[key] is None:
                raise ConfigError(f"config.json: missing required key {where}{key!r}")
            return obj[key]

        layers = []
        for i, L in enumerate(need(d, "layers")):
            where = f"layers[{i}]."
            kind = need(L, "type", where)
            m = need(L, "mixer", where)
            mw = where + "mixer."
            if kind in ("attention", "attention_2"):
                # what the entry does not mention does not exist: no `mask` means every earlier key, no `rot` no rotation
                window = 0
                if m.get("mask") is not None:
                    window = int(need(m["mask"], "size", mw + "mask."))
                    if window <= 0:
                        raise ConfigError(f"config.json: {mw}mask.size must be positive")
                rot = m.get("rot")
                if kind == "attention_2":
                    rot = need(m, "rot", mw)
                scaling, rot_base, rot_dims, layout = None, 0.0, 0, "halves"
                if rot is not None:
                    sc = rot.get("scaling")
                    if sc:
                        sw = mw + "rot.scaling."
                        scaling = RopeScaling("llama3", float(need(sc, "factor", sw)), float(need(sc, "low", sw)),
                                              float(need(sc, "high", sw)), int(need(sc, "original", sw)))
                    rot_base, rot_dims = float(need(rot, "base", mw + "rot.")), int(need(rot, "dims", mw + "rot."))
                    layout = str(rot.get("value_layout", "halves"))
                second = kind == "attention_2"
                spec = AttentionSpec(
                    heads=int(need(m, "heads", mw)), kv_heads=int(need(m, "kv_heads", mw)), dim=int(need(m, "dim", mw)),
                    vdim=int(need(m, "vdim", mw)), scale=float(need(m, "scale", mw)), window=window,
                    distance_penalty=not second, gate=not second, rot_base=rot_base, rot_dims=rot_dims, rot_scaling=scaling,
                    unit_norm=second, rotate_values=second, value_layout=layout)
            elif kind == "mamba2":
                spec = Mamba2Spec(heads=int(need(m, "heads", mw)), vdim=int(need(m, "vdim", mw)), state=int(need(m, "state", mw)),
                                  groups=int(need(m, "groups", mw)), norm_groups=int(need(m, "norm_groups", mw)),
                                  conv=int(need(m, "conv", mw)))
            else:
                raise ConfigError(f"config.json: {where}type {kind!r} is not a mixer of this design")
            mlp = L.get("mlp")
            if mlp is not None:
                if need(mlp, "kind", where + "mlp.") != "dense":
                    raise ConfigError(f"config.json: {where}mlp.kind {mlp['kind']!r} is not a feed-forward of this design")
                mlp = DenseMlpSpec(ff=int(need(mlp, "ff", where + "mlp.")))
            layers.append(LayerSpec(kind, spec, mlp))
        loop = d.get("loop")
        if loop:
            loop = LoopSpec(int(need(loop, "start", "loop.")), int(need(loop, "stop", "loop.")), int(need(loop, "times", "loop.")))
        side = d.get("token_side") or {}
        return VikupelConfig(
            architecture=str(d.get("architecture") or (d.get("architectures") or ["Vikupel"])[0]),
            n_vocab=int(need(d, "vocab")), n_embd=int(need(d, "width")), norm_eps=float(need(need(d, "norm"), "eps", "norm.")),
            residual_mult=float(d.get("residual_mult", 1.0)), side_dim=int(side.get("dim", 0)), layers=tuple(layers),
            loop=loop or None, n_ctx_train=int(d.get("max_positions", 8192)),
            stored_dtype=str(d.get("torch_dtype", "bfloat16")), extra={})
