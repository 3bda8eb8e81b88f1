"""The Vikupel decoder, built from parts, and its entry in the registry.

Token embedding; layers that are parallel blocks (one RMS norm read by the mixer and by a dense
gated feed-forward, their sum scaled by `residual_mult`) followed by a per-layer token input from
a second embedding table; a mixer per layer out of three: attention in a sliding window with a
logarithmic distance penalty and an output gate, causal attention with rotary positions,
unit-norm queries and keys and values turned by position, or a Mamba-2 state-space mixer.  A
range of layers may run several times in a row with the same weights: the schedule names those
blocks once per pass, and every pass gets cache planes and state rows of its own.  Final RMS norm
and an output matrix of its own.

The checkpoint's tensor names are short (`embed`, `side.embed`, `l<i>.norm1`, `l<i>.mix.q`,
`l<i>.mlp.gate`, `l<i>.side.gate`, `final.norm`, `head`); `file_names` maps them onto the
canonical names that the parts declare.
"""
from __future__ import annotations

from ..config.registry import Architecture, register
from ..config.vikupel import AttentionSpec, VikupelConfig
from ..parts import (Mamba2Mixer, OutputHead, ParallelBlock, RMSNorm, RotaryEmbedding, ShapedAttention, SwiGLU, TokenEmbedding,
                     TokenSideInput, TokenSideTable)
from .decoder import DecoderModel, Run

_VALUE_PAIRING = {"halves": "half", "interleaved": "adjacent"}


def build_vikupel(config: VikupelConfig, dtype, device, max_positions=None):
    c = config
    E = c.n_embd
    n_pos = int(max_positions or c.n_ctx_train)
    tables = {}     # rotary tables shared by the layers that turn alike

    def rotary(head_dim, dims, base, scaling, pairing):
        key = (head_dim, dims, base, scaling, pairing)
        if key not in tables:
            tables[key] = RotaryEmbedding(head_dim, dims, base, scaling, pairing, n_pos, device)
        return tables[key]

    side_table = TokenSideTable(c.n_vocab, c.n_layer * c.side_dim) if c.side_dim else None
    blocks = []
    for i, layer in enumerate(c.layers):
        m = layer.mixer
        if isinstance(m, AttentionSpec):
            rot = rotary(m.dim, m.rot_dims, m.rot_base, m.rot_scaling, "half") if m.rot_dims else None
            vrot = rotary(m.vdim, m.vdim, m.rot_base, None, _VALUE_PAIRING[m.value_layout]) if m.rotate_values else None
            mixer = ShapedAttention(E, m.heads, m.kv_heads, m.dim, m.vdim, dtype, m.scale, eps=c.norm_eps, window=m.window,
                                    rotary=rot, unit_norm=m.unit_norm, value_rotary=vrot, distance_penalty=m.distance_penalty,
                                    gate=m.gate)
        else:
            mixer = Mamba2Mixer(E, m.heads, m.vdim, m.state, m.groups, m.norm_groups, m.conv, c.norm_eps, dtype)
        ffn = SwiGLU(E, layer.mlp.ff, dtype, wide_products=True) if layer.mlp is not None else None
        side = TokenSideInput(E, c.side_dim, i * c.side_dim, side_table, c.norm_eps, dtype) if side_table is not None else None
        blocks.append(ParallelBlock(RMSNorm(E, c.norm_eps, dtype), mixer, ffn, mult=c.residual_mult, side=side))
    schedule = [Run(i) for i in c.run_order()]
    emb = TokenEmbedding(c.n_vocab, E)
    head = OutputHead(c.n_vocab, E, tied=False)
    shared = [("side_embd.", side_table)] if side_table is not None else []
    return DecoderModel(c, dtype, emb, None, blocks, RMSNorm(E, c.norm_eps, dtype), head, schedule=schedule, shared=shared)


_ATTENTION = {"mix.q": "mix.q.weight", "mix.k": "mix.k.weight", "mix.v": "mix.v.weight", "mix.o": "mix.output.weight"}
_PENALTY = {"mix.r1": "mix.r1", "mix.r2": "mix.r2"}
_GATE = {"mix.g": "mix.g.weight"}
_MAMBA2 = {"mix.in": "mix.in.weight", "mix.conv": "mix.conv.weight", "mix.conv.b": "mix.conv.bias", "mix.dt_bias": "mix.dt_bias",
           "mix.A_log": "mix.A_log", "mix.D": "mix.D", "mix.norm": "mix.norm.weight", "mix.o": "mix.o.weight"}
_MLP = {"mlp.gate": "mlp.gate.weight", "mlp.up": "mlp.up.weight", "mlp.down": "mlp.down.weight"}
_SIDE = {"side.gate": "side.gate.weight", "side.proj": "side.proj.weight", "side.norm": "side.norm.weight"}


def file_names(config: VikupelConfig):
    """{name in the checkpoint: canonical name}, for the tensors this configuration has."""
    out = {"embed": "token_embd.weight", "final.norm": "output_norm.weight", "head": "output.weight"}
    if config.side_dim:
        out["side.embed"] = "side_embd.weight"
    for i, layer in enumerate(config.layers):
        names = {"norm1": "norm1.weight"}
        m = layer.mixer
        if isinstance(m, AttentionSpec):
            names.update(_ATTENTION)
            names.update(_PENALTY if m.distance_penalty else {})
            names.update(_GATE if m.gate else {})
        else:
            names.update(_MAMBA2)
        names.update(_MLP if layer.mlp is not None else {})
        names.update(_SIDE if config.side_dim else {})
        for short, ours in names.items():
            out[f"l{i}.{short}"] = f"blk.{i}.{ours}"
    return out


register(Architecture("Vikupel", VikupelConfig.from_dict, build_vikupel, file_names), "vikupel")
