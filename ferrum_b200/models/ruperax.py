"""The Ruperax decoder, built from parts, and its entry in the registry.

Scaled token embedding plus learned positions; layers that are parallel gated blocks (one grouped
RMS norm with two weight vectors, token shift on the mixer's input, sigmoid gates on both
sublayers' results) around latent attention with a look-back window and a dense, biased, gated
feed-forward; grouped final norm; an output matrix of its own.  A layer with `kv_from` runs as a
schedule entry that reads the rows its source layer cached.

The checkpoint's tensor names are short (`embed`, `pos`, `l<i>.norm1`, `l<i>.mix.dq`,
`l<i>.mlp.gate.b`, `final.norm`, `head`); `file_names` maps them onto the canonical names that
the parts declare (`...weight` / `...bias`).
"""
from __future__ import annotations

from ..config.registry import Architecture, register
from ..config.ruperax import RuperaxConfig
from ..parts import (LatentAttention, LearnedPositions, OutputHead, ParallelGatedBlock, RMSNorm, RotaryEmbedding, SwiGLU,
                     TokenEmbedding)
from .decoder import DecoderModel, Run


def build_ruperax(config: RuperaxConfig, dtype, device, max_positions=None):
    c = config
    E = c.n_embd
    n_pos = int(max_positions or c.n_ctx_train)
    tables = {}     # (rot_dim, dims, base) -> rotary table, shared by the layers that turn alike

    def rotary(m):
        if m.rot_dims == 0:
            return None
        key = (m.rot_dim, m.rot_dims, m.rot_base)
        if key not in tables:
            tables[key] = RotaryEmbedding(m.rot_dim, m.rot_dims, m.rot_base, None, "half", n_pos, device)
        return tables[key]

    blocks, schedule = [], []
    for i, layer in enumerate(c.layers):
        m = layer.mixer
        mixer = LatentAttention(E, m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank, m.q_rank, c.norm_eps, m.scale, dtype,
                                rotary=rotary(m), window=m.window, own_latent=m.kv_from is None)
        ffn = SwiGLU(E, layer.mlp.ff, dtype, bias=True) if layer.mlp is not None else None
        blocks.append(ParallelGatedBlock(E, c.norm_eps, c.norm_groups, dtype, mixer, ffn))
        schedule.append(Run(i, cache_of=m.kv_from))
    positions = LearnedPositions(c.n_ctx_train, E)
    emb = TokenEmbedding(c.n_vocab, E, scale=c.embedding_scale, positions=positions)
    head = OutputHead(c.n_vocab, E, tied=False)
    return DecoderModel(c, dtype, emb, positions, blocks, RMSNorm(E, c.norm_eps, dtype, groups=c.norm_groups), head,
                        schedule=schedule)


_LAYER = {"norm1": "norm1.weight", "norm2": "norm2.weight", "shift": "shift.weight", "rg1": "rg1.weight", "rg1.b": "rg1.bias",
          "rg2": "rg2.weight", "rg2.b": "rg2.bias",
          "mix.dq": "mix.dq.weight", "mix.dq.norm": "mix.dq_norm.weight", "mix.uq": "mix.uq.weight",
          "mix.dkv": "mix.dkv.weight", "mix.dkv.norm": "mix.dkv_norm.weight", "mix.uk": "mix.uk.weight",
          "mix.uv": "mix.uv.weight", "mix.g": "mix.g.weight", "mix.o": "mix.o.weight",
          "mlp.gate": "mlp.gate.weight", "mlp.gate.b": "mlp.gate.bias", "mlp.up": "mlp.up.weight", "mlp.up.b": "mlp.up.bias",
          "mlp.down": "mlp.down.weight", "mlp.down.b": "mlp.down.bias"}


def file_names(config: RuperaxConfig):
    """{name in the checkpoint: canonical name}."""
    out = {"embed": "token_embd.weight", "pos": "position.weight", "final.norm": "output_norm.weight", "head": "output.weight"}
    for i in range(config.n_layer):
        for short, ours in _LAYER.items():
            out[f"l{i}.{short}"] = f"blk.{i}.{ours}"
    return out


register(Architecture("Ruperax", RuperaxConfig.from_dict, build_ruperax, file_names), "ruperax")
