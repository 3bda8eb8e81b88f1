"""Plain, slow Ruperax: whole sequences, no cache, one function per mechanism, float64.

The oracle of the Ruperax tests.  It shares no code with the product package (its own
safetensors reader, its own reading of config.json, its own arithmetic) and keeps every key and
value of a sequence in plain arrays: no pages, no state slots, no portions.

Notation.  x is the residual stream [T, E]; a layer computes
    n  = groupnorm(x)                      (one normalisation, two weight vectors w1, w2)
    a  = n * w1,  b = n * w2
    m  = a + (shift_down(a) - a) * s       (token shift; shift_down puts row t-1 in row t, zeros in row 0)
    x += mixer(m) * sigmoid(a G1^T + g1)  +  ff(b) * sigmoid(b G2^T + g2)
and the mixer is attention whose keys and values are expanded from a small per-token latent.
"""
from __future__ import annotations

import json
import os
import struct

import numpy as np


# --------------------------------------------------------------------------- files
def read_tensors(path):
    """name -> float64 array (integer tables stay integers) of a .safetensors file."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        blob = f.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        raw, dt = blob[lo:hi], info["dtype"]
        if dt == "BF16":
            a = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        elif dt == "F32":
            a = np.frombuffer(raw, dtype="<f4").astype(np.float64)
        elif dt == "F16":
            a = np.frombuffer(raw, dtype="<f2").astype(np.float64)
        elif dt == "I32":
            a = np.frombuffer(raw, dtype="<i4").astype(np.int64)
        else:
            raise ValueError(f"plain reader: dtype {dt} of {name}")
        out[name] = a.reshape(info["shape"])
    return out


def read_model(folder):
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_tensors(os.path.join(folder, "model.safetensors"))


def round_bf16(a):
    """Round to the nearest bfloat16 (ties to even), returned as float64."""
    u = np.asarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return u.astype(np.uint32).view(np.float32).astype(np.float64)


# --------------------------------------------------------------------------- mechanisms
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def unit_rms(v, eps):
    """v / sqrt(mean(v^2) + eps) over the last axis."""
    return v / np.sqrt((v * v).mean(axis=-1, keepdims=True) + eps)


def group_norm(x, groups, eps):
    """Every row is cut into `groups` equal consecutive parts, each divided by its own root mean
    square; no weight yet."""
    T, E = x.shape
    return unit_rms(x.reshape(T, groups, E // groups), eps).reshape(T, E)


def token_shift(a, s, before=None):
    """Row t becomes a[t] + (a[t-1] - a[t]) * s; row 0 mixes with `before` (zeros when None)."""
    prev = np.zeros_like(a)
    prev[1:] = a[:-1]
    if before is not None:
        prev[0] = before
    return a + (prev - a) * s


def rotate_half(v, pos, dims, base):
    """Rotates the first `dims` elements of the last axis: element i pairs with i + dims/2 and the
    pair turns by pos * base^(-2i/dims).  v: [T, ..., D], pos: [T]."""
    half = dims // 2
    f = base ** (-2.0 * np.arange(half) / dims)
    ang = np.asarray(pos, dtype=np.float64)[:, None] * f[None, :]
    shape = (len(pos),) + (1,) * (v.ndim - 2) + (half,)
    c, s = np.cos(ang).reshape(shape), np.sin(ang).reshape(shape)
    out = v.copy()
    u, w = v[..., :half], v[..., half:dims]
    out[..., :half] = u * c - w * s
    out[..., half:dims] = w * c + u * s
    return out


def latent_of(m, w, p, mix, eps, pos):
    """What a layer with a down-projection of its own keeps per token: (latent [T, R], rotated
    shared key part [T, Rr])."""
    R, Rr = mix["kv_rank"], mix["rot_dim"]
    d = m @ w[p + "dkv"].T
    c = unit_rms(d[:, :R], eps) * w[p + "dkv.norm"]
    kr = rotate_half(d[:, R:R + Rr], pos, mix["rot"]["dims"], mix["rot"]["base"])
    return c, kr


def latent_attention(m, w, p, mix, eps, pos, latent, rounding=None):
    """The mixer on its input rows m [T, E], given the (latent, rotated key part) of every
    position of the sequence.  Keys and values are expanded per head; a query at position i sees
    keys j with 0 <= i - j < mask.size."""
    rd = rounding or (lambda z: z)
    H, Dn, Rr, Dv = mix["heads"], mix["dim"], mix["rot_dim"], mix["vdim"]
    T = m.shape[0]
    c, kr = latent
    cq = rd(unit_rms(m @ w[p + "dq"].T, eps) * w[p + "dq.norm"])
    q = rd(cq @ w[p + "uq"].T).reshape(T, H, Dn + Rr)
    q_plain = q[:, :, :Dn]
    q_rot = rotate_half(q[:, :, Dn:], pos, mix["rot"]["dims"], mix["rot"]["base"])
    k_plain = (c @ w[p + "uk"].T).reshape(-1, H, Dn)
    v = (c @ w[p + "uv"].T).reshape(-1, H, Dv)
    size = mix["mask"]["size"]
    out = np.zeros((T, H, Dv))
    for t in range(T):
        i = int(pos[t])
        lo = max(0, i - size + 1)
        s = (np.einsum("hd,jhd->hj", q_plain[t], k_plain[lo:i + 1]) + q_rot[t] @ kr[lo:i + 1].T) * mix["scale"]
        s = s - s.max(axis=1, keepdims=True)
        pw = np.exp(s)
        pw = pw / pw.sum(axis=1, keepdims=True)
        out[t] = np.einsum("hj,jhd->hd", pw, v[lo:i + 1])
    gate = sigmoid(m @ w[p + "g"].T)                   # [T, H]
    out = rd(out * gate[:, :, None])
    return out.reshape(T, H * Dv) @ w[p + "o"].T


def dense_ff(b, w, p, rounding=None):
    rd = rounding or (lambda z: z)
    act = rd(silu(b @ w[p + "gate"].T + w[p + "gate.b"]) * (b @ w[p + "up"].T + w[p + "up.b"]))
    return act @ w[p + "down"].T + w[p + "down.b"]


def gated(y, h, w, name):
    return y * sigmoid(h @ w[name].T + w[name + ".b"])


# --------------------------------------------------------------------------- the model
def forward(cfg, w, tokens, rounding=None, layers_out=None):
    """Logits [T, vocab] of one whole sequence.  rounding: None (exact arithmetic on the stored
    weights) or a function applied where a 16-bit engine rounds its activations.  layers_out: a
    list that receives the residual stream after every layer."""
    rd = rounding or (lambda z: z)
    tokens = np.asarray(tokens)
    T = len(tokens)
    pos = np.arange(T)
    eps, groups = cfg["norm"]["eps"], cfg["norm"]["groups"]
    x = w["embed"][tokens] * cfg["embedding"]["scale"] + w["pos"][pos]
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        if layer["type"] != "latent_attention":
            raise ValueError(layer["type"])
        L, mix = f"l{i}.", layer["mixer"]
        n = group_norm(x, groups, eps)
        a = n * w[L + "norm1"]
        m = rd(token_shift(a, w[L + "shift"]))
        if "kv_from" in mix:
            latent = kept[mix["kv_from"]]
        else:
            c, kr = latent_of(m, w, L + "mix.", mix, eps, pos)
            latent = kept[i] = (rd(c), rd(kr))
        y = gated(latent_attention(m, w, L + "mix.", mix, eps, pos, latent, rounding), rd(a), w, L + "rg1")
        if layer.get("mlp") is not None:
            if layer["mlp"]["kind"] != "dense":
                raise ValueError(layer["mlp"]["kind"])
            b = rd(n * w[L + "norm2"])
            y = y + gated(dense_ff(b, w, L + "mlp.", rounding), b, w, L + "rg2")
        x = x + y
        if layers_out is not None:
            layers_out.append(x.copy())
    return rd(group_norm(x, groups, eps) * w["final.norm"]) @ w["head"].T


def generate(cfg, w, prompt, n_new):
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(np.argmax(forward(cfg, w, toks)[-1])))
    return toks[len(prompt):]
