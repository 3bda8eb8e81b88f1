"""A plain, slow Vikupel decoder in float64: whole sequences, no cache, one function per mechanism.

It shares no code with the package: it reads config.json and the safetensors file itself and
works on torch float64 tensors on the CPU.  `round_to` (a torch dtype or None) rounds where a
16-bit engine rounds: weights, the inputs of matrix products, cached keys and values.

Notation: x is the residual stream [T, E]; a layer is

    h = rms(x) * w1;   x <- x + m * (mixer(h) + ff(h))
    then the per-layer token input: e = side_table[token, i*d:(i+1)*d];  g = gelu_tanh(S_g x) * e;
    y = S_p g;  x <- x + m * rms(y) * w_s

with rms(v) = v / sqrt(mean(v^2) + eps).  A range of layers may run several times in a row with
the same weights.
"""
from __future__ import annotations

import json
import math
import os
import struct

import torch

F64 = torch.float64


# --------------------------------------------------------------------------- files
def read_safetensors(path):
    """name -> float64 (or int64) tensor."""
    with open(path, "rb") as f:
        n = struct.unpack("<Q", f.read(8))[0]
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        a, b = meta["data_offsets"]
        raw = bytearray(data[a:b])
        dt = meta["dtype"]
        if dt == "BF16":
            t = torch.frombuffer(raw, dtype=torch.bfloat16).to(F64)
        elif dt == "F16":
            t = torch.frombuffer(raw, dtype=torch.float16).to(F64)
        elif dt == "F32":
            t = torch.frombuffer(raw, dtype=torch.float32).to(F64)
        elif dt == "I32":
            t = torch.frombuffer(raw, dtype=torch.int32).to(torch.int64)
        else:
            raise ValueError(f"{name}: dtype {dt}")
        out[name] = t.reshape(meta["shape"]).clone()
    return out


def load(folder):
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(folder, "model.safetensors"))


# --------------------------------------------------------------------------- small functions
def rnd(t, round_to):
    return t if round_to is None else t.to(round_to).to(F64)


def rms(v, eps):
    return v / torch.sqrt((v * v).mean(dim=-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softplus(z):
    return torch.log1p(torch.exp(-z.abs())) + torch.clamp(z, min=0.0)


def matmul(x, w, round_to):
    """x W^T with both operands rounded as a 16-bit engine rounds them."""
    return rnd(x, round_to) @ rnd(w, round_to).T


# --------------------------------------------------------------------------- rotations
def rotary_frequencies(base, dims, scaling=None):
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    if not scaling:
        return f
    factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
    out = []
    for fi in f:
        wave = 2.0 * math.pi / fi
        if wave < orig / high:
            out.append(fi)
        elif wave > orig / low:
            out.append(fi / factor)
        else:
            s = (orig / wave - low) / (high - low)
            out.append((1.0 - s) * fi / factor + s * fi)
    return out


def rotate(v, positions, freqs, dims, layout="halves", sign=1.0):
    """v [T, heads, D]: the first `dims` elements of every head turn by sign * position * freqs;
    pairs are (i, i + dims/2) for "halves" and (2i, 2i+1) for "interleaved"."""
    out = v.clone()
    half = dims // 2
    ang = sign * positions.to(F64)[:, None] * torch.tensor(freqs, dtype=F64)[None, :]      # [T, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    if layout == "halves":
        a, b = v[..., :half], v[..., half:dims]
        out[..., :half] = a * c - b * s
        out[..., half:dims] = b * c + a * s
    else:
        a, b = v[..., 0:dims:2], v[..., 1:dims:2]
        out[..., 0:dims:2] = a * c - b * s
        out[..., 1:dims:2] = b * c + a * s
    return out


# --------------------------------------------------------------------------- mixers
def softmax_attention(q, k, v, scale, allowed, bias=None):
    """q [T, H, D], k [T, G, D], v [T, G, Dv]; allowed [T, T] bool; bias [H, T, T] is subtracted."""
    T, H, _ = q.shape
    G = k.shape[1]
    rep = H // G
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for h in range(H):
        g = h // rep
        s = (q[:, h] @ k[:, g].T) * scale
        if bias is not None:
            s = s - bias[h]
        s = s.masked_fill(~allowed, float("-inf"))
        out[:, h] = torch.softmax(s, dim=-1) @ v[:, g]
    return out


def mixer_window_attention(h, w, p, mc, round_to):
    """Sliding window, a logarithmic distance penalty r1 * ln(1 + r2 * distance) per head, no rotation,
    and a sigmoid gate on the heads' outputs."""
    T = h.shape[0]
    H, G, D, Dv = mc["heads"], mc["kv_heads"], mc["dim"], mc["vdim"]
    q = matmul(h, w[p + "q"], round_to).view(T, H, D)
    k = matmul(h, w[p + "k"], round_to).view(T, G, D)
    v = matmul(h, w[p + "v"], round_to).view(T, G, Dv)
    q, k, v = rnd(q, round_to), rnd(k, round_to), rnd(v, round_to)
    i = torch.arange(T)
    dist = (i[:, None] - i[None, :])
    window = mc["mask"]["size"]
    allowed = (dist >= 0) & (dist < window)
    d = dist.clamp(min=0).to(F64)
    bias = w[p + "r1"][:, None, None] * torch.log1p(w[p + "r2"][:, None, None] * d[None])
    o = softmax_attention(q, k, v, mc["scale"], allowed, bias)
    gate = torch.sigmoid(matmul(h, w[p + "g"], round_to)).view(T, H, Dv)
    return matmul((o * gate).reshape(T, H * Dv), w[p + "o"], round_to)


def mixer_rotary_attention(h, w, p, mc, eps, round_to):
    """Causal; q and k turn (scaled frequencies) and are then divided by their root mean square per
    head; the value of position j turns by j over all of vdim (unscaled frequencies) and every
    head's output at position i turns back by i."""
    T = h.shape[0]
    H, G, D, Dv = mc["heads"], mc["kv_heads"], mc["dim"], mc["vdim"]
    rot = mc["rot"]
    value_layout = rot.get("value_layout", "halves")
    pos = torch.arange(T)
    q = matmul(h, w[p + "q"], round_to).view(T, H, D)
    k = matmul(h, w[p + "k"], round_to).view(T, G, D)
    v = matmul(h, w[p + "v"], round_to).view(T, G, Dv)
    fk = rotary_frequencies(float(rot["base"]), int(rot["dims"]), rot.get("scaling"))
    q = rms(rotate(q, pos, fk, int(rot["dims"])), eps)
    k = rms(rotate(k, pos, fk, int(rot["dims"])), eps)
    fv = rotary_frequencies(float(rot["base"]), Dv)
    v = rotate(v, pos, fv, Dv, value_layout)
    q, k, v = rnd(q, round_to), rnd(k, round_to), rnd(v, round_to)
    allowed = pos[:, None] >= pos[None, :]
    o = softmax_attention(q, k, v, mc["scale"], allowed)
    o = rotate(o, pos, fv, Dv, value_layout, sign=-1.0)
    return matmul(o.reshape(T, H * Dv), w[p + "o"], round_to)


def causal_conv(u, kernel, bias):
    """u [T, C]; kernel [C, taps], its last column multiplies the current token; zeros before the start."""
    T, C = u.shape
    taps = kernel.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=F64), u], dim=0)
    out = bias[None, :].expand(T, C).clone()
    for j in range(taps):
        out = out + padded[j:j + T] * kernel[:, j][None, :]
    return out


def mixer_mamba2(h, w, p, mc, eps, round_to):
    T = h.shape[0]
    Hh, P, N, G = mc["heads"], mc["vdim"], mc["state"], mc["groups"]
    inner = Hh * P
    proj = matmul(h, w[p + "in"], round_to)
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].view(T, Hh, P)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + w[p + "dt_bias"][None, :])                     # [T, heads]
    decay = torch.exp(-torch.exp(w[p + "A_log"])[None, :] * dt)       # [T, heads]
    y = torch.zeros(T, Hh, P, dtype=F64)
    S = torch.zeros(Hh, N, P, dtype=F64)
    per = Hh // G
    for t in range(T):
        for hd in range(Hh):
            g = hd // per
            S[hd] = decay[t, hd] * S[hd] + dt[t, hd] * torch.outer(B[t, g], x[t, hd])
            y[t, hd] = S[hd].T @ C[t, g] + w[p + "D"][hd] * x[t, hd]
    y = y.reshape(T, inner) * silu(z)
    ng = mc["norm_groups"]
    y = rms(y.view(T, ng, inner // ng), eps).reshape(T, inner) * w[p + "norm"][None, :]
    return matmul(y, w[p + "o"], round_to)


# --------------------------------------------------------------------------- feed-forward, side input
def dense_ff(h, w, p, round_to):
    a = silu(matmul(h, w[p + "gate"], round_to)) * matmul(h, w[p + "up"], round_to)
    return matmul(a, w[p + "down"], round_to)


def side_input(x, tokens, i, w, cfg, eps, round_to):
    d = cfg["token_side"]["dim"]
    e = rnd(w["side.embed"], round_to)[tokens][:, i * d:(i + 1) * d]
    g = gelu_tanh(matmul(x, w[f"l{i}.side.gate"], round_to)) * e
    y = matmul(g, w[f"l{i}.side.proj"], round_to)
    return rms(y, eps) * w[f"l{i}.side.norm"][None, :]


# --------------------------------------------------------------------------- the model
def run_order(cfg):
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def layer(x, tokens, i, w, cfg, round_to):
    L = cfg["layers"][i]
    eps, m = float(cfg["norm"]["eps"]), float(cfg.get("residual_mult", 1.0))
    h = rms(x, eps) * w[f"l{i}.norm1"][None, :]
    p = f"l{i}.mix."
    kind = L["type"]
    if kind == "mamba2":
        y = mixer_mamba2(h, w, p, L["mixer"], eps, round_to)
    elif kind == "attention":
        y = mixer_window_attention(h, w, p, L["mixer"], round_to)
    elif kind == "attention_2":
        y = mixer_rotary_attention(h, w, p, L["mixer"], eps, round_to)
    else:
        raise ValueError(kind)
    if L.get("mlp") is not None:
        y = y + dense_ff(h, w, f"l{i}.mlp.", round_to)
    x = x + m * y
    if cfg.get("token_side"):
        x = x + m * side_input(x, tokens, i, w, cfg, eps, round_to)
    return x


def forward(cfg, w, tokens, round_to=None, taps=None):
    """Logits [T, vocab] of one sequence; `taps` (a list) receives the residual stream after every layer run."""
    tokens = torch.as_tensor(tokens, dtype=torch.int64)
    x = rnd(w["embed"], round_to)[tokens].clone()
    for i in run_order(cfg):
        x = layer(x, tokens, i, w, cfg, round_to)
        if taps is not None:
            taps.append(x.clone())
    eps = float(cfg["norm"]["eps"])
    x = rms(x, eps) * w["final.norm"][None, :]
    return matmul(x, w["head"], round_to)
