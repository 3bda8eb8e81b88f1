"""Vikupel on the GPU against the plain implementation (plain_vikupel.py): every mechanism alone,
then whole models under every way of cutting the work, then generation through the engine."""
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_vikupel as P
from helpers import Replay, assert_close_16bit, assert_close_f32, mixed_schedule, pages_were_reused, peak_pages
from vikupel_configs import VIKUPEL, write_model

pytestmark = pytest.mark.gpu
TD = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}
F64 = torch.float64


def rounding_of(dtype):
    return None if dtype == "float32" else TD[dtype]


def close(x, ref, dtype, what):
    (assert_close_f32 if dtype == "float32" else assert_close_16bit)(x, ref, what)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: write_model(cfg, str(tmp_path_factory.mktemp("vikupel_" + name)), seed) for name, (cfg, seed) in VIKUPEL.items()}


def plain(folder, dtype, tokens):
    cfg, w = P.load(folder)
    return P.forward(cfg, w, tokens, rounding_of(dtype)).numpy()


def session(folder, dtype, max_tokens, **kw):
    from ferrum_b200.engine.trace import TraceSession
    return TraceSession(folder, dtype, max_tokens, **kw)


def tokens_for(name, n, seed):
    return np.random.default_rng(seed).integers(0, VIKUPEL[name][0]["vocab"], n).tolist()


def make_ctx(entries, slots=None, max_tokens=1024, max_requests=8, widths=()):
    """A step context for [(pos0, n tokens)] entries, with explicit block tables per group."""
    from ferrum_b200.engine.batch import StepContext, StepEntry
    ctx = StepContext("cuda", max_tokens, max_requests, [len(t[0]) for t in widths])
    es = [StepEntry(slots[i] if slots else i, p0, list(range(n))) for i, (p0, n) in enumerate(entries)]
    ctx.fill(es, [list(t) for t in widths])
    return ctx


class OneMixer:
    """The least a cache needs of a model: a schedule and the needs of its runs."""

    def __init__(self, mixers):
        from ferrum_b200.models import Run
        self.mixers, self.schedule = mixers, [Run(i) for i in range(len(mixers))]

    def cache_needs(self):
        return [m.cache_need() for m in self.mixers]


def fill_part(part, seed, td, prefix, std=0.3, fixed=None):
    """Random parameters for a part; returns them under the plain implementation's names (float64)."""
    from ferrum_b200.weights.random_init import _tensor
    w = {}
    for name, ps in part.param_specs().items():
        t = _tensor(f"{prefix}{name}", ps, seed, "cuda", std if ps.kind == "matrix" else 0.2)
        if fixed and name in fixed:
            t = fixed[name].to("cuda")
        t = t.to(td) if ps.kind == "matrix" else t.float()
        part.assign(name, t.contiguous())
        short = name.replace("output.weight", "o").replace("conv.bias", "conv.b").replace(".weight", "")
        w[prefix + short] = t.double().cpu()
    part.finalize()
    return w


# ================================================================= the attention kernel alone
def attention_reference(q, k, v, pos, H, G, scale, window, r1=None, r2=None):
    """q [n, H, D] of queries at `pos`; k, v [keys, G, D]: float64 softmax over the visible keys."""
    out = np.zeros((len(pos), H, v.shape[2]))
    for t, p in enumerate(pos):
        lo = max(0, p - window + 1) if window > 0 else 0
        for h in range(H):
            g = h // (H // G)
            s = k[lo:p + 1, g] @ q[t, h] * scale
            if r1 is not None:
                s = s - r1[h] * np.log1p(r2[h] * (p - np.arange(lo, p + 1)))
            w = np.exp(s - s.max())
            out[t, h] = (w / w.sum()) @ v[lo:p + 1, g]
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,D,page,window,penalty", [(3, 1, 14, 8, 19, True), (4, 2, 64, 16, 0, False), (6, 2, 80, 16, 130, True),
                                                         (5, 5, 40, 32, 64, False), (8, 2, 128, 16, 0, True), (2, 1, 200, 8, 257, True)])
def test_attention_sees_exactly_its_window_and_takes_the_penalty(cuda, dtype, H, G, D, page, window, penalty):
    """The CUDA-core attention kernel on keys and values written straight into pages that lie
    scattered in the pool, float32 results out.  One key is made to dominate: it is scaled up and
    every query points at it.  Placed at the last position a query may see (the first row of a
    page), its value is the output; one query later it is gone.  Without a window it sits far back
    among hundreds.  A prompt portion, a single token over the whole range, and a single token
    whose key range is cut among CTAs."""
    from ferrum_b200.ops import lib as ops
    rng = np.random.default_rng(H * 1000 + D)
    n_keys, td = 700, TD[dtype]
    n_pages = -(-n_keys // page)
    order = rng.permutation(n_pages + 5)[:n_pages]
    k = rng.standard_normal((n_keys, G, D)) * 0.3
    v = rng.standard_normal((n_keys, G, D))
    hot = 37 if window == 0 else (n_keys - 1 - (window - 1) - 3) // page * page
    k[hot] *= 5.0
    kt, vt = torch.tensor(k, device="cuda").to(td), torch.tensor(v, device="cuda").to(td)
    k, v = kt.double().cpu().numpy(), vt.double().cpu().numpy()
    plane = torch.zeros(n_pages + 5, 2, G, page, D, device="cuda", dtype=td)
    for lp in range(n_pages):
        n = min(page, n_keys - lp * page)
        plane[order[lp], 0, :, :n] = kt[lp * page:lp * page + n].transpose(0, 1)
        plane[order[lp], 1, :, :n] = vt[lp * page:lp * page + n].transpose(0, 1)
    r1 = torch.rand(H, device="cuda") * 1.5 if penalty else None
    r2 = torch.rand(H, device="cuda") + 0.05 if penalty else None
    scale = 0.5
    for pos0, n in ((n_keys - 40, 40), (n_keys - 1, 1), (hot + max(window, 1) - 2, 3), (0, 9)):
        ctx = make_ctx([(pos0, n)], widths=[[list(order)]])
        pos = list(range(pos0, pos0 + n))
        q = np.tile(k[hot].repeat(H // G, axis=0).reshape(1, H * D) * 4.0, (n, 1)) + rng.standard_normal((n, H * D)) * 0.1
        qt = torch.tensor(q, device="cuda").to(td)
        ref = attention_reference(qt.double().cpu().numpy().reshape(n, H, D), k, v, pos, H, G, scale, window,
                                  r1.double().cpu().numpy() if penalty else None, r2.double().cpu().numpy() if penalty else None)
        for mode in (["rows", "tokens", "split"] if n == 1 else ["rows", "tokens"]):
            out = torch.full((n, H * D), float("nan"), device="cuda")
            part, slots, q_start = None, 0, None
            if mode == "split":
                split = ops.attention_generic_split()
                slots = (min(n_keys, window + split) if window else n_keys) // split + 2
                part = torch.full((n * H * slots * (D + 2),), float("nan"), device="cuda")
            if mode == "tokens":
                q_start = ctx.q_start
            ops.attention_generic(qt, out, n, ctx.positions, ctx.req_of_token, ctx.block_tables[0], plane, plane.stride(0), page,
                                  H, G, D, scale, window, ctx.err, part=part, split_slots=slots, q_start=q_start, n_reqs=1,
                                  distance_penalty=(r1, r2) if penalty else None)
            got = out.double().cpu().numpy().reshape(n, H, D)
            assert np.abs(got - ref).max() < (2e-5 if dtype == "float32" else 2e-2) * np.abs(ref).max(), (pos0, n, mode)
            assert ctx.err.item() == 0
        if window > 0 and pos0 > 0:
            for t, p in enumerate(pos):
                if p - window + 1 <= hot <= p and not penalty:
                    assert np.abs(got[t, 0] - v[hot, 0]).max() < 0.05 * np.abs(v[hot]).max(), (p, hot)
                elif p - window + 1 == hot + 1:
                    assert np.abs(got[t, 0] - v[hot, 0]).max() > 0.3 * np.abs(v[hot, 0]).max(), (p, hot)
        if window == 0 and pos0 > 0 and not penalty:
            assert np.abs(got[-1, 0] - v[hot, 0]).max() < 0.05 * np.abs(v[hot]).max()      # the far key among hundreds


# ================================================================= shaping of heads
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("Hq,Hkv,Dk,Dv,R,pair,vpair,norm", [(3, 1, 10, 14, 6, "half", "adjacent", True), (4, 2, 64, 64, 64, "half", "half", True),
                                                             (2, 2, 12, 6, 0, "half", None, False), (5, 5, 32, 48, 16, "adjacent", "half", False)])
def test_heads_are_shaped_cached_and_turned_back(cuda, dtype, Hq, Hkv, Dk, Dv, R, pair, vpair, norm):
    from ferrum_b200.ops import lib as ops
    from ferrum_b200.parts import RotaryEmbedding
    td, eps, page, T = TD[dtype], 1e-3, 8, 21
    Dp = max(Dk, Dv)
    g = torch.Generator(device="cuda").manual_seed(Dk)
    scaling = {"factor": 2.0, "low": 1.0, "high": 2.0, "original": 16}
    rot = RotaryEmbedding(Dk, R, 100.0, None, pair, 64, "cuda", frequencies=P.rotary_frequencies(100.0, R, scaling)) if R else None
    vrot = RotaryEmbedding(Dv, Dv, 100.0, None, vpair, 64, "cuda") if vpair else None
    entries, slots = [(30, 12), (0, 9)], None
    order = [[5, 2, 7, 0, 9, 1], [3, 8, 4, 6, -1, -1]]
    ctx = make_ctx(entries, widths=[order])
    proj = torch.randn(T, Hq * Dk + Hkv * (Dk + Dv) + Hq * Dv + 3, device="cuda", generator=g) * 2
    plane = torch.full((10, 2, Hkv, page, Dp), 7.0, device="cuda", dtype=td)
    q = torch.full((T, Hq * Dp), 7.0, device="cuda", dtype=td)
    ops.qkv_shape(proj, T, ctx, ctx.block_tables[0], rot, rot.pairing if rot else 0, vrot.cos_sin if vrot else None,
                  vrot.pairing if vrot else 0, norm, eps, q, plane, plane.stride(0), page, Hq, Hkv, Dk, Dv, Dp, True)
    assert ctx.err.item() == 0
    pos = torch.tensor(list(range(30, 42)) + list(range(9)))
    pd = proj.double().cpu()
    layout = {"half": "halves", "adjacent": "interleaved"}
    fk = P.rotary_frequencies(100.0, R, scaling) if R else []
    qr = pd[:, :Hq * Dk].view(T, Hq, Dk)
    kr = pd[:, Hq * Dk:(Hq + Hkv) * Dk].view(T, Hkv, Dk)
    vr = pd[:, (Hq + Hkv) * Dk:(Hq + Hkv) * Dk + Hkv * Dv].view(T, Hkv, Dv)
    if R:
        qr, kr = P.rotate(qr, pos, fk, R, layout[pair]), P.rotate(kr, pos, fk, R, layout[pair])
    if norm:
        qr, kr = P.rms(qr, eps), P.rms(kr, eps)
    fv = P.rotary_frequencies(100.0, Dv)
    if vpair:
        vr = P.rotate(vr, pos, fv, Dv, layout[vpair])
    tol = 1e-5 if dtype == "float32" else 1e-2
    got_q = q.double().cpu().view(T, Hq, Dp)
    assert (got_q[..., :Dk] - qr).abs().max() < tol * max(1.0, qr.abs().max()) and got_q[..., Dk:].abs().sum() == 0
    for t in range(T):
        r, p = (0, int(pos[t])) if t < 12 else (1, int(pos[t]))
        pg = order[r][p // page]
        krow, vrow = plane[pg, 0, :, p % page].double().cpu(), plane[pg, 1, :, p % page].double().cpu()
        assert (krow[:, :Dk] - kr[t]).abs().max() < tol * max(1.0, kr.abs().max()) and krow[:, Dk:].abs().sum() == 0
        assert (vrow[:, :Dv] - vr[t]).abs().max() < tol * max(1.0, vr.abs().max()) and vrow[:, Dv:].abs().sum() == 0
    # the way back: heads' results turn by minus the position and meet the gate
    o = torch.randn(T, Hq * Dp, device="cuda", generator=g)
    off = Hq * Dk + Hkv * (Dk + Dv)
    for gated in (True, False):
        out = torch.zeros(T, Hq * Dv, device="cuda", dtype=td)
        ops.attention_finish(o, T, ctx, vrot.cos_sin if vrot else None, vrot.pairing if vrot else 0,
                             proj[:, off:off + Hq * Dv] if gated else None, out, Hq, Dv, Dp)
        ref = o.double().cpu().view(T, Hq, Dp)[..., :Dv]
        if vpair:
            ref = P.rotate(ref, pos, fv, Dv, layout[vpair], sign=-1.0)
        if gated:
            ref = ref * torch.sigmoid(pd[:, off:off + Hq * Dv].view(T, Hq, Dv))
        assert (out.double().cpu().view(T, Hq, Dv) - ref).abs().max() < tol * max(1.0, ref.abs().max())
    # a page that is missing from the table raises the step's flag instead of a wild write
    ctx2 = make_ctx([(30, 12), (0, 9)], widths=[[[5, 2, 7, -1, 9, 1], order[1]]])
    ops.qkv_shape(proj, T, ctx2, ctx2.block_tables[0], rot, rot.pairing if rot else 0, None, 0, norm, eps, q, plane,
                  plane.stride(0), page, Hq, Hkv, Dk, Dv, Dp, True)
    assert ctx2.err.item() == 4


# ================================================================= mixers alone, whole and in portions
def run_mixer_in_portions(mixer, x, cuts, td, max_tokens=128, page=8):
    from ferrum_b200.cache import CacheStorage
    from ferrum_b200.engine.batch import StepContext, StepEntry
    cache = CacheStorage(OneMixer([mixer]), td, "cuda", page_size=page, max_tokens=max_tokens, max_requests=3, max_model_len=max_tokens)
    ctx = StepContext("cuda", max_tokens, 3, [cache.table_width] * cache.n_groups)
    cache.open()                              # the request under test takes the second slot
    slot = cache.open()
    got, at = [], 0
    for n in cuts:
        cache.manager.grow(slot, at + n)
        ctx.fill([StepEntry(slot, at, list(range(n)))], cache.manager if cache.n_groups else [])
        y = torch.zeros(n, x.shape[1], device="cuda")
        mixer.forward(x[at:at + n].contiguous(), ctx, cache.layer_cache(0), y, accumulate=False)
        assert ctx.err.item() == 0
        got.append(y.double().cpu())
        cache.manager.commit(slot, at + n)
        at += n
    return torch.cat(got)


CUTS = ([61], [20, 1, 1, 2, 30, 7], [2] * 30 + [1])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,P_,N,G,ng,taps", [(4, 6, 20, 2, 3, 3), (8, 16, 64, 1, 1, 4), (2, 64, 16, 2, 4, 2), (1, 8, 8, 1, 1, 1),
                                                   (3, 40, 130, 3, 5, 5)])
def test_state_space_mixer_alone(cuda, dtype, heads, P_, N, G, ng, taps):
    """The recurrent mixer on given rows: whole, in portions (the state and the convolution's last
    inputs carried in the request's state row), and token pairs."""
    from ferrum_b200.parts import Mamba2Mixer
    td, E, eps = TD[dtype], 40, 1e-5
    mx = Mamba2Mixer(E, heads, P_, N, G, ng, taps, eps, td)
    # slow decays, so that a state lost at a portion's border would show for many tokens
    w = fill_part(mx, 7, td, "p.", fixed={"A_log": torch.linspace(-3.5, -1.0, heads), "dt_bias": torch.linspace(-1.0, 0.5, heads)})
    w = {k.replace("p.o.weight", "p.o"): v for k, v in w.items()}
    x = torch.randn(61, E, device="cuda", generator=torch.Generator(device="cuda").manual_seed(8)).to(td)
    mc = {"heads": heads, "vdim": P_, "state": N, "groups": G, "norm_groups": ng}
    ref = P.mixer_mamba2(x.double().cpu(), w, "p.", mc, eps, rounding_of(dtype))
    for cuts in CUTS:
        got = run_mixer_in_portions(mx, x, cuts, td)
        assert (got - ref).abs().max() < (2e-4 if dtype == "float32" else 4e-2) * ref.abs().max(), cuts


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind,H,G,Dk,Dv", [("window", 3, 1, 10, 14), ("window", 6, 2, 80, 80), ("rotary", 4, 2, 64, 64), ("rotary", 2, 2, 12, 10),
                                            ("rotary", 4, 1, 8, 24)])
def test_attention_mixers_alone(cuda, dtype, kind, H, G, Dk, Dv):
    from ferrum_b200.parts import RotaryEmbedding, ShapedAttention
    td, E, eps = TD[dtype], 40, 1e-5
    scaling = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 32}
    if kind == "window":
        mx = ShapedAttention(E, H, G, Dk, Dv, td, 0.3, eps=eps, window=17, distance_penalty=True, gate=True)
        mc = {"heads": H, "kv_heads": G, "dim": Dk, "vdim": Dv, "scale": 0.3, "mask": {"size": 17}}
    else:
        R = Dk // 4 * 2
        rot = RotaryEmbedding(Dk, R, 1000.0, None, "half", 128, "cuda", frequencies=P.rotary_frequencies(1000.0, R, scaling))
        vrot = RotaryEmbedding(Dv, Dv, 1000.0, None, "half", 128, "cuda")
        mx = ShapedAttention(E, H, G, Dk, Dv, td, 0.9, eps=eps, rotary=rot, unit_norm=True, value_rotary=vrot)
        mc = {"heads": H, "kv_heads": G, "dim": Dk, "vdim": Dv, "scale": 0.9, "rot": {"base": 1000.0, "dims": R, "scaling": scaling}}
    w = fill_part(mx, 9, td, "p.")
    x = torch.randn(61, E, device="cuda", generator=torch.Generator(device="cuda").manual_seed(10)).to(td)
    rd = rounding_of(dtype)
    ref = (P.mixer_window_attention(x.double().cpu(), w, "p.", mc, rd) if kind == "window"
           else P.mixer_rotary_attention(x.double().cpu(), w, "p.", mc, eps, rd))
    for cuts in CUTS:
        got = run_mixer_in_portions(mx, x, cuts, td)
        assert (got - ref).abs().max() < (2e-4 if dtype == "float32" else 4e-2) * ref.abs().max(), cuts


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_parallel_sum_and_token_side_input(cuda, dtype):
    from ferrum_b200.ops import lib as ops
    from ferrum_b200.parts import TokenSideInput, TokenSideTable
    td, E, dim, V, T, eps, mult = TD[dtype], 56, 6, 31, 11, 1e-4, 0.7
    g = torch.Generator(device="cuda").manual_seed(11)
    x, y1, y2 = (torch.randn(T + 2, E, device="cuda", generator=g) for _ in range(3))
    ref = x.double() + mult * (y1.double() + y2.double())
    xc = torch.zeros(T + 2, E, device="cuda", dtype=td)
    x1 = x.clone()
    ops.scaled_sum(x1, y1, y2, mult, T, xc)
    assert (x1[:T].double() - ref[:T]).abs().max().item() < 1e-5 and torch.equal(x1[T:], x[T:])        # rows past the batch stay
    assert torch.equal(xc[:T], x1[:T].to(td))
    x2 = x.clone()
    ops.scaled_sum(x2, y1, None, mult, T)
    assert (x2[:T].double() - (x.double() + mult * y1.double())[:T]).abs().max().item() < 1e-5
    table = TokenSideTable(V, 3 * dim)
    wt = fill_part(table, 12, td, "side.")
    side = TokenSideInput(E, dim, 2 * dim, table, eps, td)
    w = fill_part(side, 13, td, "l2.side.")
    w["side.embed"] = wt["side.weight"] if "side.weight" in wt else wt["side."]
    ctx = make_ctx([(0, T)])
    toks = torch.tensor([30, 0, 5, 5, 17, 2, 29, 30, 1, 8, 9], dtype=torch.int32, device="cuda")
    ctx.token_ids.copy_(toks)
    h = x[:T].clone()
    side.forward(h, h.to(td) if td != torch.float32 else h, ctx, mult)
    cfg = {"token_side": {"dim": dim}}
    ref = x[:T].double().cpu() + mult * P.side_input(x[:T].double().cpu(), toks.long().cpu(), 2, w, cfg, eps, rounding_of(dtype))
    assert (h.double().cpu() - ref).abs().max() < (1e-5 if dtype == "float32" else 2e-2) * ref.abs().max()
    assert ctx.err.item() == 0


# ================================================================= whole models, every way of cutting the work
CASES = [(n, d) for n in ("A", "B") for d in ("float32", "bfloat16")]


@pytest.mark.parametrize("name,dtype", CASES + [("C", "float32"), ("C", "bfloat16")])
def test_whole_prompt_and_first_tokens(cuda, folders, name, dtype):
    toks = tokens_for(name, 140, 10)
    r = Replay(session(folders[name], dtype, 160))
    r.step([("a", toks, "all")], end=["a"])
    close(r.logits("a", len(toks)), plain(folders[name], dtype, toks), dtype, f"{name} whole")
    r = Replay(session(folders[name], dtype, 64))
    r.step([("b", toks[:1], "all")])
    r.step([("b", toks[1:3], "all")])
    r.step([("b", toks[3:4], "all")], end=["b"])
    close(r.logits("b", 4), plain(folders[name], dtype, toks[:4]), dtype, f"{name} first tokens")


def test_residual_rows_after_every_run(cuda, folders):
    """The stream after each run of the schedule (a looped layer counts every pass) against the plain layers."""
    toks = tokens_for("A", 25, 11)
    cfg, w = P.load(folders["A"])
    taps = []
    P.forward(cfg, w, toks, None, taps)
    s = session(folders["A"], "float32", 64)
    got = []
    s.model.on_run = lambda k, h: got.append(h[:len(toks)].double().cpu())
    s.run_step({"step": 0, "entries": [{"id": "a", "tokens": toks, "want": []}], "end": ["a"]})
    assert len(got) == len(taps) == 8
    for k, (g, t) in enumerate(zip(got, taps)):
        assert (g - t).abs().max() < 1e-4 * t.abs().max(), k


@pytest.mark.parametrize("name,dtype", CASES)
def test_prefill_then_long_decoding_past_every_window(cuda, folders, name, dtype):
    """30 tokens at once, then 120 one by one: the windows (19 and 33 keys) pass over decoded tokens,
    pages behind them are given back meanwhile, the recurrent state is carried 120 times."""
    toks = tokens_for(name, 150, 12)
    ref = plain(folders[name], dtype, toks)
    s = session(folders[name], dtype, 160, page_size=8)
    r = Replay(s)
    r.step([("a", toks[:30], "all")])
    for t in toks[30:]:
        r.step([("a", [t], "all")])
    close(r.logits("a", len(toks)), ref, dtype, f"{name} prefill+decode")
    assert s.runner.graph_replays > 0          # single tokens ran from a captured graph


@pytest.mark.parametrize("name,dtype", CASES + [("C", "float32")])
@pytest.mark.parametrize("sizes", [[2], [5, 2, 7, 3, 2, 16, 17, 2, 31, 1, 33, 2], [64, 3, 1]])
def test_portions(cuda, folders, name, dtype, sizes):
    toks = tokens_for(name, 131, 13)
    ref = plain(folders[name], dtype, toks)
    r = Replay(session(folders[name], dtype, 144, page_size=16))
    i = k = 0
    while i < len(toks):
        n = min(sizes[k % len(sizes)], len(toks) - i)
        r.step([("a", toks[i:i + n], "all")])
        i += n
        k += 1
    close(r.logits("a", len(toks)), ref, dtype, f"{name} portions {sizes[:3]}")


@pytest.mark.parametrize("name,dtype", CASES)
@pytest.mark.parametrize("page_size", [8, 32])
def test_mixed_batches_reuse_pages_and_slots(cuda, folders, name, dtype, page_size):
    """Six requests through four slots, portions beside single tokens; the pool has fewer pages than
    all requests need together: finished requests' pages and state rows go to later ones."""
    lens = {"a": 70, "b": 45, "c": 33, "d": 90, "e": 50, "f": 21}
    toks = {k: tokens_for(name, n, 20 + i) for i, (k, n) in enumerate(lens.items())}
    schedule = mixed_schedule(lens)
    pool = peak_pages(schedule, page_size)
    s = session(folders[name], dtype, pool * page_size, page_size=page_size, max_requests=4)
    slots_seen, owners = {}, {}
    r = Replay(s)
    for entries, ended in schedule:
        r.step([(k, toks[k][first:first + n], "all") for k, first, n in entries], end=ended)
        for k, slot in s.slots.items():
            slots_seen.setdefault(slot, set()).add(k)
        for g in range(s.cache.manager.n_groups):
            for k, slot in s.slots.items():
                for p in s.cache.manager.table(g, slot):
                    if p >= 0:
                        owners.setdefault((g, p), set()).add(k)
        assert s.cache.manager.check() == ""
    assert pages_were_reused(owners) and any(len(v) > 1 for v in slots_seen.values())
    for k in toks:
        close(r.logits(k, lens[k]), plain(folders[name], dtype, toks[k]), dtype, f"{name} mixed {k}")


@pytest.mark.parametrize("name", ["A", "B"])
def test_logits_do_not_depend_on_the_batch(cuda, folders, name):
    """float32: a request's logits beside three others equal those it gets alone to rounding."""
    toks = {k: tokens_for(name, n, 40 + i) for i, (k, n) in enumerate({"a": 50, "b": 9, "c": 31, "d": 2}.items())}
    alone = {}
    for k, t in toks.items():
        r = Replay(session(folders[name], "float32", 64))
        r.step([(k, t, "all")], end=[k])
        alone[k] = r.logits(k, len(t))
    r = Replay(session(folders[name], "float32", 128))
    r.step([(k, t[:len(t) // 2], "all") for k, t in toks.items()])
    r.step([(k, t[len(t) // 2:], "all") for k, t in reversed(list(toks.items()))], end=list(toks))
    for k, t in toks.items():
        assert np.abs(r.logits(k, len(t)) - alone[k]).max() < 2e-5 * max(1.0, np.abs(alone[k]).max()), k


def plain_generate(cfg, w, prompt, n, rd=None):
    seq = list(prompt)
    for _ in range(n):
        seq.append(int(P.forward(cfg, w, seq, rd)[-1].argmax()))
    return seq[len(prompt):]


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "float32"), ("B", "bfloat16")])
def test_greedy_generation_through_the_engine(cuda, folders, name, dtype):
    """Engine.generate (scheduler, sampler, chunked prompts, several requests) against the plain
    implementation; in bfloat16 a token may differ only at a near-tie of the plain logits."""
    from ferrum_b200.engine.api import Engine
    cfg, w = P.load(folders[name])
    prompts = [tokens_for(name, n, 60 + n) for n in (23, 5, 41)]
    eng = Engine(folders[name], dtype=dtype, page_size=8, num_pages=40, max_batch_tokens=32, max_batch_seqs=4, chunk_size=16,
                 max_model_len=96)
    outs = eng.generate(prompts, max_new_tokens=20)
    for p, got in zip(prompts, outs):
        if dtype == "float32":
            assert got == plain_generate(cfg, w, p, 20)
            continue
        seq = list(p)
        for t in got:
            logits = P.forward(cfg, w, seq, rounding_of(dtype))[-1].numpy()
            if t != int(np.argmax(logits)):
                assert logits.max() - logits[t] <= 0.2 * logits.std(), (len(seq), t)
            seq.append(t)
    assert eng.stats()["pages_used"] == [0] * eng.cache.manager.n_groups


def test_trace_run_program_and_command_line(cuda, folders, tmp_path):
    """bin/trace_run as a user runs it on a Vikupel folder (a subprocess, JSON lines in, .f32 files
    out), and `ferrum generate` on the same folder against the plain implementation."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    toks = tokens_for("A", 40, 16)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": toks[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": toks[30:], "want": []}, {"id": "y", "tokens": toks[:2], "want": [1]}], "end": ["y"]},
             {"step": 2, "entries": [{"id": "x", "tokens": toks[:1], "want": [0]}], "end": ["x"]}]
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folders["A"], "--dtype", "float32",
                        "--out", str(out), "--max-tokens", "128"],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-2000:]
    assert p.stdout.split() == ["done", "0", "done", "1", "done", "2"]
    ref = plain(folders["A"], "float32", toks + toks[:1])
    assert_close_f32(np.fromfile(out / "0.f32", dtype="<f4").reshape(2, -1), ref[[0, 29]], "trace_run step 0")
    assert_close_f32(np.fromfile(out / "1.f32", dtype="<f4").reshape(1, -1), ref[[1]], "trace_run step 1")
    assert_close_f32(np.fromfile(out / "2.f32", dtype="<f4").reshape(1, -1), ref[[40]], "trace_run step 2")
    cfg, w = P.load(folders["A"])
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "ferrum"), "generate", "--model", folders["A"], "--dtype", "float32",
                        "--prompt-tokens", ",".join(str(t) for t in toks[:12]), "--max-new-tokens", "6"],
                       capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-2000:]
    want = plain_generate(cfg, w, toks[:12], 6)
    assert ",".join(str(t) for t in want) in p.stdout.replace(" ", ""), (p.stdout, want)


@pytest.mark.parametrize("name", ["A", "B"])
def test_float16_prefill_and_decoding(cuda, folders, name):
    """The kernels with float16 storage (weights, activations, cached keys and values): a prompt, then
    single tokens, against the plain implementation rounding to float16 where the engine does."""
    toks = tokens_for(name, 150, 14)
    ref = plain(folders[name], "float16", toks)
    r = Replay(session(folders[name], "float16", 192))
    r.step([("a", toks[:100], "all")])
    for t in toks[100:]:
        r.step([("a", [t], "all")])
    assert_close_16bit(r.logits("a", len(toks)), ref, f"{name} float16", "float16")
