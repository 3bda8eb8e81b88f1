"""Ruperax on the GPU against the plain implementation (plain_ruperax.py): every mechanism
alone, then whole models under every way of cutting the work, then generation through the engine."""
import numpy as np
import pytest
import torch

import plain_ruperax as P
from helpers import Replay, assert_close_16bit, assert_close_f32, mixed_schedule, pages_were_reused, peak_pages, run_mixed
from ruperax_configs import RUPERAX, write_model

pytestmark = pytest.mark.gpu
TD = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def rounding_of(dtype):
    return None if dtype == "float32" else P.round_bf16


def close(x, ref, dtype, what):
    (assert_close_f32 if dtype == "float32" else assert_close_16bit)(x, ref, what)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: write_model(cfg, str(tmp_path_factory.mktemp("ruperax_" + name)), seed) for name, (cfg, seed) in RUPERAX.items()}


def plain(folder, dtype, tokens):
    cfg, w = P.read_model(folder)
    return P.forward(cfg, w, tokens, rounding=rounding_of(dtype))


def session(folder, dtype, max_tokens, **kw):
    from ferrum_b200.engine.trace import TraceSession
    return TraceSession(folder, dtype, max_tokens, **kw)


def tokens_for(name, n, seed):
    return np.random.default_rng(seed).integers(0, RUPERAX[name][0]["vocab"], n).tolist()


# ================================================================= mechanisms alone
def make_ctx(entries, slots=None, max_tokens=512, max_requests=8, widths=()):
    """A step context for [(pos0, n tokens)] entries, with explicit block tables per group."""
    from ferrum_b200.engine.batch import StepContext, StepEntry
    ctx = StepContext("cuda", max_tokens, max_requests, [len(t[0]) for t in widths])
    es = [StepEntry(slots[i] if slots else i, p0, list(range(n))) for i, (p0, n) in enumerate(entries)]
    ctx.fill(es, [list(t) for t in widths])
    return ctx


def test_scaled_embedding_with_positions(cuda):
    from ferrum_b200.ops import lib as ops
    g = torch.Generator(device="cuda").manual_seed(1)
    V, E, NP = 37, 50, 23
    for dt in (torch.float32, torch.bfloat16):
        table = torch.randn(V, E, device="cuda", generator=g).to(dt)
        pos = torch.randn(NP, E, device="cuda", generator=g).to(dt)
        ids = torch.tensor([3, 36, 0, 7], dtype=torch.int32, device="cuda")
        where = torch.tensor([22, 0, 5, 5], dtype=torch.int32, device="cuda")
        out = torch.empty(4, E, device="cuda")
        err = torch.zeros(1, dtype=torch.int32, device="cuda")
        ops.embedding(table, ids, out, err, scale=1.75, pos_table=pos, positions=where)
        ref = table.double()[ids.long()] * 1.75 + pos.double()[where.long()]
        assert (out.double() - ref).abs().max().item() < 1e-5 and err.item() == 0
        ops.embedding(table, ids, out, err, scale=0.25)
        assert (out.double() - table.double()[ids.long()] * 0.25).abs().max().item() < 1e-6
        where[1] = NP          # past the table: the step's error flag, no wild read
        ops.embedding(table, ids, out, err, scale=1.0, pos_table=pos, positions=where)
        assert err.item() == 2


@pytest.mark.parametrize("E,groups", [(48, 1), (48, 3), (130, 5), (512, 2), (96, 32)])
def test_grouped_norm(cuda, E, groups):
    from ferrum_b200.ops import lib as ops
    g = torch.Generator(device="cuda").manual_seed(2)
    x = torch.randn(9, E, device="cuda", generator=g) * torch.linspace(0.1, 30, E, device="cuda")     # groups of very different size
    w = torch.randn(E, device="cuda", generator=g)
    rows = torch.tensor([8, 0, 3], dtype=torch.int32, device="cuda")
    out = torch.empty(3, E, device="cuda")
    ops.rmsnorm(x, w, out, 1e-3, rows=rows, n_rows=3, groups=groups)
    ref = P.group_norm(x.double().cpu().numpy()[[8, 0, 3]], groups, 1e-3) * w.double().cpu().numpy()
    assert np.abs(out.double().cpu().numpy() - ref).max() < 1e-5 * max(1.0, np.abs(ref).max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_two_norms_and_token_shift_with_state(cuda, dtype):
    """Three requests in one batch: one at its start (zeros before the first token), one that goes
    on from a state row, one single token that goes on; the staged rows are the last a of each."""
    from ferrum_b200.ops import lib as ops
    g = torch.Generator(device="cuda").manual_seed(3)
    E, groups, eps = 72, 3, 2e-4
    entries = [(0, 5), (9, 4), (4, 1)]
    slots = [2, 0, 5]
    ctx = make_ctx(entries, slots)
    T = ctx.n_tokens
    x = torch.randn(T, E, device="cuda", generator=g) * 3
    w1, w2, s = (torch.randn(E, device="cuda", generator=g) for _ in range(3))
    state = torch.randn(8, E, device="cuda", generator=g)
    stage = torch.zeros(8, E, device="cuda")
    a, m, b = (torch.empty(T, E, device="cuda", dtype=TD[dtype]) for _ in range(3))
    ops.norm_pair_shift(x, w1, w2, s, a, m, b, T, ctx, state, stage, groups, eps)
    xn, w1n, w2n, sn = (t.double().cpu().numpy() for t in (x, w1, w2, s))
    n = P.group_norm(xn, groups, eps)
    tol = 1e-5 if dtype == "float32" else 2e-2
    t0 = 0
    for r, (p0, cnt) in enumerate(entries):
        ar = n[t0:t0 + cnt] * w1n
        before = None if p0 == 0 else state[slots[r]].double().cpu().numpy()
        mr = P.token_shift(ar, sn, before)
        assert np.abs(a[t0:t0 + cnt].double().cpu().numpy() - ar).max() < tol * max(1, np.abs(ar).max())
        assert np.abs(m[t0:t0 + cnt].double().cpu().numpy() - mr).max() < tol * max(1, np.abs(mr).max())
        assert np.abs(b[t0:t0 + cnt].double().cpu().numpy() - n[t0:t0 + cnt] * w2n).max() < tol * 10
        assert np.abs(stage[r].double().cpu().numpy() - ar[-1]).max() < 1e-5 * max(1, np.abs(ar).max())      # float32 in both modes
        t0 += cnt
    # without a second sublayer and without a shift
    ops.norm_pair_shift(x, w1, None, None, a, m, None, T, ctx, None, None, groups, eps)
    assert torch.equal(a, m)


def test_biased_glu_and_gated_sum(cuda):
    from ferrum_b200.ops import lib as ops
    g = torch.Generator(device="cuda").manual_seed(4)
    T, F, E = 7, 45, 40
    gu = torch.randn(T, 2 * F + E, device="cuda", generator=g) * 2
    bg, bu = torch.randn(F, device="cuda", generator=g), torch.randn(F, device="cuda", generator=g)
    act = torch.empty(T, F, device="cuda")
    ops.bias_glu(gu, bg, bu, act, T, F, "silu")
    z = (gu[:, :F] + bg).double().cpu().numpy()
    u = (gu[:, F:2 * F] + bu).double().cpu().numpy()
    assert np.abs(act.double().cpu().numpy() - P.silu(z) * u).max() < 1e-5
    ops.bias_glu(gu, bg, None, act, T, F, "gelu_tanh")
    gelu = 0.5 * z * (1 + np.tanh(np.sqrt(2 / np.pi) * (z + 0.044715 * z ** 3)))
    assert np.abs(act.double().cpu().numpy() - gelu * gu[:, F:2 * F].double().cpu().numpy()).max() < 1e-5
    # x += y1 * sigmoid(g1 + c1) + (y2 + c2) * sigmoid(g2 + c3), g2 a slice of a wider buffer
    x, y1, g1, y2 = (torch.randn(T, E, device="cuda", generator=g) for _ in range(4))
    c1, c2, c3 = (torch.randn(E, device="cuda", generator=g) for _ in range(3))
    g2 = gu[:, 2 * F:]
    ref = x.double() + y1.double() * torch.sigmoid(g1.double() + c1.double()) + (y2.double() + c2.double()) * torch.sigmoid(g2.double() + c3.double())
    ref1 = x.double() + y1.double() * torch.sigmoid(g1.double() + c1.double())
    x2 = x.clone()
    ops.gated_residual(x, T, y1, g1, c1, y2, c2, g2, c3)
    ops.gated_residual(x2, T, y1, g1, c1)
    assert (x.double() - ref).abs().max().item() < 1e-5 and (x2.double() - ref1).abs().max().item() < 1e-5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("M,H,N,K", [(5, 3, 22, 10), (64, 2, 7, 37), (9, 16, 128, 64), (70, 3, 24, 16), (300, 5, 200, 72), (129, 2, 130, 8)])
def test_one_product_per_head(cuda, dtype, M, H, N, K):
    """y[t, h, :] = W_h x[t, h, :] for every head in one launch: few tokens (CUDA cores), many
    (tensor cores in 16-bit), inside wider rows."""
    from ferrum_b200.ops import lib as ops
    g = torch.Generator(device="cuda").manual_seed(M + N)
    td = TD[dtype]
    pad = 8
    x = torch.randn(M, H * (K + pad), device="cuda", generator=g).to(td)
    w = (torch.randn(H, N, K, device="cuda", generator=g) * 0.3).to(td)
    y = torch.zeros(M, H * (N + 2), device="cuda", dtype=td)
    if M > ops.head_linear_max_tokens() and not ops.head_linear_mma_supported(x, K + pad, w, y, N + 2):
        pytest.skip("many tokens of this shape run as one product per head on the product kernels")
    ops.head_linear(x, K + pad, w, y, N + 2, M)
    ref = torch.einsum("thk,hnk->thn", x.double().view(M, H, K + pad)[:, :, :K], w.double())
    got = y.double().view(M, H, N + 2)
    tol = 1e-5 if dtype == "float32" else 1e-2
    assert (got[:, :, :N] - ref).abs().max().item() < tol * max(1.0, ref.abs().max().item())
    assert got[:, :, N:].abs().max().item() == 0          # nothing written between the heads' outputs


def attention_rows_reference(qf, rows, pos, H, Dk, Dv, scale, window, gate):
    """out[t, h] = gate * sum_j softmax_j(qf[t, h] . rows[j] * scale) rows[j, :Dv] over j in (pos - window, pos]."""
    out = np.zeros((len(pos), H, Dv))
    for t, p in enumerate(pos):
        lo = max(0, p - window + 1) if window > 0 else 0
        s = qf[t].reshape(H, Dk) @ rows[lo:p + 1].T * scale
        s = s - s.max(axis=1, keepdims=True)
        w = np.exp(s)
        w /= w.sum(axis=1, keepdims=True)
        out[t] = (w @ rows[lo:p + 1, :Dv]) * gate[t][:, None]
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,R,Rr,page,window", [(3, 24, 8, 8, 19), (5, 40, 0, 16, 64), (9, 100, 12, 32, 0), (2, 300, 20, 16, 130),
                                                (16, 64, 16, 16, 70), (5, 128, 32, 8, 0), (20, 96, 16, 32, 130), (2, 512, 64, 16, 19),
                                                (1, 32, 0, 16, 64)])
def test_attention_over_cached_rows_sees_exactly_its_window(cuda, dtype, H, R, Rr, page, window):
    """The attention kernel alone on rows written straight into pages that lie scattered in the
    pool.  One cached row is made to dominate: it is scaled up and every query points at it.
    Placed at the last position a query may see, the output is that row; one position further
    back, it is gone.  The same for a prompt portion and for single tokens, with the row at a
    page border and far back among hundreds."""
    from ferrum_b200.ops import lib as ops
    rng = np.random.default_rng(H * 1000 + R)
    Dk, n_keys, td = R + Rr, 300, TD[dtype]
    n_pages = -(-n_keys // page)
    order = rng.permutation(n_pages + 5)[:n_pages]                     # logical page -> a scattered page of the pool
    rows = rng.standard_normal((n_keys, Dk)) * 0.3
    hot = 137 if window == 0 else n_keys - 1 - (window - 1) - 3       # the last query's window starts 3 keys after it ...
    hot = hot // page * page                                           # ... and it is the first row of its page
    rows[hot] *= 6.0
    rows_t = torch.tensor(rows, device="cuda").to(td)
    rows = rows_t.double().cpu().numpy()
    plane = torch.zeros(n_pages + 5, page, Dk, device="cuda", dtype=td)
    for lp in range(n_pages):
        chunk = rows_t[lp * page:(lp + 1) * page]
        plane[order[lp], :len(chunk)] = chunk
    # 16-bit rows whose sizes the tensor-core kernel takes run on it; the others, and float32, on the CUDA cores
    on_tensor_cores = dtype != "float32" and (R + Rr) % 16 == 0 and R % 32 == 0
    for pos0, n in ((n_keys - 40, 40), (n_keys - 1, 1), (hot + max(window, 1) - 2, 3)):
        ctx = make_ctx([(pos0, n)], widths=[[list(order)]])
        pos = list(range(pos0, pos0 + n))
        qf = np.tile(rows[hot] * 4.0, (n, H)) + rng.standard_normal((n, H * Dk)) * 0.1
        qf_t = torch.tensor(qf, device="cuda").to(td)
        gate = torch.rand(n, H, device="cuda") + 0.5
        out = torch.zeros(n, H * R, device="cuda", dtype=td)
        scale = 0.7
        for single in ([False, True, "split"] if n == 1 else [False]):
            part, slots = None, 0
            if single == "split":        # the token's keys cut at multiples of the split size among CTAs, then folded
                slots = (min(n_keys, window + ops.attention_latent_split()) if window else n_keys) // ops.attention_latent_split() + 2
                part = torch.full((n * H * slots * (R + 2),), float("nan"), device="cuda")
            out.zero_()
            assert ops.attention_latent_mma_supported(qf_t, out, plane, plane.stride(0), Dk, R) == on_tensor_cores
            ops.attention_latent(qf_t, out, gate, n, ctx, ctx.block_tables[0], plane, plane.stride(0), page, H, Dk, R, scale, window,
                                 bool(single), part=part, split_slots=slots)
            if on_tensor_cores:          # the other stage size of the kernel, and the CUDA-core kernel, on the same rows
                for stage in (32, 64, None):
                    other = torch.zeros_like(out)
                    ops.attention_latent_mma_stage(stage or 0)
                    try:
                        ops.attention_latent(qf_t, other, gate, n, ctx, ctx.block_tables[0], plane, plane.stride(0), page, H, Dk, R,
                                             scale, window, bool(single), part=part, split_slots=slots,
                                             tensor_cores=None if stage else False)
                    finally:
                        ops.attention_latent_mma_stage(0)
                    assert (other.double() - out.double()).abs().max().item() < 3e-2 * out.double().abs().max().item(), stage
            ref = attention_rows_reference(qf_t.double().cpu().numpy(), rows, pos, H, Dk, R, scale, window, gate.double().cpu().numpy())
            got = out.double().cpu().numpy().reshape(n, H, R)
            tol = 1e-4 if dtype == "float32" else 3e-2
            assert np.abs(got - ref).max() < tol * np.abs(ref).max(), (pos0, n, single)
            assert ctx.err.item() == 0
        if window > 0:
            # the rows for which the hot key is the oldest visible one are (nearly) that row; the next query has lost it
            for t, p in enumerate(pos):
                lead = got[t, 0] / gate[t, 0].item()
                if p - window + 1 <= hot <= p:
                    assert np.abs(lead - rows[hot, :R]).max() < 0.05 * np.abs(rows[hot]).max(), (p, hot)
                elif p - window + 1 == hot + 1:
                    assert np.abs(lead - rows[hot, :R]).max() > 0.5 * np.abs(rows[hot, :R]).max(), (p, hot)


class OneMixer:
    """The least a cache and a runner need of a model: a schedule and the needs of its runs."""

    def __init__(self, mixers, schedule):
        from ferrum_b200.models import Run
        self.mixers, self.schedule = mixers, [Run(i, cache_of=c) for i, c in enumerate(schedule)]

    def cache_needs(self):
        return [m.cache_need() for m in self.mixers]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_latent_mixer_alone_and_a_reader_of_its_rows(cuda, dtype):
    """Two mixers on given input rows: one caches its rows, the other reads them with maps, head
    count and window of its own.  Whole sequence at once, then in portions against the cache."""
    from ferrum_b200.cache import CacheStorage
    from ferrum_b200.engine.batch import StepContext, StepEntry
    from ferrum_b200.parts import LatentAttention, RotaryEmbedding
    from ferrum_b200.weights.random_init import _tensor
    td = TD[dtype]
    E, eps, T = 40, 1e-5, 61
    rot = RotaryEmbedding(8, 8, 300.0, None, "half", 128, "cuda")
    spec = [dict(heads=3, dim=8, rot_dim=8, vdim=12, kv_rank=16, q_rank=20, scale=0.3, window=17, own=True),
            dict(heads=2, dim=12, rot_dim=8, vdim=5, kv_rank=16, q_rank=8, scale=0.21, window=30, own=False)]
    mixers = [LatentAttention(E, s["heads"], s["dim"], s["rot_dim"], s["vdim"], s["kv_rank"], s["q_rank"], eps, s["scale"], td,
                              rotary=rot, window=s["window"], own_latent=s["own"]) for s in spec]
    weights = []
    for i, mx in enumerate(mixers):
        w = {}
        for name, ps in mx.param_specs().items():
            t = _tensor(f"{i}.{name}", ps, 5, "cuda", 0.3 if ps.kind == "matrix" else 0.1)
            t = t.to(td) if ps.kind == "matrix" else t
            mx.assign(name, t.contiguous())
            w["p." + name.replace("_norm.weight", ".norm").replace(".weight", "")] = t.double().cpu().numpy()
        mx.finalize()
        weights.append(w)
    model = OneMixer(mixers, [None, 0])
    cache = CacheStorage(model, td, "cuda", page_size=8, max_tokens=64, max_requests=2, max_model_len=64)
    assert cache.layout.group_keys == [(1, 24, 30, 1)]          # the plane keeps what its widest reader needs
    ctx = StepContext("cuda", 64, 2, [cache.table_width])
    x = (torch.randn(T, E, device="cuda", generator=torch.Generator(device="cuda").manual_seed(6))).to(td)
    xn = x.double().cpu().numpy()
    pos = np.arange(T)
    rd = rounding_of(dtype)
    cfgs = [dict(heads=s["heads"], dim=s["dim"], rot_dim=s["rot_dim"], vdim=s["vdim"], kv_rank=s["kv_rank"], scale=s["scale"],
                 mask={"size": s["window"]}, rot={"dims": 8, "base": 300.0}) for s in spec]
    c, kr = P.latent_of(xn, weights[0], "p.", cfgs[0], eps, pos)
    latent = (c, kr) if rd is None else (rd(c), rd(kr))
    refs = [P.latent_attention(xn, weights[i], "p.", cfgs[i], eps, pos, latent, rd) for i in range(2)]
    for cuts in ([T], [20, 1, 1, 2, 30, 7]):
        slot = cache.open()
        got = [[], []]
        at = 0
        for n in cuts:
            cache.manager.grow(slot, at + n)
            ctx.fill([StepEntry(slot, at, list(range(n)))], cache.manager)
            for i, mx in enumerate(mixers):
                y = torch.zeros(n, E, device="cuda")
                mx.forward(x[at:at + n].contiguous(), ctx, cache.layer_cache(i), y, accumulate=False)
                got[i].append(y.double().cpu().numpy())
            assert ctx.err.item() == 0
            cache.manager.commit(slot, at + n)
            at += n
        cache.close(slot)
        for i in range(2):
            g = np.concatenate(got[i])
            tol = 2e-4 if dtype == "float32" else 4e-2
            assert np.abs(g - refs[i]).max() < tol * np.abs(refs[i]).max(), (i, cuts)


# ================================================================= whole models, every way of cutting the work
CASES = [(n, d) for n in RUPERAX for d in ("float32", "bfloat16")]


@pytest.mark.parametrize("name,dtype", CASES)
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


@pytest.mark.parametrize("name,dtype", CASES)
def test_prefill_then_long_decoding_past_every_window(cuda, folders, name, dtype):
    """30 tokens at once, then 120 one by one: every window of the configurations (7 to 48 keys)
    passes over decoded tokens, pages behind the widest window are given back meanwhile."""
    toks = tokens_for(name, 150, 12)
    ref = plain(folders[name], dtype, toks)
    s = session(folders[name], dtype, 160, page_size=8)
    r = Replay(s)
    r.step([("a", toks[:30], "all")])
    for t in toks[30:]:
        r.step([("a", [t], "all")])
    close(r.logits("a", len(toks)), ref, dtype, f"{name} prefill+decode")
    assert s.runner.graph_replays > 0          # single tokens ran from a captured graph


@pytest.mark.parametrize("name,dtype", CASES)
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
    """Six requests through four slots, portions beside single tokens; the windowless pool would
    need more pages than it has: finished requests' pages and slots go to later ones."""
    lens = {"a": 70, "b": 45, "c": 33, "d": 90, "e": 50, "f": 21}
    toks = {k: tokens_for(name, n, 20 + i) for i, (k, n) in enumerate(lens.items())}
    schedule = mixed_schedule(lens)
    pool = peak_pages(schedule, page_size)
    s = session(folders[name], dtype, pool * page_size, page_size=page_size, max_requests=4)
    slots_seen = {}
    r = Replay(s)
    owners = {}
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


@pytest.mark.parametrize("name", list(RUPERAX))
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


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "float32"), ("B", "bfloat16")])
def test_greedy_generation_through_the_engine(cuda, folders, name, dtype):
    """Engine.generate (scheduler, sampler, chunked prompts, several requests) against the plain
    implementation; in bfloat16 a token may differ only at a near-tie of the plain logits."""
    from ferrum_b200.engine.api import Engine
    cfg, w = P.read_model(folders[name])
    prompts = [tokens_for(name, n, 60 + n) for n in (23, 5, 41)]
    eng = Engine(folders[name], dtype=dtype, page_size=8, num_pages=40, max_batch_tokens=32, max_batch_seqs=4, chunk_size=16,
                 max_model_len=96)
    outs = eng.generate(prompts, max_new_tokens=20)
    for p, got in zip(prompts, outs):
        if dtype == "float32":
            assert got == P.generate(cfg, w, p, 20)
            continue
        seq = list(p)
        for t in got:
            logits = P.forward(cfg, w, seq, rounding=P.round_bf16)[-1]
            if t != int(np.argmax(logits)):
                assert logits.max() - logits[t] <= 0.2 * logits.std(), (len(seq), t)
            seq.append(t)
    assert eng.stats()["pages_used"] == [0] * eng.cache.manager.n_groups


def test_trace_run_program_and_command_line(cuda, folders, tmp_path):
    """bin/trace_run as a user runs it on a Ruperax folder (a subprocess, JSON lines in, .f32 files
    out), and `ferrum generate` on the same folder against the plain implementation."""
    import json, os, subprocess, sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    toks = tokens_for("A", 40, 16)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": toks[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": toks[30:], "want": []}, {"id": "y", "tokens": toks[:2], "want": [1]}], "end": ["y"]},
             {"step": 2, "entries": [{"id": "x", "tokens": toks[:1], "want": [0]}], "end": ["x"]}]
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folders["A"], "--dtype", "float32",
                        "--out", str(out), "--max-tokens", "128"],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert p.stdout.split() == ["done", "0", "done", "1", "done", "2"]
    ref = plain(folders["A"], "float32", toks + toks[:1])
    assert_close_f32(np.fromfile(out / "0.f32", dtype="<f4").reshape(2, -1), ref[[0, 29]], "trace_run step 0")
    assert_close_f32(np.fromfile(out / "1.f32", dtype="<f4").reshape(1, -1), ref[[1]], "trace_run step 1")
    assert_close_f32(np.fromfile(out / "2.f32", dtype="<f4").reshape(1, -1), ref[[40]], "trace_run step 2")
    cfg, w = P.read_model(folders["A"])
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "ferrum"), "generate", "--model", folders["A"], "--dtype", "float32",
                        "--prompt-tokens", ",".join(str(t) for t in toks[:12]), "--max-new-tokens", "6"],
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    want = P.generate(cfg, w, toks[:12], 6)
    assert ",".join(str(t) for t in want) in p.stdout.replace(" ", ""), (p.stdout, want)


@pytest.mark.parametrize("name", list(RUPERAX))
def test_float16_prefill_and_decoding(cuda, folders, name):
    """The 16-bit kernels with float16 storage (weights, activations, cached rows): a prompt, then
    single tokens, against exact arithmetic on the stored weights."""
    toks = tokens_for(name, 150, 14)
    cfg, w = P.read_model(folders[name])
    ref = P.forward(cfg, w, toks)
    r = Replay(session(folders[name], "float16", 192))
    r.step([("a", toks[:100], "all")])
    for t in toks[100:]:
        r.step([("a", [t], "all")])
    assert_close_16bit(r.logits("a", len(toks)), ref, f"{name} float16", "float16")
