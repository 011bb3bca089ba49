"""The Relurax decoder in the engine against the plain implementation (tests/plain_relurax.py):
each mechanism alone, then whole models through the step function, the cache and state
manager, the scheduler and the entry point, under every kind of schedule."""
import numpy as np
import pytest
import torch

import plain_relurax as P
import relurax_util as U

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = ["float32", "bfloat16"]
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def rnd(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (scale * torch.randn(*shape, generator=g)).to(torch.bfloat16)


def runtime(dtype):
    from mstar_b200.parts import Runtime
    return Runtime(dtype=TORCH[dtype], device=torch.device(DEV))


def dev(t, dtype):
    return t.to(TORCH[dtype]).to(DEV)


def step_ctx(q_lens, starts, slots=None):
    from test_gpu_parts import simple_ctx
    ctx = simple_ctx(q_lens, starts)
    if slots is not None:
        ctx.slots = torch.tensor(slots, dtype=torch.int32, device=DEV)
        ctx.host_slots = list(slots)
    return ctx


def close(got, want, dtype, what, f32=2e-5, bf16=4e-2):
    """Worst difference relative to the largest wanted value."""
    want = torch.as_tensor(np.asarray(want))
    err = (got.double().cpu() - want.double()).abs().max().item() / want.abs().max().item()
    assert err < (f32 if dtype == "float32" else bf16), (what, dtype, err)


def mixer_part(m, width, dtype, seed, sharp=1.3, conv_last=None, weights=None, eps=1e-5):
    """A mixer of a one-layer configuration as the engine builds it from a checkpoint: the
    stacked first product, the small tensors beside it.  Returns (part, spec, its tensors by
    their short names as float64 arrays)."""
    from mstar_b200.config.registry import config_from_dict
    from mstar_b200.parts import build_part

    cfg = U.config([U.layer(m)], width=width, eps=eps)
    w = weights if weights is not None else U.random_weights(cfg, seed, sharp=sharp,
                                                             conv_last=conv_last)
    spec = config_from_dict(cfg).layout().blocks[0].mixer
    p = "l0.mix."
    if spec.kind == "attention":
        params = {"qkv.weight": torch.cat([w[p + "q"], w[p + "k"], w[p + "g"]]),
                  "q_conv.weight": w[p + "q.conv"], "k_conv.weight": w[p + "k.conv"],
                  "q_norm.weight": w[p + "q.norm"], "k_norm.weight": w[p + "k.norm"],
                  "o.weight": w[p + "o"]}
    else:
        params = {"in.weight": torch.cat([w[p + "dq"], w[p + "dkv"], w[p + "g"]]),
                  "q_norm.weight": w[p + "dq.norm"], "uq.weight": w[p + "uq"],
                  "kv_norm.weight": w[p + "dkv.norm"], "uk.weight": w[p + "uk"],
                  "uv.weight": w[p + "uv"], "o.weight": w[p + "o"]}
    part = build_part("mixer", spec, {k: dev(v, dtype) for k, v in params.items()}, runtime(dtype))
    return part, spec, U.mixer_tensors(w)


def paged_cache(spec, tokens, page, dtype, slots=None, seed=1):
    """Pages scattered over a pool that holds leftovers of other requests; state slots that
    hold leftovers too, but for the one in use."""
    from mstar_b200.parts import LayerCache, part_class

    need = part_class("mixer", spec).cache_need(spec)
    pages = -(-tokens // page)
    kv_need = need.kv
    if kv_need.planes == 1:
        shape = (pages + 3, 1, 1, page, kv_need.head_dim)
    else:
        shape = (pages + 3, 2 * kv_need.num_kv_heads * page * kv_need.head_dim)
    kv = torch.full(shape, 7.0, dtype=TORCH[dtype], device=DEV)
    table = (torch.randperm(pages + 3, generator=torch.Generator().manual_seed(seed))[:pages]
             .to(torch.int32).to(DEV)[None])
    state = None
    if need.state is not None:
        state = torch.randn((slots or 1) + 1, *need.state.shape, device=DEV)
    return LayerCache(kv=kv, page_size=page, block_table=table, state=state)


def run_cut(part, x, cuts, cache, dtype, slot=0):
    """The sequence ``x`` through the mixer in portions of the sizes ``cuts``."""
    if cache.state is not None:
        cache.state[slot].zero_()
    outs, at = [], 0
    for n in cuts:
        outs.append(part.forward(dev(x[at:at + n], dtype), step_ctx([n], [at], [slot]), cache))
        at += n
    assert at == x.shape[0]
    return torch.cat(outs)


# ------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", DTYPES)
def test_gelu_gated_feed_forward(dtype):
    from mstar_b200.config.layout import GatedMLPSpec
    from mstar_b200.parts import build_part

    # a few rows and many; a width of whole 64-byte pieces and one that is not
    for rows, width, ff in ((9, 96, 200), (70, 96, 200), (5, 72, 50), (150, 40, 24)):
        x = rnd(rows, width, seed=6)
        gate, up = rnd(ff, width, seed=3, scale=0.2), rnd(ff, width, seed=4, scale=0.1)
        down = rnd(width, ff, seed=5, scale=0.1)
        part = build_part("ffn", GatedMLPSpec(hidden_size=width, intermediate_size=ff,
                                              activation="gelu_tanh"),
                          {"gate_up.weight": dev(torch.cat([gate, up]), dtype),
                           "down.weight": dev(down, dtype)}, runtime(dtype))
        want = P.plain_dense_ff(x.double().numpy(), gate.double().numpy(), up.double().numpy(),
                                down.double().numpy())
        close(part.forward(dev(x, dtype), None), want, dtype, ("gelu gate", rows, width), bf16=2e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_sandwich_norms_around_a_sublayer(dtype):
    """h += norm_b(y) in float, and the new residual normed for the next sublayer, by the
    kernel that the block's norms use."""
    from mstar_b200 import ops

    for width in (64, 200, 1000):
        h, y = rnd(7, width, seed=1).float(), rnd(7, width, seed=2, scale=3.0)
        wb, wn = rnd(width, seed=3, scale=0.5).float(), rnd(width, seed=4).float()
        after = h.double().numpy() + P.plain_rms_norm(y.double().numpy(), wb.double().numpy(), 1e-5)
        want = P.plain_rms_norm(after, wn.double().numpy(), 1e-5)
        resid = h.clone().to(DEV)
        rows = ops.add_postnorm_rmsnorm(resid, dev(y, dtype), wb.to(DEV), 1e-5, 0.0,
                                        weight=wn.to(DEV), eps=1e-5, out_dtype=TORCH[dtype])
        close(resid, after, "float32", "residual")
        close(rows, want, dtype, "normed rows", bf16=1e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,dim,size,taps,page",
                         [(4, 2, 24, 11, 3, 4), (3, 3, 16, 9, 1, 8), (6, 2, 20, 5, 5, 16),
                          (2, 1, 32, None, 2, 4), (2, 2, 64, 1, 4, 8), (8, 1, 16, 16, 4, 16),
                          (5, 5, 96, 33, 2, 16), (4, 2, 128, 20, 4, 16), (2, 1, 160, 7, 3, 8),
                          (34, 1, 16, 12, 6, 4), (1, 1, 8, 70, 7, 4)])
def test_conv_attention_alone(dtype, heads, kv_heads, dim, size, taps, page):
    """The sliding-window mixer alone, with scores so sharp that a query's weight lies on a few
    keys: a key that a window one too long or too short takes in or leaves out, a value taken
    after the norm instead of before it, or a convolution that forgets the rows before a
    portion changes the output by a value's size.  Portions down to two tokens and single
    tokens (fewer than the convolution has taps); pages scattered over the pool; a slot that
    held another request's rows."""
    m = U.attention(heads, kv_heads, dim, size=size, conv=taps, scale=6.0 / dim)
    part, spec, p = mixer_part(m, 96, dtype, seed=7, sharp=3.0)
    T = 70
    x = rnd(T, 96, seed=8)
    want = P.plain_conv_attention(x.double().numpy(), p, m, 1e-5, {})
    cache = paged_cache(spec, T, page, dtype, slots=3)
    got = run_cut(part, x, (23, 2, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 29, 3, 2), cache, dtype, slot=2)
    close(got, want, dtype, "conv attention", bf16=6e-2)
    whole = run_cut(part, x, (T,), paged_cache(spec, T, page, dtype, seed=5), dtype)
    close(whole, want, dtype, "conv attention, one portion", bf16=6e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_convolution_rows_carry_over_between_portions_and_requests(dtype):
    """Two sequences in one batch in other slots than their entry numbers, then single tokens
    of both: each equals itself alone, and the slots not named stay as they were."""
    m = U.attention(3, 1, 16, size=9, conv=4, scale=0.4)
    part, spec, p = mixer_part(m, 48, dtype, seed=2)
    xa, xb = rnd(30, 48, seed=1), rnd(12, 48, seed=2)
    wa = P.plain_conv_attention(xa.double().numpy(), p, m, 1e-5, {})
    wb = P.plain_conv_attention(xb.double().numpy(), p, m, 1e-5, {})
    from mstar_b200.parts import LayerCache

    ca, cb = paged_cache(spec, 30, 4, dtype, slots=3, seed=1), paged_cache(spec, 12, 4, dtype, seed=2)
    pool = torch.cat([ca.kv, cb.kv])
    table = torch.full((2, ca.block_table.shape[1]), 0, dtype=torch.int32, device=DEV)
    table[0] = ca.block_table[0]
    table[1, :cb.block_table.shape[1]] = cb.block_table[0] + ca.kv.shape[0]
    state = torch.randn(4, *ca.state.shape[1:], device=DEV)
    state[3].zero_()
    state[1].zero_()
    kept = state[[0, 2]].clone()
    cache = LayerCache(kv=pool, page_size=4, block_table=table, state=state)
    got = [part.forward(dev(torch.cat([xa[:25], xb[:2]]), dtype), step_ctx([25, 2], [0, 0], [3, 1]), cache)]
    outs_a, outs_b = [got[0][:25]], [got[0][25:]]
    for t in range(5):                      # a decodes 5, b brings 2 tokens a step
        o = part.forward(dev(torch.cat([xa[25 + t:26 + t], xb[2 + 2 * t:4 + 2 * t]]), dtype),
                         step_ctx([1, 2], [25 + t, 2 + 2 * t], [3, 1]), cache)
        outs_a.append(o[:1])
        outs_b.append(o[1:])
    close(torch.cat(outs_a), wa, dtype, "first of two", bf16=6e-2)
    close(torch.cat(outs_b), wb, dtype, "second of two", bf16=6e-2)
    assert torch.equal(state[[0, 2]], kept)


def marked_conv_inputs(p, m, width, T, marked, queries):
    """Inputs in which the key of token ``marked`` carries the weight of the ``queries``: the
    query tokens lie along a direction d, the marked token along a direction whose projected
    key equals the projected query of d (a solution of W_k d' = W_q d for the first head).
    The convolution's tap on the token itself is near one and its others are small, so a key
    belongs to one token.  A query token's own key points elsewhere."""
    x = rnd(T, width, seed=4, scale=0.3)
    d = rnd(width, seed=5).double().numpy()
    if p["g"][0] @ d < 0:                   # the first head's gate is open for the queries
        d = -d
    dim = m["dim"]
    target = p["q"][:dim] @ d
    d_key = np.linalg.lstsq(p["k"][:dim], target, rcond=None)[0]
    x[marked] = torch.from_numpy(4.0 * d_key).to(torch.bfloat16)
    for q in queries:
        x[q] += torch.from_numpy(4.0 * d).to(torch.bfloat16)
    return x


CONV_EDGES = [  # (marked key, query that sees it, query that does not, window)
    (50, 50 + 40 - 1, 50 + 40, 40),        # the window's far edge
    (0, 22, 23, 23),                       # the sequence's first key, a window of odd size
    (15, 15 + 16 - 1, 15 + 16, 16),        # a window of one page, the key at a page's end
    (16, 16 + 48 - 1, 16 + 48, 48),        # a window of three pages, the key at a page's start
    (20, 320, 321, 301),                   # 300 back, through a window of 301
    (7, None, 8, 1),                       # a window of one: the token before is not seen
]


def conv_edge_case(marked, seen_from, unseen_from, win, width=64, T=330):
    m = U.attention(2, 1, 32, size=win, conv=3, scale=1.0)
    cfg = U.config([U.layer(m)], width=width)
    weights = U.random_weights(cfg, 3, sharp=1.0, conv_last=1.0)
    p = U.mixer_tensors(weights)
    queries = [q for q in (seen_from, unseen_from) if q is not None]
    x = marked_conv_inputs(p, m, width, T, marked, queries)
    xn = x.double().numpy()
    want = P.plain_conv_attention(xn, p, m, 1e-5, {})
    # how much hangs on the one key: the plain output with a window one shorter (for the
    # query that sees it) or one longer (for the one that does not)
    for q, delta in ((seen_from, -1), (unseen_from, +1)):
        if q is None or win + delta < 1:
            continue
        other = dict(m, mask={"size": win + delta})
        shifted = P.plain_conv_attention(xn, p, other, 1e-5, {})
        assert np.abs(shifted[q] - want[q]).max() > 0.5 * np.abs(want[q]).max(), (marked, q)
    return m, weights, x, want


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("marked,seen_from,unseen_from,win", CONV_EDGES)
def test_one_key_that_stands_out_at_a_windows_edge(dtype, marked, seen_from, unseen_from, win):
    """One key is made to carry all of a query's weight: the query just inside the window sees
    it, the next one does not.  Queries in a prompt portion and decoded alone."""
    m, weights, x, want = conv_edge_case(marked, seen_from, unseen_from, win)
    part, spec, _ = mixer_part(m, 64, dtype, seed=3, weights=weights)
    T = x.shape[0]
    for first in (T, 5):                      # one prompt; a short prompt and decoded tokens
        cache = paged_cache(spec, T, 16, dtype, seed=first)
        got = run_cut(part, x, (first,) + (1,) * (T - first), cache, dtype)
        close(got, want, dtype, ("edge", marked, first), bf16=6e-2)


LATENT_SHAPES = [  # heads, dim, rot_dim, vdim, kv_rank, q_rank, rotated dims, page
    (3, 16, 8, 24, 40, 20, 8, 4),          # rows of whole 16s, a rank that is no multiple of 32
    (4, 12, 12, 8, 24, 36, 8, 8),          # rows of 36; part of the rotated features rotated
    (2, 32, 16, 32, 64, 24, 16, 16),       # rank and row of whole tiles
    (1, 24, 2, 16, 30, 8, 2, 4),           # one head, one rotary pair
    (5, 8, 32, 40, 96, 50, 32, 8),         # a rotated part wider than the plain one
    (17, 16, 16, 16, 32, 16, 16, 4),       # more heads than a block takes
    (2, 128, 64, 128, 512, 192, 64, 16),   # the sizes of a large model's layer
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,dim,rot,vdim,rank,q_rank,dims,page", LATENT_SHAPES)
def test_latent_attention_alone(dtype, heads, dim, rot, vdim, rank, q_rank, dims, page):
    """The latent mixer alone, cut into portions down to two tokens and single tokens, pages
    scattered over the pool, against the plain attention over explicit keys and values."""
    m = U.latent(heads, dim, rot, vdim, rank, q_rank, base=100.0, dims=dims,
                 scale=4.0 * (dim + rot) ** -0.5)
    part, spec, p = mixer_part(m, 96, dtype, seed=11, sharp=2.0)
    T = 75
    x = rnd(T, 96, seed=9)
    want = P.plain_latent_attention(x.double().numpy(), p, m, 1e-5, {})
    got = run_cut(part, x, (21, 2, 1, 1, 1, 1, 1, 30, 3, 2, 12), paged_cache(spec, T, page, dtype), dtype)
    close(got, want, dtype, "latent attention", bf16=6e-2)
    whole = run_cut(part, x, (T,), paged_cache(spec, T, page, dtype, seed=4), dtype)
    close(whole, want, dtype, "latent attention, one portion", bf16=6e-2)


def marked_latent_inputs(p, m, width, T, marked, queries):
    """Inputs in which the latent of token ``marked`` answers the first head's plain query of
    the ``queries``: its down-projection is solved for the latent whose up-projected key
    equals that query."""
    x = rnd(T, width, seed=14, scale=0.3)
    d = rnd(width, seed=15).double().numpy()
    if p["g"][0] @ d < 0:                   # the first head's gate is open for the queries
        d = -d
    dim, rank = m["dim"], m["kv_rank"]
    cq = P.plain_rms_norm(p["dq"] @ (4.0 * d), p["dq.norm"], 1e-5)
    q_plain = (p["uq"] @ cq)[:dim]
    latent = np.linalg.lstsq(p["uk"][:dim], q_plain, rcond=None)[0] / p["dkv.norm"]
    d_key = np.linalg.lstsq(p["dkv"][:rank], latent, rcond=None)[0]
    x[marked] = torch.from_numpy(4.0 * d_key / np.abs(d_key).max()).to(torch.bfloat16)
    for q in queries:
        x[q] = torch.from_numpy(4.0 * d).to(torch.bfloat16)
    return x


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("marked,queries", [(0, (640, 700)), (1, (2, 701)), (15, (16, 500)),
                                            (16, (17, 650)), (333, (334, 690))])
def test_one_latent_far_back_stands_out(dtype, marked, queries):
    """One row among hundreds carries a query's weight: the sequence's first rows and rows at a
    page's end and start, asked for by the next token and from hundreds of tokens away, in a
    prompt and decoded alone.  Without that row the plain output is another."""
    m = U.latent(2, 16, 8, 16, 32, 24, base=10000.0, scale=3.0)
    cfg = U.config([U.layer(m)], width=64)
    weights = U.random_weights(cfg, 5, sharp=1.0)
    p = U.mixer_tensors(weights)
    T = 704
    x = marked_latent_inputs(p, m, 64, T, marked, queries)
    xn = x.double().numpy()
    want = P.plain_latent_attention(xn, p, m, 1e-5, {})
    other = xn.copy()
    other[marked] = rnd(64, seed=99, scale=0.3).double().numpy()
    without = P.plain_latent_attention(other, p, m, 1e-5, {})
    for q in queries:
        assert np.abs(without[q] - want[q]).max() > 0.5 * np.abs(want[q]).max(), (marked, q)
    part, spec, _ = mixer_part(m, 64, dtype, seed=5, weights=weights)
    first = min(queries[-1] - 40, 600)
    for cuts in ((T,), (first,) + (1,) * (T - first)):
        got = run_cut(part, x, cuts, paged_cache(spec, T, 16, dtype, seed=len(cuts)), dtype)
        # scores this sharp magnify the rounding of a bfloat16 query; a lost row moves the
        # output by more than half its size (checked above)
        close(got, want, dtype, ("far row", marked, len(cuts)), bf16=0.12)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_layer_reads_the_rows_another_layer_cached(dtype):
    """Two latent mixers on one cache: the second has no down-projection, other head sizes and
    its own up-projections, and reads what the first wrote, portion by portion."""
    from mstar_b200.config.registry import config_from_dict
    from mstar_b200.parts import build_part

    owner = U.latent(3, 16, 8, 24, 40, 20, base=500.0, scale=0.6)
    reader = U.latent(2, 8, 8, 12, 40, 28, kv_from=0, scale=0.9)
    cfg = U.config([U.layer(owner), U.layer(reader)], width=80)
    w = U.random_weights(cfg, 17, sharp=2.0)
    first, spec, p0 = mixer_part(owner, 80, dtype, seed=0, weights=w)
    spec1 = config_from_dict(cfg).layout().blocks[1].mixer
    assert spec1.shares_kv
    q = "l1.mix."
    params = {"in.weight": torch.cat([w[q + "dq"], w[q + "g"]]), "q_norm.weight": w[q + "dq.norm"],
              "uq.weight": w[q + "uq"], "uk.weight": w[q + "uk"], "uv.weight": w[q + "uv"],
              "o.weight": w[q + "o"]}
    second = build_part("mixer", spec1, {k: dev(v, dtype) for k, v in params.items()}, runtime(dtype))
    p1 = U.mixer_tensors(w, 1)
    T = 50
    xa, xb = rnd(T, 80, seed=1), rnd(T, 80, seed=2)
    kept = {}
    want0 = P.plain_latent_attention(xa.double().numpy(), p0, owner, 1e-5, kept)
    want1 = P.plain_latent_attention(xb.double().numpy(), p1, cfg["layers"][1]["mixer"], 1e-5, {}, kept)
    cache = paged_cache(spec, T, 8, dtype)
    got0, got1, at = [], [], 0
    for n in (19, 2, 1, 1, 25, 2):
        ctx = step_ctx([n], [at])
        got0.append(first.forward(dev(xa[at:at + n], dtype), ctx, cache))
        got1.append(second.forward(dev(xb[at:at + n], dtype), ctx, cache))
        at += n
    close(torch.cat(got0), want0, dtype, "the layer that caches", bf16=6e-2)
    close(torch.cat(got1), want1, dtype, "the layer that reads", bf16=6e-2)


@pytest.mark.parametrize("heads,rank,rot,window", [(8, 64, 16, 0), (3, 256, 32, 0), (16, 320, 64, 0),
                                                    (20, 128, 16, 0), (5, 96, 32, 70), (1, 32, 16, 33),
                                                    (16, 512, 64, 0), (2, 192, 0, 300)])
def test_long_portions_share_key_tiles_among_tokens(heads, rank, rot, window):
    """The latent attention kernel alone on a step of long and short portions of several
    requests (the form where a block takes the rows of several tokens, portions ending inside
    a block) against float64 sums: every key before the token, or a window; one token of each
    long portion has a score that stands out on a key far back, or just outside the window."""
    from mstar_b200 import ops

    page, D = 16, rank + rot
    lens, starts = [301, 7, 1, 64, 130, 2], [0, 40, 500, 17, 222, 0]
    g = torch.Generator().manual_seed(heads * 1000 + rank)
    pages_of = [-(-(s + n) // page) for s, n in zip(starts, lens)]
    order = torch.randperm(sum(pages_of) + 2, generator=g)
    table = torch.zeros(len(lens), max(pages_of), dtype=torch.int32)
    at = 0
    for r, n in enumerate(pages_of):
        table[r, :n] = order[at:at + n]
        at += n
    cache = torch.randn(sum(pages_of) + 2, 1, 1, page, D, generator=g).to(torch.bfloat16)
    cache[..., :rank] *= 0.5
    tokens = sum(lens)
    q_abs = torch.randn(tokens, heads, rank, generator=g) * 0.4
    q_rot = (torch.randn(tokens, heads, rot, generator=g) * 0.4).to(torch.bfloat16)
    token_req = torch.cat([torch.full((n,), r) for r, n in enumerate(lens)]).to(torch.int32)
    pos = torch.cat([torch.arange(s, s + n) for s, n in zip(starts, lens)]).to(torch.int32)

    def row(r, key):
        return cache[int(table[r, key // page]), 0, 0, key % page]

    # a query that points at one key: far back, or one key outside the window
    first = {r: sum(lens[:r]) for r in range(len(lens))}
    for r in (0, 4):
        t = first[r] + lens[r] - 3
        key = 1 if not window else int(pos[t]) - window
        q_abs[t, 0] = 6.0 * row(r, key)[:rank].float() / row(r, key)[:rank].float().norm()
    scale = 0.7 * D ** -0.5
    want = torch.zeros(tokens, heads, rank, dtype=torch.float64)
    keys = {}
    for r in range(len(lens)):
        keys[r] = torch.stack([row(r, k) for k in range(starts[r] + lens[r])]).double()
    for t in range(tokens):
        r, p = int(token_req[t]), int(pos[t])
        lo = max(0, p - window + 1) if window else 0
        k = keys[r][lo:p + 1]
        s = (q_abs[t].double() @ k[:, :rank].T + q_rot[t].double() @ k[:, rank:].T) * scale
        want[t] = torch.softmax(s, -1) @ k[:, :rank]
    got = ops.latent_attention(q_abs.to(DEV), q_rot.to(DEV), cache.to(DEV), table.to(DEV),
                               token_req.to(DEV), pos.to(DEV), heads, rank, rot, page, window,
                               scale, max_keys=max(s + n for s, n in zip(starts, lens)),
                               entries=len(lens))
    close(got, want, "float32", "rows of several tokens", f32=2e-4)
    alone = ops.latent_attention(q_abs.to(DEV), q_rot.to(DEV), cache.to(DEV), table.to(DEV),
                                 token_req.to(DEV), pos.to(DEV), heads, rank, rot, page, window,
                                 scale, max_keys=max(s + n for s, n in zip(starts, lens)))
    close(alone, want, "float32", "a token a block", f32=2e-4)


# ------------------------------------------------------------------ whole models
@pytest.fixture(scope="module")
def mixed_model():
    weights = U.random_weights(U.MIXED, seed=3)
    reqs = {"a": U.tokens(U.MIXED, 61, 1), "b": U.tokens(U.MIXED, 24, 2),
            "c": U.tokens(U.MIXED, 1, 3), "d": U.tokens(U.MIXED, 37, 4),
            "e": U.tokens(U.MIXED, 90, 5)}
    want = {r: U.plain_logits(U.MIXED, weights, t) for r, t in reqs.items()}
    models = {}

    def get(dtype):
        if dtype not in models:
            models[dtype] = U.load(U.MIXED, weights, dtype)
        return models[dtype]

    return weights, reqs, want, get


def check_all(got, want, dtype, what):
    for r in want:
        U.assert_close(got[r], want[r], dtype, (what, r))


def stepper_for(model, **kw):
    from mstar_b200.engine.step import make_stepper
    kw.setdefault("page_size", 4)
    kw.setdefault("num_pages", 64)
    kw.setdefault("num_slots", 3)
    return make_stepper(model, **kw)


@pytest.mark.parametrize("dtype", DTYPES)
def test_residual_after_every_layer(mixed_model, dtype):
    """The float residual after each layer of a short prompt, against the plain model's."""
    from mstar_b200.engine.step import StepEntry

    weights, reqs, _, get = mixed_model
    model = get(dtype)
    _, after = P.PlainRelurax(U.MIXED, U.as_numpy(weights)).forward(reqs["b"])
    seen, plain_forward = [], [b.forward for b in model.blocks]

    def watched(forward):
        def run(stream, ctx, cache):
            forward(stream, ctx, cache)
            stream.settle()
            seen.append(stream.h.clone())
        return run

    try:
        for b in model.blocks:
            b.forward = watched(b.forward)
        st = stepper_for(model, cuda_graphs=False)
        st.add_request("b")
        st.step([StepEntry("b", reqs["b"], [])])
    finally:
        for b, f in zip(model.blocks, plain_forward):
            b.forward = f
    assert len(seen) == len(after)
    for i, (got, want) in enumerate(zip(seen, after)):
        assert got.dtype == torch.float32
        close(got, want, dtype, ("residual after layer", i), f32=1e-5, bf16=3e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_whole_prompts_and_token_by_token(mixed_model, dtype):
    """Each request alone: its prompt in one step, and every token as a step of its own (with
    and without captured graphs); the three agree with the plain model."""
    _, reqs, want, get = mixed_model
    model = get(dtype)
    whole = U.run_schedule(stepper_for(model), reqs, [[(r, len(t))] for r, t in reqs.items()])
    check_all(whole, want, dtype, "whole")
    for graphs in (False, True):
        st = stepper_for(model, cuda_graphs=graphs)
        single = U.run_schedule(st, reqs, [[(r, 1)] for r, t in reqs.items() for _ in t])
        check_all(single, want, dtype, f"token by token, graphs={graphs}")
        assert (st.graph_replays > 0) == graphs


@pytest.mark.parametrize("dtype", DTYPES)
def test_portions_of_every_size(mixed_model, dtype):
    """Prompts cut into portions of changing size, down to two tokens, ends decoded one by one:
    cuts fall inside pages, inside windows and between a convolution's taps."""
    _, reqs, want, get = mixed_model
    schedule = []
    for r, t in reqs.items():
        left, sizes, k = len(t), (2, 17, 3, 2, 16, 5, 33, 2), 0
        while left > 6:
            n = min(sizes[k % len(sizes)], left - 6)
            schedule.append([(r, n)])
            left -= n
            k += 1
        schedule += [[(r, 1)]] * left
    got = U.run_schedule(stepper_for(get(dtype)), reqs, schedule)
    check_all(got, want, dtype, "portions")


@pytest.mark.parametrize("dtype", DTYPES)
def test_mixed_batches_reuse_pages_and_slots(mixed_model, dtype):
    """Up to three live requests in a batch, portions beside single tokens, a request sitting
    out a step; five requests go through three slots and a pool of pages that holds less than
    all of them, so that slots and pages are used again; each agrees with itself alone."""
    _, reqs, want, get = mixed_model
    schedule = [
        [("a", 2), ("b", 3), ("c", 1)],               # c ends here: its slot goes to d
        [("a", 29), ("b", 1), ("d", 16)],
        [("a", 1), ("d", 2)],
        [("a", 1), ("b", 18), ("d", 1)],
        [("b", 1), ("a", 20), ("d", 17)],
        [("b", 1), ("a", 1), ("d", 1)],               # b and d end
        [("a", 1), ("e", 2)],
        [("a", 6), ("e", 64)],                        # a ends
        [("e", 1)], [("e", 21)], [("e", 1)], [("e", 1)],
    ]
    st = stepper_for(get(dtype), num_pages=40, num_slots=3)
    got = U.run_schedule(st, reqs, schedule)
    check_all(got, want, dtype, "mixed")
    assert st.manager.num_requests() == 0 and st.manager.check() == 0
    assert st.manager.free_slots() == 3


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_past_many_windows(dtype):
    """A short prompt and 400 decoded tokens through captured graphs: the windows pass over
    decoded tokens many times and their pages return and are taken again, the convolution's
    rows are carried 400 steps, and the latent layers' rows grow past many pages."""
    cfg = U.config([U.layer(U.attention(2, 1, 16, size=13, conv=4, scale=0.4), U.dense(64)),
                    U.layer(U.latent(2, 8, 8, 16, 32, 12, base=50.0, scale=0.5), U.dense(32)),
                    U.layer(U.attention(4, 2, 32, size=9, conv=2, scale=0.3), None),
                    U.layer(U.latent(3, 16, 8, 8, 32, 20, kv_from=1, scale=0.4), U.dense(48))],
                   width=64, vocab=97)
    weights = U.random_weights(cfg, 11)
    toks = U.tokens(cfg, 410, 12)
    want = U.plain_logits(cfg, weights, toks)
    st = stepper_for(U.load(cfg, weights, dtype), page_size=4, num_pages=[9, 110, 9], num_slots=1)
    got = U.run_schedule(st, {"r": toks}, [[("r", 10)]] + [[("r", 1)]] * 400)
    U.assert_close(got["r"], want, dtype, "long decoding")
    assert st.graph_replays == 400


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_prompts_in_one_step(dtype):
    """Two prompts of some hundred tokens in one step (what the prompt forms of the attention
    kernels take: several tokens a block, a portion ending inside a block), a third admitted
    beside their decoding."""
    cfg = U.config([U.layer(U.latent(4, 16, 16, 16, 64, 32, base=1000.0, scale=0.3), U.dense(64)),
                    U.layer(U.attention(4, 2, 32, size=150, conv=3, scale=0.25), U.dense(48)),
                    U.layer(U.latent(6, 8, 16, 24, 64, 24, kv_from=0, scale=0.35), None)],
                   width=64, vocab=120)
    weights = U.random_weights(cfg, 41)
    reqs = {"x": U.tokens(cfg, 333, 1), "y": U.tokens(cfg, 301, 2), "z": U.tokens(cfg, 310, 3)}
    want = {r: U.plain_logits(cfg, weights, t) for r, t in reqs.items()}
    st = stepper_for(U.load(cfg, weights, dtype), page_size=16, num_pages=64, num_slots=3)
    got = U.run_schedule(st, reqs, [[("x", 330), ("y", 299)], [("x", 1), ("y", 1), ("z", 309)],
                                    [("x", 2), ("y", 1), ("z", 1)]])
    check_all(got, want, dtype, "long prompts")


@pytest.mark.parametrize("dtype", DTYPES)
def test_sizes_that_are_one_or_equal(dtype):
    """One query head on one key head, a window of one, one tap, a query latent as wide as the
    key latent, one latent head, a rotated part of one pair; a model of latent layers only and
    one of window layers only; a latent layer first, read by the last; and sizes that are
    multiples of nothing (a width of 100, heads of 12 and 10, a vocabulary of 53)."""
    for layers, width, vocab in (
            ([U.layer(U.attention(1, 1, 16, size=1, conv=1, scale=0.25), U.dense(8)),
              U.layer(U.latent(1, 8, 2, 8, 16, 16, dims=2, scale=0.3), None)], 32, 50),
            ([U.layer(U.latent(2, 8, 4, 8, 8, 8, base=20.0, scale=0.5), U.dense(16)),
              U.layer(U.latent(2, 8, 4, 8, 8, 8, kv_from=0, scale=0.5), None),
              U.layer(U.latent(1, 4, 4, 4, 8, 4, kv_from=0, scale=0.5), U.dense(16))], 32, 50),
            ([U.layer(U.attention(2, 2, 8, size=3, conv=2, scale=0.5), None),
              U.layer(U.attention(4, 1, 8, size=64, conv=3, scale=0.5), U.dense(16))], 32, 50),
            ([U.layer(U.latent(3, 12, 6, 10, 20, 14, base=77.0, scale=0.4), U.dense(36)),
              U.layer(U.attention(3, 1, 12, size=6, conv=3, scale=0.4), U.dense(20)),
              U.layer(U.attention(6, 3, 10, size=9, conv=2, scale=0.4), None),
              U.layer(U.latent(5, 10, 6, 12, 20, 30, kv_from=0, scale=0.4), U.dense(28))], 100, 53)):
        cfg = U.config(layers, width=width, vocab=vocab)
        weights = U.random_weights(cfg, 21)
        reqs = {"x": U.tokens(cfg, 33, 1), "y": U.tokens(cfg, 12, 2)}
        want = {r: U.plain_logits(cfg, weights, t) for r, t in reqs.items()}
        st = stepper_for(U.load(cfg, weights, dtype))
        got = U.run_schedule(st, reqs, [[("x", 7), ("y", 2)], [("x", 1), ("y", 10)],
                                        [("x", 25)]])
        check_all(got, want, dtype, "small sizes")


@pytest.mark.parametrize("dtype", DTYPES)
def test_layers_of_a_larger_model(dtype):
    """Head sizes, ranks and widths as a model of some billion weights has them (what the
    tensor-core kernels and the large-product paths take), on a few tokens."""
    cfg = U.config([U.layer(U.attention(8, 2, 128, size=24, conv=4, scale=128 ** -0.5), U.dense(640)),
                    U.layer(U.latent(4, 128, 64, 128, 256, 192, base=10000.0, scale=192 ** -0.5),
                            U.dense(512)),
                    U.layer(U.latent(8, 64, 64, 64, 256, 128, kv_from=1, scale=128 ** -0.5), None)],
                   width=512, vocab=300)
    weights = U.random_weights(cfg, 31)
    reqs = {"x": U.tokens(cfg, 70, 1), "y": U.tokens(cfg, 40, 2)}
    want = {r: U.plain_logits(cfg, weights, t) for r, t in reqs.items()}
    st = stepper_for(U.load(cfg, weights, dtype), page_size=16, num_pages=16)
    got = U.run_schedule(st, reqs, [[("x", 50), ("y", 2)], [("x", 1), ("y", 37)], [("x", 1), ("y", 1)],
                                    [("x", 18)]])
    check_all(got, want, dtype, "larger layers")


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_entry_point(mixed_model, dtype, tmp_path):
    """LLM.generate with its scheduler (portions under a small token budget, several requests
    at once) picks the tokens the plain model picks; in bfloat16 a pick may differ only where
    the plain model's own margin is small, but for one token in twenty."""
    import json

    from safetensors.torch import save_file

    from mstar_b200 import LLM, SamplingParams

    weights, reqs, _, _ = mixed_model
    (tmp_path / "config.json").write_text(json.dumps(U.MIXED))
    save_file({k: v.contiguous() for k, v in weights.items()}, str(tmp_path / "model.safetensors"))
    llm = LLM(str(tmp_path), dtype=dtype, page_size=8, max_num_pages=48,
              max_num_batched_tokens=16, max_concurrent_requests=3)
    prompts = [reqs["a"][:40], reqs["b"][:5], reqs["d"][:19], reqs["e"][:2]]
    n_new = 12
    results = llm.generate(prompts, SamplingParams(temperature=0.0, ignore_eos=True,
                                                   max_output_tokens=n_new))
    far_off = 0
    for prompt, res in zip(prompts, results):
        assert len(res.token_ids) == n_new
        for tok, (best, margin) in zip(res.token_ids,
                                       U.plain_greedy_check(U.MIXED, weights, prompt, res.token_ids)):
            assert tok == best or dtype == "bfloat16", (tok, best, margin)
            far_off += tok != best and margin >= 0.25
    assert far_off <= len(prompts) * n_new // 20, far_off


def test_trace_replay_of_a_model_folder(mixed_model, tmp_path):
    """bin/trace_run on a folder of this design: the registry picks the model by config.json."""
    import json
    import subprocess
    import sys
    from pathlib import Path

    from safetensors.torch import save_file

    weights, reqs, want, _ = mixed_model
    folder = tmp_path / "model"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(U.MIXED))
    save_file({k: v.contiguous() for k, v in weights.items()}, str(folder / "model.safetensors"))
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": reqs["a"][:50], "want": [3, 49]},
                                     {"id": "b", "tokens": reqs["b"][:2], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "b", "tokens": reqs["b"][2:], "want": [0]},
                                     {"id": "a", "tokens": reqs["a"][50:51], "want": [0]}],
              "end": ["b"]}]
    exe = Path(__file__).resolve().parent.parent / "bin" / "trace_run"
    out = tmp_path / "out"
    done = subprocess.run([sys.executable, str(exe), "--model", str(folder), "--dtype", "float32",
                           "--out", str(out), "--max-tokens", "128"],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", text=True,
                          capture_output=True, timeout=900)
    assert done.returncode == 0, done.stderr[-2000:]
    assert [l for l in done.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1"]
    got0 = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(2, -1))
    got1 = torch.from_numpy(np.fromfile(out / "1.f32", dtype="<f4").reshape(2, -1))
    U.assert_close(got0, want["a"][[3, 49]], "float32", "trace step 0")
    U.assert_close(got1, torch.stack([want["b"][2], want["a"][50]]), "float32", "trace step 1")
