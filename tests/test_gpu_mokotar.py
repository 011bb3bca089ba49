"""The Mokotar decoder in the engine against the plain implementation (tests/plain_mokotar.py):
each mechanism alone, then whole models through the step function, the cache and state
manager, the scheduler and the entry point, under every kind of schedule."""
import numpy as np
import pytest
import torch

import mokotar_util as U
import plain_mokotar as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = ["float32", "bfloat16"]
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}
EPS = 1e-5


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


# ------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("streams,width", [(1, 64), (2, 200), (3, 1000), (8, 72)])
def test_hyper_connection_kernel(dtype, streams, width):
    """First read from the embedding output, a write with one output, a write with two
    weighted outputs and a bias, and the sum of the copies of chosen rows with a write still
    pending: against the plain read and write."""
    from mstar_b200 import ops

    T, m = 7, 0.35
    g = torch.Generator().manual_seed(streams)
    emb = rnd(T, width, seed=1).float()
    tabs = [(torch.randn(streams, generator=g), torch.randn(streams, generator=g),
             torch.randn(streams, streams, generator=g)) for _ in range(3)]
    norm_w = (rnd(width, seed=2).float() + 1.0).to(torch.bfloat16).float()
    y1, y2 = rnd(T, width, seed=3, scale=2.0), rnd(T, width, seed=4, scale=2.0)
    bias = rnd(width, seed=5)
    x = torch.empty(T, streams, width, device=DEV)
    f = lambda t: t.contiguous().to(DEV)
    eye, zero = torch.eye(streams), torch.zeros(streams)
    # the copies start as the embedding output
    xs = np.stack([emb.double().numpy()] * streams)
    got = ops.hyper_step(x, init=f(emb), mix=f(eye), out=f(zero), read=f(tabs[0][0]),
                         norm_weight=dev(norm_w, dtype), eps=EPS, out_dtype=TORCH[dtype])
    want = P.plain_rms_norm(P.plain_hyper_read(xs, tabs[0][0].double().numpy()), norm_w.double().numpy(), EPS)
    close(got, want, dtype, "first read", bf16=8e-3)
    close(x.transpose(0, 1), xs, "float32", "copies written")
    # one output
    xs = P.plain_hyper_write(xs, y1.double().numpy(), tabs[0][2].double().numpy(),
                             tabs[0][1].double().numpy(), m)
    got = ops.hyper_step(x, y=dev(y1, dtype), mix=f(tabs[0][2]), out=f(tabs[0][1] * m),
                         read=f(tabs[1][0]), norm_weight=dev(norm_w, dtype), eps=EPS,
                         out_dtype=TORCH[dtype])
    want = P.plain_rms_norm(P.plain_hyper_read(xs, tabs[1][0].double().numpy()), norm_w.double().numpy(), EPS)
    close(x.transpose(0, 1), xs, "float32", "write")
    close(got, want, dtype, "read after write", bf16=8e-3)
    # two weighted outputs and a bias, left pending; the sum of rows sees them
    y = 1.2 * y1.double().numpy() + 0.9 * y2.double().numpy() + bias.double().numpy()
    after = P.plain_hyper_write(xs, y, tabs[1][2].double().numpy(), tabs[1][1].double().numpy(), m)
    rows = torch.tensor([T - 1, 0, 3, 3], dtype=torch.int32, device=DEV)
    before = x.clone()
    got = ops.hyper_step(x, y=dev(y1, dtype), y2=dev(y2, dtype), y_scales=(1.2, 0.9),
                         y_bias=dev(bias, dtype), mix=f(tabs[1][2]), out=f(tabs[1][1] * m), rows=rows)
    close(got, after.sum(0)[[T - 1, 0, 3, 3]], "float32", "sum of copies")
    assert torch.equal(x, before)                      # a sum leaves the copies alone


@pytest.mark.parametrize("dtype", DTYPES)
def test_block_with_one_copy_is_the_plain_residual(dtype):
    """streams 0: x += m * mixer(norm1(x)); x += m * ff(norm2(x)) through the same kernels,
    the feed-forward's three biases included; and a block without a feed-forward."""
    for mlp in ("dense", None):
        cfg = U.config([U.layer("attention", U.attention(2, 1, 16, 24), mlp=mlp)], width=48,
                       vocab=31, streams=0, mult=0.6)
        w = U.random_weights(cfg, 5)
        toks = U.tokens(cfg, 12, 1)
        want = U.plain_logits(cfg, w, toks)
        st = stepper_for(U.load(cfg, w, dtype))
        got = U.run_schedule(st, {"r": toks}, [[("r", 5)], [("r", 2)]] + [[("r", 1)]] * 5)
        U.assert_close(got["r"], want, dtype, ("one copy", mlp))


@pytest.mark.parametrize("dtype", DTYPES)
def test_biased_gated_feed_forward(dtype):
    from mstar_b200.config.layout import GatedMLPSpec
    from mstar_b200.parts import build_part
    from mstar_b200.parts.mlp import OutputWithBias

    for rows, width, ff in ((9, 96, 200), (150, 72, 40)):
        x = rnd(rows, width, seed=6)
        w = {"gate": rnd(ff, width, seed=1, scale=0.1), "up": rnd(ff, width, seed=2, scale=0.1),
             "down": rnd(width, ff, seed=3, scale=0.1), "gate.b": rnd(ff, seed=4),
             "up.b": rnd(ff, seed=5), "down.b": rnd(width, seed=7)}
        part = build_part("ffn", GatedMLPSpec(hidden_size=width, intermediate_size=ff, bias=True),
                          {"gate_up.weight": dev(torch.cat([w["gate"], w["up"]]), dtype),
                           "gate_up.bias": dev(torch.cat([w["gate.b"], w["up.b"]]), dtype),
                           "down.weight": dev(w["down"], dtype), "down.bias": dev(w["down.b"], dtype)},
                          runtime(dtype))
        out = part.forward(dev(x, dtype), None)
        assert isinstance(out, OutputWithBias)           # the last bias travels with the output
        want = P.plain_feed_forward(x.double().numpy(), {k: v.double().numpy() for k, v in w.items()}, "")
        close(out.materialize(), want, dtype, ("biased feed-forward", rows), bf16=2e-2)


def attention_part(kind, m, width, dtype, seed, sharp=3.0):
    from mstar_b200.config.registry import config_from_dict
    from mstar_b200.parts import build_part

    if kind == "left":
        cfg = U.config([U.layer("parallel", U.parallel(l=m))], width=width)
        p = "l0.mix.left."
    else:
        cfg = U.config([U.layer(kind, m)], width=width)
        p = "l0.mix."
    w = U.random_weights(cfg, seed, sharp=sharp)
    mixer = config_from_dict(cfg).layout().blocks[0].mixer
    spec = mixer.branches[0] if kind == "left" else mixer
    stack = [w[p + "q"], w[p + "k"], w[p + "v"]] + ([w[p + "g"]] if kind != "left" else [])
    params = {"qkv.weight": torch.cat(stack), "q_norm.weight": w[p + "q.norm"],
              "k_norm.weight": w[p + "k.norm"], "o.weight": w[p + "o"]}
    if kind != "left":
        params["sink"] = w[p + "sink"]
    part = build_part("mixer", spec, {k: dev(v, dtype) for k, v in params.items()}, runtime(dtype))
    return part, spec, U.sub(w, p)


def paged_cache(part_spec, tokens, page, dtype, seed=1):
    """Pages scattered over a pool that holds leftovers of other requests."""
    from mstar_b200 import ops
    from mstar_b200.parts import LayerCache

    pages = -(-tokens // page)
    elems = ops.sink_page_elements(part_spec.num_kv_heads, page, part_spec.head_dim,
                                   part_spec.value_dim)
    kv = torch.full((pages + 3, elems), 7.0, dtype=TORCH[dtype], device=DEV)
    table = (torch.randperm(pages + 3, generator=torch.Generator().manual_seed(seed))[:pages]
             .to(torch.int32).to(DEV)[None])
    return LayerCache(kv=kv, page_size=page, block_table=table)


def plain_attention(kind, x, p, m, positions=None):
    positions = np.arange(x.shape[0]) if positions is None else positions
    return P.plain_attention(x, positions, p, "", m, EPS, {}, kind)


ATTENTIONS = [
    ("attention", U.attention(4, 2, 24, 40, scale=6.0 / 24, coef=0.4, every=7, softcap=5.0), 4),
    ("attention", U.attention(3, 3, 16, 8, scale=0.4, coef=1.0, every=1, softcap=50.0), 8),
    ("attention", U.attention(34, 1, 16, 24, scale=0.4, coef=0.1, every=64, softcap=1.0), 16),
    ("attention", U.attention(2, 1, 160, 256, scale=0.04, coef=0.3, every=16, softcap=30.0), 8),
    ("attention", U.attention(2, 2, 12, 10, scale=0.5, coef=0.3, every=5, softcap=4.0), 4),
    ("attention_2", U.attention_2(4, 2, 32, 16, scale=0.2, rot_dims=12, base=300.0), 4),
    ("attention_2", U.attention_2(4, 2, 128, 128, scale=0.06, rot_dims=128, base=70000.0), 16),
    ("attention_2", U.attention_2(1, 1, 20, 20, scale=0.3, rot_dims=2, base=10.0), 8),
    ("attention_2", U.attention_2(5, 5, 96, 72, scale=0.1, rot_dims=32), 16),
    ("left", U.left(4, 1, 16, 24, scale=0.5, rot_dims=16), 4),
    ("left", U.left(4, 2, 64, 64, scale=0.125, rot_dims=16, base=1e5), 16),
    ("left", U.left(3, 3, 20, 12, scale=0.3, rot_dims=8, base=50.0), 8),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind,m,page", ATTENTIONS)
def test_attention_alone(dtype, kind, m, page):
    """Each of the three attentions alone with scores so sharp that a query's weight lies on
    a few keys and on the sink; a prompt portion, portions of two, single tokens (several
    temperature steps are crossed), pages scattered over the pool."""
    part, spec, p = attention_part(kind, m, 96, dtype, seed=7, sharp=3.0)
    T = 70
    x = rnd(T, 96, seed=8)
    want = plain_attention(kind, x.double().numpy(), p, m)
    if kind != "left":            # the sink matters: without it the output differs
        other = plain_attention(kind, x.double().numpy(), dict(p, sink=p["sink"] - 30.0), m)
        assert np.abs(other - want).max() > 0.05 * np.abs(want).max()
    cache = paged_cache(spec, T, page, dtype)
    outs, at = [], 0
    for n in (23, 2, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 29, 3, 2):
        outs.append(part.forward(dev(x[at:at + n], dtype), step_ctx([n], [at]), cache))
        at += n
    assert at == T
    close(torch.cat(outs), want, dtype, ("attention", kind), bf16=6e-2)


def marked_inputs(p, m, width, T, marked, queries, gain=4.0):
    """Inputs in which the key at ``marked`` carries the weight of the ``queries``: the query
    tokens lie along a direction d, the marked token along the direction whose key equals
    the query of d (a solution of W_k d' = W_q d), so that its score stands out among
    hundreds.  A query token's own key points elsewhere."""
    x = rnd(T, width, seed=4, scale=0.3)
    d = rnd(width, seed=5).double().numpy()
    dim = m["dim"]
    target = p["q"][:dim] @ d                                  # the first query head
    d_key = np.linalg.lstsq(p["k"][:dim], target, rcond=None)[0]
    x[marked] = torch.from_numpy(gain * d_key).to(torch.bfloat16)
    for q in queries:
        x[q] += torch.from_numpy(gain * d).to(torch.bfloat16)
    return x


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("marked,page", [(0, 16), (15, 16), (16, 16), (3, 4), (257, 8)])
def test_one_far_key_stands_out(dtype, marked, page):
    """One key hundreds of tokens back (the first token, the last of a page, the first of the
    next) carries a query's weight; a wrong page or a lost first key changes the output by
    that key's whole value.  The query in a prompt portion and decoded alone."""
    m = U.attention(2, 1, 32, 32, scale=1.0, coef=0.2, every=100, softcap=40.0)
    T, queries = 330, [300, 329]
    part, spec, p = attention_part("attention", m, 64, dtype, seed=3, sharp=1.0)
    x = marked_inputs(p, m, 64, T, marked, queries)
    xn = x.double().numpy()
    want = plain_attention("attention", xn, p, m)
    hidden = xn.copy()
    hidden[marked] = 0.0
    blind = plain_attention("attention", hidden, p, m)
    for q in queries:             # how much hangs on the one key
        assert np.abs(blind[q] - want[q]).max() > 0.3 * np.abs(want[q]).max(), (marked, q)
    for first in (T, 290):                    # one prompt; a prompt and decoded tokens
        cache = paged_cache(spec, T, page, dtype, seed=first)
        outs = [part.forward(dev(x[:first], dtype), step_ctx([first], [0]), cache)]
        outs += [part.forward(dev(x[t:t + 1], dtype), step_ctx([1], [t]), cache)
                 for t in range(first, T)]
        close(torch.cat(outs), want, dtype, ("far key", marked, first), bf16=6e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_soft_cap_and_temperature_change_what_wins(dtype):
    """Scores far above the cap: the cap flattens them, the temperature (a large coefficient,
    a step every two positions) sharpens later queries; leaving either out gives another
    output, and the engine gives the one with both."""
    m = U.attention(2, 1, 16, 16, scale=2.0, coef=2.0, every=2, softcap=3.0)
    part, spec, p = attention_part("attention", m, 64, dtype, seed=9, sharp=3.0)
    x = rnd(40, 64, seed=2)
    xn = x.double().numpy()
    want = plain_attention("attention", xn, p, m)
    no_cap = plain_attention("attention", xn, p, dict(m, softcap=None))
    no_temp = plain_attention("attention", xn, p, dict(m, q_temp=None))
    assert np.abs(no_cap - want).max() > 0.2 * np.abs(want).max()
    assert np.abs(no_temp - want).max() > 0.05 * np.abs(want).max()
    cache = paged_cache(spec, 40, 8, dtype)
    got = torch.cat([part.forward(dev(x[:31], dtype), step_ctx([31], [0]), cache)] +
                    [part.forward(dev(x[t:t + 1], dtype), step_ctx([1], [t]), cache)
                     for t in range(31, 40)])
    close(got, want, dtype, "cap and temperature", bf16=6e-2)


def delta_part(m, width, dtype, seed, ranks=U.RANKS):
    from mstar_b200.config.layout import GatedDeltaSpec
    from mstar_b200.parts import build_part

    cfg = U.config([U.layer("parallel", U.parallel(r=m))], width=width)
    w = U.random_weights(cfg, seed, ranks=ranks)
    p = "l0.mix.right."
    spec = GatedDeltaSpec(hidden_size=width, num_heads=m["heads"], num_kv_heads=m["kv_heads"],
                          qk_dim=m["dim"], v_dim=m["vdim"], conv=m["conv"], decay_rank=ranks[0],
                          gate_rank=ranks[1], norm_eps=EPS)
    params = {"in.weight": torch.cat([w[p + n] for n in ("q", "k", "v", "b", "a1", "g1")]),
              "conv.weight": torch.cat([w[p + n + ".conv"] for n in ("q", "k", "v")]),
              "a2.weight": w[p + "a2"], "dt_bias": w[p + "dt_bias"], "A_log": w[p + "A_log"],
              "g2.weight": w[p + "g2"], "norm.weight": w[p + "norm"], "o.weight": w[p + "o"]}
    part = build_part("mixer", spec, {k: dev(v, dtype) for k, v in params.items()}, runtime(dtype))
    return part, spec, U.sub(w, p)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,taps",
                         [(4, 2, 24, 20, 3), (3, 3, 10, 36, 4), (1, 1, 64, 32, 1), (4, 4, 64, 48, 3),
                          (6, 2, 72, 130, 2), (2, 1, 130, 8, 5), (8, 2, 300, 16, 2)])
def test_gated_delta_rule_alone(dtype, heads, kv_heads, dim, vdim, taps):
    """The recurrent branch over a sequence cut into a portion, a two-token portion, single
    tokens (fewer than the convolution has taps) and more portions, in a slot that held
    another request's state, against the token-by-token recurrence; then two sequences in one
    batch in other slots."""
    from mstar_b200 import ops
    from mstar_b200.parts import LayerCache

    m = U.right(heads, kv_heads, dim, vdim, taps)
    part, spec, p = delta_part(m, 96, dtype, seed=dim)
    T = 45
    x = rnd(T, 96, seed=5)
    want = P.plain_gated_delta(x.double().numpy(), p, "", m, EPS, {})
    size = ops.gated_delta_state_size(heads, kv_heads, dim, vdim, taps)
    slots = torch.randn(4, size, device=DEV)               # leftovers of earlier requests
    slots[2].zero_()
    cache = LayerCache(state=slots)
    outs, at = [], 0
    for n in (19, 2, 1, 1, 1, 17, 4):
        outs.append(part.forward(dev(x[at:at + n], dtype), step_ctx([n], [at], [2]), cache))
        at += n
    assert at == T
    close(torch.cat(outs), want, dtype, "gated delta rule", bf16=5e-2)
    slots2 = torch.zeros(4, size, device=DEV)
    both = part.forward(dev(torch.cat([x[:9], x[:30]]), dtype), step_ctx([9, 30], [0, 0], [3, 0]),
                        LayerCache(state=slots2))
    close(both[:9], want[:9], dtype, "first of two", bf16=5e-2)
    close(both[9:], want[:30], dtype, "second of two", bf16=5e-2)
    assert float(slots2[1].abs().max()) == 0.0 and float(slots2[3].abs().max()) > 0.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,taps",
                         [(4, 2, 24, 20, 3), (2, 1, 128, 40, 2), (2, 2, 200, 9, 1), (5, 1, 64, 64, 3),
                          (2, 2, 32, 12, 3), (2, 1, 256, 20, 2), (3, 1, 64, 7, 4)])
def test_delta_rule_long_portions_in_pieces(dtype, heads, kv_heads, dim, vdim, taps):
    """A portion long enough to be scanned in pieces of 16 tokens (what does not depend on the
    state made ahead for all pieces, a scalar chain within a piece; key sizes of 32, 64, 128
    and 256 take that form, the others and a state that does not start on a 16-byte boundary
    the token-by-token kernel), beside a short portion
    of another request in the same batch; then more tokens of both, a portion that is no
    multiple of 16 and a last one of a single token: against the token-by-token recurrence."""
    from mstar_b200 import ops
    from mstar_b200.parts import LayerCache

    m = U.right(heads, kv_heads, dim, vdim, taps)
    part, spec, p = delta_part(m, 96, dtype, seed=dim + 1)
    T = ops.DELTA_PIECES_FROM + 3 * ops.DELTA_PIECE + 5
    x = rnd(T + 80, 96, seed=6)
    want = P.plain_gated_delta(x.double().numpy(), p, "", m, EPS, {})
    short = P.plain_gated_delta(x[:9].double().numpy(), p, "", m, EPS, {})
    size = ops.gated_delta_state_size(heads, kv_heads, dim, vdim, taps)
    slots = torch.randn(3, size, device=DEV)
    slots[:2].zero_()
    cache = LayerCache(state=slots)
    got = part.forward(dev(torch.cat([x[:5], x[:T]]), dtype), step_ctx([5, T], [0, 0], [1, 0]), cache)
    close(got[5:], want[:T], dtype, "pieces", bf16=5e-2)
    close(got[:5], short[:5], dtype, "short beside pieces", bf16=5e-2)
    more = part.forward(dev(torch.cat([x[5:9], x[T:T + 79]]), dtype), step_ctx([4, 79], [5, T], [1, 0]),
                        cache)
    close(more[4:], want[T:T + 79], dtype, "after pieces", bf16=5e-2)
    close(more[:4], short[5:], dtype, "short after pieces", bf16=5e-2)
    last = part.forward(dev(x[T + 79:], dtype), step_ctx([1], [T + 79], [0]), cache)
    close(last, want[T + 79:], dtype, "one more token", bf16=5e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_delta_rule_state_is_carried_a_long_way(dtype):
    """Decays close to one: what the first tokens wrote is still read hundreds of tokens on, so
    a state lost or reset at a portion's edge shows.  The plain model without its first
    tokens gives another output at the end."""
    from mstar_b200 import ops
    from mstar_b200.parts import LayerCache

    m = U.right(2, 1, 64, 12, 2)
    part, spec, p = delta_part(m, 64, dtype, seed=21)
    part.dt_bias.fill_(-9.0)                                # decays of about 0.9999 a token
    p["dt_bias"] = np.full_like(p["dt_bias"], -9.0)
    T = 300
    x = rnd(T, 64, seed=6)
    xn = x.double().numpy()
    want = P.plain_gated_delta(xn, p, "", m, EPS, {})
    late = P.plain_gated_delta(xn[200:], p, "", m, EPS, {})
    assert np.abs(late[-1] - want[-1]).max() > 0.05 * np.abs(want[-1]).max()
    size = ops.gated_delta_state_size(2, 1, 64, 12, 2)
    cache = LayerCache(state=torch.zeros(1, size, device=DEV))
    outs, at = [], 0
    for n in [130, 2, 101] + [1] * 67:
        outs.append(part.forward(dev(x[at:at + n], dtype), step_ctx([n], [at], [0]), cache))
        at += n
    close(torch.cat(outs), want, dtype, "long carry", bf16=5e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_weighted_sum_of_two_branches(dtype):
    from mstar_b200 import ops

    a, b = rnd(9, 130, seed=1), rnd(9, 130, seed=2)
    s = ops.WeightedSum([dev(a, dtype), dev(b, dtype)], (1.3, -0.4))
    close(s.materialize(), 1.3 * a.double() - 0.4 * b.double(), dtype, "weighted sum", bf16=8e-3)


# ------------------------------------------------------------------ whole models
@pytest.fixture(scope="module")
def mixed_model():
    weights = U.random_weights(U.MIXED, seed=3)
    reqs = {"a": U.tokens(U.MIXED, 61, 1), "b": U.tokens(U.MIXED, 24, 2),
            "c": [52], "d": U.tokens(U.MIXED, 37, 4),
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
def test_residual_after_every_layer_run(mixed_model, dtype):
    """The sum of the residual's copies after each of the eight layer runs (a looped stretch
    counts every pass) against the plain model's: a fault shows in the run it enters."""
    from mstar_b200.engine.step import StepEntry
    from mstar_b200.parts import block as B

    weights, reqs, _, get = mixed_model
    want = []
    P.plain_forward(reqs["b"], U.as_numpy(weights), U.MIXED, layer_outputs=want)
    seen = []
    orig = B.HyperBlock.forward

    def recording(self, stream, ctx, cache):
        orig(self, stream, ctx, cache)
        rows = torch.arange(stream.copies.x.shape[0], dtype=torch.int32, device=DEV)
        seen.append(stream.copies.gather(rows).cpu())

    B.HyperBlock.forward = recording
    try:
        st = stepper_for(get(dtype))
        st.add_request("b")
        st.step([StepEntry("b", reqs["b"], [0])])
    finally:
        B.HyperBlock.forward = orig
    assert len(seen) == len(want) == U.runs(U.MIXED)
    for run, (g, w) in enumerate(zip(seen, want)):
        close(g, w, dtype, ("layer run", run), f32=2e-5, bf16=3e-2)


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
    cuts fall inside pages, inside the convolutions' taps, across temperature steps and
    inside the scan's token chunks."""
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
def test_long_decoding(dtype):
    """A short prompt and 400 decoded tokens through captured graphs: many temperature steps,
    keys over a hundred pages, the delta rule's matrix and the convolutions' rows carried 400
    steps."""
    cfg = U.config([U.layer("attention", U.attention(2, 1, 16, 24, scale=0.4, coef=0.5, every=32,
                                                     softcap=6.0), U.dense(64)),
                    U.layer("parallel", U.parallel(U.left(2, 2, 32, 16, scale=0.3, rot_dims=32),
                                                   U.right(2, 1, 24, 8, conv=4)), U.dense(32)),
                    U.layer("attention_2", U.attention_2(2, 1, 24, 24, scale=0.3, rot_dims=8),
                            mlp=None)],
                   width=64, vocab=97, streams=2, loop=(1, 3, 2))
    weights = U.random_weights(cfg, 11)
    toks = U.tokens(cfg, 410, 12)
    want = U.plain_logits(cfg, weights, toks)
    st = stepper_for(U.load(cfg, weights, dtype), page_size=4, num_pages=104, num_slots=1)
    got = U.run_schedule(st, {"r": toks}, [[("r", 10)]] + [[("r", 1)]] * 400)
    U.assert_close(got["r"], want, dtype, "long decoding")
    assert st.graph_replays == 400


@pytest.mark.parametrize("dtype", DTYPES)
def test_sizes_that_are_one_or_equal(dtype):
    """One query head on one key head, a value as wide as a key, one tap, one copy of the
    residual, a temperature step at every position, a multiplier of one, ranks of one, a
    loop of one layer run three times, a loop that is the whole model, no loop; and sizes
    that are multiples of nothing (a width of 100, heads of 12 and 10, a vocabulary of 53)."""
    for layers, kw, ranks in (
            ([U.layer("attention", U.attention(1, 1, 16, 16, scale=0.25, coef=1.0, every=1, softcap=1.0)),
              U.layer("parallel", U.parallel(U.left(1, 1, 8, 8, rot_dims=8), U.right(1, 1, 8, 8, conv=1),
                                             1.0, 1.0), mlp=None)],
             dict(width=32, vocab=50, mult=1.0, streams=1, loop=(1, 2, 3)), (1, 1)),
            ([U.layer("attention_2", U.attention_2(2, 2, 8, 8, scale=0.5, rot_dims=8)),
              U.layer("parallel", U.parallel(U.left(2, 2, 8, 8, rot_dims=2), U.right(2, 2, 8, 8, conv=2)))],
             dict(width=32, vocab=50, mult=0.7, streams=4, loop=(0, 2, 2)), (8, 8)),
            ([U.layer("parallel", U.parallel(U.left(3, 1, 12, 10, rot_dims=6),
                                             U.right(5, 1, 12, 10, conv=3)), U.dense(36)),
              U.layer("attention", U.attention(3, 3, 12, 10, scale=0.4, coef=0.3, every=4, softcap=9.0),
                      U.dense(20)),
              U.layer("attention_2", U.attention_2(3, 1, 10, 12, scale=0.4, rot_dims=10))],
             dict(width=100, vocab=53, mult=0.6, streams=2, loop=None), (3, 6))):
        cfg = U.config(layers, **kw)
        weights = U.random_weights(cfg, 21, ranks=ranks)
        reqs = {"x": U.tokens(cfg, 33, 1), "y": U.tokens(cfg, 12, 2)}
        want = {r: U.plain_logits(cfg, weights, t) for r, t in reqs.items()}
        st = stepper_for(U.load(cfg, weights, dtype))
        got = U.run_schedule(st, reqs, [[("x", 7), ("y", 2)], [("x", 1), ("y", 10)],
                                        [("x", 25)]])
        check_all(got, want, dtype, "small sizes")


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
    w = U.as_numpy(weights)
    far_off = 0
    for prompt, res in zip(prompts, results):
        assert len(res.token_ids) == n_new
        states = [{} for _ in range(U.runs(U.MIXED))]
        logits = P.plain_forward(list(prompt), w, U.MIXED, states)[-1]
        for tok in res.token_ids:
            best = int(np.argmax(logits))
            margin = float(logits[best] - logits[tok])
            assert tok == best or dtype == "bfloat16", (tok, best, margin)
            far_off += tok != best and margin >= 0.25
            logits = P.plain_forward([tok], w, U.MIXED, states)[-1]
    assert far_off <= len(prompts) * n_new // 20, far_off


def test_trace_replay_of_a_model_folder(mixed_model, tmp_path):
    """bin/trace_run on a folder of this design: the registry picks the model by config.json,
    the ranks of the low-rank projections come from the tensors."""
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
