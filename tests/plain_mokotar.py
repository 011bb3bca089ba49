"""A plain, slow implementation of the Mokotar decoder in numpy float64: one function per
mechanism, written from the design's equations and sharing nothing with the engine.

The residual is ``streams`` copies of the embedding output (hyper-connections): a sublayer
reads a weighted sum of the copies through an RMS norm, and every copy becomes a mix of the
old copies plus its own share of the sublayer's output times ``residual_mult``.  Without
``streams`` it is the plain ``x += m * sublayer(norm(x))``.  A mixer is one of

* ``attention``: grouped queries, an RMS norm per query and key head, no rotation; the query
  is multiplied by a temperature that grows with the logarithm of the position; scores are
  scaled, soft-capped by a tanh, and the softmax has a learned sink a head in its
  denominator; the heads are gated feature by feature by a sigmoid of the mixer's input;
* ``attention_2``: the RMS norm runs over all heads of q (and of k) at once, rotary pairs
  ``(2i, 2i + 1)`` over the first ``rot.dims`` features, sink and gate as above;
* ``parallel``: a softmax attention with one added to its denominator (norm a head, rotary
  pairs) beside a gated delta rule (short causal convolutions with SiLU on q, k and v, unit
  q and k, a decay per head and key channel, a write strength a head), summed with two
  weights.

The feed-forward is ``down(silu(gate h) * up h)`` with biases, or absent.  Layers
``loop.start .. loop.stop - 1`` run ``loop.times`` times with the same tensors and a cache of
their own each time.

Everything works on one sequence; ``states`` (a dict per layer run) carries keys, values, the
delta rule's matrix and the convolutions' last inputs from call to call, so that a sequence
can be fed whole, in portions, or token by token.
"""
from __future__ import annotations

import math

import numpy as np

F = np.float64


def plain_rms_norm(x, weight, eps):
    x = np.asarray(x, F)
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * np.asarray(weight, F)


def plain_sigmoid(z):
    return 1.0 / (1.0 + np.exp(-np.asarray(z, F)))


def plain_silu(z):
    z = np.asarray(z, F)
    return z * plain_sigmoid(z)


def plain_softplus(z):
    z = np.asarray(z, F)
    return np.maximum(z, 0.0) + np.log1p(np.exp(-np.abs(z)))


def plain_rotate_pairs(x, positions, dims, base):
    """x: [tokens, heads, dim]; feature 2i is rotated with feature 2i + 1 by the angle
    position * base^(-2i/dims), for i < dims / 2."""
    x = np.array(x, F)
    for i in range(dims // 2):
        ang = np.asarray(positions, F) * float(base) ** (-2.0 * i / dims)
        c, s = np.cos(ang)[:, None], np.sin(ang)[:, None]
        u, v = x[..., 2 * i].copy(), x[..., 2 * i + 1].copy()
        x[..., 2 * i] = u * c - v * s
        x[..., 2 * i + 1] = v * c + u * s
    return x


def plain_query_temperature(positions, coef, every):
    """1 + coef * ln(floor((p + 1) / every) + 1) per position."""
    p = np.asarray(positions, np.int64)
    return 1.0 + float(coef) * np.log(np.floor_divide(p + 1, int(every)).astype(F) + 1.0)


def plain_sink_softmax(scores, sink):
    """Weights over the last axis of ``scores`` whose denominator also holds exp(sink);
    ``sink`` None is the ordinary softmax."""
    z = np.asarray(scores, F)
    m = z.max(axis=-1, keepdims=True)
    if sink is not None:
        m = np.maximum(m, sink)
    e = np.exp(z - m)
    den = e.sum(axis=-1, keepdims=True)
    if sink is not None:
        den = den + np.exp(sink - m)
    return e / den


def plain_causal_attention(q, keys, values, first_position, scale, softcap=None, sinks=None):
    """q: [tokens, heads, dim], the tokens at positions first_position ..; keys [n, kv_heads,
    dim] and values [n, kv_heads, vdim] of positions 0 .. n - 1.  Query head h reads key head
    h // (heads / kv_heads).  ``sinks``: None, or one number a head."""
    T, H, _ = q.shape
    G = keys.shape[1]
    out = np.zeros((T, H, values.shape[2]), F)
    for t in range(T):
        n = first_position + t + 1
        for h in range(H):
            g = h // (H // G)
            s = keys[:n, g] @ q[t, h] * scale
            if softcap is not None:
                s = softcap * np.tanh(s / softcap)
            p = plain_sink_softmax(s, None if sinks is None else float(sinks[h]))
            out[t, h] = p @ values[:n, g]
    return out


def _grow(state, name, rows):
    state[name] = rows if name not in state else np.concatenate([state[name], rows], axis=0)
    return state[name]


def plain_attention(h, positions, w, p, m, eps, state, kind):
    """The three softmax attentions.  ``kind``: "attention" (norm a head, temperature, soft
    cap, learned sink, gate), "attention_2" (norm over the whole projection, rotary pairs,
    learned sink, gate), "left" (norm a head, rotary pairs, a sink of zero, no gate)."""
    T = h.shape[0]
    H, G, D, VD = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = h @ w[p + "q"].T, h @ w[p + "k"].T, h @ w[p + "v"].T
    if kind == "attention_2":
        q = plain_rms_norm(q, w[p + "q.norm"], eps)
        k = plain_rms_norm(k, w[p + "k.norm"], eps)
    q, k, v = q.reshape(T, H, D), k.reshape(T, G, D), v.reshape(T, G, VD)
    if kind != "attention_2":
        q = plain_rms_norm(q, w[p + "q.norm"], eps)
        k = plain_rms_norm(k, w[p + "k.norm"], eps)
    rot = m.get("rot")
    if rot is not None:
        q = plain_rotate_pairs(q, positions, rot["dims"], rot["base"])
        k = plain_rotate_pairs(k, positions, rot["dims"], rot["base"])
    temp = m.get("q_temp")
    if temp is not None:
        q = q * plain_query_temperature(positions, temp["coef"], temp["every"])[:, None, None]
    keys, values = _grow(state, "k", k), _grow(state, "v", v)
    sinks = np.zeros(H, F) if kind == "left" else w[p + "sink"]
    o = plain_causal_attention(q, keys, values, int(positions[0]), m["scale"], m.get("softcap"),
                               sinks).reshape(T, H * VD)
    if kind != "left":
        o = o * plain_sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def plain_short_conv(x, weight, state, name):
    """Causal convolution over time per channel: x [tokens, channels], weight [channels, taps]
    whose last column meets the token itself; zeros before the sequence's start.  The last
    taps - 1 inputs are carried in ``state[name]``."""
    taps = weight.shape[1]
    before = state.get(name)
    if before is None:
        before = np.zeros((taps - 1, x.shape[1]), F)
    padded = np.concatenate([before, x], axis=0)
    out = np.zeros_like(x)
    for t in range(x.shape[0]):
        out[t] = np.sum(padded[t:t + taps].T * weight, axis=1)
    state[name] = padded[padded.shape[0] - (taps - 1):]
    return out


def plain_delta_rule(q, k, v, beta, decay, S):
    """One head, token after token: S [dim, vdim] is first decayed row by row, the write is
    beta (v - S^T k), and the read-out S^T q sees it.  Returns the outputs [tokens, vdim];
    S is changed in place."""
    out = np.zeros((q.shape[0], v.shape[1]), F)
    for t in range(q.shape[0]):
        S *= decay[t][:, None]
        u = beta[t] * (v[t] - S.T @ k[t])
        S += np.outer(k[t], u)
        out[t] = S.T @ q[t]
    return out


def plain_gated_delta(h, w, p, m, eps, state):
    T = h.shape[0]
    H, G, D, VD = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = plain_silu(plain_short_conv(h @ w[p + "q"].T, w[p + "q.conv"], state, "cq")).reshape(T, G, D)
    k = plain_silu(plain_short_conv(h @ w[p + "k"].T, w[p + "k.conv"], state, "ck")).reshape(T, G, D)
    v = plain_silu(plain_short_conv(h @ w[p + "v"].T, w[p + "v.conv"], state, "cv")).reshape(T, H, VD)
    q = q / np.sqrt(np.sum(q * q, axis=-1, keepdims=True) + 1e-6) * D ** -0.5
    k = k / np.sqrt(np.sum(k * k, axis=-1, keepdims=True) + 1e-6)
    beta = plain_sigmoid(h @ w[p + "b"].T)                                      # [T, H]
    step = plain_softplus((h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]).reshape(T, H, D)
    decay = np.exp(-np.exp(np.asarray(w[p + "A_log"], F))[None, :, None] * step)
    if "S" not in state:
        state["S"] = np.zeros((H, D, VD), F)
    o = np.zeros((T, H, VD), F)
    for hd in range(H):
        g = hd // (H // G)
        o[:, hd] = plain_delta_rule(q[:, g], k[:, g], v[:, hd], beta[:, hd], decay[:, hd],
                                    state["S"][hd])
    o = plain_rms_norm(o, w[p + "norm"], eps)
    gate = plain_sigmoid((h @ w[p + "g1"].T) @ w[p + "g2"].T)
    return (o.reshape(T, H * VD) * gate) @ w[p + "o"].T


def plain_mixer(kind, h, positions, w, p, m, eps, state):
    if kind in ("attention", "attention_2"):
        return plain_attention(h, positions, w, p, m, eps, state, kind)
    if kind == "parallel":
        left = plain_attention(h, positions, w, p + "left.", m["left"], eps, state, "left")
        right = plain_gated_delta(h, w, p + "right.", m["right"], eps, state)
        return m["left_scale"] * left + m["right_scale"] * right
    raise ValueError(kind)


def plain_feed_forward(h, w, p):
    gate = h @ w[p + "gate"].T + w[p + "gate.b"]
    up = h @ w[p + "up"].T + w[p + "up.b"]
    return (plain_silu(gate) * up) @ w[p + "down"].T + w[p + "down.b"]


def plain_hyper_read(xs, w_in):
    """xs: [streams, tokens, width] -> sum_s in[s] xs[s]."""
    return np.tensordot(np.asarray(w_in, F), xs, axes=(0, 0))


def plain_hyper_write(xs, y, w_mix, w_out, mult):
    """new[t] = sum_s mix[s, t] xs[s] + mult * out[t] * y, every t from the old copies."""
    new = np.tensordot(np.asarray(w_mix, F).T, xs, axes=(1, 0))
    return new + mult * np.asarray(w_out, F)[:, None, None] * y[None]


def plain_run_order(cfg):
    """Layer indices in the order they run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def plain_forward(tokens, w, cfg, states=None, layer_outputs=None):
    """float64 logits [len(tokens), vocab].  ``states``: a list with one dict per layer run;
    given, the tokens continue the sequence it holds.  ``layer_outputs``: a list that takes
    the residual (the sum of the copies) after every layer run."""
    order = plain_run_order(cfg)
    if states is None:
        states = [{} for _ in order]
    eps, mult = cfg["norm"]["eps"], cfg["residual_mult"]
    start = states[0].get("len", 0) if states else 0
    positions = np.arange(start, start + len(tokens))
    x = np.asarray(w["embed"], F)[np.asarray(tokens)]
    streams = cfg.get("streams")
    xs = np.stack([x] * streams) if streams else None
    for run, i in enumerate(order):
        layer, state, p = cfg["layers"][i], states[run], f"l{i}."
        state["len"] = start + len(tokens)
        for q, sub in ((1, "mix"), (2, "mlp")):
            if sub == "mlp" and layer.get("mlp") is None:
                continue
            u = plain_hyper_read(xs, w[f"{p}hc{q}.in"]) if streams else x
            hn = plain_rms_norm(u, w[f"{p}norm{q}"], eps)
            if sub == "mix":
                y = plain_mixer(layer["type"], hn, positions, w, p + "mix.", layer["mixer"], eps,
                                state)
            else:
                y = plain_feed_forward(hn, w, p + "mlp.")
            if streams:
                xs = plain_hyper_write(xs, y, w[f"{p}hc{q}.mix"], w[f"{p}hc{q}.out"], mult)
            else:
                x = x + mult * y
        if layer_outputs is not None:
            layer_outputs.append(xs.sum(axis=0) if streams else x.copy())
    if streams:
        x = xs.sum(axis=0)
    return plain_rms_norm(x, w["final.norm"], eps) @ np.asarray(w["head"], F).T
