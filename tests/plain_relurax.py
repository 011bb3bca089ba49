"""A plain, slow implementation of the Relurax decoder in numpy float64: one function per
mechanism, written from the design's equations and sharing nothing with the engine.

A layer is ``x += norm1b(mixer(norm1(x))); x += norm2b(ff(norm2(x)))`` with RMS norms of plain
weights.  The mixer is one of two attentions:

* a sliding-window grouped-query attention without positions: q and k are projected, pass a
  short causal convolution per channel, and are RMS-normed per head; the values are the
  convolved keys before their norm; every head's output is scaled by one sigmoid gate;
* a causal latent attention: queries come from a normed latent of their own, keys and
  values are up-projections of one normed latent per token, a rotated key part is shared
  by all heads (rotate-half pairs), every head's output is scaled by one sigmoid gate; a
  layer may read the latents that an earlier layer left instead of making its own.

The feed-forward is ``down(gelu_tanh(gate h) * up h)``.

Everything works on one sequence; ``state`` (a dict per layer) carries what a layer keeps
from call to call, so that a sequence can be fed whole, in portions, or token by token.
"""
from __future__ import annotations

import math

import numpy as np

F = np.float64


def plain_rms_norm(x, weight, eps):
    x = np.asarray(x, F)
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * np.asarray(weight, F)


def plain_gelu_tanh(z):
    z = np.asarray(z, F)
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def plain_sigmoid(z):
    return 1.0 / (1.0 + np.exp(-np.asarray(z, F)))


def plain_softmax(z):
    z = np.asarray(z, F)
    e = np.exp(z - z.max(axis=-1, keepdims=True))
    return e / e.sum(axis=-1, keepdims=True)


def plain_rotary_frequencies(dims, base):
    return np.asarray([float(base) ** (-2.0 * i / dims) for i in range(dims // 2)], F)


def plain_rotate_half(x, positions, freqs):
    """x: [tokens, ..., dim]; the first 2*len(freqs) features are rotated, feature i paired
    with feature i + len(freqs)."""
    x = np.array(x, F)
    half = len(freqs)
    if half == 0:
        return x
    ang = np.asarray(positions, F)[:, None] * freqs[None, :]
    while ang.ndim < x.ndim:
        ang = ang[:, None]
    c, s = np.cos(ang), np.sin(ang)
    u, v = x[..., :half].copy(), x[..., half:2 * half].copy()
    x[..., :half] = u * c - v * s
    x[..., half:2 * half] = v * c + u * s
    return x


def plain_causal_conv(u, weight, before):
    """y_t = sum_j weight[:, j] * u_(t - taps + 1 + j).  ``u``: [tokens, channels] of this call,
    ``before``: [taps - 1, channels], the inputs that came before it (zeros at a sequence's
    start).  Returns (y, the last taps - 1 inputs, for the next call)."""
    u = np.asarray(u, F)
    w = np.asarray(weight, F)
    taps = w.shape[1]
    full = np.concatenate([np.asarray(before, F), u], axis=0)
    y = np.zeros_like(u)
    for t in range(u.shape[0]):
        for j in range(taps):
            y[t] += w[:, j] * full[t + j]
    return y, full[full.shape[0] - (taps - 1):]


def plain_window_visible(i, j, size=None):
    """Whether position i sees position j: itself and the size - 1 before it (all before it
    without a size)."""
    return j <= i and (size is None or i - j < size)


def plain_dense_ff(h, w_gate, w_up, w_down):
    h = np.asarray(h, F)
    return (plain_gelu_tanh(h @ np.asarray(w_gate, F).T) * (h @ np.asarray(w_up, F).T)) \
        @ np.asarray(w_down, F).T


def plain_conv_attention(h, w, m, eps, state):
    """The sliding-window attention of one layer on the next tokens ``h`` [tokens, width] of a
    sequence.  ``w``: the mixer's tensors by their short names, ``m``: its configuration,
    ``state``: dict carrying the sequence's keys, values and convolution inputs."""
    h = np.asarray(h, F)
    n = h.shape[0]
    heads, groups, dim = m["heads"], m["kv_heads"], m["dim"]
    taps = m["conv"]
    if not state:
        state.update(k=np.zeros((0, groups, dim), F), v=np.zeros((0, groups, dim), F),
                     q_before=np.zeros((taps - 1, heads * dim), F),
                     k_before=np.zeros((taps - 1, groups * dim), F))
    q, state["q_before"] = plain_causal_conv(h @ np.asarray(w["q"], F).T, w["q.conv"],
                                             state["q_before"])
    k, state["k_before"] = plain_causal_conv(h @ np.asarray(w["k"], F).T, w["k.conv"],
                                             state["k_before"])
    q = q.reshape(n, heads, dim)
    k = k.reshape(n, groups, dim)
    v = k.copy()                                   # the values: keys as they leave the convolution
    q = plain_rms_norm(q, w["q.norm"], eps)
    k = plain_rms_norm(k, w["k.norm"], eps)
    start = state["k"].shape[0]
    state["k"] = np.concatenate([state["k"], k], axis=0)
    state["v"] = np.concatenate([state["v"], v], axis=0)
    gate = plain_sigmoid(h @ np.asarray(w["g"], F).T)         # [tokens, heads]
    out = np.zeros((n, heads, dim), F)
    per = heads // groups
    size = m["mask"]["size"] if m.get("mask") else None
    for t in range(n):
        i = start + t
        js = [j for j in range(i + 1) if plain_window_visible(i, j, size)]
        for hd in range(heads):
            g = hd // per
            s = np.asarray([q[t, hd] @ state["k"][j, g] for j in js], F) * m["scale"]
            p = plain_softmax(s)
            out[t, hd] = sum(pj * state["v"][j, g] for pj, j in zip(p, js)) * gate[t, hd]
    return out.reshape(n, heads * dim) @ np.asarray(w["o"], F).T


def plain_latent_attention(h, w, m, eps, state, borrowed=None):
    """The latent attention of one layer on the next tokens ``h`` of a sequence.  ``borrowed``:
    the state dict of the layer whose latents and rotated keys this layer reads (it then has
    no down-projection of its own); that layer has run on the same tokens before."""
    h = np.asarray(h, F)
    n = h.shape[0]
    heads, dim, rot, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    freqs = plain_rotary_frequencies(m["rot"]["dims"], m["rot"]["base"])
    if borrowed is None:
        if not state:
            state.update(c=np.zeros((0, rank), F), kr=np.zeros((0, rot), F))
        start = state["c"].shape[0]
        positions = np.arange(start, start + n)
        d = h @ np.asarray(w["dkv"], F).T
        c = plain_rms_norm(d[:, :rank], w["dkv.norm"], eps)
        kr = plain_rotate_half(d[:, rank:], positions, freqs)
        state["c"] = np.concatenate([state["c"], c], axis=0)
        state["kr"] = np.concatenate([state["kr"], kr], axis=0)
        kept = state
    else:
        kept = borrowed
        start = kept["c"].shape[0] - n
        positions = np.arange(start, start + n)
    cq = plain_rms_norm(h @ np.asarray(w["dq"], F).T, w["dq.norm"], eps)
    q = (cq @ np.asarray(w["uq"], F).T).reshape(n, heads, dim + rot)
    q_plain = q[:, :, :dim]
    q_rot = plain_rotate_half(q[:, :, dim:], positions, freqs)
    keys = (kept["c"] @ np.asarray(w["uk"], F).T).reshape(-1, heads, dim)
    values = (kept["c"] @ np.asarray(w["uv"], F).T).reshape(-1, heads, vdim)
    gate = plain_sigmoid(h @ np.asarray(w["g"], F).T)
    out = np.zeros((n, heads, vdim), F)
    for t in range(n):
        i = start + t
        for hd in range(heads):
            s = (keys[:i + 1, hd] @ q_plain[t, hd] + kept["kr"][:i + 1] @ q_rot[t, hd]) * m["scale"]
            p = plain_softmax(s)
            out[t, hd] = (p @ values[:i + 1, hd]) * gate[t, hd]
    return out.reshape(n, heads * vdim) @ np.asarray(w["o"], F).T


def layer_tensors(tensors, i, part):
    """The tensors of layer i's ``part`` ("mix" or "mlp") by their short names."""
    prefix = f"l{i}.{part}."
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


class PlainRelurax:
    """The whole model on one sequence; ``forward`` takes the sequence's next tokens and
    returns (logits [tokens, vocab], the residual after every layer [layers, tokens, width])."""

    def __init__(self, config, tensors):
        self.config = config
        self.t = {k: np.asarray(v, F) for k, v in tensors.items()}
        self.eps = config["norm"]["eps"]
        self.reset()

    def reset(self):
        self.states = [dict() for _ in self.config["layers"]]

    def forward(self, tokens):
        cfg, t, eps = self.config, self.t, self.eps
        x = t["embed"][np.asarray(tokens, dtype=np.int64)]
        after = []
        for i, layer in enumerate(cfg["layers"]):
            m = layer["mixer"]
            h = plain_rms_norm(x, t[f"l{i}.norm1"], eps)
            w = layer_tensors(t, i, "mix")
            if layer["type"] == "attention":
                y = plain_conv_attention(h, w, m, eps, self.states[i])
            elif layer["type"] == "latent_attention":
                src = m.get("kv_from")
                y = plain_latent_attention(h, w, m, eps, self.states[i],
                                           None if src is None else self.states[src])
            else:
                raise ValueError(layer["type"])
            x = x + plain_rms_norm(y, t[f"l{i}.norm1b"], eps)
            if layer.get("mlp") is not None:
                h = plain_rms_norm(x, t[f"l{i}.norm2"], eps)
                f = layer_tensors(t, i, "mlp")
                y = plain_dense_ff(h, f["gate"], f["up"], f["down"])
                x = x + plain_rms_norm(y, t[f"l{i}.norm2b"], eps)
            after.append(x.copy())
        logits = plain_rms_norm(x, t["final.norm"], eps) @ t["head"].T
        return logits, np.stack(after)
