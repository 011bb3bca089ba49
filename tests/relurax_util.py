"""Small Relurax configurations with random weights for the tests, and the plumbing to run
them through the plain implementation (the engine side is shared with the other decoders'
tests: ``tifosun_util.run_schedule`` and its comparisons)."""
from __future__ import annotations

import copy

import numpy as np
import torch

import plain_relurax as P
from tifosun_util import assert_close, relative_error, row_errors, run_schedule, tokens  # noqa: F401


def attention(heads=4, kv_heads=2, dim=24, size=11, conv=3, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "conv": conv,
         "scale": 4.0 / dim if scale is None else scale}
    if size is not None:
        m["mask"] = {"size": size}
    return m


def latent(heads=3, dim=16, rot_dim=8, vdim=24, kv_rank=40, q_rank=20, base=10000.0, dims=None,
           scale=None, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
         "q_rank": q_rank, "rot": {"base": base, "dims": rot_dim if dims is None else dims},
         "scale": 1.5 * (dim + rot_dim) ** -0.5 if scale is None else scale}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def dense(ff=72):
    return {"kind": "dense", "ff": ff}


def layer(mixer, mlp=None):
    kind = "latent_attention" if "kv_rank" in mixer else "attention"
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def config(layers, width=64, vocab=157, eps=1e-5):
    layers = copy.deepcopy(layers)
    for l in layers:                # a layer that reads another's rows repeats its sizes
        src = l["mixer"].get("kv_from")
        if src is not None:
            for key in ("kv_rank", "rot_dim", "rot"):
                l["mixer"][key] = copy.deepcopy(layers[src]["mixer"][key])
    return {"architecture": "Relurax", "width": width, "vocab": vocab, "norm": {"eps": eps},
            "layers": layers}


# Layers that differ in every size: query groups of 2, 1 and 3, head sizes that are and are
# not multiples of 16, windows shorter and longer than a page, a layer without a window, one
# to five taps, latent layers with all and with part of the rotated features rotated, two
# layers that read the rows of an earlier one (one of them with other head sizes), a layer
# without a feed-forward.
MIXED = config([
    layer(attention(4, 2, 24, size=11, conv=3), dense(72)),
    layer(latent(3, 16, 8, 24, 40, 20, base=10000.0), dense(40)),
    layer(attention(3, 3, 16, size=21, conv=1, scale=0.3), None),
    layer(latent(2, 8, 8, 12, 40, 28, kv_from=1), dense(56)),
    layer(attention(6, 2, 20, size=5, conv=5), dense(24)),
    layer(latent(4, 12, 12, 8, 24, 36, base=50.0, dims=8), None),
    layer(attention(2, 1, 32, size=None, conv=2), dense(48)),
    layer(latent(1, 24, 12, 16, 24, 8, kv_from=5), dense(32)),
])


def random_weights(cfg: dict, seed: int, sharp: float = 1.3, conv_last: float = None) -> dict:
    """Checkpoint tensors (bfloat16 values).  Projections keep activations of order one; the
    query and key norm weights are ``sharp`` so that a query's weight lies on a few keys.
    ``conv_last``: the tap on the token itself is that much and the earlier taps are small (a
    key then belongs to one token), else all taps are of order one."""
    g = torch.Generator().manual_seed(seed)
    w: dict = {}

    def mat(name, rows, cols, gain=1.0):
        w[name] = (gain * torch.randn(rows, cols, generator=g) / cols ** 0.5).to(torch.bfloat16)

    def vec(name, n, mean=0.0, std=0.1):
        w[name] = (mean + std * torch.randn(n, generator=g)).to(torch.bfloat16)

    def taps(name, channels, n):
        t = torch.randn(channels, n, generator=g) * 0.6
        if conv_last is not None:
            t = t * 0.05
            t[:, -1] = conv_last + 0.1 * torch.randn(channels, generator=g)
        w[name] = t.to(torch.bfloat16)

    W = cfg["width"]
    w["embed"] = torch.randn(cfg["vocab"], W, generator=g).to(torch.bfloat16)
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.", l["mixer"]
        vec(p + "norm1", W, 1.0, 0.2)
        vec(p + "norm1b", W, 0.5, 0.1)
        H = m["heads"]
        if l["type"] == "attention":
            G, D = m["kv_heads"], m["dim"]
            mat(p + "mix.q", H * D, W)
            mat(p + "mix.k", G * D, W)
            taps(p + "mix.q.conv", H * D, m["conv"])
            taps(p + "mix.k.conv", G * D, m["conv"])
            vec(p + "mix.q.norm", D, sharp, 0.3)
            vec(p + "mix.k.norm", D, sharp, 0.3)
            mat(p + "mix.g", H, W, 2.0)
            mat(p + "mix.o", W, H * D)
        else:
            D, R, V = m["dim"], m["rot_dim"], m["vdim"]
            mat(p + "mix.dq", m["q_rank"], W)
            vec(p + "mix.dq.norm", m["q_rank"], 1.0, 0.2)
            mat(p + "mix.uq", H * (D + R), m["q_rank"], sharp)
            if m.get("kv_from") is None:
                mat(p + "mix.dkv", m["kv_rank"] + R, W)
                vec(p + "mix.dkv.norm", m["kv_rank"], 1.0, 0.2)
            mat(p + "mix.uk", H * D, m["kv_rank"], sharp)
            mat(p + "mix.uv", H * V, m["kv_rank"])
            mat(p + "mix.g", H, W, 2.0)
            mat(p + "mix.o", W, H * V)
        mlp = l["mlp"]
        if mlp is None:
            continue
        vec(p + "norm2", W, 1.0, 0.2)
        vec(p + "norm2b", W, 0.5, 0.1)
        mat(p + "mlp.gate", mlp["ff"], W, 1.5)
        mat(p + "mlp.up", mlp["ff"], W)
        mat(p + "mlp.down", W, mlp["ff"])
    vec("final.norm", W, 1.0, 0.2)
    mat("head", cfg["vocab"], W)
    return w


def as_numpy(weights: dict) -> dict:
    return {k: v.double().numpy() for k, v in weights.items()}


def mixer_tensors(weights: dict, i: int = 0) -> dict:
    return P.layer_tensors(as_numpy(weights), i, "mix")


def plain_logits(cfg: dict, weights: dict, toks: list) -> torch.Tensor:
    """float64 logits [len(toks), vocab] of one sequence."""
    return torch.from_numpy(P.PlainRelurax(cfg, as_numpy(weights)).forward(list(toks))[0])


def plain_greedy_check(cfg: dict, weights: dict, prompt: list, picked: list):
    """For every token of ``picked`` (what an engine appended to ``prompt``, greedily): the
    plain model's own best token and its margin over the picked one, the plain model fed the
    picked tokens."""
    model = P.PlainRelurax(cfg, as_numpy(weights))
    logits = model.forward(list(prompt))[0][-1]
    out = []
    for tok in picked:
        best = int(np.argmax(logits))
        out.append((best, float(logits[best] - logits[tok])))
        logits = model.forward([tok])[0][-1]
    return out


def load(cfg: dict, weights: dict, dtype: str):
    from mstar_b200.config.registry import config_from_dict
    from mstar_b200.engine.model import load_model

    return load_model(None, dtype=dtype, device="cuda:0", config=config_from_dict(cfg),
                      tensors=weights)
