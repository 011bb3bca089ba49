"""Small Mokotar configurations with random weights for the tests, and the plumbing to run
them through the plain implementation (the engine side is shared with the other decoders'
tests: ``tifosun_util.run_schedule`` and its comparisons)."""
from __future__ import annotations

import copy

import numpy as np
import torch

import plain_mokotar as P
from tifosun_util import assert_close, relative_error, row_errors, run_schedule, tokens  # noqa: F401


def attention(heads=4, kv_heads=2, dim=24, vdim=40, scale=None, coef=0.4, every=7, softcap=8.0):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
            "scale": dim ** -0.5 if scale is None else scale,
            "q_temp": {"coef": coef, "every": every}, "softcap": softcap}


def attention_2(heads=4, kv_heads=2, dim=32, vdim=16, scale=None, rot_dims=12, base=300.0):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
            "scale": dim ** -0.5 if scale is None else scale,
            "rot": {"base": base, "dims": rot_dims}}


def left(heads=4, kv_heads=1, dim=16, vdim=24, scale=None, rot_dims=16, base=1000.0):
    return attention_2(heads, kv_heads, dim, vdim, scale, rot_dims, base)


def right(heads=4, kv_heads=2, dim=24, vdim=20, conv=3):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def parallel(l=None, r=None, left_scale=1.3, right_scale=0.8):
    return {"left": l or left(), "right": r or right(), "left_scale": left_scale,
            "right_scale": right_scale}


def dense(ff=72):
    return {"kind": "dense", "ff": ff}


def layer(kind, mixer, mlp="dense"):
    return {"type": kind, "mixer": mixer, "mlp": dense() if mlp == "dense" else mlp}


def config(layers, width=64, vocab=157, eps=1e-5, mult=0.4, streams=3, loop=None):
    out = {"architecture": "Mokotar", "width": width, "vocab": vocab, "norm": {"eps": eps},
           "residual_mult": mult, "layers": copy.deepcopy(layers)}
    if streams:
        out["streams"] = streams
    if loop is not None:
        out["loop"] = dict(zip(("start", "stop", "times"), loop))
    return out


# Layers that differ in every size: query groups of 2, 4, 1 and 3, value sizes above and below
# the key size, head sizes that are no multiple of 16, all and part of a head rotated, one to
# four taps, delta-rule heads that share keys and that do not, a layer without a feed-forward,
# a stretch of three layers that runs twice, three copies of the residual.
MIXED = config([
    layer("attention", attention(4, 2, 24, 40, scale=0.3, coef=0.4, every=7, softcap=8.0)),
    layer("parallel", parallel(left(4, 1, 16, 24, rot_dims=16), right(4, 2, 24, 20, conv=3))),
    layer("attention_2", attention_2(3, 3, 40, 8, scale=0.2, rot_dims=12), mlp=None),
    layer("parallel", parallel(left(6, 2, 20, 12, rot_dims=8, base=50.0), right(3, 3, 10, 36, conv=4),
                               left_scale=0.7, right_scale=1.6), dense(40)),
    layer("attention", attention(6, 2, 16, 16, scale=0.35, coef=1.0, every=3, softcap=2.5), dense(24)),
], loop=(1, 4, 2))

RANKS = (5, 7)      # of the delta rule's decay and gate projections, where nothing else is said


def random_weights(cfg: dict, seed: int, sharp: float = 1.0, ranks=RANKS) -> dict:
    """Checkpoint tensors (bfloat16 values).  Projections keep activations of order one; the
    query and key norm weights are ``sharp`` (at 3 a query's weight lies on a few keys, which
    the tests of the attention alone use; whole models take one, or eight layer runs of such
    attention amplify the rounding of bfloat16 activations beyond any use as a yardstick);
    sinks lie where they hold a good part of a row's weight; the delta rule's decays spread
    from nearly one to a half a token, its write strengths over (0, 1)."""
    g = torch.Generator().manual_seed(seed)
    w: dict = {}

    def mat(name, rows, cols, gain=1.0):
        w[name] = (gain * torch.randn(rows, cols, generator=g) / cols ** 0.5).to(torch.bfloat16)

    def vec(name, n, mean=0.0, std=0.1):
        w[name] = (mean + std * torch.randn(n, generator=g)).to(torch.bfloat16)

    def attn(p, a, kind):
        H, G, D, VD = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
        mat(p + "q", H * D, W)
        mat(p + "k", G * D, W)
        mat(p + "v", G * VD, W)
        whole = kind == "attention_2"
        vec(p + "q.norm", H * D if whole else D, sharp, 0.3)
        vec(p + "k.norm", G * D if whole else D, sharp, 0.3)
        if kind != "left":
            vec(p + "sink", H, 1.0, 1.5)
            mat(p + "g", H * VD, W, 2.0)
        mat(p + "o", W, H * VD)

    W, S = cfg["width"], cfg.get("streams", 0)
    w["embed"] = torch.randn(cfg["vocab"], W, generator=g).to(torch.bfloat16)
    for i, l in enumerate(cfg["layers"]):
        p = f"l{i}."
        for q in (1, 2) if l["mlp"] is not None else (1,):
            vec(f"{p}norm{q}", W, 1.0, 0.2)
            if S:
                vec(f"{p}hc{q}.in", S, 1.0 / S, 0.3)
                vec(f"{p}hc{q}.out", S, 1.0, 0.4)
                w[f"{p}hc{q}.mix"] = (torch.eye(S) * 0.8 + 0.25 * torch.randn(S, S, generator=g)).to(
                    torch.bfloat16)
        if l["type"] != "parallel":
            attn(p + "mix.", l["mixer"], l["type"])
        else:
            attn(p + "mix.left.", l["mixer"]["left"], "left")
            m, r = l["mixer"]["right"], p + "mix.right."
            H, G, D, VD, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            ra, rg = m.get("decay_rank", ranks[0]), m.get("gate_rank", ranks[1])
            for n, rows in (("q", G * D), ("k", G * D), ("v", H * VD)):
                mat(r + n, rows, W, 1.5)
                mat(r + n + ".conv", rows, taps, 1.5)
            mat(r + "b", H, W, 2.0)
            mat(r + "a1", ra, W)
            mat(r + "a2", H * D, ra, 2.0)
            w[r + "dt_bias"] = (-3.0 + 3.0 * torch.rand(H * D, generator=g)).to(torch.bfloat16)
            w[r + "A_log"] = torch.log(0.3 + 2.0 * torch.rand(H, generator=g)).to(torch.bfloat16)
            mat(r + "g1", rg, W)
            mat(r + "g2", H * VD, rg, 2.0)
            vec(r + "norm", VD, 1.0, 0.3)
            mat(r + "o", W, H * VD)
        if l["mlp"] is not None:
            ff = l["mlp"]["ff"]
            for n, rows, cols in (("gate", ff, W), ("up", ff, W), ("down", W, ff)):
                mat(f"{p}mlp.{n}", rows, cols)
                vec(f"{p}mlp.{n}.b", rows, 0.0, 0.3)
    vec("final.norm", W, 1.0, 0.2)
    mat("head", cfg["vocab"], W)
    return w


def as_numpy(weights: dict) -> dict:
    return {k: v.double().numpy() for k, v in weights.items()}


def sub(weights: dict, prefix: str) -> dict:
    return {k[len(prefix):]: v.double().numpy() for k, v in weights.items() if k.startswith(prefix)}


def plain_logits(cfg: dict, weights: dict, toks: list) -> torch.Tensor:
    """float64 logits [len(toks), vocab] of one sequence."""
    return torch.from_numpy(P.plain_forward(list(toks), as_numpy(weights), cfg))


def load(cfg: dict, weights: dict, dtype: str):
    from mstar_b200.config.registry import config_from_dict
    from mstar_b200.engine.model import load_model

    return load_model(None, dtype=dtype, device="cuda:0", config=config_from_dict(cfg),
                      tensors=weights)


def runs(cfg: dict) -> int:
    return len(P.plain_run_order(cfg))


assert P.plain_run_order(MIXED) == [0, 1, 2, 3, 1, 2, 3, 4]
assert np.isclose(P.plain_query_temperature([20], 0.4, 7)[0], 1 + 0.4 * np.log(4.0))
