"""Checkpoint tensor names of the Mokotar decoder and where each goes.

Layer i's tensors start with ``l<i>.``: ``norm1`` / ``norm2``, the hyper-connection tables
``hc1.{in,out,mix}`` / ``hc2.{in,out,mix}`` (with ``streams``), the mixer under ``mix.`` (the two
halves of a parallel mixer under ``mix.left.`` / ``mix.right.``), the feed-forward under
``mlp.``; the model's ends are ``embed``, ``final.norm``, ``head``.  Stacked into one engine
parameter: an attention's ``[q; k; v; g]``, the delta rule's ``[q; k; v; b; a1; g1]`` and
their convolutions, the feed-forward's ``[gate; up]`` with their biases.
"""
from __future__ import annotations

from ..config.layout import ModelLayout
from .names import CheckpointMap, TensorSource
from .tifosun import _stack


def _attention_sources(src: list, ck: str, me: str, a, width: int) -> None:
    q_rows = a.num_heads * a.head_dim
    k_rows = a.num_kv_heads * a.head_dim
    v_rows = a.num_kv_heads * a.value_dim
    parts = [(f"{ck}.q", q_rows), (f"{ck}.k", k_rows), (f"{ck}.v", v_rows)]
    if a.feature_gate:
        parts.append((f"{ck}.g", a.num_heads * a.value_dim))
    _stack(src, f"{me}.qkv.weight", parts)
    src.append(TensorSource(f"{ck}.q.norm", f"{me}.q_norm.weight", 0,
                            q_rows if a.qk_norm_whole else a.head_dim))
    src.append(TensorSource(f"{ck}.k.norm", f"{me}.k_norm.weight", 0,
                            k_rows if a.qk_norm_whole else a.head_dim))
    if a.sink == "learned":
        src.append(TensorSource(f"{ck}.sink", f"{me}.sink", 0, a.num_heads))
    src.append(TensorSource(f"{ck}.o", f"{me}.o.weight", 0, width))


def _delta_sources(src: list, ck: str, me: str, d, width: int) -> None:
    qk, vv = d.num_kv_heads * d.qk_dim, d.num_heads * d.v_dim
    _stack(src, f"{me}.in.weight", [(f"{ck}.q", qk), (f"{ck}.k", qk), (f"{ck}.v", vv),
                                    (f"{ck}.b", d.num_heads), (f"{ck}.a1", d.decay_rank),
                                    (f"{ck}.g1", d.gate_rank)])
    _stack(src, f"{me}.conv.weight", [(f"{ck}.q.conv", qk), (f"{ck}.k.conv", qk),
                                      (f"{ck}.v.conv", vv)])
    src.append(TensorSource(f"{ck}.a2", f"{me}.a2.weight", 0, d.num_heads * d.qk_dim))
    src.append(TensorSource(f"{ck}.dt_bias", f"{me}.dt_bias", 0, d.num_heads * d.qk_dim))
    src.append(TensorSource(f"{ck}.A_log", f"{me}.A_log", 0, d.num_heads))
    src.append(TensorSource(f"{ck}.g2", f"{me}.g2.weight", 0, vv))
    src.append(TensorSource(f"{ck}.norm", f"{me}.norm.weight", 0, d.v_dim))
    src.append(TensorSource(f"{ck}.o", f"{me}.o.weight", 0, width))


def mokotar_checkpoint_map(config, layout: ModelLayout) -> CheckpointMap:
    src: list = []
    width = layout.hidden_size
    src.append(TensorSource("embed", "embed.weight", 0, layout.vocab_size))
    for i, block in enumerate(layout.blocks):
        ck, me = f"l{i}", f"blocks.{i}"
        subs = (1,) if block.ffn is None else (1, 2)
        for q in subs:
            src.append(TensorSource(f"{ck}.norm{q}", f"{me}.norm{q}.weight", 0, width))
            if block.streams:
                for t in ("in", "out", "mix"):
                    src.append(TensorSource(f"{ck}.hc{q}.{t}", f"{me}.hc{q}.{t}", 0, block.streams))
        m = block.mixer
        if m.kind == "attention":
            _attention_sources(src, f"{ck}.mix", f"{me}.mixer", m, width)
        elif m.kind == "parallel" and len(m.branches) == 2:
            _attention_sources(src, f"{ck}.mix.left", f"{me}.mixer.branch0", m.branches[0], width)
            _delta_sources(src, f"{ck}.mix.right", f"{me}.mixer.branch1", m.branches[1], width)
        else:
            raise ValueError(f"no checkpoint names for a mixer of kind {m.kind!r}")
        f = block.ffn
        if f is None:
            continue
        ff = f.intermediate_size
        _stack(src, f"{me}.ffn.gate_up.weight", [(f"{ck}.mlp.gate", ff), (f"{ck}.mlp.up", ff)])
        _stack(src, f"{me}.ffn.gate_up.bias", [(f"{ck}.mlp.gate.b", ff), (f"{ck}.mlp.up.b", ff)])
        src.append(TensorSource(f"{ck}.mlp.down", f"{me}.ffn.down.weight", 0, width))
        src.append(TensorSource(f"{ck}.mlp.down.b", f"{me}.ffn.down.bias", 0, width))
    src.append(TensorSource("final.norm", "final_norm.weight", 0, layout.final_norm.size))
    src.append(TensorSource("head", "head.weight", 0, layout.vocab_size))
    return CheckpointMap(sources=src)
