"""Checkpoint tensor names of the Relurax decoder and where each goes.

Layer i's tensors start with ``l<i>.``: its four norms (``norm1``, ``norm1b``, ``norm2``,
``norm2b``), its mixer under ``mix.`` and its feed-forward under ``mlp.``; the model's ends
are ``embed``, ``final.norm`` and ``head``.  Matrices that read the same input are stacked
into one engine parameter so that one product serves them:

  attention          qkv = [q; k; g]            (no value matrix: the values are the keys)
  latent attention   in  = [dq; dkv; g]         ([dq; g] for a layer that reads another's rows)
  feed-forward       gate_up = [gate; up]

The convolution weights (``q.conv``, ``k.conv``: [channels, taps]), the head norms
(``q.norm``, ``k.norm``) and the latent norms (``dq.norm``, ``dkv.norm``) stay tensors of
their own.
"""
from __future__ import annotations

from ..config.layout import ModelLayout
from .names import CheckpointMap, TensorSource
from .tifosun import _stack


def relurax_checkpoint_map(config, layout: ModelLayout) -> CheckpointMap:
    src: list = []
    unused: set = set()     # norms of a second sublayer that a layer without a feed-forward lacks
    width = layout.hidden_size
    src.append(TensorSource("embed", "embed.weight", 0, layout.vocab_size))
    for i, block in enumerate(layout.blocks):
        ck, me = f"l{i}", f"blocks.{i}"
        for ck_norm, part in (("norm1", "norm1"), ("norm1b", "norm1_post"), ("norm2", "norm2"),
                              ("norm2b", "norm2_post")):
            spec = getattr(block, part)
            if spec is not None:
                src.append(TensorSource(f"{ck}.{ck_norm}", f"{me}.{part}.weight", 0, spec.size))
        m = block.mixer
        if m.kind == "attention":
            q_rows, k_rows = m.num_heads * m.head_dim, m.num_kv_heads * m.head_dim
            _stack(src, f"{me}.mixer.qkv.weight", [(f"{ck}.mix.q", q_rows), (f"{ck}.mix.k", k_rows),
                                                   (f"{ck}.mix.g", m.num_heads)])
            src.append(TensorSource(f"{ck}.mix.q.conv", f"{me}.mixer.q_conv.weight", 0, q_rows))
            src.append(TensorSource(f"{ck}.mix.k.conv", f"{me}.mixer.k_conv.weight", 0, k_rows))
            src.append(TensorSource(f"{ck}.mix.q.norm", f"{me}.mixer.q_norm.weight", 0, m.head_dim))
            src.append(TensorSource(f"{ck}.mix.k.norm", f"{me}.mixer.k_norm.weight", 0, m.head_dim))
            src.append(TensorSource(f"{ck}.mix.o", f"{me}.mixer.o.weight", 0, width))
        elif m.kind == "latent_attention":
            parts = [(f"{ck}.mix.dq", m.q_rank)]
            if not m.shares_kv:
                parts.append((f"{ck}.mix.dkv", m.kv_rank + m.rot_dim))
            parts.append((f"{ck}.mix.g", m.num_heads))
            _stack(src, f"{me}.mixer.in.weight", parts)
            src.append(TensorSource(f"{ck}.mix.dq.norm", f"{me}.mixer.q_norm.weight", 0, m.q_rank))
            src.append(TensorSource(f"{ck}.mix.uq", f"{me}.mixer.uq.weight", 0,
                                    m.num_heads * (m.qk_dim + m.rot_dim)))
            if not m.shares_kv:
                src.append(TensorSource(f"{ck}.mix.dkv.norm", f"{me}.mixer.kv_norm.weight", 0,
                                        m.kv_rank))
            src.append(TensorSource(f"{ck}.mix.uk", f"{me}.mixer.uk.weight", 0,
                                    m.num_heads * m.qk_dim))
            src.append(TensorSource(f"{ck}.mix.uv", f"{me}.mixer.uv.weight", 0,
                                    m.num_heads * m.v_dim))
            src.append(TensorSource(f"{ck}.mix.o", f"{me}.mixer.o.weight", 0, width))
        else:
            raise ValueError(f"no checkpoint names for a mixer of kind {m.kind!r}")
        f = block.ffn
        if f is None:
            unused.update((f"{ck}.norm2", f"{ck}.norm2b"))      # present or not: never read
            continue
        if f.kind == "gated_mlp":
            _stack(src, f"{me}.ffn.gate_up.weight", [(f"{ck}.mlp.gate", f.intermediate_size),
                                                     (f"{ck}.mlp.up", f.intermediate_size)])
            src.append(TensorSource(f"{ck}.mlp.down", f"{me}.ffn.down.weight", 0, width))
        else:
            raise ValueError(f"no checkpoint names for a feed-forward of kind {f.kind!r}")
    src.append(TensorSource("final.norm", "final_norm.weight", 0, layout.final_norm.size))
    src.append(TensorSource("head", "head.weight", 0, layout.vocab_size))
    return CheckpointMap(sources=src, ignore=unused.__contains__)
