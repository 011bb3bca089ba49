"""Typed configuration of the Mokotar decoder (``"architecture": "Mokotar"``).

config.json gives ``width``, ``vocab``, ``norm.eps``, ``residual_mult``, optionally ``streams``
(hyper-connections: that many copies of the residual) and ``loop`` (``start``, ``stop``,
``times``: layers ``start .. stop - 1`` run ``times`` times in a row with the same tensors, each
pass with a cache and a state of its own), and the layers one by one: ``layers[i] = {"type":
..., "mixer": {...}, "mlp": {"kind": "dense", "ff": n} | null}``.

Layer types, each a pre-norm layer ``x += m * mixer(norm1(x)); x += m * ff(norm2(x))`` (with
``streams`` the sums become the hyper-connection's read and write):

* ``attention``: grouped-query attention over every earlier key without rotation: an RMS norm
  per query and key head, a query temperature ``q_temp.{coef, every}``, scores scaled by
  ``scale`` and soft-capped at ``softcap``, a learned sink a head in the softmax's
  denominator, a sigmoid gate a feature on the heads' outputs;
* ``attention_2``: the RMS norm runs over the whole q (and k) projection, rotary pairs ``(2i,
  2i + 1)`` over ``rot.dims`` features with base ``rot.base``, sink and gate as above;
* ``parallel``: ``left_scale * left + right_scale * right`` of an attention (norm a head,
  rotary pairs, one added to the softmax's denominator) and a gated delta rule (``conv`` taps
  on q, k and v; the ranks of its decay and gate projections come from the tensors' shapes).

The feed-forward is ``down(silu(gate h) * up h)`` with biases.  Nothing has a size default;
every size may differ from layer to layer.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Mapping, Optional

from .base import ConfigError, ModelConfig
from .layout import (AttentionSpec, BlockSpec, GatedDeltaSpec, GatedMLPSpec, ModelLayout,
                     NormSpec, ParallelMixerSpec, PositionSpec, RunEntry)
from .tifosun import _Reader

LAYER_TYPES = ("attention", "attention_2", "parallel")


@dataclass
class MokotarConfig(ModelConfig):
    width: int
    vocab: int
    norm_eps: float
    residual_mult: float
    streams: int = 0                                   # 0: one residual, no hyper-connections
    loop: Optional[tuple] = None                       # (start, stop, times)
    layers: list = field(default_factory=list)        # the raw layer objects of config.json
    stop_tokens: tuple = ()

    architecture = "Mokotar"

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "MokotarConfig":
        rd = _Reader()
        width = rd.get(raw, "config", "width", int)
        vocab = rd.get(raw, "config", "vocab", int)
        eps = rd.get(rd.get(raw, "config", "norm", dict), "config.norm", "eps", float)
        mult = rd.get(raw, "config", "residual_mult", float, default=1.0, required=False)
        streams = rd.get(raw, "config", "streams", int, default=0, required=False)
        if streams < 0 or streams > 8:
            rd.problems.append(f"config.streams must lie in 1..8, got {streams}")
        layers = raw.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            rd.problems.append("config.layers must be a non-empty list")
            layers = []
        loop = None
        lp = rd.get(raw, "config", "loop", dict, default=None, required=False)
        if lp is not None:
            start, stop, times = (rd.get(lp, "config.loop", k, int) for k in
                                  ("start", "stop", "times"))
            if not (0 <= start <= stop <= len(layers)) or times < 1:
                rd.problems.append(f"config.loop must name layers start <= stop within the "
                                   f"model and times >= 1, got {dict(lp)!r}")
            else:
                loop = (start, stop, times)
        stops = raw.get("eos_token_id")
        if stops is None:
            stops = ()
        elif not isinstance(stops, (list, tuple)):
            stops = (stops,)
        cfg = cls(width=width, vocab=vocab, norm_eps=eps, residual_mult=mult, streams=streams,
                  loop=loop, layers=copy.deepcopy(list(layers)),
                  stop_tokens=tuple(int(t) for t in stops))
        rd.positive("config", width=width, vocab=vocab, **{"norm.eps": eps})
        if width > 0:
            cfg._blocks(rd)
        if rd.problems:
            raise ConfigError("unusable Mokotar configuration: " + "; ".join(rd.problems))
        return cfg

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "width": self.width, "vocab": self.vocab,
               "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult,
               "layers": copy.deepcopy(self.layers)}
        if self.streams:
            out["streams"] = self.streams
        if self.loop is not None:
            out["loop"] = dict(zip(("start", "stop", "times"), self.loop))
        if self.stop_tokens:
            out["eos_token_id"] = list(self.stop_tokens)
        return out

    # -- what a checkpoint adds ---------------------------------------------
    def with_shapes(self, shape_of) -> "MokotarConfig":
        """The ranks of the delta rule's decay and gate projections are sizes that only the
        tensors give (``shape_of(name)``: a checkpoint tensor's shape, or None); they are
        written into the layer's ``mixer.right`` as ``decay_rank`` and ``gate_rank``, the keys
        under which a configuration may also state them itself."""
        for i, layer in enumerate(self.layers):
            if not isinstance(layer, Mapping) or layer.get("type") != "parallel":
                continue
            right = layer.get("mixer", {}).get("right")
            if not isinstance(right, dict):
                continue
            for key, name in (("decay_rank", "a1"), ("gate_rank", "g1")):
                shape = shape_of(f"l{i}.mix.right.{name}")
                if shape is not None and len(shape) == 2:
                    right[key] = int(shape[0])
        return self

    # -- layers -------------------------------------------------------------
    def _attention(self, rd: _Reader, path: str, m: Mapping, kind: str) -> AttentionSpec:
        heads, kv_heads, dim, vdim = (rd.get(m, path, k, int)
                                      for k in ("heads", "kv_heads", "dim", "vdim"))
        scale = rd.get(m, path, "scale", float)
        rd.positive(path, heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale)
        if kv_heads > 0 and heads % kv_heads:
            rd.problems.append(f"{path}.heads ({heads}) is no multiple of kv_heads ({kv_heads})")
        position = PositionSpec(kind="none", head_dim=dim)
        # the first type has no rotation; the other two always rotate
        rot = None if kind == "attention" else rd.get(m, path, "rot", dict)
        if rot is not None:
            base = rd.get(rot, path + ".rot", "base", float)
            dims = rd.get(rot, path + ".rot", "dims", int)
            rd.positive(path, **{"rot.base": base})
            if dims % 2 or not 0 <= dims <= dim:
                rd.problems.append(f"{path}.rot.dims must be even and at most dim, got {dims}")
            elif dims:
                position = PositionSpec(kind="rope", head_dim=dim, rotary_dim=dims, theta=base,
                                        interleaved=True)
        q_temp = softcap = None
        # temperature and soft cap belong to the first type only
        temp = rd.get(m, path, "q_temp", dict) if kind == "attention" else None
        if temp is not None:
            coef = rd.get(temp, path + ".q_temp", "coef", float)
            every = rd.get(temp, path + ".q_temp", "every", int)
            rd.positive(path, **{"q_temp.every": every})
            q_temp = (coef, every)
        cap = rd.get(m, path, "softcap", float) if kind == "attention" else None
        if cap is not None:
            rd.positive(path, softcap=cap)
            softcap = cap
        return AttentionSpec(hidden_size=self.width, num_heads=heads, num_kv_heads=kv_heads,
                             head_dim=dim, position=position, window=None, scale=scale,
                             v_head_dim=vdim, qk_norm_eps=self.norm_eps,
                             qk_norm_whole=kind == "attention_2",
                             feature_gate=kind != "left", q_temp=q_temp, softcap=softcap,
                             sink="zero" if kind == "left" else "learned")

    def _delta(self, rd: _Reader, path: str, m: Mapping, layer: int) -> GatedDeltaSpec:
        heads, kv_heads, dim, vdim, taps = (rd.get(m, path, k, int) for k in
                                            ("heads", "kv_heads", "dim", "vdim", "conv"))
        rd.positive(path, heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=taps)
        if kv_heads > 0 and heads % kv_heads:
            rd.problems.append(f"{path}.heads ({heads}) is no multiple of kv_heads ({kv_heads})")
        decay_rank = rd.get(m, path, "decay_rank", int, default=0, required=False)
        gate_rank = rd.get(m, path, "gate_rank", int, default=0, required=False)
        return GatedDeltaSpec(hidden_size=self.width, num_heads=heads, num_kv_heads=kv_heads,
                              qk_dim=dim, v_dim=vdim, conv=taps, decay_rank=decay_rank,
                              gate_rank=gate_rank, norm_eps=self.norm_eps)

    def _mixer(self, rd: _Reader, i: int, layer: Mapping):
        kind = rd.get(layer, f"layers[{i}]", "type", str)
        if kind not in LAYER_TYPES:
            rd.problems.append(f"layers[{i}].type {kind!r} is not known (known: {LAYER_TYPES})")
            return None
        path = f"layers[{i}].mixer"
        m = rd.get(layer, f"layers[{i}]", "mixer", dict)
        if kind != "parallel":
            return self._attention(rd, path, m, kind)
        left = self._attention(rd, path + ".left", rd.get(m, path, "left", dict), "left")
        right = self._delta(rd, path + ".right", rd.get(m, path, "right", dict), i)
        scales = (rd.get(m, path, "left_scale", float), rd.get(m, path, "right_scale", float))
        return ParallelMixerSpec(hidden_size=self.width, branches=(left, right),
                                 norm_eps=self.norm_eps, merge="weighted_sum", scales=scales)

    def _ffn(self, rd: _Reader, i: int, layer: Mapping):
        mlp = layer.get("mlp")
        if mlp is None:
            return None
        path = f"layers[{i}].mlp"
        kind = rd.get(mlp, path, "kind", str)
        if kind != "dense":
            rd.problems.append(f"{path}.kind {kind!r} is not known (known: dense)")
            return None
        ff = rd.get(mlp, path, "ff", int)
        rd.positive(path, ff=ff)
        return GatedMLPSpec(hidden_size=self.width, intermediate_size=ff, activation="silu",
                            bias=True)

    def _blocks(self, rd: Optional[_Reader] = None) -> list:
        rd = rd or _Reader()
        norm = NormSpec(kind="rmsnorm", size=self.width, eps=self.norm_eps)
        blocks = []
        for i, layer in enumerate(self.layers):
            if not isinstance(layer, Mapping):
                rd.problems.append(f"layers[{i}] must be an object")
                continue
            ffn = self._ffn(rd, i, layer)
            blocks.append(BlockSpec(kind="hyper", mixer=self._mixer(rd, i, layer), ffn=ffn,
                                    norm1=norm, norm2=None if ffn is None else norm,
                                    residual_mult=self.residual_mult, streams=self.streams))
        return blocks

    def run_order(self) -> list:
        """Layer indices in the order they run (a looped stretch several times)."""
        n = len(self.layers)
        if self.loop is None:
            return list(range(n))
        start, stop, times = self.loop
        return list(range(start)) + list(range(start, stop)) * times + list(range(stop, n))

    def layout(self) -> ModelLayout:
        norm = NormSpec(kind="rmsnorm", size=self.width, eps=self.norm_eps)
        order = [RunEntry(block=i, cache=run) for run, i in enumerate(self.run_order())]
        layout = ModelLayout(vocab_size=self.vocab, hidden_size=self.width,
                             blocks=self._blocks(), order=order, final_norm=norm,
                             tie_word_embeddings=False, max_positions=None)
        layout.validate()
        return layout

    def stop_token_ids(self) -> tuple:
        return tuple(self.stop_tokens)

    def max_positions(self):
        return None
