"""Typed configuration of the Relurax decoder (``"architecture": "Relurax"``).

config.json gives ``width``, ``vocab``, ``norm.eps`` and the layers one by one:
``layers[i] = {"type", "mixer": {...}, "mlp": {...} | null}``.  Every layer is a sandwich
block (an RMS norm with a plain weight before and after each sublayer) around one of two
mixers:

* ``"attention"``: grouped-query attention without positions.  q and k pass a causal
  convolution of ``conv`` taps per channel right after their projections and an RMS norm
  per head; the values are the convolved keys before that norm (there is no value
  projection); a sliding window ``mask.size``; the score scale ``scale``; one sigmoid gate
  a head on the output.
* ``"latent_attention"``: causal attention over one cached latent row per token
  (``kv_rank`` normed features and ``rot_dim`` rotated key features shared by the heads),
  queries through a normed latent of ``q_rank`` features, rotate-half rotary pairs over the
  first ``rot.dims`` of the rotated part, one sigmoid gate a head.  ``"kv_from": j`` makes
  the layer read the rows that layer j cached instead of projecting its own.

The feed-forward is ``down(gelu_tanh(gate h) * up h)`` (``mlp.kind`` "dense") or absent.
Nothing has a size default; every size may differ from layer to layer.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Mapping, Optional

from .base import ConfigError, ModelConfig
from .layout import (AttentionSpec, BlockSpec, GatedMLPSpec, LatentAttentionSpec, ModelLayout,
                     NormSpec, PositionSpec, RunEntry)
from .tifosun import _Reader

LAYER_TYPES = ("attention", "latent_attention")


@dataclass
class ReluraxConfig(ModelConfig):
    width: int
    vocab: int
    norm_eps: float
    layers: list = field(default_factory=list)        # the raw layer objects of config.json
    stop_tokens: tuple = ()

    architecture = "Relurax"

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "ReluraxConfig":
        rd = _Reader()
        width = rd.get(raw, "config", "width", int)
        vocab = rd.get(raw, "config", "vocab", int)
        eps = rd.get(rd.get(raw, "config", "norm", dict), "config.norm", "eps", float)
        layers = raw.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            rd.problems.append("config.layers must be a non-empty list")
            layers = []
        stops = raw.get("eos_token_id")
        if stops is None:
            stops = ()
        elif not isinstance(stops, (list, tuple)):
            stops = (stops,)
        cfg = cls(width=width, vocab=vocab, norm_eps=eps, layers=copy.deepcopy(list(layers)),
                  stop_tokens=tuple(int(t) for t in stops))
        rd.positive("config", width=width, vocab=vocab, **{"norm.eps": eps})
        if not rd.problems:
            cfg._plan(rd)
        if rd.problems:
            raise ConfigError("unusable Relurax configuration: " + "; ".join(rd.problems))
        return cfg

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "width": self.width, "vocab": self.vocab,
               "norm": {"eps": self.norm_eps}, "layers": copy.deepcopy(self.layers)}
        if self.stop_tokens:
            out["eos_token_id"] = list(self.stop_tokens)
        return out

    # -- layers -------------------------------------------------------------
    def _attention(self, rd: _Reader, path: str, m: Mapping):
        heads, groups, dim, vdim, taps = (rd.get(m, path, k, int)
                                          for k in ("heads", "kv_heads", "dim", "vdim", "conv"))
        scale = rd.get(m, path, "scale", float)
        mask = rd.get(m, path, "mask", dict, default=None, required=False)
        window = None if mask is None else rd.get(mask, path + ".mask", "size", int)
        rd.positive(path, heads=heads, kv_heads=groups, dim=dim, vdim=vdim, conv=taps, scale=scale)
        if window is not None:
            rd.positive(path, **{"mask.size": window})
        if groups > 0 and heads % groups:
            rd.problems.append(f"{path}.heads ({heads}) must be a multiple of kv_heads ({groups})")
        if vdim != dim:
            rd.problems.append(f"{path}.vdim ({vdim}) must equal dim ({dim}): the values are "
                               "the keys")
        return AttentionSpec(hidden_size=self.width, num_heads=heads, num_kv_heads=groups,
                             head_dim=dim, position=PositionSpec(kind="none", head_dim=dim),
                             window=window, scale=scale, qk_norm_eps=self.norm_eps,
                             conv_taps=taps, value_from_key=True, head_gate=True)

    def _latent(self, rd: _Reader, i: int, path: str, m: Mapping):
        heads, dim, vdim, rank, rot_dim, q_rank = (
            rd.get(m, path, k, int) for k in ("heads", "dim", "vdim", "kv_rank", "rot_dim", "q_rank"))
        rot = rd.get(m, path, "rot", dict)
        base = rd.get(rot, path + ".rot", "base", float)
        dims = rd.get(rot, path + ".rot", "dims", int, default=rot_dim, required=False)
        scale = rd.get(m, path, "scale", float)
        rd.positive(path, heads=heads, dim=dim, vdim=vdim, kv_rank=rank, rot_dim=rot_dim,
                    q_rank=q_rank, scale=scale, **{"rot.base": base})
        if dims % 2 or not 0 <= dims <= rot_dim:
            rd.problems.append(f"{path}.rot.dims must be even and at most rot_dim, got {dims}")
        source = m.get("kv_from") if isinstance(m, Mapping) else None
        if source is not None:
            ok = (not isinstance(source, bool) and isinstance(source, int) and 0 <= source < i
                  and isinstance(self.layers[source], Mapping)
                  and self.layers[source].get("type") == "latent_attention"
                  and isinstance(self.layers[source].get("mixer"), Mapping)
                  and self.layers[source]["mixer"].get("kv_from") is None)
            if not ok:
                rd.problems.append(f"{path}.kv_from must name an earlier latent_attention layer "
                                   f"with a down-projection of its own, got {source!r}")
                source = None
            else:
                theirs = self.layers[source]["mixer"]
                for key in ("kv_rank", "rot_dim", "rot"):
                    if theirs.get(key) != m.get(key):
                        rd.problems.append(f"{path}.{key} must equal that of layer {source}, "
                                           "whose rows it reads")
        position = PositionSpec(kind="rope", head_dim=rot_dim, rotary_dim=dims, theta=base,
                                interleaved=False)
        return LatentAttentionSpec(hidden_size=self.width, num_heads=heads, qk_dim=dim,
                                   rot_dim=rot_dim, v_dim=vdim, kv_rank=rank, position=position,
                                   window=None, scale=scale, norm_eps=self.norm_eps, gated=True,
                                   gate_per_head=True, q_rank=q_rank,
                                   shares_kv=source is not None), source

    def _ffn(self, rd: _Reader, i: int, layer: Mapping):
        mlp = layer.get("mlp")
        if mlp is None:
            return None
        path = f"layers[{i}].mlp"
        kind = rd.get(mlp, path, "kind", str)
        if kind == "dense":
            ff = rd.get(mlp, path, "ff", int)
            rd.positive(path, ff=ff)
            return GatedMLPSpec(hidden_size=self.width, intermediate_size=ff,
                                activation="gelu_tanh")
        rd.problems.append(f"{path}.kind {kind!r} is not known (known: dense)")
        return None

    def _plan(self, rd: Optional[_Reader] = None):
        """(blocks, order): a block per layer; a layer that caches something gets the next
        cache number, a layer that reads another's rows runs on that layer's cache."""
        rd = rd or _Reader()
        norm = NormSpec(kind="rmsnorm", size=self.width, eps=self.norm_eps)
        blocks, order, cache_of = [], [], {}
        for i, layer in enumerate(self.layers):
            if not isinstance(layer, Mapping):
                rd.problems.append(f"layers[{i}] must be an object")
                continue
            path = f"layers[{i}].mixer"
            kind = rd.get(layer, f"layers[{i}]", "type", str)
            m = rd.get(layer, f"layers[{i}]", "mixer", dict)
            source = None
            if kind == "attention":
                mixer = self._attention(rd, path, m)
            elif kind == "latent_attention":
                mixer, source = self._latent(rd, i, path, m)
            else:
                rd.problems.append(f"layers[{i}].type {kind!r} is not known (known: {LAYER_TYPES})")
                continue
            ffn = self._ffn(rd, i, layer)
            if source is None:
                cache_of[i] = len(set(cache_of.values()))
            elif source in cache_of:
                cache_of[i] = cache_of[source]
            else:
                continue
            order.append(RunEntry(block=len(blocks), cache=cache_of[i]))
            blocks.append(BlockSpec(kind="sandwich", mixer=mixer, ffn=ffn, norm1=norm,
                                    norm2=None if ffn is None else norm, norm1_post=norm,
                                    norm2_post=None if ffn is None else norm))
        return blocks, order

    def layout(self) -> ModelLayout:
        norm = NormSpec(kind="rmsnorm", size=self.width, eps=self.norm_eps)
        blocks, order = self._plan()
        layout = ModelLayout(vocab_size=self.vocab, hidden_size=self.width, blocks=blocks,
                             order=order, final_norm=norm, tie_word_embeddings=False,
                             max_positions=None)
        layout.validate()
        return layout

    def stop_token_ids(self) -> tuple:
        return tuple(self.stop_tokens)

    def max_positions(self):
        return None
