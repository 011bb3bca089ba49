"""Block arrangements: how a mixer, a feed-forward and norms are wired.

"prenorm" is the reference's DecoderLayer (mstar/model/components/decoder_layer.py:
58-71): h += mixer(norm1(h)); h += ffn(norm2(h)).  The two adds are not separate
passes: each part's output stays pending on the residual stream and the next norm
(the next block's norm1, or the final norm) adds it in float while normalising.
"""
from __future__ import annotations

import torch

from ..weights.names import ParamSpec
from .base import ResidualStream, Runtime
from .registry import build_part, part_class, register_part


def _sub(params: dict, prefix: str) -> dict:
    p = prefix + "."
    return {k[len(p):]: v for k, v in params.items() if k.startswith(p)}


class PreNormBlock:
    SUBPARTS = (("norm1", "norm"), ("mixer", "mixer"), ("norm2", "norm"), ("ffn", "ffn"))

    @classmethod
    def param_specs(cls, spec) -> dict:
        out = {}
        for name, category in cls.SUBPARTS:
            sub = getattr(spec, name)
            for local, ps in part_class(category, sub).param_specs(sub).items():
                out[f"{name}.{local}"] = ps
        return out

    @classmethod
    def cache_need(cls, spec):
        return part_class("mixer", spec.mixer).cache_need(spec.mixer)

    def __init__(self, spec, params: dict, runtime: Runtime):
        self.spec = spec
        self.norm1 = build_part("norm", spec.norm1, _sub(params, "norm1"), runtime)
        self.mixer = build_part("mixer", spec.mixer, _sub(params, "mixer"), runtime)
        self.norm2 = build_part("norm", spec.norm2, _sub(params, "norm2"), runtime)
        self.ffn = build_part("ffn", spec.ffn, _sub(params, "ffn"), runtime)
        # replayable as part of a captured decode step only if every sub-part says so itself
        self.graph_safe = all(getattr(p, "graph_safe", False) is True
                              for p in (self.norm1, self.mixer, self.norm2, self.ffn))

    def forward(self, stream: ResidualStream, ctx, cache) -> None:
        x = self.norm1.add_norm(stream)
        stream.push(self.mixer.forward(x, ctx, cache))
        y = self.norm2.add_norm(stream)
        stream.push(self.ffn.forward(y, ctx))


class SandwichBlock:
    """h += norm1_post(mixer(norm1(h))); h += norm2_post(ffn(norm2(h))).  A sublayer's output
    is pushed together with its own norm; the next norm on the stream (this block's norm2, the
    next block's norm1, or the model's final norm) applies it, adds and normalises in one
    kernel.  A block without a feed-forward has the first sublayer only."""

    @staticmethod
    def _subparts(spec):
        parts = [("norm1", "norm"), ("mixer", "mixer"), ("norm1_post", "norm")]
        if spec.ffn is not None:
            parts += [("norm2", "norm"), ("ffn", "ffn"), ("norm2_post", "norm")]
        return parts

    @classmethod
    def param_specs(cls, spec) -> dict:
        out = {}
        for name, category in cls._subparts(spec):
            sub = getattr(spec, name)
            if sub is None:
                raise ValueError(f"a sandwich block needs {name}")
            for local, ps in part_class(category, sub).param_specs(sub).items():
                out[f"{name}.{local}"] = ps
        return out

    @classmethod
    def cache_need(cls, spec):
        return part_class("mixer", spec.mixer).cache_need(spec.mixer)

    def __init__(self, spec, params: dict, runtime: Runtime):
        self.spec = spec
        self.parts = {name: build_part(category, getattr(spec, name), _sub(params, name), runtime)
                      for name, category in self._subparts(spec)}
        self.norm1, self.mixer, self.norm1_post = (self.parts[k] for k in
                                                   ("norm1", "mixer", "norm1_post"))
        self.norm2, self.ffn, self.norm2_post = (self.parts.get(k) for k in
                                                 ("norm2", "ffn", "norm2_post"))
        self.graph_safe = all(getattr(p, "graph_safe", False) is True for p in self.parts.values())

    def forward(self, stream: ResidualStream, ctx, cache) -> None:
        x = self.norm1.add_norm(stream)
        stream.push(self.mixer.forward(x, ctx, cache), post=self.norm1_post)
        if self.ffn is not None:
            y = self.norm2.add_norm(stream)
            stream.push(self.ffn.forward(y, ctx), post=self.norm2_post)


class PostNormBlock:
    """h += m * norm1_post(mixer(h)); h += m * norm2_post(ffn(h)): the sublayers read the
    residual itself, only their outputs are normed (and multiplied by ``residual_mult``).  A
    sublayer's output stays pending with its norm; the kernel that adds it also hands the new
    residual, in the compute dtype, to the sublayer that reads it next."""

    @staticmethod
    def _subparts(spec):
        parts = [("mixer", "mixer"), ("norm1_post", "norm")]
        if spec.ffn is not None:
            parts += [("ffn", "ffn"), ("norm2_post", "norm")]
        return parts

    @classmethod
    def param_specs(cls, spec) -> dict:
        out = {}
        for name, category in cls._subparts(spec):
            sub = getattr(spec, name)
            if sub is None:
                raise ValueError(f"a postnorm block needs {name}")
            for local, ps in part_class(category, sub).param_specs(sub).items():
                out[f"{name}.{local}"] = ps
        return out

    @classmethod
    def cache_need(cls, spec):
        return part_class("mixer", spec.mixer).cache_need(spec.mixer)

    def __init__(self, spec, params: dict, runtime: Runtime):
        self.spec = spec
        self.runtime = runtime
        self.parts = {name: build_part(category, getattr(spec, name), _sub(params, name), runtime)
                      for name, category in self._subparts(spec)}
        self.mixer, self.norm1_post = self.parts["mixer"], self.parts["norm1_post"]
        self.ffn, self.norm2_post = self.parts.get("ffn"), self.parts.get("norm2_post")
        self.graph_safe = all(getattr(p, "graph_safe", False) is True for p in self.parts.values())

    def forward(self, stream: ResidualStream, ctx, cache) -> None:
        m = self.spec.residual_mult
        x = stream.rows(self.runtime.dtype)
        stream.push(self.mixer.forward(x, ctx, cache), post=self.norm1_post, scale=m)
        if self.ffn is not None:
            y = stream.rows(self.runtime.dtype)
            stream.push(self.ffn.forward(y, ctx), post=self.norm2_post, scale=m)


class ResidualCopies:
    """The residual as ``streams`` copies per token, float [tokens, streams, width], with the
    last sublayer's output still to be written into them.  It hangs on the residual stream
    from the first hyper-connection block to the model's end."""

    def __init__(self, x: torch.Tensor, init: torch.Tensor):
        self.x = x
        self.init = init            # the embedding output, until the copies are first written
        self.pending = None         # dict of hyper_step's write arguments

    def step(self, **read):
        """Write what is pending, then read (``read=...``) or sum (``rows=...``)."""
        from .. import ops

        write = self.pending or {}
        if not write:                # nothing to write yet: the kernel still wants its tables
            write = dict(zip(("mix", "out"), _no_write_tables(self.x.shape[1], self.x.device)))
        out = ops.hyper_step(self.x, init=self.init, **write, **read)
        if "rows" not in read:      # a sum leaves the copies as they were
            self.init = None
            self.pending = None
        return out

    def gather(self, rows: torch.Tensor) -> torch.Tensor:
        return self.step(rows=rows)


_NO_WRITE: dict = {}


def _no_write_tables(n: int, device) -> tuple:
    """(identity mix, zero out) for a step that writes nothing; made once per size and device."""
    key = (n, str(device))
    if key not in _NO_WRITE:
        _NO_WRITE[key] = (torch.eye(n, dtype=torch.float32, device=device).contiguous(),
                          torch.zeros(n, dtype=torch.float32, device=device))
    return _NO_WRITE[key]


class HyperBlock:
    """Pre-norm sublayers on a residual of several copies (hyper-connections): sublayer q
    reads ``norm_q(sum_s in_q[s] x_s)`` and writes ``x_t = sum_s mix_q[s, t] x_s + m * out_q[t] *
    y`` into every copy at once.  What lies between two sublayers (the write of the one, the
    read and the norm of the next) is one kernel; a sublayer's output stays pending until
    then, with its bias or its second branch where it has one.  ``streams`` 0 is the ordinary
    ``x += m * sublayer(norm(x))`` through the same kernel (one copy, tables of ones)."""

    @staticmethod
    def _subparts(spec):
        parts = [("norm1", "norm"), ("mixer", "mixer")]
        if spec.ffn is not None:
            parts += [("norm2", "norm"), ("ffn", "ffn")]
        return parts

    @classmethod
    def param_specs(cls, spec) -> dict:
        out = {}
        for name, category in cls._subparts(spec):
            sub = getattr(spec, name)
            if sub is None:
                raise ValueError(f"a hyper-connection block needs {name}")
            for local, ps in part_class(category, sub).param_specs(sub).items():
                out[f"{name}.{local}"] = ps
        s = spec.streams
        if s:
            for q in (1, 2) if spec.ffn is not None else (1,):
                out[f"hc{q}.in"] = ParamSpec((s,), role="vector", init="ones")
                out[f"hc{q}.out"] = ParamSpec((s,), role="vector", init="ones")
                out[f"hc{q}.mix"] = ParamSpec((s, s), role="vector", init="identity")
        return out

    @classmethod
    def cache_need(cls, spec):
        return part_class("mixer", spec.mixer).cache_need(spec.mixer)

    def __init__(self, spec, params: dict, runtime: Runtime):
        self.spec = spec
        self.runtime = runtime
        self.parts = {name: build_part(category, getattr(spec, name), _sub(params, name), runtime)
                      for name, category in self._subparts(spec)}
        self.norm1, self.mixer = self.parts["norm1"], self.parts["mixer"]
        self.norm2, self.ffn = self.parts.get("norm2"), self.parts.get("ffn")
        self.streams = max(1, spec.streams)
        self.tables = {}
        for q in (1, 2) if spec.ffn is not None else (1,):
            if spec.streams:
                t_in, t_out, t_mix = (params[f"hc{q}.{t}"].float() for t in ("in", "out", "mix"))
            else:
                t_in = t_out = torch.ones(1, dtype=torch.float32, device=runtime.device)
                t_mix = torch.ones((1, 1), dtype=torch.float32, device=runtime.device)
            # the residual multiplier is folded into the write weights (float)
            self.tables[q] = (t_in.contiguous(), (t_out * spec.residual_mult).contiguous(),
                              t_mix.contiguous())
        for norm in (self.norm1, self.norm2):
            if norm is not None and (norm.spec.kind != "rmsnorm" or norm.spec.weight_offset):
                raise ValueError("a hyper-connection block reads through a plain RMS norm")
        self.graph_safe = all(getattr(p, "graph_safe", False) is True for p in self.parts.values())

    def _pending(self, y, q: int) -> dict:
        from .. import ops
        from .mlp import OutputWithBias

        _, t_out, t_mix = self.tables[q]
        write = {"mix": t_mix, "out": t_out}
        if isinstance(y, OutputWithBias):
            write.update(y=y.y, y_bias=y.bias)
        elif isinstance(y, ops.WeightedSum) and len(y.branches) == 2:
            write.update(y=y.branches[0], y2=y.branches[1], y_scales=tuple(y.scales))
        else:
            write["y"] = y.materialize() if hasattr(y, "materialize") else y
        return write

    def forward(self, stream: ResidualStream, ctx, cache) -> None:
        copies = stream.copies
        if copies is None:
            if stream.delta is not None:                 # a block of another kind came before
                stream.h.add_(stream.take_delta().float())
            x = torch.empty((stream.h.shape[0], self.streams, stream.h.shape[1]),
                            dtype=torch.float32, device=stream.h.device)
            copies = stream.copies = ResidualCopies(x, stream.h)
        elif copies.x.shape[1] != self.streams:
            raise ValueError("blocks of one model keep the same number of residual copies")
        dtype = self.runtime.dtype
        x = copies.step(read=self.tables[1][0], norm_weight=self.norm1.weight,
                        eps=self.norm1.spec.eps, out_dtype=dtype)
        copies.pending = self._pending(self.mixer.forward(x, ctx, cache), 1)
        if self.ffn is not None:
            y = copies.step(read=self.tables[2][0], norm_weight=self.norm2.weight,
                            eps=self.norm2.spec.eps, out_dtype=dtype)
            copies.pending = self._pending(self.ffn.forward(y, ctx), 2)


register_part("block", "hyper", HyperBlock)
register_part("block", "prenorm", PreNormBlock)
register_part("block", "postnorm", PostNormBlock)
register_part("block", "sandwich", SandwichBlock)
