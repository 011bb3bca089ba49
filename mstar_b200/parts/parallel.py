"""Parallel mixer: several mixers side by side on the same input.  With ``merge``
"weighted_sum" the result is ``sum_b scales[b] * branch_b``, handed on uncomputed
(``ops.WeightedSum``) for the block's kernel to add.  Otherwise the result is the mean of
their outputs, each divided by its root mean square over the model width and scaled by a
weight of its own; the mean is float.  The mixer hands it on uncomputed (``ops.MeanOfNorms``):
the norm that adds it to the residual does both in one kernel, or computes it first.  At most one branch may keep keys and values in pages
and at most one a state slot: the layer's cache entry then serves both.

The branches do not depend on one another, so each after the first runs on a stream of its
own, forked from and joined to the stream of the step (in a captured decode step they become
parallel branches of the graph): the short kernels of one branch fill the gaps between those
of the other.  MSTAR_PARALLEL_STREAMS=0 runs them one after the other.
"""
from __future__ import annotations

import os

import torch

from .. import ops
from ..weights.names import ParamSpec
from .base import CacheNeed, LayerCache, Runtime, StepContext
from .registry import build_part, part_class, register_part


def _sub(params: dict, prefix: str) -> dict:
    p = prefix + "."
    return {k[len(p):]: v for k, v in params.items() if k.startswith(p)}


class ParallelMixer:
    @classmethod
    def param_specs(cls, spec) -> dict:
        out = {}
        for b, branch in enumerate(spec.branches):
            for local, ps in part_class("mixer", branch).param_specs(branch).items():
                out[f"branch{b}.{local}"] = ps
            if spec.merge == "mean_of_norms":
                out[f"out{b}.weight"] = ParamSpec((spec.hidden_size,), role="vector", init="ones")
        return out

    @classmethod
    def cache_need(cls, spec) -> CacheNeed:
        kv = state = None
        for branch in spec.branches:
            need = part_class("mixer", branch).cache_need(branch)
            if need is None:
                continue
            if need.kv is not None:
                if kv is not None:
                    raise ValueError("two branches of a parallel mixer ask for key/value pages")
                kv = need.kv
            if need.state is not None:
                if state is not None:
                    raise ValueError("two branches of a parallel mixer ask for a state slot")
                state = need.state
        return CacheNeed(kv=kv, state=state)

    def __init__(self, spec, params: dict, runtime: Runtime):
        if not 1 <= len(spec.branches) <= 4:
            raise ValueError("a parallel mixer has one to four branches")
        self.spec = spec
        self.runtime = runtime
        self.branches = [build_part("mixer", branch, _sub(params, f"branch{b}"), runtime)
                         for b, branch in enumerate(spec.branches)]
        if spec.merge not in ("mean_of_norms", "weighted_sum"):
            raise ValueError(f"a parallel mixer merges by mean_of_norms or weighted_sum, not "
                             f"{spec.merge!r}")
        if spec.merge == "weighted_sum" and len(spec.scales) != len(spec.branches):
            raise ValueError("a weighted sum needs one scale per branch")
        self.weights = [params[f"out{b}.weight"].float().contiguous()
                        for b in range(len(spec.branches))] if spec.merge == "mean_of_norms" else []
        self.graph_safe = all(getattr(p, "graph_safe", False) is True for p in self.branches)
        self.side_streams = None
        if len(self.branches) > 1 and os.environ.get("MSTAR_PARALLEL_STREAMS") != "0":
            self.side_streams = [torch.cuda.Stream(device=runtime.device)
                                 for _ in self.branches[1:]]

    def forward(self, x, ctx: StepContext, cache: LayerCache):
        if self.side_streams is None:
            outs = [branch.forward(x, ctx, cache) for branch in self.branches]
            return self._merge(outs)
        main = torch.cuda.current_stream(self.runtime.device)
        outs = [None] * len(self.branches)
        for b, side in enumerate(self.side_streams, start=1):
            side.wait_stream(main)                       # x is ready there
            with torch.cuda.stream(side):
                outs[b] = self.branches[b].forward(x, ctx, cache)
        outs[0] = self.branches[0].forward(x, ctx, cache)
        for side in self.side_streams:
            main.wait_stream(side)
        # what the side streams allocated is used on the step's stream from here on
        for out in outs[1:]:
            out.record_stream(main)
        return self._merge(outs)

    def _merge(self, outs):
        # (left to the kernel that adds it to the residual: one kernel for both where it can)
        if self.spec.merge == "weighted_sum":
            return ops.WeightedSum(outs, self.spec.scales)
        return ops.MeanOfNorms(outs, self.weights, self.spec.norm_eps)


register_part("mixer", "parallel", ParallelMixer)
