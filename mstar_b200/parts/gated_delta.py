"""Gated delta rule mixer: a matrix memory per head that is decayed per key channel, corrected
towards the token's value along its key and read with its query; the matrix (float) and the
last inputs of its short convolutions live in a state slot.

One product, with float output, gives ``[q | k | v | b | a1 | g1]``; two small products give
the decay's pre-activation (``W_a2 a1``, float) and the output gate (``W_g2 g1``).  A kernel
runs the convolutions with SiLU, makes q and k unit vectors, the write strengths and the
decays (all float); a second moves the slot's convolution rows on; the scan walks each
entry's tokens from the matrix in its slot; a last kernel norms each head's output, gates it
and hands it to the output product.  A prompt portion, a decoded token and any mix are the
same launches.
"""
from __future__ import annotations

import torch

from .. import ops
from ..weights.names import ParamSpec
from .base import CacheNeed, LayerCache, Runtime, StateNeed, StepContext
from .registry import register_part


class GatedDelta:
    graph_safe = True       # the forward pass reads the step's device arrays only

    @classmethod
    def param_specs(cls, spec) -> dict:
        qk, vv = spec.num_kv_heads * spec.qk_dim, spec.num_heads * spec.v_dim
        rows = 2 * qk + vv + spec.num_heads + spec.decay_rank + spec.gate_rank
        return {
            "in.weight": ParamSpec((rows, spec.hidden_size)),
            "conv.weight": ParamSpec((2 * qk + vv, spec.conv), role="vector"),
            "a2.weight": ParamSpec((spec.num_heads * spec.qk_dim, spec.decay_rank)),
            "dt_bias": ParamSpec((spec.num_heads * spec.qk_dim,), role="vector", init="zeros"),
            "A_log": ParamSpec((spec.num_heads,), role="vector", init="zeros"),
            "g2.weight": ParamSpec((vv, spec.gate_rank)),
            "norm.weight": ParamSpec((spec.v_dim,), role="vector", init="ones"),
            "o.weight": ParamSpec((spec.hidden_size, vv)),
        }

    @classmethod
    def cache_need(cls, spec) -> CacheNeed:
        size = ops.gated_delta_state_size(spec.num_heads, spec.num_kv_heads, spec.qk_dim,
                                          spec.v_dim, spec.conv)
        return CacheNeed(state=StateNeed(shape=(size,), dtype="float32"))

    def __init__(self, spec, params: dict, runtime: Runtime):
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"num_heads {spec.num_heads} is not a multiple of num_kv_heads "
                             f"{spec.num_kv_heads}")
        if spec.decay_rank <= 0 or spec.gate_rank <= 0:
            raise ValueError("the ranks of the decay and gate projections are not known: they "
                             "come from the checkpoint's tensor shapes or the configuration")
        self.spec = spec
        self.runtime = runtime
        self.w_in = params["in.weight"]
        self.w_a2 = params["a2.weight"]
        self.w_g2 = params["g2.weight"]
        self.w_out = params["o.weight"]
        self.conv_w = params["conv.weight"].contiguous()
        # everything that enters the recurrence besides q, k and v is float
        self.dt_bias = params["dt_bias"].float().contiguous()
        self.a_exp = torch.exp(params["A_log"].float()).contiguous()
        self.norm_weight = params["norm.weight"].float().contiguous()
        # a caller that sums this mixer's output with a weight may fold the weight in here
        self.out_scale = 1.0

    def forward(self, x, ctx: StepContext, cache: LayerCache):
        s = self.spec
        H, G, D, VD = s.num_heads, s.num_kv_heads, s.qk_dim, s.v_dim
        channels = 2 * G * D + H * VD
        proj = ops.linear(x, self.w_in, out_dtype=torch.float32, static_weights=True)
        low = proj[:, channels + H:]
        if self.runtime.dtype != torch.float32:
            low = ops.convert(low.contiguous(), self.runtime.dtype)
        a1, g1 = low[:, :s.decay_rank], low[:, s.decay_rank:]
        a_proj = ops.linear(a1.contiguous(), self.w_a2, out_dtype=torch.float32,
                            static_weights=True)
        gate = ops.linear(g1.contiguous(), self.w_g2, static_weights=True)
        q, k, v, beta, decay = ops.delta_prepare(
            proj, self.conv_w, a_proj, self.dt_bias, self.a_exp, ctx.token_req, ctx.qo_indptr,
            ctx.slots, cache.state, H, G, D, VD, s.conv, s.unit_eps)
        ops.conv_state_advance(proj, channels, s.conv, ctx.qo_indptr, ctx.slots, cache.state,
                               ctx.num_entries)
        o = ops.delta_scan(q, k, v, beta, decay, ctx.qo_indptr, ctx.slots, cache.state,
                           ctx.num_entries, H, G, D, VD, s.conv, max_q_len=ctx.max_q_len)
        y = ops.delta_finish(o, gate, self.norm_weight, H, VD, s.norm_eps, self.runtime.dtype,
                             self.out_scale)
        return ops.linear(y, self.w_out, static_weights=True)


register_part("mixer", "gated_delta", GatedDelta)
