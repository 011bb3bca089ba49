"""Grouped-query attention mixer over the paged cache.

Order of operations as in the reference (mstar/model/components/distributed/
attention.py:98-110, 138-149): one fused QKV product, split [q | k | v], position
encoding on q and k, write of k and v into the cache, attention, output product.
Query head i uses key/value head i // (num_heads / num_kv_heads); scores are scaled
by head_dim ** -0.5 unless the spec says otherwise; the mask is causal and aligned
to the end of the key sequence, optionally limited to a window of keys.

A layer with ``shares_kv`` has only the query and output products and reads the
cache that an earlier layer wrote.

Beyond that plain form a spec may ask for biases on q, k and v, an RMS norm per query and
key head before the position encoding, a value size other than the key size, and a window
that keeps the sequence's first keys visible (``keep_first``).  Such a layer takes the fused
product in float, a kernel that adds the bias, norms, rotates and fills the cache pages, and
an attention kernel that walks the kept first keys and the window's keys.  The same path
takes a short causal convolution over time on the q and k channels (its last inputs are
per-request state in a slot), values that are the keys before their norm, and one sigmoid
gate a head on the output; the gate's rows ride in the fused first product.  Further
options of that path: an RMS norm over the whole q (and k) projection instead of a head,
rotary pairs of neighbouring features, a query temperature that grows with the logarithm of
the position, a tanh soft cap on the scores, a sink in the softmax's denominator (a learned
number a head, or zero), and a sigmoid gate a feature on the heads' outputs.
"""
from __future__ import annotations

import torch

from .. import ops
from ..weights.names import ParamSpec
from .base import CacheNeed, KVNeed, LayerCache, Runtime, StateNeed, StepContext
from .registry import build_part, register_part


class Attention:
    # everything the forward pass does depends on the step's device arrays and on host
    # values that are fixed for a batch shape, so a decode step can be replayed as a
    # CUDA graph
    graph_safe = True

    @classmethod
    def param_specs(cls, spec) -> dict:
        q_rows = spec.num_heads * spec.head_dim
        kv_rows = spec.num_kv_heads * (spec.head_dim + (0 if spec.value_from_key
                                                        else spec.value_dim))
        if spec.head_gate:
            kv_rows += spec.num_heads           # the gate's rows come last
        if spec.feature_gate:
            kv_rows += spec.num_heads * spec.value_dim
        if spec.shares_kv:
            first = {"q.weight": ParamSpec((q_rows, spec.hidden_size))}
        else:
            first = {"qkv.weight": ParamSpec((q_rows + kv_rows, spec.hidden_size))}
            if spec.bias:
                first["qkv.bias"] = ParamSpec((q_rows + kv_rows,), role="vector", init="zeros")
        if spec.qk_norm_eps is not None:
            per_q, per_k = (spec.num_heads, spec.num_kv_heads) if spec.qk_norm_whole else (1, 1)
            first["q_norm.weight"] = ParamSpec((per_q * spec.head_dim,), role="vector", init="ones")
            first["k_norm.weight"] = ParamSpec((per_k * spec.head_dim,), role="vector", init="ones")
        if spec.sink == "learned":
            first["sink"] = ParamSpec((spec.num_heads,), role="vector", init="zeros")
        if spec.conv_taps:
            first["q_conv.weight"] = ParamSpec((q_rows, spec.conv_taps), role="vector")
            first["k_conv.weight"] = ParamSpec((spec.num_kv_heads * spec.head_dim, spec.conv_taps),
                                               role="vector")
        first["o.weight"] = ParamSpec((spec.hidden_size, spec.num_heads * spec.value_dim))
        return first

    @classmethod
    def cache_need(cls, spec) -> CacheNeed:
        state = None
        if spec.conv_taps > 1:                  # the convolution's last inputs, q then k channels
            channels = (spec.num_heads + spec.num_kv_heads) * spec.head_dim
            state = StateNeed(shape=((spec.conv_taps - 1) * channels,), dtype="float32")
        return CacheNeed(kv=KVNeed(num_kv_heads=spec.num_kv_heads, head_dim=spec.head_dim,
                                   window=spec.window, keep_first=spec.keep_first if spec.window
                                   else 0,
                                   v_head_dim=None if spec.value_dim == spec.head_dim
                                   else spec.value_dim), state=state)

    def __init__(self, spec, params: dict, runtime: Runtime):
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"num_heads {spec.num_heads} is not a multiple of num_kv_heads "
                             f"{spec.num_kv_heads}")
        if spec.plain and spec.head_dim % 16:
            raise ValueError(f"head_dim {spec.head_dim} must be a multiple of 16")
        if not spec.plain and spec.shares_kv:
            raise ValueError("a layer that reads another layer's keys takes the plain attention")
        self.spec = spec
        self.runtime = runtime
        self.w_in = params["q.weight"] if spec.shares_kv else params["qkv.weight"]
        self.w_out = params["o.weight"]
        self.bias = params.get("qkv.bias")
        self.q_norm, self.k_norm = params.get("q_norm.weight"), params.get("k_norm.weight")
        self.q_conv, self.k_conv = params.get("q_conv.weight"), params.get("k_conv.weight")
        if spec.value_from_key and spec.value_dim != spec.head_dim:
            raise ValueError("values that are the keys have the keys' size")
        if spec.conv_taps and spec.bias:
            raise ValueError("a convolution on biased projections is not defined here")
        if spec.head_gate and spec.feature_gate:
            raise ValueError("an attention has a gate a head or a gate a feature, not both")
        if spec.qk_norm_whole and (spec.conv_taps or spec.qk_norm_eps is None):
            raise ValueError("a norm over the whole projection needs qk_norm_eps and no "
                             "convolution")
        if spec.sink not in (None, "learned", "zero"):
            raise ValueError(f"sink {spec.sink!r} is not known (learned, zero)")
        self.sink = None
        if spec.sink == "learned":
            self.sink = params["sink"].float().contiguous()
        elif spec.sink == "zero":
            self.sink = torch.zeros(spec.num_heads, dtype=torch.float32, device=runtime.device)
        small = [w for w in (self.bias, self.q_norm, self.k_norm, self.q_conv, self.k_conv)
                 if w is not None]
        if len({w.dtype for w in small}) > 1:   # the input kernel takes them in one type
            self.bias, self.q_norm, self.k_norm, self.q_conv, self.k_conv = (
                None if w is None else w.float().contiguous()
                for w in (self.bias, self.q_norm, self.k_norm, self.q_conv, self.k_conv))
        if not spec.plain:
            from .rope import rope_inverse_frequencies

            p = spec.position
            if p.kind not in ("rope", "none"):
                raise ValueError("this attention rotates pairs of features (a rope position "
                                 "spec) or nothing")
            if p.interleaved and p.scaling is not None:
                raise ValueError("frequency scaling goes with split-half pairs here")
            self.rot = p.rotary_dim if p.kind == "rope" else 0
            self.freq = None
            if self.rot:
                self.freq = torch.tensor(rope_inverse_frequencies(p), dtype=torch.float64,
                                         device=runtime.device)
        self.position = build_part("position", spec.position, {}, runtime)
        # a position part may offer the first product and its own work as one call
        self._fused_projection = getattr(self.position, "project_and_apply", None)
        self.scale = spec.scale if spec.scale is not None else spec.head_dim ** -0.5

    def forward(self, x, ctx: StepContext, cache: LayerCache):
        s = self.spec
        if not s.plain:
            return self._forward_general(x, ctx, cache)
        write_heads = 0 if s.shares_kv else s.num_kv_heads
        qkv = None
        if self._fused_projection is not None and not s.shares_kv:
            # queries only, [tokens, heads * head_dim]; keys and values are in the cache
            qkv = self._fused_projection(x, self.w_in, ctx, cache.kv, cache.block_table,
                                         cache.page_size, s.num_heads, write_heads)
        if qkv is None:
            qkv = ops.linear(x, self.w_in, static_weights=True)
            self.position.apply(qkv, ctx, None if s.shares_kv else cache.kv, cache.block_table,
                                cache.page_size, s.num_heads, write_heads)
        out = qkv.new_empty((ctx.num_tokens, s.num_heads * s.head_dim))
        self.attend(qkv, out, ctx, cache)
        return ops.linear(out, self.w_out, static_weights=True)

    def _forward_general(self, x, ctx: StepContext, cache: LayerCache):
        s = self.spec
        qkv = ops.linear(x, self.w_in, out_dtype=torch.float32, static_weights=True)
        conv = None
        if s.conv_taps:
            conv = (self.q_conv, self.k_conv, ctx.qo_indptr, ctx.slots, cache.state)
        q = ops.sink_prepare(qkv, self.bias, self.q_norm, self.k_norm, self.freq, ctx.positions,
                             ctx.cache_pos, ctx.token_req, cache.block_table, cache.kv,
                             s.num_heads, s.num_kv_heads, s.head_dim, s.value_dim, self.rot,
                             cache.page_size, s.qk_norm_eps or 0.0, self.runtime.dtype,
                             conv=conv, value_from_key=s.value_from_key,
                             interleaved=s.position.interleaved and self.rot > 0,
                             norm_whole=s.qk_norm_whole, q_temp=s.q_temp)
        if s.conv_taps > 1:
            ops.conv_state_advance(qkv, (s.num_heads + s.num_kv_heads) * s.head_dim, s.conv_taps,
                                   ctx.qo_indptr, ctx.slots, cache.state, ctx.num_entries)
        gate = qkv[:, qkv.shape[1] - s.num_heads:] if s.head_gate else None
        if s.feature_gate:
            gate = qkv[:, qkv.shape[1] - s.num_heads * s.value_dim:]
        out = ops.sink_attention(q, cache.kv, cache.block_table, ctx.token_req, ctx.cache_pos,
                                 s.num_heads, s.num_kv_heads, s.head_dim, s.value_dim,
                                 cache.page_size, s.window or 0, s.keep_first if s.window else 0,
                                 self.scale, ctx=ctx, gate=gate, softcap=s.softcap,
                                 sink=self.sink)
        return ops.linear(out, self.w_out, static_weights=True)

    def attend(self, qkv, out, ctx: StepContext, cache: LayerCache) -> None:
        """bfloat16 with a head size the tensor-core kernels take: single-token entries
        (they come first in the batch) go to the split-K decode kernel, prompt portions
        to the prefill kernel.  Everything else, float32 included, runs the generic
        kernel."""
        s = self.spec
        if ops.fast_attention_supported(qkv.dtype, s.num_heads, s.num_kv_heads, s.head_dim):
            nd = ctx.num_decode
            if nd:
                ops.paged_decode_attention(
                    qkv, qkv.stride(0), out, cache.kv, cache.block_table, ctx.token_req,
                    ctx.cache_pos, nd, s.num_heads, s.num_kv_heads, s.head_dim,
                    cache.page_size, s.window or 0, self.scale, max(ctx.kv_lens[:nd]),
                    static_keys=True)
            if ctx.num_entries > nd:
                ops.paged_prefill_attention(
                    qkv, qkv.stride(0), out, cache.kv, cache.block_table, ctx.qo_indptr,
                    ctx.kv_len, nd, ctx.num_entries - nd, max(ctx.q_lens[nd:]), s.num_heads,
                    s.num_kv_heads, s.head_dim, cache.page_size, s.window or 0, self.scale)
            return
        ops.paged_attention_generic(
            qkv, qkv.stride(0), out, cache.kv, cache.block_table, ctx.token_req, ctx.cache_pos,
            ctx.num_tokens, s.num_heads, s.num_kv_heads, s.head_dim, cache.page_size,
            s.window or 0, self.scale)


register_part("mixer", "attention", Attention)
