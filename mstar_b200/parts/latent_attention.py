"""Latent attention mixer: softmax attention whose keys and values are up-projections of
one cached latent row per token.

A token leaves ``kv_rank`` normalised latent features c and ``rot_dim`` rotated key features
in its cache row; nothing per head is cached.  The key up-projection is folded into the
query (a_h = W_uk[h]^T q_h, so that q_h . (W_uk[h] c) = a_h . c) and the value up-projection
is applied to the attention's output (sum_j p_j W_uv[h] c_j = W_uv[h] sum_j p_j c_j): the
attention kernel then reads the same rows for every head, in prompts and in decoding alike.
One product gives the queries, the down-projection and the output gate.  Scores,
probabilities and the weighted sum are float; the folded query is kept in float as well.

Options of the spec: queries through a normed latent of their own (the first product then
gives that latent instead of the queries, and a second one the queries), rotary pairs
interleaved or split in halves, a gate per feature or one a head, and a layer without a
down-projection that reads the rows an earlier layer cached (``shares_kv``).
"""
from __future__ import annotations

import torch

from .. import ops
from ..weights.names import ParamSpec
from .base import CacheNeed, KVNeed, LayerCache, Runtime, StepContext
from .registry import register_part


class LatentAttention:
    graph_safe = True       # nothing per-step is read from the host

    @staticmethod
    def _gate_rows(spec) -> int:
        if not spec.gated:
            return 0
        return spec.num_heads if spec.gate_per_head else spec.num_heads * spec.v_dim

    @classmethod
    def param_specs(cls, spec) -> dict:
        h = spec.num_heads
        q_rows = h * (spec.qk_dim + spec.rot_dim)
        # the fused first product: [q or its latent; down-projection; gate]
        rows = spec.q_rank if spec.q_rank is not None else q_rows
        if not spec.shares_kv:
            rows += spec.kv_rank + spec.rot_dim
        rows += cls._gate_rows(spec)
        out = {"in.weight": ParamSpec((rows, spec.hidden_size))}
        if spec.q_rank is not None:
            out["q_norm.weight"] = ParamSpec((spec.q_rank,), role="vector", init="ones")
            out["uq.weight"] = ParamSpec((q_rows, spec.q_rank))
        if not spec.shares_kv:
            out["kv_norm.weight"] = ParamSpec((spec.kv_rank,), role="vector", init="ones")
        out.update({
            "uk.weight": ParamSpec((h * spec.qk_dim, spec.kv_rank)),
            "uv.weight": ParamSpec((h * spec.v_dim, spec.kv_rank)),
            "o.weight": ParamSpec((spec.hidden_size, h * spec.v_dim)),
        })
        return out

    @classmethod
    def cache_need(cls, spec) -> CacheNeed:
        return CacheNeed(kv=KVNeed(num_kv_heads=1, head_dim=spec.kv_rank + spec.rot_dim,
                                   window=spec.window, planes=1))

    def __init__(self, spec, params: dict, runtime: Runtime):
        p = spec.position
        if p.kind != "rope":
            raise ValueError("latent attention rotates the shared key part (a rope position spec)")
        if p.scaling is not None:
            raise ValueError("latent attention has no frequency scaling")
        if p.rotary_dim % 2 or p.rotary_dim > spec.rot_dim:
            raise ValueError(f"rotary_dim {p.rotary_dim} must be even and at most rot_dim "
                             f"{spec.rot_dim}")
        self.spec = spec
        self.runtime = runtime
        h = spec.num_heads
        self.w_in = params["in.weight"]
        self.w_out = params["o.weight"]
        self.norm_weight = None
        if not spec.shares_kv:
            self.norm_weight = params["kv_norm.weight"].float().contiguous()
        self.w_uq = self.q_norm_weight = None
        if spec.q_rank is not None:
            self.w_uq = params["uq.weight"]
            self.q_norm_weight = params["q_norm.weight"].float().contiguous()
        # per head: [rank, qk_dim] rows so that a = q @ uk_t[h]^T, and [v_dim, rank]
        self.uk_t = params["uk.weight"].view(h, spec.qk_dim, spec.kv_rank).transpose(1, 2).contiguous()
        self.uv = params["uv.weight"].view(h, spec.v_dim, spec.kv_rank)
        half = p.rotary_dim // 2
        self.freq = torch.tensor([p.theta ** (-(2.0 * i) / p.rotary_dim) for i in range(half)],
                                 dtype=torch.float64, device=runtime.device)
        self.scale = spec.scale if spec.scale is not None else (spec.qk_dim + spec.rot_dim) ** -0.5

    def forward(self, x, ctx: StepContext, cache: LayerCache):
        s = self.spec
        h, per_head = s.num_heads, s.qk_dim + s.rot_dim
        q_cols = h * per_head
        down = 0 if s.shares_kv else s.kv_rank + s.rot_dim
        fill = dict(positions=ctx.positions, cache_pos=ctx.cache_pos, token_req=ctx.token_req,
                    block_table=cache.block_table, heads=h, qk_dim=s.qk_dim, rot=s.rot_dim,
                    rot_dims=s.position.rotary_dim, rank=s.kv_rank, page_size=cache.page_size,
                    eps=s.norm_eps, interleaved=s.position.interleaved)
        if s.q_rank is None:
            # queries straight from the input: rotate them and fill the cache in one launch
            proj = ops.linear(x, self.w_in, static_weights=True)
            q = proj[:, :q_cols]
            ops.latent_fill(q, None if s.shares_kv else proj[:, q_cols:q_cols + down],
                            self.norm_weight, self.freq, cache=cache.kv, **fill)
            gate = proj[:, q_cols + down:]
        else:
            # queries through a latent: the product's sums stay float up to the norms
            proj = ops.linear(x, self.w_in, out_dtype=torch.float32, static_weights=True)
            lat_q = ops.latent_fill(None, None if s.shares_kv else proj[:, s.q_rank:s.q_rank + down],
                                    self.norm_weight, self.freq, cache=cache.kv,
                                    q_latent=proj[:, :s.q_rank],
                                    q_latent_weight=self.q_norm_weight, **fill)
            q = ops.linear(lat_q, self.w_uq, static_weights=True)
            ops.latent_fill(q, None, None, self.freq, cache=cache.kv, **fill)
            gate = proj[:, s.q_rank + down:]
        q = q.view(-1, h, per_head)
        q_abs = ops.linear_per_head(q[:, :, :s.qk_dim], self.uk_t, out_dtype=torch.float32)
        lat = ops.latent_attention(q_abs, q[:, :, s.qk_dim:], cache.kv, cache.block_table,
                                   ctx.token_req, ctx.cache_pos, h, s.kv_rank, s.rot_dim,
                                   cache.page_size, s.window or 0, self.scale,
                                   max_keys=ctx.max_kv_len, entries=ctx.num_entries)
        if s.gated and s.gate_per_head:
            # one gate a head commutes with the head's value up-projection
            lat = ops.head_gate_mul(lat.view(-1, h * s.kv_rank), gate, h,
                                    out_dtype=self.runtime.dtype).view(-1, h, s.kv_rank)
        else:
            lat = ops.convert(lat, self.runtime.dtype)
        y = ops.linear_per_head(lat, self.uv)
        y = y.view(-1, h * s.v_dim)
        if s.gated and not s.gate_per_head:
            ops.sigmoid_gate_mul(y, gate)
        return ops.linear(y, self.w_out, static_weights=True)


register_part("mixer", "latent_attention", LatentAttention)
