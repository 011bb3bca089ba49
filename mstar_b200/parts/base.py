"""What parts and the step function share: the runtime, the step context, the
residual stream and the description of a mixer's cache needs."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch


@dataclass(frozen=True)
class KVNeed:
    """Keys and values in pages: [pages, planes, num_kv_heads, page_size, head_dim].
    ``window`` None keeps every key; W keeps the last W, and the first ``keep_first`` beside
    them.  ``planes``: 2 for keys and values, 1 for a mixer that keeps one row per token (a
    latent that both are made from).  ``v_head_dim``: not None and other than ``head_dim``
    makes a page [num_kv_heads, page_size, head_dim] keys followed by [num_kv_heads,
    page_size, v_head_dim] values, and the cache tensor [pages, elements of a page]."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    planes: int = 2
    keep_first: int = 0
    v_head_dim: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """Per-request state of fixed size: one ``shape`` tensor per state slot,
    zeroed when a request takes the slot."""

    shape: tuple
    dtype: str = "float32"


@dataclass(frozen=True)
class CacheNeed:
    kv: Optional[KVNeed] = None
    state: Optional[StateNeed] = None


@dataclass
class Runtime:
    """Compute dtype and device of a model instance."""

    dtype: torch.dtype
    device: torch.device


@dataclass
class LayerCache:
    """The cache of one run-order entry, as its mixer sees it."""

    kv: Optional[torch.Tensor] = None           # [pages, planes, kv_heads, page_size, head_dim]
    page_size: int = 0
    block_table: Optional[torch.Tensor] = None  # int32 [entries, width] of the cache's group
    state: Optional[torch.Tensor] = None        # [slots, *shape]


@dataclass
class StepContext:
    """Index arrays of one step on the device (int32) plus host copies.

    Tokens are packed entry after entry.  ``token_req[t]`` is the entry of token
    t, ``positions[t]`` its position id, ``cache_pos[t]`` the index of its key in
    the request's key sequence (kept apart from the position id, as the reference
    keeps position_id_start apart from seq_len, mstar/engine/kv_store.py:112-116).
    """

    num_tokens: int
    num_entries: int
    token_req: torch.Tensor
    positions: torch.Tensor
    cache_pos: torch.Tensor
    qo_indptr: torch.Tensor
    kv_len: torch.Tensor
    slots: torch.Tensor
    # host copies (python lists) for parts that plan on the host
    q_lens: list = field(default_factory=list)
    kv_lens: list = field(default_factory=list)
    host_slots: list = field(default_factory=list)
    max_q_len: int = 0
    max_kv_len: int = 0
    # entries [0, num_decode) bring exactly one token each (tokens [0, num_decode))
    num_decode: int = 0
    # (src, prev) or None: where src[t] >= 0, token t is prev[src[t]], a token that the step
    # before sampled and that only the device holds yet (int32 tensors)
    token_source: Optional[tuple] = None
    extras: dict = field(default_factory=dict)


class ResidualStream:
    """The float residual ``h`` and the not-yet-added output ``delta`` of the last
    part.  Norm parts fold ``h += delta`` into the normalisation that follows, so
    the residual sum is a 32-bit sum and costs no pass of its own.  A delta may be pushed
    with a norm of its own (``post``: a norm part), which is applied to it on its way into
    the residual, together with a multiplier: ``h += scale * post(delta)``."""

    def __init__(self, h: torch.Tensor):
        assert h.dtype == torch.float32
        self.h = h
        self.delta: Optional[torch.Tensor] = None
        self.post = None
        self.post_scale = 1.0
        # set by a block that keeps the residual as several copies (hyper-connections): an
        # object with ``gather(rows)``; ``h`` is then no longer the residual
        self.copies = None

    def gather(self, rows: torch.Tensor) -> torch.Tensor:
        """The float residual of the rows asked for, everything pending added."""
        from .. import ops

        if self.copies is not None:
            return self.copies.gather(rows)
        return ops.gather_add_rows(self.h, self.take_delta(), rows)

    def push(self, delta: torch.Tensor, post=None, scale: float = 1.0) -> None:
        if self.delta is not None:
            raise RuntimeError("a part's output was pushed before the previous one was added")
        if post is None and scale != 1.0:
            raise ValueError("a multiplier goes with a norm on the part's output")
        self.delta = delta
        self.post = post
        self.post_scale = float(scale)

    def take_delta(self) -> Optional[torch.Tensor]:
        """The pending delta as it is to be added.  One that carries a norm of its own is
        added here and now (by that norm part), and nothing is left pending."""
        if self.post is not None:
            self.settle()
        d, self.delta = self.delta, None
        if hasattr(d, "materialize"):           # a part's output that is not computed yet
            d = d.materialize()
        return d

    def take_pending(self):
        """(delta, its own norm part or None), for a norm that folds both in itself."""
        d, post = self.delta, self.post
        self.delta = self.post = None
        return d, post

    def settle(self) -> None:
        """Add a pending delta that carries its own norm into ``h`` now."""
        if self.delta is not None and self.post is not None:
            scale = self.post_scale
            d, post = self.take_pending()
            post.add_normed(self.h, d, scale)

    def rows(self, dtype: torch.dtype) -> torch.Tensor:
        """The residual itself, everything pending added, as rows of ``dtype`` for a sublayer
        that reads it without a norm (the float residual tensor when ``dtype`` is float)."""
        from .. import ops

        if self.delta is not None and self.post is not None:
            scale = self.post_scale
            d, post = self.take_pending()
            return post.add_normed(self.h, d, scale, rows_dtype=dtype)
        if self.delta is not None:
            d = self.take_delta()
            self.h.add_(d.float() if d.dtype != torch.float32 else d)
        return ops.convert(self.h, dtype)
