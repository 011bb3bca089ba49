"""Python entry points of the hand-written kernels.

Each function validates shapes and dtypes, then launches a kernel from
``csrc/`` on the current CUDA stream.  Tensors must live on the GPU; nothing
here computes on the CPU.  Matrix products in bfloat16: this package's
weight-streaming kernels for up to 16 rows, its tcgen05 kernels for the LM head and
for gate/up at prompt size, and the library GEMM (cuBLAS through ``torch.mm``)
elsewhere, as the reference uses for every linear layer
(mstar/model/components/distributed/linear.py:101, 412); the float32 product
is this package's own true-32-bit kernel.
"""
from __future__ import annotations

import os

import torch

from . import lib
from .lib import BF16, F32, KernelError, check

_DT = {torch.float32: F32, torch.bfloat16: BF16}


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"dtype {t.dtype} is not supported (float32 and bfloat16 are)") from None


def _stream() -> int:
    """Handle of the current CUDA stream of the current device (the raw accessors cost a
    tenth of ``torch.cuda.current_stream()``, which matters at some 300 launches a step)."""
    return torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice())


def _need_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("mstar_b200 kernels run on CUDA tensors only; got a "
                              f"{t.device} tensor (there is no CPU path)")


def _ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def embed_rows(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor | None = None,
               source=None, scale: float = 1.0):
    """out[t] = float(table[ids[t]]) * scale; the residual stream is float in both dtypes.
    ``source`` = (src, prev): where src[t] >= 0 the token is prev[src[t]] instead, a token
    that is on the device only (int32 tensors, src as long as ids)."""
    _need_cuda(table, ids)
    assert ids.dtype == torch.int32 and table.dim() == 2 and table.is_contiguous()
    n, (vocab, hidden) = ids.numel(), table.shape
    if out is None:
        out = torch.empty((n, hidden), dtype=torch.float32, device=table.device)
    src = prev = None
    if source is not None:
        src, prev = source
        _need_cuda(src, prev)
        assert src.dtype == torch.int32 and prev.dtype == torch.int32 and src.numel() == n
    check(lib.get("elementwise").mstar_embed_rows(
        table.data_ptr(), _dt(table), ids.data_ptr(), _ptr(src), _ptr(prev), out.data_ptr(), n,
        vocab, hidden, float(scale), _stream()), "embed_rows")
    return out


def scale_softcap(x: torch.Tensor, scale: float = 1.0, cap: float | None = None):
    """In place on float ``x``: x *= scale, then x = cap * tanh(x / cap) if ``cap``."""
    _need_cuda(x)
    assert x.dtype == torch.float32 and x.is_contiguous()
    check(lib.get("elementwise").mstar_scale_softcap(
        x.data_ptr(), x.numel(), float(scale), float(cap or 0.0), _stream()), "scale_softcap")
    return x


def add_rmsnorm(resid: torch.Tensor, delta, weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, weight_offset: float = 0.0, out=None,
                resid_static: bool = False):
    """resid += delta (if given), in place in float; returns rmsnorm(resid)*weight.
    ``resid_static`` promises that the kernel before this one on the stream did not write
    ``resid`` (it wrote ``delta``): the residual is then read while that kernel drains."""
    _need_cuda(resid, delta, weight)
    assert resid.dtype == torch.float32 and resid.dim() == 2 and resid.is_contiguous()
    rows, hidden = resid.shape
    assert weight.numel() == hidden and weight.is_contiguous()
    if delta is not None:
        assert delta.shape == resid.shape and delta.dtype == out_dtype and delta.is_contiguous()
    if out is None:
        out = torch.empty((rows, hidden), dtype=out_dtype, device=resid.device)
    check(lib.get("elementwise").mstar_add_rmsnorm(
        resid.data_ptr(), _ptr(delta), weight.data_ptr(), _dt(weight), out.data_ptr(), _dt(out),
        rows, hidden, float(eps), float(weight_offset), int(resid_static), _stream()),
        "add_rmsnorm")
    return out


def gather_add_rows(resid: torch.Tensor, delta, rows: torch.Tensor):
    """float(resid[rows] + delta[rows]) as a new [len(rows), hidden] tensor."""
    _need_cuda(resid, delta, rows)
    assert resid.dtype == torch.float32 and resid.is_contiguous() and rows.dtype == torch.int32
    hidden = resid.shape[1]
    out = torch.empty((rows.numel(), hidden), dtype=torch.float32, device=resid.device)
    act = _dt(delta) if delta is not None else F32
    if delta is not None:
        assert delta.shape == resid.shape and delta.is_contiguous()
    check(lib.get("elementwise").mstar_gather_add_rows(
        resid.data_ptr(), _ptr(delta), act, rows.data_ptr(), out.data_ptr(), rows.numel(),
        hidden, _stream()), "gather_add_rows")
    return out


GATE_ACTIVATIONS = {"gelu_tanh": 1, "silu": 2}


def silu_mul(gate_up: torch.Tensor, out=None, kind: str = "silu"):
    """act(gate_up[:, :I]) * gate_up[:, I:], act the SiLU or (``kind`` "gelu_tanh") the tanh
    form of gelu."""
    _need_cuda(gate_up)
    if kind not in GATE_ACTIVATIONS:
        raise KernelError(f"gate activation {kind!r} has no kernel (known: "
                          f"{sorted(GATE_ACTIVATIONS)})")
    assert gate_up.dim() == 2 and gate_up.is_contiguous() and gate_up.shape[1] % 2 == 0
    rows, inter = gate_up.shape[0], gate_up.shape[1] // 2
    if out is None:
        out = torch.empty((rows, inter), dtype=gate_up.dtype, device=gate_up.device)
    check(lib.get("elementwise").mstar_silu_mul(
        gate_up.data_ptr(), out.data_ptr(), _dt(gate_up), rows, inter, GATE_ACTIVATIONS[kind],
        _stream()), "silu_mul")
    return out


def bias_act_mul(gate_up: torch.Tensor, bias: torch.Tensor, out_dtype: torch.dtype,
                 kind: str = "silu") -> torch.Tensor:
    """act(gate_up[:, :I] + bias[:I]) * (gate_up[:, I:] + bias[I:]) from the float product
    ``gate_up``; the result has ``out_dtype``."""
    _need_cuda(gate_up, bias)
    if kind not in GATE_ACTIVATIONS:
        raise KernelError(f"gate activation {kind!r} has no kernel (known: "
                          f"{sorted(GATE_ACTIVATIONS)})")
    assert gate_up.dtype == torch.float32 and gate_up.dim() == 2 and gate_up.is_contiguous()
    assert gate_up.shape[1] % 2 == 0 and bias.numel() == gate_up.shape[1] and bias.is_contiguous()
    rows, inter = gate_up.shape[0], gate_up.shape[1] // 2
    out = torch.empty((rows, inter), dtype=out_dtype, device=gate_up.device)
    check(lib.get("elementwise").mstar_bias_act_mul(
        gate_up.data_ptr(), bias.data_ptr(), _dt(bias), out.data_ptr(), _DT[out_dtype], rows,
        inter, GATE_ACTIVATIONS[kind], _stream()), "bias_act_mul")
    return out


def convert(src: torch.Tensor, dtype: torch.dtype):
    _need_cuda(src)
    if src.dtype == dtype:
        return src
    assert src.is_contiguous()
    out = torch.empty(src.shape, dtype=dtype, device=src.device)
    check(lib.get("elementwise").mstar_convert(
        src.data_ptr(), _dt(src), out.data_ptr(), _dt(out), src.numel(), _stream()), "convert")
    return out


def rope_kv_write(qkv: torch.Tensor, positions, cache_pos, token_req, block_table,
                  inv_freq, kv_cache, num_heads: int, num_kv_heads: int, head_dim: int,
                  rotary_dim: int, interleaved: bool, page_size: int) -> None:
    """Rotate queries in place; rotate keys and copy values into their cache pages.

    ``kv_cache``: [pages, 2, kv_heads, page_size, head_dim] or None (queries only).
    ``inv_freq``: float [rotary_dim / 2] or None when rotary_dim == 0."""
    _need_cuda(qkv, positions, cache_pos, token_req, block_table, inv_freq, kv_cache)
    assert qkv.dim() == 2 and qkv.is_contiguous()
    n = qkv.shape[0]
    assert qkv.shape[1] == (num_heads + 2 * num_kv_heads) * head_dim
    assert rotary_dim % 2 == 0 and 0 <= rotary_dim <= head_dim
    if rotary_dim:
        assert inv_freq is not None and inv_freq.dtype == torch.float32
        assert inv_freq.numel() == rotary_dim // 2
    if kv_cache is not None:
        assert kv_cache.dtype == qkv.dtype and kv_cache.is_contiguous()
        assert tuple(kv_cache.shape[1:]) == (2, num_kv_heads, page_size, head_dim)
    check(lib.get("elementwise").mstar_rope_kv_write(
        qkv.data_ptr(), _dt(qkv), positions.data_ptr(), cache_pos.data_ptr(),
        token_req.data_ptr(), block_table.data_ptr(), block_table.stride(0), _ptr(inv_freq),
        _ptr(kv_cache), n, num_heads, num_kv_heads, head_dim, rotary_dim, int(interleaved),
        page_size, _stream()), "rope_kv_write")


def paged_attention_generic(q: torch.Tensor, q_stride: int, out: torch.Tensor, kv_cache,
                            block_table, token_req, cache_pos, num_tokens: int, num_heads: int,
                            num_kv_heads: int, head_dim: int, page_size: int, window: int,
                            scale: float) -> None:
    """Attention of ``num_tokens`` query rows (portions and decoded tokens alike)
    over the paged cache; ``q`` may be a view into the fused qkv buffer with
    ``q_stride`` elements between tokens."""
    _need_cuda(q, out, kv_cache, block_table, token_req, cache_pos)
    assert out.is_contiguous() and kv_cache.is_contiguous()
    code = lib.get("attention_generic").mstar_paged_attention_generic(
        q.data_ptr(), q_stride, out.data_ptr(), kv_cache.data_ptr(), block_table.data_ptr(),
        block_table.stride(0), token_req.data_ptr(), cache_pos.data_ptr(), num_tokens,
        num_heads, num_kv_heads, head_dim, page_size, window, float(scale), _dt(out), _stream())
    if code == -1:
        raise KernelError(
            f"paged attention refuses heads={num_heads}, kv_heads={num_kv_heads}, "
            f"head_dim={head_dim}: it needs head_dim <= 256 and (heads/kv_heads)*head_dim <= 4096")
    check(code, "paged_attention_generic")


FAST_ATTENTION_HEAD_DIMS = (16, 32, 64, 128, 256)

_sm_counts: dict = {}


def num_sms(device=None) -> int:
    """SMs of ``device`` (default: the current CUDA device), asked once per device."""
    index = torch.cuda.current_device() if device is None else (
        torch.device(device).index or 0)
    if index not in _sm_counts:
        _sm_counts[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return _sm_counts[index]


def fast_attention_supported(dtype: torch.dtype, num_heads: int, num_kv_heads: int,
                             head_dim: int) -> bool:
    """Whether the tensor-core attention kernels take this shape (else the generic
    kernel does)."""
    return (dtype == torch.bfloat16 and head_dim in FAST_ATTENTION_HEAD_DIMS
            and num_heads % num_kv_heads == 0 and num_heads // num_kv_heads <= 16)


# CTAs of the decode attention grid per SM that the split of the keys aims for (the kernel
# with one CTA per work item), and CTAs per SM of the persistent ring kernel
DECODE_FILL = 6
RING_CTAS_PER_SM = 2


def decode_split(tokens: int, num_kv_heads: int, max_len: int, ring: bool = False,
                 sms: int | None = None) -> tuple:
    """(chunk, splits) of the keys for split-K decode attention, chunks in whole tiles of 64
    keys.  One CTA per work item (token, kv head, split): enough items to fill the GPU a
    few times over.  Persistent ring kernel: as many items as CTAs are resident or fewer
    (each CTA then streams one item of equal size), of at least 128 keys.  ``sms``: the
    device's SM count (default: asked of the current device)."""
    if sms is None:
        sms = num_sms()
    pairs = max(tokens * num_kv_heads, 1)
    if ring:
        want = max(1, (sms * RING_CTAS_PER_SM) // pairs)
        chunk = max(128, -(-(-(-max_len // want)) // 64) * 64)
    else:
        fill = int(os.environ.get("MSTAR_DECODE_FILL", DECODE_FILL))
        want = max(1, -(-sms * fill // pairs))
        want = min(want, 256)                   # the merge kernel takes up to 256 splits
        chunk = max(64, -(-(-(-max_len // want)) // 64) * 64)
    splits = max(1, -(-max_len // chunk))
    while splits > 256:                         # the merge kernel takes up to 256 splits
        chunk *= 2
        splits = max(1, -(-max_len // chunk))
    return chunk, splits


# page sizes whose caches the TMA kernels take: boxes of min(page, 64) keys
TMA_PAGE_SIZES = (8, 16, 32, 64, 128, 256)

_kv_maps: dict = {}


def kv_tensor_map(kv_cache: torch.Tensor):
    """The TMA tensor map (a 128-byte host buffer) of a cache tensor [pages, 2, kv_heads,
    page_size, head_dim], or None when the TMA kernels do not take its shape."""
    pages, _, nkv, page_size, hd = kv_cache.shape
    key = (kv_cache.data_ptr(), tuple(kv_cache.shape))
    if key not in _kv_maps:
        import ctypes

        buf = ctypes.create_string_buffer(128 + 64)
        addr = (ctypes.addressof(buf) + 63) & ~63          # the driver wants 64-byte alignment
        code = lib.get("attention_decode").mstar_make_kv_tensor_map(
            addr, kv_cache.data_ptr(), pages, nkv, page_size, hd)
        if code == -1:
            _kv_maps[key] = None
        elif code != 0:
            raise KernelError(f"could not make the TMA tensor map of a cache (code {code})")
        else:
            _kv_maps[key] = (buf, addr)
    entry = _kv_maps[key]
    return None if entry is None else entry[1]


def paged_decode_attention(q: torch.Tensor, q_stride: int, out: torch.Tensor, kv_cache,
                           block_table, token_req, cache_pos, tokens: int, num_heads: int,
                           num_kv_heads: int, head_dim: int, page_size: int, window: int,
                           scale: float, max_len: int, static_keys: bool = False) -> None:
    """bfloat16 attention of ``tokens`` single-query rows (token i of q/out/token_req/
    cache_pos); ``max_len`` bounds the keys any of them sees.  ``static_keys`` promises that
    the kernel before this one on the stream wrote nothing that is read here but the queries
    and each token's own key and value (a decode step of the engine: the keys before are from
    earlier steps, the index arrays from before the step's first kernel); the copies of the
    earlier keys then start while that kernel is still draining."""
    _need_cuda(q, out, kv_cache, block_table, token_req, cache_pos)
    assert q.dtype == torch.bfloat16 and kv_cache.dtype == torch.bfloat16
    assert (q_stride * 2) % 16 == 0 and q.data_ptr() % 16 == 0 and out.is_contiguous()
    if window:
        max_len = min(max_len, window)
    kv_map = kv_tensor_map(kv_cache) if not window else None
    ring = kv_map is not None and os.environ.get("MSTAR_DECODE_ATTENTION") != "per_item"
    if not ring and page_size > 64:
        kv_map = None                       # the per-item TMA kernel copies whole pages
    chunk, splits = decode_split(tokens, num_kv_heads, max(max_len, 1), ring=ring,
                                 sms=num_sms(q.device))
    scratch = None
    if splits > 1:
        scratch = torch.empty(tokens * num_heads * splits * (head_dim + 2), dtype=torch.float32,
                              device=q.device)
    if kv_map is not None:
        code = lib.get("attention_decode").mstar_paged_decode_attention_bf16_tma(
            kv_map, q.data_ptr(), q_stride, out.data_ptr(), kv_cache.data_ptr(),
            block_table.data_ptr(), block_table.stride(0), token_req.data_ptr(),
            cache_pos.data_ptr(), tokens, num_heads, num_kv_heads, head_dim, page_size,
            float(scale), chunk, splits, int(static_keys), _ptr(scratch),
            tcgen05_error_word(q.device).data_ptr(), _stream())
        if code == -1:
            raise KernelError("TMA decode attention refuses this shape")
        check(code, "paged_decode_attention_tma")
        if splits > 1:
            lib.add_launches(1)                 # the merge kernel
        return
    code = lib.get("attention_decode").mstar_paged_decode_attention_bf16(
        q.data_ptr(), q_stride, out.data_ptr(), kv_cache.data_ptr(), block_table.data_ptr(),
        block_table.stride(0), token_req.data_ptr(), cache_pos.data_ptr(), tokens, num_heads,
        num_kv_heads, head_dim, page_size, window, float(scale), chunk, splits, _ptr(scratch),
        _stream())
    if code == -1:
        raise KernelError(f"decode attention refuses heads={num_heads}, kv_heads={num_kv_heads}, "
                          f"head_dim={head_dim} (head_dim in {FAST_ATTENTION_HEAD_DIMS}, at most "
                          "16 query heads per kv head)")
    check(code, "paged_decode_attention")
    if splits > 1:
        lib.add_launches(1)                     # the merge kernel


def prefill_attention_kernel(has_kv_map: bool, head_dim: int, page_size: int, group: int = 1) -> str:
    """"tcgen05" or "mma": which prefill attention kernel runs.  The tcgen05 kernel takes
    head_dim 64, 128 or 256, no window, the page sizes of ``TMA_PAGE_SIZES`` and up to 128
    query heads per kv head (``group``), and is the faster one from the shortest portions on;
    MSTAR_PREFILL_ATTENTION=mma selects the other."""
    import os

    takes = (has_kv_map and head_dim in (64, 128, 256) and page_size in TMA_PAGE_SIZES
             and group <= 128)
    if not takes or os.environ.get("MSTAR_PREFILL_ATTENTION") == "mma":
        return "mma"
    return "tcgen05"


def paged_prefill_attention(q: torch.Tensor, q_stride: int, out: torch.Tensor, kv_cache,
                            block_table, qo_indptr, kv_len, first_entry: int, entries: int,
                            max_q_len: int, num_heads: int, num_kv_heads: int, head_dim: int,
                            page_size: int, window: int, scale: float) -> None:
    """bfloat16 attention of the new tokens of batch entries [first_entry, first_entry +
    entries); q and out hold all tokens of the step, indexed through qo_indptr."""
    _need_cuda(q, out, kv_cache, block_table, qo_indptr, kv_len)
    assert q.dtype == torch.bfloat16 and kv_cache.dtype == torch.bfloat16
    assert (q_stride * 2) % 16 == 0 and q.data_ptr() % 16 == 0 and out.is_contiguous()
    kv_map = kv_tensor_map(kv_cache) if not window else None
    if prefill_attention_kernel(kv_map is not None, head_dim, page_size,
                                num_heads // num_kv_heads) == "tcgen05":
        code = lib.get("attention_prefill_tc").mstar_paged_prefill_attention_tc(
            kv_map, q.data_ptr(), q_stride, q.shape[0], out.data_ptr(), block_table.data_ptr(),
            block_table.stride(0), qo_indptr.data_ptr(), kv_len.data_ptr(), first_entry, entries,
            max_q_len, num_heads, num_kv_heads, head_dim, page_size, float(scale),
            tcgen05_error_word(q.device).data_ptr(), _stream())
        if code == -1:
            raise KernelError("tcgen05 prefill attention refuses this shape")
        check(code, "paged_prefill_attention_tc")
        return
    code = lib.get("attention_prefill").mstar_paged_prefill_attention_bf16(
        kv_map or 0, q.data_ptr(), q_stride, out.data_ptr(), kv_cache.data_ptr(),
        block_table.data_ptr(), block_table.stride(0), qo_indptr.data_ptr(), kv_len.data_ptr(),
        first_entry, entries, max_q_len, num_heads, num_kv_heads, head_dim, page_size, window,
        float(scale), tcgen05_error_word(q.device).data_ptr(), _stream())
    if code == -1:
        raise KernelError(f"prefill attention refuses heads={num_heads}, kv_heads={num_kv_heads}, "
                          f"head_dim={head_dim} (head_dim in {FAST_ATTENTION_HEAD_DIMS})")
    check(code, "paged_prefill_attention")


def sgemm_nt(a: torch.Tensor, w: torch.Tensor, out=None):
    """a[M,K] @ w[N,K]^T in true float32 (FMA, no tensor-core reduced precision)."""
    _need_cuda(a, w)
    assert a.dtype == torch.float32 and w.dtype == torch.float32
    assert a.dim() == 2 and w.dim() == 2 and a.shape[1] == w.shape[1]
    assert a.stride(1) == 1 and w.stride(1) == 1
    m, k = a.shape
    n = w.shape[0]
    if out is None:
        out = torch.empty((m, n), dtype=torch.float32, device=a.device)
    assert out.stride(1) == 1
    check(lib.get("gemm_f32").mstar_sgemm_nt(
        a.data_ptr(), w.data_ptr(), out.data_ptr(), m, n, k, a.stride(0), w.stride(0),
        out.stride(0), _stream()), "sgemm_nt")
    return out


# Rows up to which the weight-streaming kernel is used (it takes up to 16); beyond, the
# library GEMM.
SMALL_M = 16


def _smallm_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and 0 < x.shape[0] <= SMALL_M
            and x.shape[1] % 32 == 0 and x.stride(1) == 1 and w.stride(1) == 1
            and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def _gemm_smallm(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype, gated,
                 static_weights: bool = False):
    """``gated``: False or 0 for the plain product; True or 1 gates by the SiLU, 2 by the tanh
    form of gelu."""
    m, k = x.shape
    n = w.shape[0]
    out = torch.empty((m, n // 2 if gated else n), dtype=out_dtype, device=x.device)
    code = lib.get("gemm_smallm_bulk").mstar_gemm_smallm_bulk_bf16(
        x.data_ptr(), w.data_ptr(), out.data_ptr(), m, n, k, x.stride(0), w.stride(0),
        out.stride(0), int(gated), _dt(out), int(static_weights),
        tcgen05_error_word(x.device).data_ptr(), _stream())
    if code == -1:
        raise KernelError(f"small-M GEMM refuses M={m}, N={n}, K={k}")
    check(code, "gemm_smallm_bulk")
    return out


# Rows up to which the swapped-operand tcgen05 kernel is used (tokens are the MMA's N
# dimension: 32, 64 or 128), the rows of W to one of its tiles, and the tiles per SM from
# which on it is used: each CTA takes one tile and all of K, so only a matrix of many tiles
# (a vocabulary-wide head) fills the GPU several times over; with few tiles the library's
# cut along K wins.
SKINNY_MAX = 128
SKINNY_ROWS = 128
SKINNY_TILES_PER_SM = 4


def _skinny_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the product of ``SMALL_M`` < M <= ``SKINNY_MAX`` bfloat16 rows goes to the
    swapped-operand tcgen05 kernel (MSTAR_SKINNY=0: nowhere, 1: for every width)."""
    if not (SMALL_M < x.shape[0] <= SKINNY_MAX and _tc_ok(x, w)):
        return False
    forced = os.environ.get("MSTAR_SKINNY")
    if forced is not None:
        return forced != "0"
    return -(-w.shape[0] // SKINNY_ROWS) >= SKINNY_TILES_PER_SM * num_sms(x.device)


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None,
                static_weights: bool = False):
    """x[M,K] @ w[N,K]^T for up to 128 bfloat16 rows on the tcgen05 tensor cores with the
    operands swapped (rows of W are the MMA's M dimension, the tokens its N dimension)."""
    _need_cuda(x, w)
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    assert x.stride(1) == 1 and w.stride(1) == 1 and x.shape[1] == w.shape[1]
    m, k = x.shape
    n = w.shape[0]
    out_dtype = out_dtype or torch.bfloat16
    out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    code = lib.get("gemm_skinny").mstar_gemm_skinny_bf16(
        x.data_ptr(), w.data_ptr(), out.data_ptr(), m, n, k, x.stride(0), w.stride(0),
        out.stride(0), _dt(out), int(static_weights),
        tcgen05_error_word(x.device).data_ptr(), _stream())
    if code == -1:
        raise KernelError(f"skinny GEMM refuses M={m}, N={n}, K={k} (at most {SKINNY_MAX} rows, "
                          "K and row strides multiples of 8, operands 16-byte aligned)")
    if code in (-3, -4):
        raise KernelError(f"skinny GEMM could not make its TMA tensor map (code {code})")
    check(code, "gemm_skinny")
    return out


def qkv_rope_write(x: torch.Tensor, w_qkv: torch.Tensor, positions, cache_pos, token_req,
                   block_table, inv_freq, kv_cache, num_heads: int, num_kv_heads: int,
                   head_dim: int, page_size: int, static_weights: bool = False):
    """For few bfloat16 rows (decoded tokens): the product x Wqkv^T, the split-half rotary
    encoding of q and k over the whole head, and the write of k and v into their cache
    pages, as one kernel.  Returns q [M, num_heads * head_dim], rotated; or None when this
    form does not apply (more than ``SMALL_M`` rows, another dtype, no cache to write, or
    MSTAR_FUSED_ROPE=0), and the caller runs ``linear`` and ``rope_kv_write`` instead."""
    if (kv_cache is None or inv_freq is None or not _smallm_ok(x, w_qkv)
            or kv_cache.dtype != torch.bfloat16 or head_dim % 16
            or inv_freq.numel() != head_dim // 2
            or w_qkv.shape[0] != (num_heads + 2 * num_kv_heads) * head_dim
            or os.environ.get("MSTAR_FUSED_ROPE") == "0"):
        return None
    _need_cuda(x, w_qkv, positions, cache_pos, token_req, block_table, inv_freq, kv_cache)
    assert kv_cache.is_contiguous() and inv_freq.dtype == torch.float32
    assert tuple(kv_cache.shape[1:]) == (2, num_kv_heads, page_size, head_dim)
    m, k = x.shape
    q = torch.empty((m, num_heads * head_dim), dtype=torch.bfloat16, device=x.device)
    code = lib.get("gemm_smallm_bulk").mstar_qkv_rope_write_bulk_bf16(
        x.data_ptr(), w_qkv.data_ptr(), q.data_ptr(), m, k, x.stride(0), w_qkv.stride(0),
        q.stride(0), positions.data_ptr(), cache_pos.data_ptr(), token_req.data_ptr(),
        block_table.data_ptr(), block_table.stride(0), inv_freq.data_ptr(), kv_cache.data_ptr(),
        num_heads, num_kv_heads, head_dim, page_size, int(static_weights),
        tcgen05_error_word(x.device).data_ptr(), _stream())
    if code == -1:
        raise KernelError(f"fused qkv/rotary product refuses M={m}, K={k}, heads={num_heads}, "
                          f"kv_heads={num_kv_heads}, head_dim={head_dim}")
    check(code, "qkv_rope_write")
    return q


_tc_error_words: dict = {}


def tcgen05_error_word(device) -> torch.Tensor:
    """Device int32 that a kernel with bounded mbarrier waits sets when one of them ran out:
    1-3 tcgen05 GEMM (producer, MMA issuer, epilogue), 4 decode attention copies, 6-12 tcgen05
    prefill attention, 13-14 bulk-copy small-M GEMM, 15-17 swapped-operand tcgen05 GEMM; zero
    otherwise."""
    key = torch.device(device).index or 0
    if key not in _tc_error_words:
        _tc_error_words[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _tc_error_words[key]


WAIT_CODES = {
    1: "tcgen05 GEMM: the producer waited for a free operand stage",
    2: "tcgen05 GEMM: the MMA issuer waited for operand tiles",
    3: "tcgen05 GEMM: the epilogue waited for an accumulator",
    4: "decode attention: a wait for a key/value tile",
    5: "attention: a wait for the query tile or a key/value tile copied by TMA",
    13: "bulk-copy small-M GEMM: the producer waited for a free stage",
    14: "bulk-copy small-M GEMM: a consumer waited for weights",
}
WAIT_CODES.update({15: "swapped-operand tcgen05 GEMM: the producer waited for a free stage",
                   16: "swapped-operand tcgen05 GEMM: the MMA issuer waited for operand tiles",
                   17: "swapped-operand tcgen05 GEMM: the epilogue waited for the accumulator"})
WAIT_CODES.update({c: "tcgen05 prefill attention: a wait on one of its barriers ran out"
                   for c in range(6, 13)})


def raise_on_wait_code(code: int) -> None:
    """``code``: a value read from ``tcgen05_error_word``.  Non-zero means that a bounded
    wait inside a kernel ran out and the kernel returned with partial output, so whatever
    was computed since the word was last zero must not be used."""
    code = int(code)
    if code == 0:
        return
    what = WAIT_CODES.get(code, "an unknown kernel")
    raise KernelError(f"a kernel gave up a bounded wait (code {code}: {what}); the results "
                      "of the steps since the last check are not valid")


def check_error_word(device) -> None:
    """Read the device's error word (this waits for the work queued so far), zero it if it
    is set, and raise ``KernelError`` naming the code.  The engine's entry points call this
    (or read the word along with a step's results) before they hand results out."""
    word = tcgen05_error_word(device)
    code = int(word.item())
    if code:
        word.zero_()
        raise_on_wait_code(code)


def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None,
                 bn: int = 256):
    """x[M,K] @ w[N,K]^T on the tcgen05 tensor cores (TMA operand tiles, TMEM
    accumulator).  bfloat16 operands, K and the row strides multiples of 8."""
    _need_cuda(x, w)
    out_dtype = out_dtype or torch.bfloat16
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    assert x.dim() == 2 and w.dim() == 2 and x.shape[1] == w.shape[1]
    assert x.stride(1) == 1 and w.stride(1) == 1
    m, k = x.shape
    n = w.shape[0]
    out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    code = lib.get("gemm_tcgen05").mstar_gemm_tcgen05_bf16(
        x.data_ptr(), w.data_ptr(), out.data_ptr(), m, n, k, x.stride(0), w.stride(0),
        out.stride(0), _dt(out), bn, tcgen05_error_word(x.device).data_ptr(), _stream())
    if code == -1:
        raise KernelError(f"tcgen05 GEMM refuses M={m}, N={n}, K={k} (K and row strides must be "
                          "multiples of 8, operands 16-byte aligned)")
    if code in (-3, -4):
        raise KernelError(f"tcgen05 GEMM could not make its TMA tensor map (code {code})")
    check(code, "gemm_tcgen05")
    return out


def gemm_tcgen05_gated(x: torch.Tensor, w_gate_up: torch.Tensor, kind: str = "silu"):
    """act(x Wg^T) * (x Wu^T) for the fused [Wg; Wu] on pairs of CTAs (cta_group::2), the
    activation (``kind``: "silu" or "gelu_tanh") applied in the epilogue straight from tensor
    memory."""
    assert kind in ("silu", "gelu_tanh")
    _need_cuda(x, w_gate_up)
    assert x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16
    assert x.stride(1) == 1 and w_gate_up.stride(1) == 1 and x.shape[1] == w_gate_up.shape[1]
    m, k = x.shape
    n = w_gate_up.shape[0]
    out = torch.empty((m, n // 2), dtype=torch.bfloat16, device=x.device)
    code = lib.get("gemm_tcgen05").mstar_gemm_tcgen05_gated_bf16(
        x.data_ptr(), w_gate_up.data_ptr(), out.data_ptr(), m, n, k, x.stride(0),
        w_gate_up.stride(0), out.stride(0), tcgen05_error_word(x.device).data_ptr(),
        0 if kind == "silu" else 1, _stream())
    if code == -1:
        raise KernelError(f"gated tcgen05 GEMM refuses M={m}, N={n}, K={k}")
    if code in (-3, -4):
        raise KernelError(f"tcgen05 GEMM could not make its TMA tensor map (code {code})")
    check(code, "gemm_tcgen05_gated")
    return out


def _tc_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[1] % 8 == 0
            and x.stride(1) == 1 and w.stride(1) == 1 and x.stride(0) % 8 == 0
            and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def tcgen05_tile(m: int, n: int, sms: int | None = None) -> int | None:
    """Which tcgen05 kernel takes an [m, K] x [n, K]^T product of more than ``SKINNY_MAX``
    rows, or None for the library GEMM: 256 = lone CTAs with 128 x 256 tiles, 1024 =
    persistent CTA pairs with 256 x 256 tiles (512: the same pairs, one tile each).
    The hand-written kernels are used where their tiles fill the GPU: up to 256 rows when
    there is a 128 x 256 tile or more for every SM (a vocabulary-wide head), beyond when the
    256 x 256 tiles make three waves or more over the CTA pairs (below, the library's finer
    tiles win: measured at 96 to 160 tiles on 74 pairs).
    ``MSTAR_GEMM=tcgen05`` forces them everywhere, ``MSTAR_GEMM=library`` nowhere."""
    forced = os.environ.get("MSTAR_GEMM", "")
    if forced == "library":
        return None
    if sms is None:
        sms = num_sms()
    if m <= 256:
        if -(-n // 256) >= sms:
            return 256
    elif -(-m // 256) * -(-n // 256) >= 3 * (sms // 2):
        return 1024
    if forced == "tcgen05":
        return 1024 if m > 128 else 256
    return None


def linear(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None,
           static_weights: bool = False):
    """x[M,K] @ w[N,K]^T.  bfloat16: this package's weight-streaming kernel for at most
    ``SMALL_M`` rows, its swapped-operand tcgen05 kernel up to ``SKINNY_MAX`` rows, its
    tiled tcgen05 kernels where ``tcgen05_tile`` says so, else the library GEMM; anything
    involving a float32 operand runs in true float32.  ``static_weights`` promises that no
    kernel earlier on the stream writes ``w`` (model parameters): the kernels for few rows
    then start their weight copies while the kernel before them is still draining."""
    bf16 = x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.is_cuda and w.is_cuda
    m, n = x.shape[0], w.shape[0]
    if bf16 and out_dtype is None and m > SKINNY_MAX and tcgen05_tile(m, n) is None:
        # the common case of a prompt portion on a narrow projection, decided first: this
        # function runs a hundred times in a step that the host has to get launched
        return torch.mm(x, w.t())
    _need_cuda(x, w)
    out_dtype = out_dtype or x.dtype
    if out_dtype in (torch.bfloat16, torch.float32) and _smallm_ok(x, w):
        return _gemm_smallm(x, w, out_dtype, gated=False, static_weights=static_weights)
    if out_dtype in (torch.bfloat16, torch.float32) and _skinny_ok(x, w):
        return gemm_skinny(x, w, out_dtype, static_weights=static_weights)
    if out_dtype in (torch.bfloat16, torch.float32) and _tc_ok(x, w):
        tile = tcgen05_tile(x.shape[0], w.shape[0])
        if tile is not None:
            return gemm_tcgen05(x, w, out_dtype, tile)
    if x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        if out_dtype == torch.float32:
            try:
                return torch.mm(x, w.t(), out_dtype=torch.float32)
            except (TypeError, RuntimeError):
                return torch.mm(x, w.t()).float()
        return torch.mm(x, w.t())
    xf = convert(x, torch.float32)
    wf = convert(w, torch.float32)
    y = sgemm_nt(xf, wf)
    return convert(y, out_dtype)


def linear_act(x: torch.Tensor, w: torch.Tensor, kind: str, static_weights: bool = False):
    """act(x W^T) for a feed-forward without a gate (``kind``: see ``ACTIVATIONS``): one kernel
    for few bfloat16 rows and the square of relu (MSTAR_FUSED_ACT=0: never), else the product
    followed by the activation kernel."""
    _need_cuda(x, w)
    if (kind == "relu2" and _smallm_ok(x, w) and os.environ.get("MSTAR_FUSED_ACT") != "0"):
        m, k = x.shape
        n = w.shape[0]
        out = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
        code = lib.get("gemm_smallm_bulk").mstar_gemm_smallm_bulk_relu2_bf16(
            x.data_ptr(), w.data_ptr(), out.data_ptr(), m, n, k, x.stride(0), w.stride(0),
            out.stride(0), int(static_weights), tcgen05_error_word(x.device).data_ptr(), _stream())
        if code == -1:
            raise KernelError(f"small-M GEMM refuses M={m}, N={n}, K={k}")
        check(code, "gemm_smallm_bulk_relu2")
        return out
    return activation(linear(x, w, static_weights=static_weights), kind)


def gated_up(x: torch.Tensor, w_gate_up: torch.Tensor, static_weights: bool = False,
             kind: str = "silu"):
    """act(x Wg^T) * (x Wu^T) for the fused matrix [Wg; Wu], act the SiLU or (``kind``
    "gelu_tanh") the tanh form of gelu: one kernel for bfloat16 rows whose shapes the small-M
    or the tcgen05 kernel takes (MSTAR_FUSED_ACT=0: never for the gelu), else the product
    followed by the activation-multiply kernel."""
    _need_cuda(x, w_gate_up)
    if kind == "silu" or (kind == "gelu_tanh" and os.environ.get("MSTAR_FUSED_ACT") != "0"):
        if _smallm_ok(x, w_gate_up) and w_gate_up.shape[0] % 2 == 0:
            return _gemm_smallm(x, w_gate_up, torch.bfloat16, gated=1 if kind == "silu" else 2,
                                static_weights=static_weights)
        if (_tc_ok(x, w_gate_up) and w_gate_up.shape[0] % 16 == 0
                and tcgen05_tile(x.shape[0], w_gate_up.shape[0]) is not None):
            return gemm_tcgen05_gated(x, w_gate_up, kind)
    return silu_mul(linear(x, w_gate_up, static_weights=static_weights), kind=kind)


_argmax_scratch: dict = {}


def _argmax_buffers(device, rows: int):
    """Zeroed scratch of the argmax kernel (a 64-bit key and a counter per row); the kernel
    leaves it zeroed.  One per device: launches that share it run on one stream."""
    key = torch.device(device).index or 0
    have = _argmax_scratch.get(key)
    if have is None or have[1].numel() < rows:
        n = max(rows, 1024)
        have = _argmax_scratch[key] = (torch.zeros(n, dtype=torch.int64, device=device),
                                       torch.zeros(n, dtype=torch.int32, device=device))
    return have


def argmax(logits: torch.Tensor):
    _need_cuda(logits)
    assert logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1
    rows, vocab = logits.shape
    out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    best, arrived = _argmax_buffers(logits.device, rows)
    check(lib.get("sampling").mstar_argmax(
        logits.data_ptr(), logits.stride(0), rows, vocab, out.data_ptr(), best.data_ptr(),
        arrived.data_ptr(), _stream()), "argmax")
    return out


def sample(logits: torch.Tensor, temperature, top_k=None, top_p=None, penalty=None,
           seen_mask=None, seen_rows=None, seed=None, offset=None):
    """One token per row.  Per-row tensors: temperature float32, top_k int32,
    top_p float32, penalty float32, seed/offset int64; ``seen_mask`` uint8
    [slots, vocab] with ``seen_rows`` int32 naming each row's slot (or -1)."""
    _need_cuda(logits, temperature, top_k, top_p, penalty, seen_mask, seen_rows, seed, offset)
    assert logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1
    rows, vocab = logits.shape
    assert temperature.dtype == torch.float32 and temperature.numel() == rows
    for t, dt in ((top_k, torch.int32), (top_p, torch.float32), (penalty, torch.float32),
                  (seen_rows, torch.int32), (seed, torch.int64), (offset, torch.int64)):
        assert t is None or (t.dtype == dt and t.numel() == rows)
    if seen_mask is not None:
        assert seen_mask.dtype == torch.uint8 and seen_mask.shape[1] == vocab
        assert seen_mask.is_contiguous()
    out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    check(lib.get("sampling").mstar_sample(
        logits.data_ptr(), logits.stride(0), rows, vocab, temperature.data_ptr(), _ptr(top_k),
        _ptr(top_p), _ptr(penalty), _ptr(seen_mask), _ptr(seen_rows), _ptr(seed), _ptr(offset),
        out.data_ptr(), _stream()), "sample")
    return out


# ------------------------------------------------------------------ sandwich norms
def add_postnorm_rmsnorm(resid: torch.Tensor, delta: torch.Tensor, post_weight: torch.Tensor,
                         post_eps: float, post_offset: float, weight=None, eps: float = 0.0,
                         weight_offset: float = 0.0, out_dtype: torch.dtype | None = None,
                         post_scale: float = 1.0, plain_out: bool = False):
    """resid += post_scale * rms(delta) * (post_weight + post_offset), in place in float; with
    ``weight``, returns rms(resid) * (weight + weight_offset) in ``out_dtype``; with
    ``plain_out`` (and no weight), returns the new residual itself in ``out_dtype`` (the
    residual tensor when that is float); else None.  ``post_weight`` is a float vector;
    ``delta`` is float or of ``out_dtype``."""
    if isinstance(delta, MeanOfNorms):
        # the mean of two normed branches that nobody has computed yet: one kernel does it
        # together with this norm and the sum, where it has a form for the case
        fused = delta.fused_postnorm(resid, post_weight, post_eps, post_offset, post_scale,
                                     weight, out_dtype, plain_out)
        if fused is not NotImplemented:
            return fused
        delta = delta.materialize()
    _need_cuda(resid, delta, post_weight, weight)
    assert resid.dtype == torch.float32 and resid.dim() == 2 and resid.is_contiguous()
    assert delta.shape == resid.shape and delta.is_contiguous()
    assert post_weight.dtype == torch.float32 and post_weight.numel() == resid.shape[1]
    rows, hidden = resid.shape
    out = None
    out_dtype = out_dtype or delta.dtype
    assert delta.dtype in (out_dtype, torch.float32)
    if weight is not None:
        assert weight.numel() == hidden and weight.is_contiguous()
        out = torch.empty((rows, hidden), dtype=out_dtype, device=resid.device)
    elif plain_out and out_dtype != torch.float32:
        out = torch.empty((rows, hidden), dtype=out_dtype, device=resid.device)
    code = lib.get("elementwise").mstar_add_postnorm_rmsnorm(
        resid.data_ptr(), delta.data_ptr(), _dt(delta), post_weight.data_ptr(), float(post_eps),
        float(post_offset), float(post_scale), _ptr(weight),
        _dt(weight) if weight is not None else F32, _ptr(out), _DT[out_dtype], rows, hidden,
        float(eps), float(weight_offset), _stream())
    if code == -1:
        raise KernelError(f"post-norm kernel refuses a width of {hidden}")
    check(code, "add_postnorm_rmsnorm")
    if plain_out and weight is None and out is None:
        return resid
    return out


def mean_of_norms(branches, weights, eps: float) -> torch.Tensor:
    """float [rows, hidden]: the mean over the branches of rms(x_b) * w_b.  ``branches``: up
    to four [rows, hidden] tensors of one dtype; ``weights``: float vectors."""
    n = len(branches)
    assert 1 <= n <= 4 and len(weights) == n
    _need_cuda(*branches, *weights)
    rows, hidden = branches[0].shape
    for x, w in zip(branches, weights):
        assert x.shape == (rows, hidden) and x.is_contiguous() and x.dtype == branches[0].dtype
        assert w.dtype == torch.float32 and w.numel() == hidden
    out = torch.empty((rows, hidden), dtype=torch.float32, device=branches[0].device)
    xs = [b.data_ptr() for b in branches] + [0] * (4 - n)
    ws = [w.data_ptr() for w in weights] + [0] * (4 - n)
    check(lib.get("elementwise").mstar_mean_of_norms(
        *xs, *ws, n, out.data_ptr(), _dt(branches[0]), rows, hidden, float(eps), _stream()),
        "mean_of_norms")
    return out


class MeanOfNorms:
    """The mean of normed branch outputs, not computed yet: ``materialize()`` runs
    ``mean_of_norms``; a norm that is to add it to the residual may take the two steps as one
    kernel (``add_postnorm_rmsnorm`` does for two branches)."""

    def __init__(self, branches, weights, eps: float):
        self.branches, self.weights, self.eps = list(branches), list(weights), float(eps)
        self.shape, self.dtype = branches[0].shape, torch.float32

    def materialize(self) -> torch.Tensor:
        return mean_of_norms(self.branches, self.weights, self.eps)

    def fused_postnorm(self, resid, post_weight, post_eps, post_offset, post_scale, weight,
                       out_dtype, plain_out):
        x0 = self.branches[0]
        hidden = resid.shape[1]
        if (len(self.branches) != 2 or weight is not None or hidden > 6144
                or os.environ.get("MSTAR_FUSED_MEAN") == "0"):
            return NotImplemented
        out_dtype = out_dtype or x0.dtype
        if out_dtype != x0.dtype:
            return NotImplemented
        _need_cuda(resid, *self.branches, *self.weights, post_weight)
        assert resid.dtype == torch.float32 and resid.is_contiguous() and resid.shape == x0.shape
        assert post_weight.dtype == torch.float32 and post_weight.numel() == hidden
        for x, w in zip(self.branches, self.weights):
            assert x.shape == x0.shape and x.dtype == x0.dtype and x.is_contiguous()
            assert w.dtype == torch.float32 and w.numel() == hidden
        out = None
        if plain_out and out_dtype != torch.float32:
            out = torch.empty(resid.shape, dtype=out_dtype, device=resid.device)
        check(lib.get("elementwise").mstar_mean2_postnorm(
            resid.data_ptr(), x0.data_ptr(), self.branches[1].data_ptr(),
            self.weights[0].data_ptr(), self.weights[1].data_ptr(), self.eps,
            post_weight.data_ptr(), float(post_eps), float(post_offset), float(post_scale),
            _ptr(out), _dt(x0), resid.shape[0], hidden, _stream()), "mean2_postnorm")
        if plain_out and out is None:
            return resid
        return out


ACTIVATIONS = {"relu2": 0, "gelu_tanh": 1, "silu": 2}


def activation(x: torch.Tensor, kind: str, inplace: bool = True) -> torch.Tensor:
    """relu(x)^2, gelu (tanh form) or silu, elementwise."""
    _need_cuda(x)
    assert x.is_contiguous()
    if kind not in ACTIVATIONS:
        raise KernelError(f"activation {kind!r} has no kernel (known: {sorted(ACTIVATIONS)})")
    out = x if inplace else torch.empty_like(x)
    check(lib.get("elementwise").mstar_activation(
        x.data_ptr(), out.data_ptr(), _dt(x), x.numel(), ACTIVATIONS[kind], _stream()),
        "activation")
    return out


def sigmoid_gate_mul(y: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """In place: y *= sigmoid(gate).  ``gate`` may be a column view of a wider product."""
    _need_cuda(y, gate)
    assert y.dim() == 2 and y.is_contiguous() and gate.shape == y.shape and gate.stride(1) == 1
    assert gate.dtype == y.dtype
    check(lib.get("elementwise").mstar_sigmoid_gate_mul(
        y.data_ptr(), gate.data_ptr(), _dt(y), y.shape[0], y.shape[1], gate.stride(0), _stream()),
        "sigmoid_gate_mul")
    return y


def head_gate_mul(y: torch.Tensor, gate: torch.Tensor, heads: int,
                  out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """y[t, h, :] * sigmoid(gate[t, h]): one gate a head.  ``y``: [tokens, heads * dim]
    contiguous (float or bfloat16), ``gate``: [tokens, heads], a column view of a wider product
    (float or bfloat16).  In place when ``out_dtype`` is y's own type or None."""
    _need_cuda(y, gate)
    assert y.dim() == 2 and y.is_contiguous() and y.shape[1] % heads == 0
    assert tuple(gate.shape) == (y.shape[0], heads) and gate.stride(1) == 1
    out_dtype = out_dtype or y.dtype
    out = y if out_dtype == y.dtype else torch.empty(y.shape, dtype=out_dtype, device=y.device)
    check(lib.get("elementwise").mstar_head_gate_mul(
        y.data_ptr(), _dt(y), out.data_ptr(), _dt(out), gate.data_ptr(), _dt(gate), gate.stride(0),
        y.shape[0], heads, y.shape[1] // heads, _stream()), "head_gate_mul")
    return out


# ------------------------------------------------------------------ matrix memory
def matrix_memory_state_size(heads: int, dim: int, vdim: int) -> int:
    """Floats of one request's state: S^T [heads, vdim, dim], n [heads, dim], m [heads]."""
    return heads * (dim * vdim + dim + 1)


def matrix_memory_scan(proj: torch.Tensor, gates: torch.Tensor, bias: torch.Tensor, qo_indptr,
                       slots, state: torch.Tensor, entries: int, heads: int, dim: int, vdim: int,
                       cap: float, q_scale: float, floor: float) -> torch.Tensor:
    """The mLSTM recurrence over the tokens of ``entries`` batch entries, each continuing
    the state in its slot (updated in place).  ``proj``: [tokens, >= 2*heads*dim + heads*vdim]
    with q, k, v side by side; ``gates``: float [tokens, 2*heads] pre-activations (input gates
    first), ``bias`` float [2*heads].  Returns float [tokens, heads*vdim]."""
    _need_cuda(proj, gates, bias, qo_indptr, slots, state)
    assert proj.dim() == 2 and proj.stride(1) == 1
    assert gates.dtype == torch.float32 and gates.is_contiguous() and gates.shape[1] == 2 * heads
    assert bias.dtype == torch.float32 and bias.numel() == 2 * heads
    assert state.dtype == torch.float32 and state.dim() == 2 and state.is_contiguous()
    tokens = proj.shape[0]
    out = torch.empty((tokens, heads * vdim), dtype=torch.float32, device=proj.device)
    code = lib.get("matrix_memory").mstar_matrix_memory_scan(
        proj.data_ptr(), _dt(proj), proj.stride(0), heads * dim, 2 * heads * dim, gates.data_ptr(),
        bias.data_ptr(), qo_indptr.data_ptr(), slots.data_ptr(), state.data_ptr(),
        state.stride(0), out.data_ptr(), entries, heads, dim, vdim, float(cap), float(q_scale),
        float(floor), _stream())
    if code == -1:
        raise KernelError(f"matrix-memory scan refuses heads={heads}, dim={dim}, vdim={vdim} "
                          "(dim at most 512)")
    check(code, "matrix_memory_scan")
    return out


def head_norm_gate(o: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, heads: int,
                   vdim: int, eps: float, out_dtype: torch.dtype) -> torch.Tensor:
    """o / rms(o per head) * weight * sigmoid(gate): float ``o`` [tokens, heads*vdim], ``gate``
    a column view in ``out_dtype``, float ``weight`` [heads*vdim]."""
    _need_cuda(o, gate, weight)
    assert o.dtype == torch.float32 and o.is_contiguous() and weight.dtype == torch.float32
    assert gate.dtype == out_dtype and gate.stride(1) == 1 and gate.shape == o.shape
    out = torch.empty(o.shape, dtype=out_dtype, device=o.device)
    check(lib.get("matrix_memory").mstar_head_norm_gate(
        o.data_ptr(), gate.data_ptr(), gate.stride(0), weight.data_ptr(), out.data_ptr(), _dt(out),
        o.shape[0], heads, vdim, float(eps), _stream()), "head_norm_gate")
    return out


# ------------------------------------------------------------------ latent attention
def latent_fill(q, dkv, norm_weight, freq: torch.Tensor, positions, cache_pos, token_req,
                block_table, cache, heads: int, qk_dim: int, rot: int, rot_dims: int, rank: int,
                page_size: int, eps: float, interleaved: bool = True, q_latent=None,
                q_latent_weight=None):
    """The elementwise work around a latent attention's products, one launch; each job is
    left out when its tensor is None.

    ``dkv`` [tokens, rank + rot] (a column view; float or the cache's type): the latent part
    is RMS-normed with ``norm_weight`` (float [rank]), the first ``rot_dims`` key features are
    rotated, and the row goes into the token's slot of ``cache`` [pages, 1, 1, page_size,
    rank + rot].  ``q`` [tokens, heads * (qk_dim + rot)] (the cache's type; a column view):
    the rotated part of every head is rotated in place.  ``q_latent`` [tokens, q_rank] (a
    column view, same type as ``dkv``): RMS-normed with ``q_latent_weight`` (float) into new
    rows of the cache's type, which are returned.  Pairs are (2i, 2i+1) when ``interleaved``,
    else (i, i + rot_dims/2); ``freq``: float64 [rot_dims / 2]."""
    _need_cuda(q, dkv, norm_weight, freq, positions, cache_pos, token_req, block_table, cache,
               q_latent, q_latent_weight)
    assert freq.dtype == torch.float64 and freq.numel() == rot_dims // 2
    first = next(t for t in (q, dkv, q_latent) if t is not None)
    tokens = first.shape[0]
    act = q.dtype if q is not None else cache.dtype
    ins = [t for t in (dkv, q_latent) if t is not None]
    in_dtype = ins[0].dtype if ins else act
    assert all(t.dtype == in_dtype and t.dim() == 2 and t.stride(1) == 1 for t in ins)
    if q is not None:
        assert q.dim() == 2 and q.stride(1) == 1 and q.shape[1] == heads * (qk_dim + rot)
    if dkv is not None:
        assert cache.dtype == act and dkv.shape[1] == rank + rot
        assert cache.is_contiguous() and tuple(cache.shape[1:]) == (1, 1, page_size, rank + rot)
        assert norm_weight.dtype == torch.float32 and norm_weight.numel() == rank
    out = None
    q_rank = 0
    if q_latent is not None:
        q_rank = q_latent.shape[1]
        assert q_latent_weight.dtype == torch.float32 and q_latent_weight.numel() == q_rank
        out = torch.empty((tokens, q_rank), dtype=act, device=q_latent.device)
    code = lib.get("attention_latent").mstar_latent_fill(
        _ptr(q), q.stride(0) if q is not None else 0, _ptr(dkv),
        dkv.stride(0) if dkv is not None else 0, _DT[in_dtype], _DT[act], _ptr(norm_weight),
        freq.data_ptr(), positions.data_ptr(), cache_pos.data_ptr(), token_req.data_ptr(),
        _ptr(block_table), block_table.stride(0) if block_table is not None else 0, _ptr(cache),
        _ptr(q_latent), q_latent.stride(0) if q_latent is not None else 0, _ptr(q_latent_weight),
        _ptr(out), q_rank, q_rank, tokens, heads, qk_dim, rot, rot_dims, rank, page_size,
        int(interleaved), float(eps), _stream())
    if code == -1:
        raise KernelError(f"latent cache fill refuses rot_dims={rot_dims} of rot={rot}, or float "
                          "activations with inputs of another type")
    check(code, "latent_fill")
    return out


def latent_attention_plan(tokens: int, heads: int, rank: int, max_keys: int,
                          sms: int | None = None) -> tuple:
    """(heads per block, splits of a token's keys) for the latent attention kernels.  The
    tensor-core kernel takes up to 16 heads a block whatever the first number says; the
    CUDA-core kernels take as many heads as a thread's 32 sums allow (they share the rows a
    block loads), fewer when tokens are few.  With few tokens a token's keys are shared among
    blocks until there are some two blocks per SM, a split keeping at least two tiles of 32
    keys."""
    if sms is None:
        sms = num_sms()
    group = max(1, min(heads, 16 if rank <= 256 else (8 if rank <= 512 else 4)))
    want = 2 * sms
    while group > 4 and tokens * -(-heads // group) < want:
        group = max(4, group // 2)
    blocks = tokens * -(-heads // 16)
    tiles = max(1, -(-max_keys // 32))
    splits = max(1, min(want // max(blocks, 1), tiles // 2, 32))
    return group, splits


def latent_attention(q_abs: torch.Tensor, q_rot: torch.Tensor, cache: torch.Tensor, block_table,
                     token_req, cache_pos, heads: int, rank: int, rot: int, page_size: int,
                     window: int, scale: float, max_keys: int | None = None,
                     entries: int | None = None) -> torch.Tensor:
    """Softmax attention of every token over the latent rows it sees.  ``q_abs``: float
    [tokens, heads, rank], the plain query part with the key up-projection folded in;
    ``q_rot``: [tokens, heads, rot] view (last stride 1) of rotated query parts.  Returns the
    float [tokens, heads, rank] probability-weighted sums of latents.  ``max_keys`` bounds the
    keys any token sees (default: the window, or one tile when there is none); it only decides
    among how many blocks a token's keys are shared.  ``entries``: how many requests the
    step's tokens belong to; where they come in runs of one request (four tokens an entry or
    more) and no token's keys are shared among blocks, a block takes several tokens."""
    _need_cuda(q_abs, q_rot, cache, block_table, token_req, cache_pos)
    assert q_abs.dtype == torch.float32 and q_abs.is_contiguous()
    tokens = q_abs.shape[0]
    assert tuple(q_abs.shape) == (tokens, heads, rank) and cache.is_contiguous()
    assert tuple(q_rot.shape) == (tokens, heads, rot) and q_rot.dtype == cache.dtype
    assert rot == 0 or q_rot.stride(2) == 1
    if max_keys is None:
        max_keys = window or 32
    if window:
        max_keys = min(max_keys, window)
    group, splits = latent_attention_plan(tokens, heads, rank, max_keys, num_sms(q_abs.device))
    out = torch.empty((tokens, heads, rank), dtype=torch.float32, device=q_abs.device)
    scratch = None
    if splits > 1:
        scratch = torch.empty(tokens * heads * splits * (rank + 2), dtype=torch.float32,
                              device=q_abs.device)
    code = lib.get("attention_latent").mstar_latent_attention(
        q_abs.data_ptr(), q_rot.data_ptr(), q_rot.stride(0), q_rot.stride(1), out.data_ptr(),
        cache.data_ptr(), block_table.data_ptr(), block_table.stride(0), token_req.data_ptr(),
        cache_pos.data_ptr(), tokens, heads, rank, rot, page_size, int(window or 0), float(scale),
        _dt(cache), group, splits, _ptr(scratch),
        int(entries is not None and tokens >= 4 * max(entries, 1)), _stream())
    if code == -1:
        raise KernelError(f"latent attention refuses rank={rank}, rot={rot} (rank at most 1024, "
                          "a tile of 32 rows within 200 KB of shared memory)")
    check(code, "latent_attention")
    if splits > 1:
        lib.add_launches(1)                     # the merge kernel
    return out


_BMM_INTO_ROWS: dict = {}       # out dtype -> False once the library refused the strided output


def linear_per_head(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None):
    """out[t, h, :] = x[t, h, :] @ w[h]^T for x [tokens, heads, K] (any token and head strides,
    last stride 1) and w [heads, N, K].  bfloat16: the library's batched GEMM; float32: this
    package's true-32-bit kernel, head by head."""
    _need_cuda(x, w)
    tokens, heads, k = x.shape
    assert w.shape[0] == heads and w.shape[2] == k and x.stride(2) == 1 and w.is_contiguous()
    n = w.shape[1]
    out_dtype = out_dtype or x.dtype
    if x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        a, b = x.transpose(0, 1), w.transpose(1, 2)
        # the library writes [heads, tokens, n] straight into the rows of [tokens, heads, n]
        # (a row stride of heads * n), so no copy follows the product
        out = torch.empty((tokens, heads, n), dtype=out_dtype, device=x.device)
        if _BMM_INTO_ROWS.get(out_dtype, True):
            try:
                if out_dtype == torch.float32:
                    torch.bmm(a, b, out_dtype=torch.float32, out=out.transpose(0, 1))
                else:
                    torch.bmm(a, b, out=out.transpose(0, 1))
                return out
            except (TypeError, RuntimeError):
                _BMM_INTO_ROWS[out_dtype] = False
        if out_dtype == torch.float32:
            try:
                return torch.bmm(a, b, out_dtype=torch.float32).transpose(0, 1).contiguous()
            except (TypeError, RuntimeError):
                return torch.bmm(a, b).transpose(0, 1).float()
        return torch.bmm(a, b).transpose(0, 1).contiguous()
    xf = x if x.dtype == torch.float32 else x.float()
    wf = w if w.dtype == torch.float32 else w.float()
    out = torch.empty((tokens, heads, n), dtype=torch.float32, device=x.device)
    for h in range(heads):
        sgemm_nt(xf[:, h], wf[h], out[:, h])
    return out if out_dtype == torch.float32 else convert(out, out_dtype)


# ------------------------------------------------------------------ routed experts
def route_topk(logits: torch.Tensor, top: int, softmax: bool = False, renormalize: bool = False,
               choice_bias=None):
    """(chosen int32 [tokens, top], weight float [tokens, top]) from float router logits.
    ``choice_bias``: float [experts] added to the scores for the choice only."""
    _need_cuda(logits, choice_bias)
    assert logits.dtype == torch.float32 and logits.dim() == 2 and logits.is_contiguous()
    tokens, experts = logits.shape
    assert choice_bias is None or (choice_bias.dtype == torch.float32
                                   and choice_bias.numel() == experts)
    chosen = torch.empty((tokens, top), dtype=torch.int32, device=logits.device)
    weight = torch.empty((tokens, top), dtype=torch.float32, device=logits.device)
    code = lib.get("routed_experts").mstar_route_topk(
        logits.data_ptr(), _ptr(choice_bias), chosen.data_ptr(), weight.data_ptr(), tokens, experts, top,
        int(softmax), int(renormalize), _stream())
    if code == -1:
        raise KernelError(f"cannot choose {top} of {experts} experts")
    check(code, "route_topk")
    return chosen, weight


def experts_by_row(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, chosen, weight,
                   ff: int, scale_input: bool, add=None, gated: bool = True,
                   real: int | None = None) -> torch.Tensor:
    """sum over a token's chosen experts of down(silu(gate u) * up u) (+ ``add``), every row
    streaming its experts' matrices.  ``w_gate_up``: [experts * 2 * ff, width] (per expert
    gate rows, then up rows), ``w_down``: [experts * width, ff].  ``gated`` False: an expert
    is down(relu(up u)^2) and ``w_gate_up`` [experts * ff, width].  ``real``: experts that
    have matrices; a chosen index at or beyond it adds weight * x (default: all are real)."""
    if real is None:
        real = w_down.shape[0] // x.shape[1]
    _need_cuda(x, w_gate_up, w_down, chosen, weight, add)
    tokens, width = x.shape
    top = chosen.shape[1]
    assert x.is_contiguous() and w_gate_up.is_contiguous() and w_down.is_contiguous()
    assert w_gate_up.dtype == x.dtype and w_down.dtype == x.dtype
    assert w_gate_up.shape[1] == width and w_down.shape[1] == ff
    assert add is None or (add.shape == x.shape and add.is_contiguous() and add.dtype == x.dtype)
    act = torch.empty((tokens * top, ff), dtype=torch.float32, device=x.device)
    out = torch.empty_like(x)
    code = lib.get("routed_experts").mstar_experts_by_row(
        x.data_ptr(), w_gate_up.data_ptr(), w_down.data_ptr(), chosen.data_ptr(),
        weight.data_ptr(), act.data_ptr(), _ptr(add), out.data_ptr(), _dt(x), tokens, width, ff,
        top, int(scale_input), int(gated), int(real), _stream())
    if code == -1:
        raise KernelError(f"the by-row expert kernels refuse width={width}, ff={ff}, top={top} "
                          "(a row of inputs, and of hidden units, within 48 KB)")
    check(code, "experts_by_row")
    lib.add_launches(1)                       # two kernels behind one call
    return out


# Rows (tokens x choices) from which on the experts' rows are sorted by expert and run as
# tiles of a tensor-core GEMM; below, every row streams its experts' matrices by itself.
GROUPED_EXPERT_ROWS = 64


def experts_grouped(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, chosen, weight,
                    experts: int, ff: int, scale_input: bool, add=None, gated: bool = True,
                    real: int | None = None) -> torch.Tensor:
    """The same sums as ``experts_by_row`` for many bfloat16 rows: rows sorted by expert on
    the device, each expert's rows through its matrices as 64-row tiles on the tensor cores
    (float sums), a token's choices added up in their order.  Nothing is read by the host."""
    _need_cuda(x, w_gate_up, w_down, chosen, weight, add)
    tokens, width = x.shape
    top = chosen.shape[1]
    assert x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16
    assert w_down.dtype == torch.bfloat16 and x.is_contiguous()
    assert w_gate_up.is_contiguous() and w_down.is_contiguous()
    real = experts if real is None else real       # ``experts`` counts identity experts too
    assert tuple(w_gate_up.shape) == (real * (2 if gated else 1) * ff, width)
    assert tuple(w_down.shape) == (real * width, ff)
    assert add is None or (add.shape == x.shape and add.is_contiguous() and add.dtype == x.dtype)
    rows = tokens * top
    ints = torch.empty(2 * rows + experts + 2 + 2 * (rows // 64 + experts), dtype=torch.int32,
                       device=x.device)
    act = torch.empty((rows, ff), dtype=torch.bfloat16, device=x.device)
    y = torch.empty((rows, width), dtype=torch.float32, device=x.device)
    out = torch.empty_like(x)
    code = lib.get("routed_experts").mstar_experts_grouped(
        x.data_ptr(), w_gate_up.data_ptr(), w_down.data_ptr(), chosen.data_ptr(),
        weight.data_ptr(), ints.data_ptr(), act.data_ptr(), y.data_ptr(), _ptr(add),
        out.data_ptr(), tokens, width, ff, top, experts, int(scale_input), int(gated), int(real),
        _stream())
    if code == -1:
        raise KernelError(f"the grouped expert kernels refuse width={width}, ff={ff}, "
                          f"experts={experts} (width and ff multiples of 8, at most 1024 experts)")
    check(code, "experts_grouped")
    lib.add_launches(3)                       # four kernels behind one call
    return out


def routed_experts(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, chosen, weight,
                   experts: int, ff: int, scale_input: bool, add=None, gated: bool = True,
                   identity: int = 0) -> torch.Tensor:
    """sum over a token's chosen experts of down(silu(gate u) * up u) (+ ``add``): sorted by
    expert on the tensor cores from ``GROUPED_EXPERT_ROWS`` bfloat16 rows on
    (MSTAR_EXPERTS=by_row: never), row by row below and in float32."""
    rows = x.shape[0] * chosen.shape[1]
    if (x.dtype == torch.bfloat16 and rows >= GROUPED_EXPERT_ROWS and x.shape[1] % 8 == 0
            and ff % 8 == 0 and experts <= 1024 and os.environ.get("MSTAR_EXPERTS") != "by_row"):
        return experts_grouped(x, w_gate_up, w_down, chosen, weight, experts + identity, ff,
                               scale_input, add, gated=gated, real=experts)
    return experts_by_row(x, w_gate_up, w_down, chosen, weight, ff, scale_input, add, gated=gated,
                          real=experts)


# ------------------------------------------------------------------ window attention with kept first keys
def sink_page_elements(num_kv_heads: int, page_size: int, head_dim: int, v_dim: int) -> int:
    """Elements of one cache page: [kv_heads, page_size, head_dim] keys, then [kv_heads,
    page_size, v_dim] values (the two-plane layout when the sizes are equal)."""
    return num_kv_heads * page_size * (head_dim + v_dim)


def sink_prepare(qkv: torch.Tensor, bias, q_norm, k_norm, freq, positions, cache_pos, token_req,
                 block_table, kv_cache: torch.Tensor, num_heads: int, num_kv_heads: int,
                 head_dim: int, v_dim: int, rot: int, page_size: int, eps: float,
                 out_dtype: torch.dtype, conv=None, value_from_key: bool = False,
                 interleaved: bool = False, norm_whole: bool = False,
                 q_temp=None) -> torch.Tensor:
    """From the float fused projection ``qkv`` [tokens, (heads + kv_heads) * head_dim +
    kv_heads * v_dim (+ columns this kernel does not read)]: add ``bias``, norm every query
    and key head (``q_norm`` / ``k_norm`` weights of ``head_dim``, or None for no norm), rotate
    their first ``rot`` features (``freq``: float64 [rot / 2]), write keys and values into the
    token's cache page, and return the queries [tokens, heads * head_dim] in ``out_dtype``.

    ``conv``: (q weights [heads * head_dim, taps], k weights [kv_heads * head_dim, taps],
    qo_indptr, slots, state) puts a causal convolution over time on every q and k channel
    before the norm; the rows before a portion come from ``state`` [slots, (taps - 1) *
    channels] (float), which ``conv_state_advance`` moves on afterwards.  ``value_from_key``:
    the row has no value part; a key head before its norm is the value head.
    ``interleaved``: feature 2i is rotated with 2i + 1 instead of i with i + rot / 2.
    ``norm_whole``: one root mean square over all query heads and one over all key heads;
    ``q_norm`` / ``k_norm`` then have ``heads * head_dim`` / ``kv_heads * head_dim`` numbers.
    ``q_temp``: (coef, every) multiplies the query of the token at position p by ``1 + coef
    * ln(floor((p + 1) / every) + 1)``."""
    _need_cuda(qkv, bias, q_norm, k_norm, freq, positions, cache_pos, token_req, block_table,
               kv_cache)
    if q_norm is not None:
        per = (num_heads, num_kv_heads) if norm_whole else (1, 1)
        assert q_norm.numel() == per[0] * head_dim and k_norm.numel() == per[1] * head_dim
    assert not (norm_whole and conv is not None)
    temp_coef, temp_every = (float(q_temp[0]), int(q_temp[1])) if q_temp else (0.0, 0)
    assert qkv.dtype == torch.float32 and qkv.dim() == 2 and qkv.stride(1) == 1
    assert kv_cache.is_contiguous()
    tokens = qkv.shape[0]
    need = (num_heads + num_kv_heads) * head_dim + (0 if value_from_key else num_kv_heads * v_dim)
    assert qkv.shape[1] >= need
    assert kv_cache.dtype == out_dtype
    assert kv_cache[0].numel() == sink_page_elements(num_kv_heads, page_size, head_dim, v_dim)
    assert (q_norm is None) == (k_norm is None)
    wq = wk = qo = slots = state = None
    taps = 0
    if conv is not None:
        wq, wk, qo, slots, state = conv
        _need_cuda(wq, wk, qo, slots, state)
        taps = wq.shape[1]
        assert tuple(wq.shape) == (num_heads * head_dim, taps) and wq.is_contiguous()
        assert tuple(wk.shape) == (num_kv_heads * head_dim, taps) and wk.is_contiguous()
        if taps > 1:
            assert state.dtype == torch.float32 and state.dim() == 2 and state.stride(1) == 1
            assert state.shape[1] >= (taps - 1) * (num_heads + num_kv_heads) * head_dim
    wd = F32
    for w in (bias, q_norm, k_norm, wq, wk):
        if w is not None:
            wd = _dt(w)
    for w in (bias, q_norm, k_norm, wq, wk):
        assert w is None or (_dt(w) == wd and w.is_contiguous())
    if rot:
        assert freq is not None and freq.dtype == torch.float64 and freq.numel() == rot // 2
    q = torch.empty((tokens, num_heads * head_dim), dtype=out_dtype, device=qkv.device)
    code = lib.get("attention_sink").mstar_sink_prepare(
        qkv.data_ptr(), _ptr(bias), _ptr(q_norm), _ptr(k_norm), wd, _ptr(freq),
        positions.data_ptr(), cache_pos.data_ptr(), token_req.data_ptr(), block_table.data_ptr(),
        block_table.stride(0), q.data_ptr(), kv_cache.data_ptr(), _DT[out_dtype], tokens, num_heads,
        num_kv_heads, head_dim, v_dim, rot, page_size, float(eps), int(q_norm is not None),
        qkv.stride(0), _ptr(wq), _ptr(wk), taps, int(value_from_key), _ptr(qo), _ptr(slots),
        _ptr(state) if taps > 1 else 0, state.stride(0) if taps > 1 else 0, int(interleaved),
        int(norm_whole and q_norm is not None), temp_coef, temp_every, _stream())
    if code == -1:
        raise KernelError(f"attention input kernel refuses head_dim={head_dim}, v_dim={v_dim}, "
                          f"rot={rot}, taps={taps}")
    check(code, "sink_prepare")
    return q


def conv_state_advance(qkv: torch.Tensor, channels: int, taps: int, qo_indptr, slots,
                       state: torch.Tensor, entries: int) -> None:
    """After ``sink_prepare`` with a convolution: every entry's slot takes the last
    ``taps - 1`` rows of the first ``channels`` columns of its sequence (what the slot held
    moves up where the portion is shorter)."""
    if taps <= 1:
        return
    _need_cuda(qkv, qo_indptr, slots, state)
    assert qkv.dtype == torch.float32 and qkv.stride(1) == 1 and qkv.shape[1] >= channels
    assert state.dtype == torch.float32 and state.dim() == 2 and state.stride(1) == 1
    assert state.shape[1] >= (taps - 1) * channels
    check(lib.get("attention_sink").mstar_conv_state_advance(
        qkv.data_ptr(), qkv.stride(0), channels, taps, qo_indptr.data_ptr(), slots.data_ptr(),
        state.data_ptr(), state.stride(0), entries, _stream()), "conv_state_advance")


def sink_attention_splits(entries: int, max_q_len: int, num_heads: int, num_kv_heads: int,
                          max_keys: int, sms: int | None = None, wide: int = 128) -> int:
    """Among how many CTAs the keys of a row tile are shared in the tensor-core kernel: one
    where the row tiles alone fill the GPU, else as many as still give every CTA an SM of its
    own (a CTA's key and value stages take most of an SM's shared memory, so a CTA beyond one
    per SM waits for a second wave: at 8 requests with 2,048 keys 8 splits take 23 us, 16
    take 29, at 32 requests 2 take 62 and 5 take 76), a split keeping at least two tiles of
    64 keys (one tile a CTA was measured and is slower: 27 against 24 us at 8 requests with
    1,028 visible keys).  ``wide``: the larger of the key and value sizes; where the stages of
    two CTAs fit an SM (sizes up to 64), two CTAs an SM are the target."""
    if sms is None:
        sms = num_sms()
    group = num_heads // num_kv_heads
    rows = max_q_len * group
    ctas = max(1, -(-rows // 64) * num_kv_heads * entries)
    padded = next((d for d in (32, 64, 96, 128, 256) if wide <= d), 256)
    stages = 4 if (rows <= 64 and padded <= 128) else 2
    smem = (2 * stages + 1) * 64 * (padded + 8) * 2
    room = sms * min(2, max(1, (227 * 1024) // smem))
    if ctas >= room:
        return 1
    return max(1, min(room // ctas, -(-max_keys // 64) // 2, 64))


def sink_attention(q: torch.Tensor, kv_cache: torch.Tensor, block_table, token_req, cache_pos,
                   num_heads: int, num_kv_heads: int, head_dim: int, v_dim: int, page_size: int,
                   window: int, keep_first: int, scale: float, ctx=None, gate=None,
                   softcap: float | None = None, sink=None) -> torch.Tensor:
    """Softmax attention of every token over the keys it sees: those of the last ``window``
    positions (0: all) and the first ``keep_first`` of the sequence.  ``q``: [tokens, heads *
    head_dim]; returns [tokens, heads * v_dim].  ``gate``: None, or float [tokens, heads] (a
    column view of a wider product): head h's output is multiplied by sigmoid(gate[t, h]),
    where the tensor-core kernel writes it out, by a kernel of its own after the other; a gate
    of [tokens, heads * v_dim] numbers multiplies feature by feature.  ``softcap``: a score
    becomes ``softcap * tanh(score / softcap)`` after the scale.  ``sink``: float [heads];
    ``exp(sink[h])`` joins the denominator of head h's softmax (no key, no value).  bfloat16 with sizes that are multiples of 8
    up to 256 and a step context (``ctx``: entries, their token ranges and lengths) runs on
    the tensor cores (MSTAR_SINK_ATTENTION=generic: never); everything else, float32
    included, on the CUDA cores."""
    _need_cuda(q, kv_cache, block_table, token_req, cache_pos, gate)
    assert q.is_contiguous() and kv_cache.is_contiguous() and kv_cache.dtype == q.dtype
    tokens = q.shape[0]
    gate_features = False
    if gate is not None:
        gate_features = gate.shape[1] == num_heads * v_dim and v_dim > 1
        assert tuple(gate.shape) == (tokens, num_heads * (v_dim if gate_features else 1))
        assert gate.dtype == torch.float32 and gate.stride(1) == 1
    if sink is not None:
        _need_cuda(sink)
        assert sink.dtype == torch.float32 and sink.numel() == num_heads and sink.is_contiguous()
    cap = float(softcap or 0.0)
    out = torch.empty((tokens, num_heads * v_dim), dtype=q.dtype, device=q.device)
    if (ctx is not None and q.dtype == torch.bfloat16 and head_dim % 8 == 0 and v_dim % 8 == 0
            and max(head_dim, v_dim) <= 256 and os.environ.get("MSTAR_SINK_ATTENTION") != "generic"):
        max_keys = ctx.max_kv_len
        if window:
            max_keys = min(max_keys, window + keep_first + ctx.max_q_len)
        splits = sink_attention_splits(ctx.num_entries, ctx.max_q_len, num_heads, num_kv_heads,
                                       max_keys, num_sms(q.device), wide=max(head_dim, v_dim))
        scratch = None
        if splits > 1:
            scratch = torch.empty(tokens * num_heads * splits * (v_dim + 2), dtype=torch.float32,
                                  device=q.device)
        code = lib.get("attention_sink_tc").mstar_sink_attention_tc(
            q.data_ptr(), q.stride(0), out.data_ptr(), kv_cache.data_ptr(), block_table.data_ptr(),
            block_table.stride(0), ctx.qo_indptr.data_ptr(), ctx.kv_len.data_ptr(),
            ctx.num_entries, tokens, ctx.max_q_len, num_heads, num_kv_heads, head_dim, v_dim,
            page_size, int(window or 0), int(keep_first), float(scale), splits, _ptr(scratch),
            _ptr(gate), gate.stride(0) if gate is not None else 0, int(gate_features), cap,
            _ptr(sink), _stream())
        if code == -1:
            raise KernelError(f"tensor-core window attention refuses heads={num_heads}, "
                              f"kv_heads={num_kv_heads}, head_dim={head_dim}, v_dim={v_dim}")
        check(code, "sink_attention_tc")
        if splits > 1:
            lib.add_launches(1)                 # the merge kernel
        return out
    code = lib.get("attention_sink").mstar_sink_attention_generic(
        q.data_ptr(), q.stride(0), out.data_ptr(), kv_cache.data_ptr(), block_table.data_ptr(),
        block_table.stride(0), token_req.data_ptr(), cache_pos.data_ptr(), tokens, num_heads,
        num_kv_heads, head_dim, v_dim, page_size, int(window or 0), int(keep_first), float(scale),
        _dt(q), cap, _ptr(sink), _ptr(gate) if gate_features else 0,
        gate.stride(0) if gate_features else 0, _stream())
    if code == -1:
        raise KernelError(f"window attention refuses heads={num_heads}, kv_heads={num_kv_heads}, "
                          f"head_dim={head_dim}, v_dim={v_dim}")
    check(code, "sink_attention")
    if gate is not None and not gate_features:
        head_gate_mul(out, gate, num_heads)
    return out


# ------------------------------------------------------------------ selective scan
def selective_scan_state_size(inner: int, n_state: int, taps: int) -> int:
    """Floats of one request's state: the convolution's last inputs [taps - 1, inner], then
    S [inner, n_state]."""
    return (taps - 1) * inner + inner * n_state


def conv_silu(xz: torch.Tensor, weight, bias, token_req, qo_indptr, slots, state: torch.Tensor,
              inner: int, taps: int, weight_t=None, bias_f32=None) -> torch.Tensor:
    """silu(causal convolution per channel) of the x half of ``xz`` [tokens, 2 * inner], the
    inputs before a portion's start taken from the request's slot.  ``weight`` [inner, taps]
    (last column: the current token), ``bias`` [inner].  With ``weight_t`` (float [taps,
    inner]) and ``bias_f32`` given and rows of whole 16-byte pieces, a thread takes 8 channels
    with 16-byte accesses."""
    _need_cuda(xz, weight, bias, token_req, qo_indptr, slots, state, weight_t, bias_f32)
    assert xz.dim() == 2 and xz.stride(1) == 1 and weight.is_contiguous() and bias.is_contiguous()
    assert tuple(weight.shape) == (inner, taps) and bias.numel() == inner
    assert weight.dtype == bias.dtype
    assert state.dtype == torch.float32 and state.dim() == 2 and state.stride(1) == 1
    tokens = xz.shape[0]
    out = torch.empty((tokens, inner), dtype=xz.dtype, device=xz.device)
    if (weight_t is not None and bias_f32 is not None and inner % 8 == 0 and xz.stride(0) % 8 == 0
            and state.stride(0) % 4 == 0 and xz.data_ptr() % 16 == 0
            and os.environ.get("MSTAR_CONV") != "scalar"):
        assert weight_t.dtype == torch.float32 and tuple(weight_t.shape) == (taps, inner)
        assert bias_f32.dtype == torch.float32 and bias_f32.numel() == inner
        assert weight_t.is_contiguous() and bias_f32.is_contiguous()
        check(lib.get("selective_scan").mstar_conv_silu_vec(
            xz.data_ptr(), xz.stride(0), weight_t.data_ptr(), bias_f32.data_ptr(),
            token_req.data_ptr(), qo_indptr.data_ptr(), slots.data_ptr(), state.data_ptr(),
            state.stride(0), out.data_ptr(), _dt(xz), tokens, inner, taps, _stream()),
            "conv_silu_vec")
        return out
    check(lib.get("selective_scan").mstar_conv_silu(
        xz.data_ptr(), xz.stride(0), weight.data_ptr(), bias.data_ptr(), _dt(weight),
        token_req.data_ptr(), qo_indptr.data_ptr(), slots.data_ptr(), state.data_ptr(),
        state.stride(0), out.data_ptr(), _dt(xz), tokens, inner, taps, _stream()), "conv_silu")
    return out


# Tokens of a piece when a long portion's recurrence is cut into pieces that run side by side
# (a multiple of the kernel's chunk of 16), and the portion length from which on it is cut.
SCAN_PIECE = 128
SCAN_PIECES_FROM = 512


def selective_scan(xc: torch.Tensor, xz: torch.Tensor, proj: torch.Tensor, w_dt, dt_bias, a_neg,
                   d_skip, qo_indptr, slots, state: torch.Tensor, entries: int, inner: int,
                   n_state: int, rank: int, taps: int, max_q_len: int | None = None) -> torch.Tensor:
    """The recurrence over the tokens of ``entries`` batch entries, each continuing the state
    in its slot (S updated in place, the convolution's window moved on by the portion).
    ``xc`` [tokens, inner] conv outputs; ``xz`` [tokens, 2 * inner] (the gate z is its second
    half, the raw x its first); ``proj`` float [tokens, rank + 2 * n_state] = [dt_in | B | C];
    float ``w_dt`` [inner, rank], ``dt_bias`` [inner], ``a_neg`` [inner, n_state] (= -exp(A_log)),
    ``d_skip`` [inner].  Returns y * silu(z) [tokens, inner] in the dtype of ``xc``.
    ``max_q_len`` (the longest portion of the batch) of ``SCAN_PIECES_FROM`` tokens or more
    cuts every portion into pieces of ``SCAN_PIECE`` tokens that run side by side: a first
    pass leaves each piece's own end state and summed step sizes, a second starts each piece
    from the state joined over the pieces before it (the recurrence is linear in the state);
    MSTAR_SCAN_PIECE sets another piece size, 0 none."""
    _need_cuda(xc, xz, proj, w_dt, dt_bias, a_neg, d_skip, qo_indptr, slots, state)
    assert xc.is_contiguous() and xz.stride(1) == 1 and xz.dtype == xc.dtype
    assert proj.dtype == torch.float32 and proj.is_contiguous()
    assert proj.shape[1] == rank + 2 * n_state
    for t, shape in ((w_dt, (inner, rank)), (dt_bias, (inner,)), (a_neg, (inner, n_state)),
                     (d_skip, (inner,))):
        assert t.dtype == torch.float32 and t.is_contiguous() and tuple(t.shape) == shape
    assert state.dtype == torch.float32 and state.dim() == 2 and state.stride(1) == 1
    assert state.shape[1] == selective_scan_state_size(inner, n_state, taps)
    out = torch.empty_like(xc)
    piece, pieces, piece_state, piece_dt, dt_pre = 0, 1, None, None, None
    if max_q_len is not None and max_q_len >= SCAN_PIECES_FROM:
        piece = int(os.environ.get("MSTAR_SCAN_PIECE", SCAN_PIECE)) // 16 * 16
    if piece:
        pieces = -(-max_q_len // piece)
        piece_state = torch.empty((entries, pieces, inner, n_state), dtype=torch.float32,
                                  device=xc.device)
        piece_dt = torch.empty((entries, pieces, inner), dtype=torch.float32, device=xc.device)
        # with many tokens the step sizes' product W_dt dt_in is a true-32-bit product of its
        # own (a third of the scan's instructions otherwise)
        dt_pre = sgemm_nt(proj[:, :rank], w_dt)
    code = lib.get("selective_scan").mstar_selective_scan(
        xc.data_ptr(), xz.data_ptr(), xz.stride(0), proj.data_ptr(), w_dt.data_ptr(),
        dt_bias.data_ptr(), a_neg.data_ptr(), d_skip.data_ptr(), qo_indptr.data_ptr(),
        slots.data_ptr(), state.data_ptr(), state.stride(0), out.data_ptr(), _dt(xc), entries,
        inner, n_state, rank, taps, piece, pieces, _ptr(piece_state), _ptr(piece_dt), _ptr(dt_pre),
        _stream())
    if piece:
        lib.add_launches(1)                     # two passes behind one call
    if code == -1:
        raise KernelError(f"selective scan refuses inner={inner}, state={n_state}, rank={rank} "
                          "(at most 256 states a channel)")
    check(code, "selective_scan")
    return out


# ------------------------------------------------------------------ hyper-connections
def hyper_step(x: torch.Tensor, *, init=None, y=None, y2=None, y_scales=(1.0, 1.0), y_bias=None,
               mix=None, out=None, read=None, norm_weight=None, eps: float = 0.0,
               out_dtype: torch.dtype | None = None, rows=None):
    """What lies between two sublayers of a residual kept as copies ``x`` [tokens, S, width]
    (float, updated in place).

    With ``y`` (a sublayer's output [tokens, width]; ``y_scales[0] * y + y_scales[1] * y2 +
    y_bias``) every copy is rewritten from the old ones: ``x_t = sum_s mix[s, t] x_s + out[t] *
    y``.  With ``init`` [tokens, width] the old copies are all that row.  Then either ``read``
    (float [S]) with ``norm_weight``: returns ``rmsnorm(sum_s read[s] x_s) * norm_weight`` in
    ``out_dtype``; or ``rows`` (int32 indices): returns float ``sum_s x_s`` of those tokens
    without writing the copies back."""
    _need_cuda(x, init, y, y2, y_bias, mix, out, read, norm_weight, rows)
    assert x.dtype == torch.float32 and x.dim() == 3 and x.is_contiguous()
    tokens, streams, width = x.shape
    assert mix.dtype == torch.float32 and mix.numel() == streams * streams and mix.is_contiguous()
    assert out.dtype == torch.float32 and out.numel() == streams
    assert (read is None) != (rows is None)
    act = out_dtype
    for t in (y, y2):
        if t is not None:
            assert tuple(t.shape) == (tokens, width) and t.is_contiguous()
            assert act is None or t.dtype == act
            act = t.dtype
    if init is not None:
        assert init.dtype == torch.float32 and tuple(init.shape) == (tokens, width)
        assert init.is_contiguous()
    wd = F32
    for w in (y_bias, norm_weight):
        if w is not None:
            wd = _dt(w)
    for w in (y_bias, norm_weight):
        assert w is None or (_dt(w) == wd and w.is_contiguous() and w.numel() == width)
    normed = sums = None
    if read is not None:
        assert read.dtype == torch.float32 and read.numel() == streams
        assert norm_weight is not None and out_dtype is not None
        normed = torch.empty((tokens, width), dtype=out_dtype, device=x.device)
        blocks = tokens
    else:
        assert rows.dtype == torch.int32 and rows.is_contiguous()
        blocks = rows.numel()
        sums = torch.empty((blocks, width), dtype=torch.float32, device=x.device)
    code = lib.get("hyper").mstar_hyper_step(
        x.data_ptr(), _ptr(init), _ptr(y), _ptr(y2), _ptr(y_bias), float(y_scales[0]),
        float(y_scales[1]), mix.data_ptr(), out.data_ptr(), _ptr(read), _ptr(norm_weight),
        _ptr(normed), _ptr(rows), _ptr(sums), blocks, streams, width, float(eps),
        _DT[act or torch.float32], wd, _stream())
    if code == -1:
        raise KernelError(f"hyper-connection kernel refuses streams={streams}, width={width}")
    check(code, "hyper_step")
    return normed if read is not None else sums


class WeightedSum:
    """``sum_b scales[b] * branches[b]`` of branch outputs, not computed yet: a block that adds
    it to the residual takes the branches into its own kernel; ``materialize()`` computes it."""

    def __init__(self, branches, scales):
        self.branches, self.scales = list(branches), [float(s) for s in scales]
        self.shape, self.dtype = branches[0].shape, branches[0].dtype

    def materialize(self) -> torch.Tensor:
        acc, scale = self.branches[0], self.scales[0]
        if len(self.branches) == 1:
            return weighted_sum2(acc, acc, scale, 0.0)
        for b, s in zip(self.branches[1:], self.scales[1:]):
            acc = weighted_sum2(acc, b, scale, s)
            scale = 1.0
        return acc


def weighted_sum2(y1: torch.Tensor, y2: torch.Tensor, a: float, b: float) -> torch.Tensor:
    """a * y1 + b * y2 with float sums."""
    _need_cuda(y1, y2)
    assert y1.shape == y2.shape and y1.dtype == y2.dtype and y1.is_contiguous() and y2.is_contiguous()
    out = torch.empty_like(y1)
    check(lib.get("hyper").mstar_weighted_sum2(y1.data_ptr(), y2.data_ptr(), out.data_ptr(),
                                               y1.numel(), float(a), float(b), _dt(y1), _stream()),
          "weighted_sum2")
    return out


# ------------------------------------------------------------------ gated delta rule
def gated_delta_state_size(heads: int, kv_heads: int, dim: int, vdim: int, taps: int) -> int:
    """Floats of one request's state: the convolutions' last inputs [taps - 1, 2 * kv_heads *
    dim + heads * vdim], then S^T [heads, vdim, dim]."""
    return (taps - 1) * (2 * kv_heads * dim + heads * vdim) + heads * vdim * dim


def delta_prepare(proj: torch.Tensor, conv_w: torch.Tensor, a_proj: torch.Tensor, dt_bias, a_exp,
                  token_req, qo_indptr, slots, state: torch.Tensor, heads: int, kv_heads: int,
                  dim: int, vdim: int, taps: int, unit_eps: float):
    """From the float fused projection ``proj`` [tokens, q | k | v | b | ...]: convolution and
    SiLU on the q, k and v channels (``conv_w`` [channels, taps]; rows before a portion from
    ``state``), unit q (times ``dim ** -0.5``) and k per head, ``beta = sigmoid(b)``, and the
    decays ``exp(-a_exp[h] * softplus(a_proj + dt_bias))``.  Returns float (q, k, v, beta,
    decay).  ``conv_state_advance`` moves the slot's rows on afterwards."""
    _need_cuda(proj, conv_w, a_proj, dt_bias, a_exp, token_req, qo_indptr, slots, state)
    tokens = proj.shape[0]
    qk, vv = kv_heads * dim, heads * vdim
    assert proj.dtype == torch.float32 and proj.stride(1) == 1 and proj.shape[1] >= 2 * qk + vv + heads
    assert tuple(conv_w.shape) == (2 * qk + vv, taps) and conv_w.is_contiguous()
    assert a_proj.dtype == torch.float32 and a_proj.is_contiguous()
    assert tuple(a_proj.shape) == (tokens, heads * dim)
    assert dt_bias.dtype == torch.float32 and dt_bias.numel() == heads * dim
    assert a_exp.dtype == torch.float32 and a_exp.numel() == heads
    assert state.dtype == torch.float32 and state.dim() == 2 and state.stride(1) == 1
    assert state.shape[1] >= gated_delta_state_size(heads, kv_heads, dim, vdim, taps)
    dev = proj.device
    q = torch.empty((tokens, qk), dtype=torch.float32, device=dev)
    k = torch.empty((tokens, qk), dtype=torch.float32, device=dev)
    v = torch.empty((tokens, vv), dtype=torch.float32, device=dev)
    beta = torch.empty((tokens, heads), dtype=torch.float32, device=dev)
    decay = torch.empty((tokens, heads * dim), dtype=torch.float32, device=dev)
    code = lib.get("gated_delta").mstar_delta_prepare(
        proj.data_ptr(), proj.stride(0), conv_w.data_ptr(), _dt(conv_w), a_proj.data_ptr(),
        dt_bias.data_ptr(), a_exp.data_ptr(), token_req.data_ptr(), qo_indptr.data_ptr(),
        slots.data_ptr(), state.data_ptr(), state.stride(0), q.data_ptr(), k.data_ptr(),
        v.data_ptr(), beta.data_ptr(), decay.data_ptr(), tokens, heads, kv_heads, dim, vdim, taps,
        float(unit_eps), _stream())
    if code == -1:
        raise KernelError(f"delta-rule input kernel refuses heads={heads}, kv_heads={kv_heads}, "
                          f"dim={dim}, vdim={vdim}, taps={taps}")
    check(code, "delta_prepare")
    return q, k, v, beta, decay


DELTA_PIECE = 16            # tokens of a piece of the delta-rule scan
DELTA_PIECES_FROM = 64      # entries of this many tokens or more are scanned in pieces
DELTA_PIECES_DIMS = (32, 64, 128, 256)     # key sizes the scan in pieces takes


def delta_scan(q, k, v, beta, decay, qo_indptr, slots, state: torch.Tensor, entries: int,
               heads: int, kv_heads: int, dim: int, vdim: int, taps: int,
               max_q_len: int = 1 << 30) -> torch.Tensor:
    """The gated delta rule over the tokens of ``entries`` batch entries, each continuing the
    matrix in its slot (updated in place).  ``max_q_len``: the longest entry (a bound will do;
    short entries stage fewer tokens at a time).  Returns float [tokens, heads * vdim].

    A step with an entry of ``DELTA_PIECES_FROM`` tokens or more (and ``dim`` 32, 64, 128 or 256) is
    scanned in pieces of 16 tokens: what does not depend on the state (decayed keys and
    queries, the keys' products among themselves) is made for all pieces side by side, and
    the chain from token to token shrinks to a scalar a token (MSTAR_DELTA_PIECES=0: never;
    1: always)."""
    _need_cuda(q, k, v, beta, decay, qo_indptr, slots, state)
    for t in (q, k, v, beta, decay):
        assert t.dtype == torch.float32 and t.is_contiguous()
    assert state.dtype == torch.float32 and state.dim() == 2 and state.stride(1) == 1
    tokens = q.shape[0]
    out = torch.empty((tokens, heads * vdim), dtype=torch.float32, device=q.device)
    offset = (taps - 1) * (2 * kv_heads * dim + heads * vdim)
    longest = int(min(max_q_len, tokens))
    forced = os.environ.get("MSTAR_DELTA_PIECES")
    pieces = (forced == "1" or (forced != "0" and longest >= DELTA_PIECES_FROM))
    if (pieces and dim in DELTA_PIECES_DIMS and tokens > 0 and offset % 4 == 0
            and state.stride(0) % 4 == 0):
        max_pieces = -(-longest // DELTA_PIECE)
        floats = (3 * tokens * heads * dim + entries * max_pieces * heads * dim
                  + 2 * tokens * heads * DELTA_PIECE)
        work = torch.empty(floats, dtype=torch.float32, device=q.device)
        code = lib.get("gated_delta").mstar_delta_scan_pieces(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), beta.data_ptr(), decay.data_ptr(),
            qo_indptr.data_ptr(), slots.data_ptr(), state.data_ptr(), state.stride(0), offset,
            out.data_ptr(), work.data_ptr(), tokens, entries, longest, heads, kv_heads, dim, vdim,
            _stream())
        if code == -1:
            raise KernelError(f"delta-rule scan in pieces refuses heads={heads}, "
                              f"kv_heads={kv_heads}, dim={dim}")
        check(code, "delta_scan_pieces")
        lib.add_launches(1)
        return out
    code = lib.get("gated_delta").mstar_delta_scan(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), beta.data_ptr(), decay.data_ptr(),
        qo_indptr.data_ptr(), slots.data_ptr(), state.data_ptr(), state.stride(0), offset,
        out.data_ptr(), entries, int(min(max_q_len, 1 << 30)), heads, kv_heads, dim, vdim,
        _stream())
    if code == -1:
        raise KernelError(f"delta-rule scan refuses heads={heads}, kv_heads={kv_heads}, dim={dim} "
                          "(dim at most 512)")
    check(code, "delta_scan")
    return out


def delta_finish(o: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, heads: int, vdim: int,
                 eps: float, out_dtype: torch.dtype, scale: float = 1.0) -> torch.Tensor:
    """o / rms(o per head) * weight * sigmoid(gate) * scale: float ``o`` [tokens, heads * vdim],
    ``gate`` of the same shape in ``out_dtype``, float ``weight`` [vdim] shared by the heads."""
    _need_cuda(o, gate, weight)
    assert o.dtype == torch.float32 and o.is_contiguous()
    assert weight.dtype == torch.float32 and weight.numel() == vdim
    assert gate.dtype == out_dtype and gate.stride(1) == 1 and gate.shape == o.shape
    out = torch.empty(o.shape, dtype=out_dtype, device=o.device)
    check(lib.get("gated_delta").mstar_delta_finish(
        o.data_ptr(), gate.data_ptr(), gate.stride(0), weight.data_ptr(), out.data_ptr(),
        _DT[out_dtype], o.shape[0], heads, vdim, float(eps), float(scale), _stream()),
        "delta_finish")
    return out
