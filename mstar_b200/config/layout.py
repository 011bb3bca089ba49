"""Architecture-neutral description of a decoder: the specs that parts are built from.

A model configuration (for instance ``LlamaConfig``) is turned into a
``ModelLayout``: one ``BlockSpec`` per set of layer weights, each naming its
mixer, feed-forward, norms and their arrangement, and a run order that says
which block runs when and which cache it uses.  The engine only ever sees
these specs, so nothing below the configuration knows which model it is in.

Every spec carries a ``kind`` string.  ``mstar_b200.parts.registry`` maps
``(category, kind)`` to the class that implements it; a new mixer,
feed-forward, norm, position encoding or block arrangement is a new spec
dataclass plus one ``register_part`` call.

The reference builds its decoder layer from interchangeable modules in the
same spirit (mstar/model/components/decoder_layer.py:45-56) but takes the
sizes from a hard-coded dataclass (mstar/model/orpheus/config.py:4-53).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence


@dataclass(frozen=True)
class RopeScalingSpec:
    """Frequency-dependent scaling of rotary frequencies ("llama3" rule)."""

    rope_type: str
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int


@dataclass(frozen=True)
class PositionSpec:
    """Position encoding applied to queries and keys inside a mixer.

    kind "rope": rotary embedding over the first ``rotary_dim`` features of
    each head, pairs ``(j, j + rotary_dim/2)`` unless ``interleaved``.
    kind "none": nothing is applied.
    """

    kind: str = "rope"
    head_dim: int = 0
    rotary_dim: int = 0
    theta: float = 10000.0
    scaling: Optional[RopeScalingSpec] = None
    interleaved: bool = False


@dataclass(frozen=True)
class NormSpec:
    """kind "rmsnorm": ``x * rsqrt(mean(x^2) + eps) * (weight + weight_offset)``."""

    kind: str = "rmsnorm"
    size: int = 0
    eps: float = 1e-6
    weight_offset: float = 0.0


@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query softmax attention over a paged key/value cache.

    ``window``: None keeps every key; ``W`` lets a token at position ``p``
    see keys ``p-W+1 .. p``.  ``shares_kv``: the layer has no key/value
    projections and reads the cache written by an earlier layer.
    ``scale``: None means ``head_dim ** -0.5``.
    ``keep_first``: with a window, the keys at positions below it stay visible to every
    later token (at their true positions).  ``v_head_dim``: size of a value head, None
    when it equals ``head_dim``.  ``bias``: the q, k and v projections add a bias.
    ``qk_norm_eps``: not None puts an RMS norm over each query and key head (one weight of
    ``head_dim`` for the queries and one for the keys, shared by the heads) before the
    position encoding.  ``conv_taps`` > 1 puts a causal convolution over time on every
    channel of q and k (``conv_taps`` weights a channel, the last one on the token itself, no
    bias) directly after the projection; the last ``conv_taps - 1`` projected rows of a
    sequence are per-request state.  ``value_from_key``: there is no value projection, a key
    head as it leaves the convolution (before its norm) is the value.  ``head_gate``: the
    output of head h is multiplied by ``sigmoid(W_g x)_h``, one number a head, before the
    output product; ``feature_gate``: the concatenated heads are multiplied feature by feature
    by ``sigmoid(W_g x)`` (W_g has ``num_heads * value_dim`` rows).  ``qk_norm_whole``: the
    RMS norm runs over all heads of q (and of k) at once, with one weight per feature of the
    whole projection.  A rope position spec with ``interleaved`` pairs feature 2i with 2i + 1.
    ``q_temp``: (coef, every) multiplies the query at position p by ``1 + coef * ln(floor((p
    + 1) / every) + 1)``.  ``softcap``: scores become ``softcap * tanh(score / softcap)`` after
    the scale.  ``sink``: "learned" puts ``exp(sink_h)``, a parameter a head, into the
    softmax's denominator (it has no key and no value); "zero" puts exp(0) = 1 there.
    """

    kind: str = "attention"
    hidden_size: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    position: PositionSpec = field(default_factory=PositionSpec)
    window: Optional[int] = None
    scale: Optional[float] = None
    shares_kv: bool = False
    keep_first: int = 0
    v_head_dim: Optional[int] = None
    bias: bool = False
    qk_norm_eps: Optional[float] = None
    conv_taps: int = 0
    value_from_key: bool = False
    head_gate: bool = False
    feature_gate: bool = False
    qk_norm_whole: bool = False
    q_temp: Optional[tuple] = None
    softcap: Optional[float] = None
    sink: Optional[str] = None

    @property
    def value_dim(self) -> int:
        return self.head_dim if self.v_head_dim is None else self.v_head_dim

    @property
    def plain(self) -> bool:
        """Whether this is the attention that the kernels of the dense decoder take."""
        return (not self.keep_first and self.v_head_dim in (None, self.head_dim)
                and not self.bias and self.qk_norm_eps is None and self.conv_taps == 0
                and not self.value_from_key and not self.head_gate and not self.feature_gate
                and self.q_temp is None and self.softcap is None and self.sink is None)


@dataclass(frozen=True)
class GatedMLPSpec:
    """``down(act(gate(x)) * up(x))`` with a fused ``[gate; up]`` matrix; ``activation``:
    "silu" or "gelu_tanh".  ``bias``: the three products add a bias."""

    kind: str = "gated_mlp"
    hidden_size: int = 0
    intermediate_size: int = 0
    activation: str = "silu"
    bias: bool = False


@dataclass(frozen=True)
class MLPSpec:
    """kind "mlp": ``down(act(up(x)))`` without a gate.  ``activation``: "relu2" (the square
    of relu), "gelu_tanh" or "silu"."""

    kind: str = "mlp"
    hidden_size: int = 0
    intermediate_size: int = 0
    activation: str = "relu2"


@dataclass(frozen=True)
class SelectiveScanSpec:
    """kind "selective_scan": the Mamba mixer, a diagonal linear recurrence per channel whose
    step size and input/output maps depend on the token.

    ``[x | z] = W_in h`` (``inner`` channels each); x passes a causal convolution of ``conv``
    taps per channel and SiLU; ``[dt_in | B | C] = W_x x`` (``dt_rank``, ``state``, ``state``);
    ``dt = softplus(W_dt dt_in + b)`` per channel; with ``A = -exp(A_log)``:
    ``S[c, n] = exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n``, ``y_c = sum_n S[c, n] C_n + D_c x_c``;
    the output is ``W_o (y * silu(z))``.  S (float) and the convolution's last ``conv - 1``
    inputs are per-request state.
    """

    kind: str = "selective_scan"
    hidden_size: int = 0
    inner: int = 0
    state: int = 0
    dt_rank: int = 0
    conv: int = 1
    shares_kv: bool = False


@dataclass(frozen=True)
class ParallelMixerSpec:
    """kind "parallel": several mixers side by side on the same input.  ``merge``
    "mean_of_norms": the result is the mean of their outputs, each RMS-normed over the model
    width with a weight of its own; "weighted_sum": ``sum_b scales[b] * branch_b``."""

    kind: str = "parallel"
    hidden_size: int = 0
    branches: tuple = ()
    norm_eps: float = 1e-6
    shares_kv: bool = False
    merge: str = "mean_of_norms"
    scales: tuple = ()


@dataclass(frozen=True)
class GatedDeltaSpec:
    """kind "gated_delta": a delta-rule matrix memory with a decay per head and key channel,
    carried from token to token as per-request state.

    ``q = W_q h`` and ``k = W_k h`` have ``num_kv_heads`` heads of ``qk_dim``, ``v = W_v h`` has
    ``num_heads`` heads of ``v_dim``; head h reads q/k head ``h // (num_heads / num_kv_heads)``.
    Each passes a causal convolution of ``conv`` taps per channel and SiLU; q and k become
    unit vectors per head (``x / sqrt(sum x^2 + unit_eps)``), q times ``qk_dim ** -0.5``.
    ``beta = sigmoid(W_b h)`` a head; ``decay = exp(-exp(A_log_h) * softplus(W_a2 W_a1 h +
    dt_bias))`` a head and key channel.  Per head, in this order: ``S = decay * S`` row by
    row, ``u = beta (v - S^T k)``, ``S += k u^T``, ``o = S^T q``.  Each head's o is divided by
    its root mean square (``norm_eps``), scaled by a weight shared by the heads, gated by
    ``sigmoid(W_g2 W_g1 h)`` and projected back.  S (float) and the convolutions' last
    ``conv - 1`` inputs are per-request state.
    """

    kind: str = "gated_delta"
    hidden_size: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    qk_dim: int = 0
    v_dim: int = 0
    conv: int = 1
    decay_rank: int = 0
    gate_rank: int = 0
    norm_eps: float = 1e-6
    unit_eps: float = 1e-6
    shares_kv: bool = False


@dataclass(frozen=True)
class MatrixMemorySpec:
    """kind "mlstm": a matrix memory per head (the mLSTM cell of xLSTM), carried from token
    to token as per-request state instead of a key/value cache.

    Per head, with q scaled by ``dim ** -0.5``, log input gate i and log forget gate f
    (both soft-capped at ``gate_cap``, f through logsigmoid), and a running maximum m that
    starts at 0:  m' = max(f + m, i);  S' = exp(f + m - m') S + exp(i - m') k v^T;  n'
    likewise with k;  out = S'^T q / (max(|n' . q|, exp(-m')) + ``denom_floor``).  Each
    head's output is divided by its root mean square (``norm_eps``), scaled by a weight,
    gated by sigmoid(W_g x) and projected back.
    """

    kind: str = "mlstm"
    hidden_size: int = 0
    num_heads: int = 0
    qk_dim: int = 0
    v_dim: int = 0
    gate_cap: float = 15.0
    norm_eps: float = 1e-6
    denom_floor: float = 1e-6
    shares_kv: bool = False


@dataclass(frozen=True)
class LatentAttentionSpec:
    """kind "latent_attention": softmax attention whose keys and values are up-projections
    of one cached latent vector per token.

    A token caches ``kv_rank`` latent features (RMS-normed, plain weight) and ``rot_dim``
    rotated key features shared by all heads.  Head h scores a key as
    ``(q_plain . W_uk[h] c + q_rot . k_rot) * scale`` and reads the value ``W_uv[h] c``.
    ``position`` rotates the ``rot_dim`` part of queries and of the shared key.
    ``window``: None keeps every key; W lets position p see p-W+1 .. p.  ``gated``:
    the concatenated heads are multiplied by sigmoid(W_g x) before the output product,
    feature by feature, or, with ``gate_per_head``, by one number a head (W_g then has
    ``num_heads`` rows).  ``q_rank``: not None sends the queries through a latent of that
    size, ``q = W_uq norm(W_dq x)`` (RMS norm with a plain weight).  ``shares_kv``: the
    layer has no down-projection and reads the rows that an earlier layer cached.
    """

    kind: str = "latent_attention"
    hidden_size: int = 0
    num_heads: int = 0
    qk_dim: int = 0
    rot_dim: int = 0
    v_dim: int = 0
    kv_rank: int = 0
    position: PositionSpec = field(default_factory=PositionSpec)
    window: Optional[int] = None
    scale: Optional[float] = None
    norm_eps: float = 1e-6
    gated: bool = True
    shares_kv: bool = False
    gate_per_head: bool = False
    q_rank: Optional[int] = None


@dataclass(frozen=True)
class RoutedExpertsSpec:
    """kind "routed_experts": ``experts`` small gated feed-forwards of which a token uses
    ``top``, plus an optional shared one (``shared_size`` > 0) that every token uses.

    Router logits are float.  ``score``: "sigmoid" or "softmax" over all experts.
    ``renormalize``: the chosen scores are divided by their sum.  ``scale_input``: True
    scales what goes into the expert by the weight, False what comes out of it.
    ``gated``: an expert is ``down(act(gate u) * up u)``; False: ``down(act(up u))``.
    ``choice_bias``: a learned correction per router output is added to the scores for the
    choice only (the weights use the scores without it).  ``identity_experts``: the router
    has that many further outputs, standing for experts without tensors whose output is
    their input.
    """

    kind: str = "routed_experts"
    hidden_size: int = 0
    num_experts: int = 0
    top: int = 1
    expert_size: int = 0
    shared_size: int = 0
    score: str = "sigmoid"
    renormalize: bool = False
    scale_input: bool = True
    activation: str = "silu"
    gated: bool = True
    choice_bias: bool = False
    identity_experts: int = 0


@dataclass(frozen=True)
class EmbeddingSpec:
    """kind "table": the residual starts as ``table[token] * multiplier`` in float."""

    kind: str = "table"
    vocab_size: int = 0
    hidden_size: int = 0
    multiplier: float = 1.0


@dataclass(frozen=True)
class HeadSpec:
    """kind "linear": ``logits = x W^T * logit_scale``, then ``softcap * tanh(logits /
    softcap)`` when a soft cap is given; float logits."""

    kind: str = "linear"
    vocab_size: int = 0
    hidden_size: int = 0
    logit_scale: float = 1.0
    softcap: Optional[float] = None


@dataclass(frozen=True)
class BlockSpec:
    """One set of layer weights and how its parts are wired.

    kind "prenorm": ``h += mixer(norm1(h)); h += ffn(norm2(h))``.
    kind "sandwich": ``h += norm1_post(mixer(norm1(h))); h += norm2_post(ffn(norm2(h)))``;
    ``ffn`` None leaves the second sublayer (and its norms) out.
    kind "postnorm": ``h += residual_mult * norm1_post(mixer(h)); h += residual_mult *
    norm2_post(ffn(h))``: the sublayers read the residual itself (``norm1`` and ``norm2`` are
    None), only their outputs are normed.
    kind "hyper": hyper-connections.  The residual is ``streams`` copies ``x_1 .. x_s`` (all
    equal to the embedding output at first); sublayer q reads ``norm_q(sum_s in_q[s] x_s)``
    and then, all copies at once from the old ones, ``x_t = sum_s mix_q[s, t] x_s +
    residual_mult * out_q[t] * y``; the model's residual is the sum of the copies.  ``streams``
    0 is the plain ``x += residual_mult * sublayer(norm(x))`` through the same kernels.
    ``ffn`` None leaves the second sublayer out.
    ``mixer`` / ``ffn`` are any registered spec; they may differ from block
    to block within one model.
    """

    kind: str
    mixer: object
    ffn: object
    norm1: Optional[NormSpec]
    norm2: Optional[NormSpec]
    norm1_post: Optional[NormSpec] = None
    norm2_post: Optional[NormSpec] = None
    residual_mult: float = 1.0
    streams: int = 0


@dataclass(frozen=True)
class RunEntry:
    """One position in the execution order.

    ``block``: index into ``ModelLayout.blocks`` (a block may appear twice,
    its weights are then shared).  ``cache``: index of the cache this run
    reads and writes; by default every run has its own.  A run whose mixer
    ``shares_kv`` names the cache of the earlier run it reads.
    """

    block: int
    cache: int


@dataclass(frozen=True)
class ModelLayout:
    vocab_size: int
    hidden_size: int
    blocks: Sequence[BlockSpec]
    order: Sequence[RunEntry]
    final_norm: NormSpec
    tie_word_embeddings: bool = False
    # position ids run over [0, max_positions); None: no limit is known
    max_positions: Optional[int] = None
    # what turns token ids into the residual and normed rows into logits; None: a plain
    # table and a plain linear head of the layout's sizes
    embedding: Optional[object] = None
    head: Optional[object] = None

    def embedding_spec(self):
        return self.embedding or EmbeddingSpec(vocab_size=self.vocab_size,
                                               hidden_size=self.hidden_size)

    def head_spec(self):
        return self.head or HeadSpec(vocab_size=self.vocab_size, hidden_size=self.hidden_size)

    def num_caches(self) -> int:
        return 1 + max((e.cache for e in self.order), default=-1)

    def validate(self) -> None:
        if not self.blocks:
            raise ValueError("a model layout needs at least one block")
        owners: dict[int, int] = {}
        for pos, entry in enumerate(self.order):
            if not 0 <= entry.block < len(self.blocks):
                raise ValueError(f"run order entry {pos} names block {entry.block}, "
                                 f"but the layout has {len(self.blocks)} blocks")
            mixer = self.blocks[entry.block].mixer
            if getattr(mixer, "shares_kv", False):
                if entry.cache not in owners:
                    raise ValueError(f"run order entry {pos} reads cache {entry.cache} "
                                     "before any earlier entry has written it")
            else:
                if entry.cache in owners:
                    raise ValueError(f"cache {entry.cache} is written by run order entries "
                                     f"{owners[entry.cache]} and {pos}")
                owners[entry.cache] = pos
        missing = sorted(set(range(self.num_caches())) - set(owners))
        if missing:
            raise ValueError(f"caches {missing} are never written")
