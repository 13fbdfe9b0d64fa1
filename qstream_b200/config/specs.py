"""Typed descriptions of the parts a model is put together from.

A spec says which part to build (`kind`, looked up in the part registries), with
which sizes and constants, and under which checkpoint names its tensors lie
(`names`: the part's own tensor name -> the name in the safetensors file).  A spec
holds no weights and no code.  An architecture's configuration produces one
`ModelSpec`; nothing below it knows the architecture's name.

Any object with a `kind` attribute may serve as a spec of a part registered under
that kind, so a new part brings its own spec class.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Mapping, Optional, Tuple


@dataclass(frozen=True)
class NormSpec:
    """LayerNorm: mean and biased variance over `size`, eps inside the root,
    weight and (if `bias`) bias (QStream src/kernels_scalar.c:151-171)."""
    size: int
    eps: float
    bias: bool = True
    kind: str = "layernorm"
    names: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class RmsNormSpec:
    """RMS norm: x / sqrt(mean(x^2) + eps) * (offset + weight), eps inside the root.  `offset` 1 is for
    weights stored around zero, 0 for plain weights."""
    size: int
    eps: float
    offset: float = 0.0
    kind: str = "rmsnorm"
    names: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class PositionSpec:
    """Rotary position encoding on the first `rotary_dim` dims of each head,
    pairs (i, i+1) (QStream src/engine.c:205-234 with head_dim -> rotary_dim)."""
    rotary_dim: int
    base: float
    max_positions: int
    kind: str = "rotary_interleaved"


@dataclass(frozen=True)
class AttentionSpec:
    """Causal softmax attention over the sequence's cache.

    `window` = 0 reads all keys, w > 0 the last w (the query's own included).
    `shares_cache`: the layer projects queries only and reads the keys and values
    that another layer of the schedule wrote.
    `v_head_dim`: the values' head size where it differs from that of queries and keys.
    `score_scale`: the factor on q.k (default head_dim^-1/2).  `softcap` c > 0: scores
    become c tanh(s / c) before the softmax.  `gate`: the concatenated heads are multiplied
    by sigmoid(W_g h) before the output projection.  `value_mix`: "first" keeps the layer's
    values for later layers of the same step, "blend" caches (1 - l) v + l v_first with its
    scalar tensor "value_mix" as l.
    """
    width: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    position: Optional[PositionSpec] = None
    window: int = 0
    qkv_bias: bool = False
    out_bias: bool = False
    shares_cache: bool = False
    kind: str = "attention"
    names: Mapping[str, str] = field(default_factory=dict)
    v_head_dim: Optional[int] = None
    score_scale: Optional[float] = None
    softcap: float = 0.0
    gate: bool = False
    value_mix: Optional[str] = None

    @property
    def scale(self) -> float:
        return self.head_dim ** -0.5 if self.score_scale is None else float(self.score_scale)

    @property
    def value_dim(self) -> int:
        return self.head_dim if self.v_head_dim is None else self.v_head_dim


@dataclass(frozen=True)
class DecayAttentionSpec:
    """Linear attention with a fixed decay per head: S_t = decay_h S_{t-1} + k_t v_t^T, o_t = S_t^T q_t, with
    `activation` on q, k and v; the concatenated heads get one RMS norm (plain weight), a sigmoid gate from
    the mixer's input, and the output projection.  State: [heads, value_dim, key_dim] in 32-bit per sequence."""
    width: int
    n_heads: int
    key_dim: int
    value_dim: int
    decay: Tuple[float, ...]
    eps: float
    activation: str = "silu"
    kind: str = "lightning"
    names: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class WkvSpec:
    """RWKV-style time mixing: five mixes of the input with the previous token's, r/k/v/gate projections,
    a decay exp(-exp(.)) per token and channel from a two-matrix bottleneck of `decay_rank` (-1: whatever
    the checkpoint holds), a bonus for the current token, a unit RMS per head, a weight, the gate, and the
    output projection.  State: [heads, head_dim, head_dim] in 32-bit and the previous input per sequence."""
    width: int
    n_heads: int
    head_dim: int
    eps: float
    decay_rank: int = -1
    kind: str = "wkv"
    names: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class MlpSpec:
    """Dense feed-forward: up projection, activation, down projection
    (QStream src/engine.c:1150-1170), with biases if `bias`."""
    width: int
    inner: int
    activation: str
    bias: bool = True
    kind: str = "mlp"
    names: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class GatedMlpSpec:
    """Gated feed-forward without biases: down(act(gate h) * (up h))."""
    width: int
    inner: int
    activation: str = "silu"
    kind: str = "gated_mlp"
    names: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class BlockSpec:
    """One layer: its norms, mixer and feed-forward, and how they are wired.

    arrangement "parallel": h = norm(x); x + mixer(h) + ffn(h)   (norms: "input")
    arrangement "sequential": x += mixer(norm_1(x)); x += ffn(norm_2(x))
                                                     (norms: "input", "post_mixer")
    arrangement "scaled_residual": the same with x kept in 32-bit whatever the engine's type and
        every branch multiplied by `residual_scale`: x += m mixer(norm_1(x)); x += m ffn(norm_2(x));
        `ffn` may be None (then only "input" is needed).
    """
    mixer: object
    ffn: object
    norms: Mapping[str, object]
    arrangement: str = "parallel"
    residual_scale: float = 1.0


@dataclass(frozen=True)
class LayerRun:
    """One entry of the schedule: run layer `layer` against cache entry `cache`.
    A layer may appear in several runs; two runs may name the same cache entry
    when the later one only reads it.  For a layer with several parts that use the
    cache, `cache` is a tuple with one entry id per such part."""
    layer: int
    cache: object


@dataclass(frozen=True)
class EmbeddingSpec:
    vocab_size: int
    width: int
    kind: str = "embedding"
    names: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class PairEmbeddingSpec:
    """x = table[token] * scale + pair[(previous token * mul_prev + token * mul_cur) mod buckets], the pair
    table's last row (number `buckets`) for a sequence's first token; `buckets` 0: no pair table.
    `stream_dtype`: the type of x where it is not the engine's ("float32": a 32-bit residual stream)."""
    vocab_size: int
    width: int
    scale: float = 1.0
    buckets: int = 0
    mul_prev: int = 0
    mul_cur: int = 0
    stream_dtype: Optional[str] = None
    kind: str = "pair_embedding"
    names: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class HeadSpec:
    """Output projection to the vocabulary, logits in 32-bit.  `tied` reuses the
    embedding table as its weight."""
    vocab_size: int
    width: int
    bias: bool = True
    tied: bool = False
    kind: str = "lm_head"
    names: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    width: int
    max_positions: int
    embedding: object
    layers: Tuple[BlockSpec, ...]
    schedule: Tuple[LayerRun, ...]
    final_norm: Optional[object]            # None: the head sees the last layer's output as it is
    head: object
    stop_tokens: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None

    def n_cache_entries(self) -> int:
        ids = [c for r in self.schedule for c in (r.cache if isinstance(r.cache, (tuple, list)) else (r.cache,))]
        return 1 + max(ids, default=-1)
