"""Descriptions of a model as data: which parts each layer is made of, with every size and
constant as a parameter, and the order in which layers run.

A description is built from a typed configuration by the architecture's `describe` function; no
part class is touched until the model is built. Each spec names its `kind`; the part registry
(parts/registry.py) maps (category, kind) to the class that implements it, so a new mixer,
feed-forward, norm or position encoding is a new spec class plus one registered part class, and a
model may use different kinds in different layers.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, FrozenSet, Optional, Tuple


@dataclass(frozen=True)
class TensorNeed:
    """One checkpoint tensor a part reads.
    precision: "compute" = a matrix that feeds matrix products, kept in the engine's dtype
               (bfloat16, or float32 on the 32-bit path);
               "float32" = always widened to float32 (norm weights and other vectors);
               "stored"  = kept as the file stores it (32-bit stays 32-bit, integer tables int32).
    init: what the random-weights mode draws for it: "normal" = N(0, std); "around_one" = N(1, std)
          (weights that multiply, such as a norm's); "zeros" (biases and other additive terms)."""
    name: str
    shape: Tuple[int, ...]
    precision: str = "compute"
    init: str = "normal"


@dataclass(frozen=True)
class NormSpec:
    kind: str
    dim: int
    eps: float
    weight: str  # checkpoint tensor name


@dataclass(frozen=True)
class PositionSpec:
    """kind "rope": rotary, half-split layout; `scaling` as in the configuration; kind "none"."""
    kind: str
    head_dim: int = 0
    theta: float = 10000.0
    max_positions: int = 0
    scaling_factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 1.0
    original_max_positions: int = 0  # 0: no rescaling of frequencies


@dataclass(frozen=True)
class ScaledRotarySpec:
    """kind "rope_ramp": rotary, half-split layout over the first `dims` numbers of the vector it is given.
    Pair i turns by position * f_i, f_i = base^(-2i/dims). With factor > 0 the frequencies are stretched
    along a ramp: turn(t) = dims * ln(original / (2 pi t)) / (2 ln base), lo = max(floor(turn(fast)), 0),
    hi = min(ceil(turn(slow)), dims - 1), ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1),
    f_i <- f_i / factor * ramp_i + f_i * (1 - ramp_i), and cos and sin are both multiplied by
    0.1 ln(factor) + 1. factor 0: plain frequencies, no multiplier."""
    kind: str
    dims: int
    base: float
    max_positions: int
    factor: float = 0.0
    original: float = 0.0
    fast: float = 0.0
    slow: float = 0.0


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Causal attention whose keys and values are maps of one cached latent per token (parts/latent_attention.py).
    heads H; per head `dim` unrotated and `rot_dim` rotated query/key numbers and `vdim` value numbers;
    `kv_rank` the latent of keys and values, `q_rank` the latent of queries. `scale` multiplies the scores as given."""
    kind: str
    hidden: int
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    eps: float
    position: object  # a position spec with rotation tables over `dims` <= rot_dim numbers
    dq_weight: str
    dq_norm: str
    uq_weight: str
    dkv_weight: str
    dkv_norm: str
    uk_weight: str
    uv_weight: str
    gate_weight: str
    o_weight: str
    window: int = 0


@dataclass(frozen=True)
class AttentionSpec:
    """Causal grouped-query attention. window = 0 keeps every key; W > 0 reads the last W."""
    kind: str
    hidden: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    position: PositionSpec
    q_weight: str
    k_weight: str
    v_weight: str
    o_weight: str
    window: int = 0
    scale: Optional[float] = None  # None: 1/sqrt(head_dim)


@dataclass(frozen=True)
class GatedMLPSpec:
    """down( act(gate(x)) * up(x) ), dense, no bias. activation "silu"."""
    kind: str
    hidden: int
    intermediate: int
    gate_weight: str
    up_weight: str
    down_weight: str
    activation: str = "silu"  # or "gelu_tanh"


@dataclass(frozen=True)
class RoutedMLPSpec:
    """Mixture of experts: logits = router x + router_bias in float32; each token uses the `top` experts with the largest
    logits, weighted by the softmax over the chosen logits; an expert is down_e(act(up_e(x))) without biases.
    up_weights / down_weights: one checkpoint name per expert. activation "gelu" (the exact, erf form)."""
    kind: str
    hidden: int
    intermediate: int
    experts: int
    top: int
    router_weight: str
    router_bias: Optional[str]
    up_weights: Tuple[str, ...]
    down_weights: Tuple[str, ...]
    activation: str = "gelu"


@dataclass(frozen=True)
class TokenSideSpec:
    """A per-layer input from the token itself, added after the layer: e = table[token, col0 : col0 + dim];
    y = proj(gelu_tanh(gate(x)) * e) for the stream x; x += y / rms(y) * norm (eps inside the root)."""
    kind: str
    hidden: int
    dim: int
    vocab_size: int
    table: str       # [vocab, table_width], shared by all layers
    table_width: int
    col0: int
    gate_weight: str  # [dim, hidden]
    proj_weight: str  # [hidden, dim]
    norm_weight: str  # [hidden]
    eps: float


@dataclass(frozen=True)
class BlockSpec:
    """kind "pre_norm": h += mixer(norm1(h)); h += feed_forward(norm2(h)).
    kind "parallel": h += mixer(norm1(h)) + feed_forward(norm2(h)), both of the same h (feed_forward and norm2 may be
    None: then the mixer alone); then, if `token_input` is given, h += token_input(h, tokens).
    mixer / feed_forward / token_input are any registered spec objects with a `kind`."""
    kind: str
    norm1: object
    mixer: object
    norm2: object
    feed_forward: object
    token_input: object = None


@dataclass(frozen=True)
class LayerRun:
    """One entry of the execution order: run `layer`; if `cache_from` names another layer, this
    run reads that layer's cache and writes none of its own. add_embedding: the embedding's output
    (the stream as it was before the first run) is added to the stream right before this run."""
    layer: int
    cache_from: Optional[int] = None
    add_embedding: bool = False


@dataclass(frozen=True)
class EmbeddingSpec:
    """kind "lookup": residual stream row = table row of the token id, widened to float32."""
    weight: str
    vocab_size: int
    dim: int
    kind: str = "lookup"


@dataclass(frozen=True)
class HeadSpec:
    """kind "linear": logits = x . W^T in float32, no bias, for the wanted rows only."""
    weight: str  # the embedding's name when input and output embeddings are tied
    vocab_size: int
    dim: int
    kind: str = "linear"


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    embedding: object  # any registered "embedding" spec with `kind`, `weight`, `vocab_size`, `dim`
    layers: Tuple[BlockSpec, ...]
    order: Tuple[LayerRun, ...]
    final_norm: object
    head: object       # any registered "head" spec with `kind`, `weight`, `vocab_size`, `dim`
    max_positions: int
    eos_token_ids: FrozenSet[int] = field(default_factory=frozenset)
    # names that may be present in the checkpoint without being read, each with the needed tensor
    # it must agree with in shape (a tied lm_head saved beside the embedding)
    duplicates: Dict[str, str] = field(default_factory=dict)
    # shell-style patterns of names that a checkpoint may carry and nobody reads (buffers that some
    # exporters save, such as "*.rotary_emb.inv_freq"); the reference maps whatever a file holds and
    # reads what it needs (src/weights.cpp:269-301), so it ignores them too
    ignore: Tuple[str, ...] = ()

    @property
    def vocab_size(self) -> int:
        return self.head.vocab_size

    @property
    def hidden_size(self) -> int:
        return self.embedding.dim
