"""What a model is made of, as data.

A `ModelSpec` lists layers; a layer names its block arrangement, its mixer, its
feed-forward and its norms; each of those is a small frozen record with a `kind` (the
key under which the part is registered in `parts.registry`) and the sizes and constants
the part needs.  `schedule` is the order in which layers run: a list of layer indices
that may name a layer twice.  A layer whose `cache_from` names another layer reads that
layer's cache and keeps none of its own.  Nothing in this file knows an architecture;
`models/` turns a config.json into these records.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional


@dataclass(frozen=True)
class NormSpec:
    size: int
    eps: float
    name: str                      # tensor name of the weight, relative to the owner's prefix
    kind: str = "rmsnorm"          # "rmsnorm", or "dyt": tanh(alpha * x) * weight + bias (`<name>.alpha`, `<name>.b`)
    offset: float = 0.0            # rmsnorm: the stored weight plus this number multiplies (1.0: the file holds weight - 1)


@dataclass(frozen=True)
class RopeSpec:
    dim: int                       # number of rotated elements of a head (<= head size, even)
    theta: float
    kind: str = "rope"
    exact_table: bool = False      # the frequency table is formed in 64-bit and rounded once (else in 32-bit)
    scaling_factor: float = 1.0    # linear scaling: every frequency is divided by this number
    layout: str = "halves"         # pairs of the rotation: "halves" (i with i + dim/2) or "interleaved" (2i with 2i + 1)


@dataclass(frozen=True)
class AttentionSpec:
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float                   # multiplies q.k before the softmax
    position: Optional[Any] = None  # a position-encoding spec, or None
    qk_norm_eps: Optional[float] = None  # per-head RMSNorm of queries and keys, or None
    window: Optional[int] = None   # keys visible to a query: the last `window`, or all
    prefix: str = "self_attn"
    kind: str = "attention"


@dataclass(frozen=True)
class GatedMLPSpec:
    hidden_size: int
    intermediate_size: int
    activation: str = "silu"
    prefix: str = "mlp"
    kind: str = "gated_mlp"


@dataclass(frozen=True)
class TwinMapsSpec:
    """Two score maps per head over the same values (the projections hold, head by head, [map 1 | map 2]):
    o = a1 - lam * a2 with lam = exp(lq1 . lk1) - exp(lq2 . lk2) + offset, one number for the layer from four
    vectors of the key size; then a weightless RMSNorm over the head's values (eps) times (1 - offset)."""
    offset: float
    eps: float
    names: tuple = ("lq1", "lk1", "lq2", "lk2")


@dataclass(frozen=True)
class GeneralAttentionSpec:
    """Causal grouped-query attention whose options are data: keys and values of different sizes; rotation of a
    leading part of every head; RMSNorm over a token's WHOLE query (key) projection; values that are the keys as
    projected; a query temperature 1 + coef * ln(floor((p + 1) / every) + 1); scores capped by tanh; softmax
    or independent sigmoid weights with a bias per head; two score maps per head; a sigmoid output gate per head
    or per element."""
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    key_dim: int
    value_dim: int
    scale: float
    position: Optional[Any] = None         # rotation of the first position.dim elements of every head, or None
    whole_norm_eps: Optional[float] = None  # RMSNorm over all heads of q (of k) at once, weights of that size
    values_from_keys: bool = False          # v = k as projected (before norm and rotation); no value projection
    query_temperature: Optional[tuple] = None   # (coef, every)
    score_cap: Optional[float] = None       # score <- cap * tanh(score / cap)
    weights: str = "softmax"                # "softmax", or "sigmoid": sigmoid(score + bias_h), not normalised
    score_bias: bool = False                # a number per head added to the score (sigmoid weights)
    twin: Optional[TwinMapsSpec] = None
    gate: Optional[str] = None              # "head": one sigmoid gate a head; "element": one per output element
    head_temperature: bool = False          # a learned number per query head multiplies its scaled scores
    # a learned bias by distance, added to the score after scale and temperature: (buckets or None = the table's own
    # row count, the distance from which the last bucket serves); see parts.general_attention.distance_buckets
    distance_bias: Optional[tuple] = None
    sink: bool = False                      # exp(a learned number per head) counts once in the softmax's denominator
    # RMSNorm of every query and key head with ONE weight vector of the key size that all heads share (the norms'
    # names serve both kinds; a layer has the whole-projection norm or this one)
    head_norm_eps: Optional[float] = None
    value_norm_eps: Optional[float] = None  # every value head divided by its root mean square (no weight); cached so
    # values rotated by their own position over their whole size (frequencies theta^(-2m/value_dim), never scaled, the
    # position encoding's theta and layout), cached so; every head's output turned back by the query's position
    rotate_values: bool = False
    window: Optional[int] = None            # a query sees its own position and the window - 1 before it
    chunk: Optional[int] = None             # a query sees the earlier positions of its chunk, chunks counted from 0
    prefix: str = "mix"
    # tensor names below the prefix: queries, keys, values, gate, output, whole-projection norms, score bias,
    # temperature, distance bias, sink
    names: tuple = ("q", "k", "v", "g", "o", "q.norm", "k.norm", "pb", "temp", "rel", "sink")
    kind: str = "general_attention"


@dataclass(frozen=True)
class StateSpaceSpec:
    """A Mamba-2 mixer (state-space duality): the input product gives [z | x | B | C | dt]; x, B and C pass a short
    causal convolution with a bias and silu; per head a state S [state, value_dim] with S <- exp(-exp(A_log) dt) S +
    dt B x^T, y = S^T C + D x, dt = softplus(dt + dt_bias); B and C are shared by the heads of a group; y times
    silu(z), RMS-normed in `norm_groups` equal parts, times a weight, then the output product."""
    hidden_size: int
    num_heads: int
    value_dim: int
    state_dim: int
    groups: int
    norm_groups: int
    conv_taps: int
    norm_eps: float
    prefix: str = "mix"
    # input product, convolution and its bias, step bias, log of the decay rate, skip, norm weight, output product
    names: tuple = ("in", "conv", "conv.b", "dt_bias", "A_log", "D", "norm", "o")
    kind: str = "state_space"


@dataclass(frozen=True)
class DeltaRuleSpec:
    """A matrix state per head under the generalized delta rule (per token: a decay per key channel, the removal of
    what the state holds along the unit key, then the new key-value pair); keys and values of one size.  The decay
    comes from a low-rank pair of matrices whose rank is the first matrix's row count."""
    hidden_size: int
    num_heads: int
    head_dim: int
    norm_eps: float                # of the per-head unit norm of the output
    decay_rank: Optional[int] = None   # None: taken from the tensor
    prefix: str = "mix"
    # receptance, key, value, output gate, removal gate and its bias, decay down- and up-projection and its bias,
    # output norm weight, output projection
    names: tuple = ("r", "k", "v", "g", "a", "a.b", "w1", "w2", "w0", "norm", "o")
    kind: str = "delta_rule"


@dataclass(frozen=True)
class MatrixMemorySpec:
    """A matrix memory per head with an exponential input gate, a sigmoid forget gate (both capped by tanh in the log
    domain), a normaliser vector and a running maximum that keeps the exponentials in range."""
    hidden_size: int
    num_heads: int
    key_dim: int
    value_dim: int
    gate_cap: float
    norm_eps: float
    prefix: str = "mix"
    # query, key, value, output gate, input gate and its bias, forget gate and its bias, output norm weight, output
    names: tuple = ("q", "k", "v", "g", "i", "i.b", "f", "f.b", "norm", "o")
    kind: str = "matrix_memory"


@dataclass(frozen=True)
class MixerPairSpec:
    """Two mixers that read the same input; the result is coef * (rms(left) * w_left + rms(right) * w_right) with a
    plain RMSNorm over the model width on each output."""
    hidden_size: int
    left: Any
    right: Any
    eps: float
    coef: float = 0.5
    prefix: str = "mix"
    names: tuple = ("left.out", "right.out")
    kind: str = "mixer_pair"


@dataclass(frozen=True)
class DenseMLPSpec:
    """A feed-forward without a gate: down(act(up(x)))."""
    hidden_size: int
    intermediate_size: int
    activation: str = "relu2"               # "relu2": relu(z)^2; "gelu": the exact (erf) gelu; "tanh"
    prefix: str = "mlp"
    names: tuple = ("up", "down")
    kind: str = "dense_mlp"


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Attention whose keys and values are made from one low-rank latent per token: a query head is
    [plain_dim | rot_dim]; a token leaves a normed latent of `latent_dim` and one rotated key part of `rot_dim`
    that all heads share; head h's key is [W_uk_h latent | rotated part], its value W_uv_h latent."""
    hidden_size: int
    num_heads: int
    plain_dim: int                 # query/key elements of a head that are not rotated
    rot_dim: int                   # rotated elements of a head (the shared key part has this size)
    value_dim: int
    latent_dim: int
    scale: float
    position: Optional[Any] = None  # rotation of the rot_dim part, or None
    latent_norm_eps: float = 1e-6  # RMSNorm of the latent
    output_gate: bool = False      # heads multiplied by sigmoid(W_g x) before the output projection
    prefix: str = "self_attn"
    # tensor names below the prefix: queries, down-projection (latent | key part), latent norm, key and value
    # up-projections, gate, output
    names: tuple = ("q", "dkv", "dkv.norm", "uk", "uv", "g", "o")
    # queries through a latent of their own: c_q = RMSNorm(W_dq x) (eps = latent_norm_eps), q = W_uq c_q; the three
    # tensors' names below the prefix.  None: q = W_q x
    query_latent_dim: Optional[int] = None
    query_names: tuple = ("dq", "dq.norm", "uq")
    window: Optional[int] = None   # a query sees its own position and the window - 1 before it
    sink: Optional[str] = None     # tensor name below the prefix of a number per head: exp(sink) counts once in the
                                   # softmax's denominator, with no key and no value
    kind: str = "latent_attention"


@dataclass(frozen=True)
class RoutedExpertsSpec:
    """A mixture of small feed-forward experts down(act(up(x))): each token uses the `top_k` experts with the
    largest router scores; with `n_groups` > 1 the experts form equal groups of neighbours, a group scores as
    its best expert, and only experts of the `keep_groups` best groups can be chosen."""
    hidden_size: int
    num_experts: int
    top_k: int
    expert_size: int
    n_groups: int = 1
    keep_groups: int = 1
    scoring: str = "softmax"       # router scores: "softmax" over all experts, or "sigmoid" of each logit
    renormalize: bool = False      # whether the chosen scores are made to sum to one
    activation: str = "gelu"       # "gelu": down(gelu(up x)), exact (erf) gelu; "clamped_glu": experts with a gate
                                   #   matrix, g = min(gate x, limit), u = clamp(up x, +-limit), down(g sigmoid(1.702 g) (u + 1))
    group_score: str = "max"       # a group's score: its best expert's ("max") or the sum of its two best ("top2_sum")
    renorm_eps: float = 0.0        # added to the chosen scores' sum before the division
    weight_scale: float = 1.0      # multiplies the weights at the end
    limit: float = 0.0             # of the clamped activation
    prefix: str = "mlp"
    kind: str = "routed_experts"


@dataclass(frozen=True)
class TokenInputSpec:
    """A per-layer input that depends on the token id: e = columns [offset, offset + dim) of a shared table
    row; branch = proj(gelu_tanh(gate(x)) * e), normed by an RMSNorm of its own."""
    hidden_size: int
    dim: int
    offset: int                    # first column of this layer's part of a table row
    table_name: str                # full tensor name of the table [vocab, table_width]
    table_width: int
    vocab_size: int
    eps: float
    prefix: str = "side"
    kind: str = "token_input"


@dataclass(frozen=True)
class LayerSpec:
    prefix: str                    # e.g. "model.layers.3"
    mixer: Any
    feed_forward: Any              # None: the layer has no feed-forward (arrangements that allow it)
    mixer_norm: NormSpec
    ffn_norm: Optional[NormSpec]
    cache_from: Optional[int] = None
    kind: str = "pre_norm"
    residual_scale: float = 1.0    # multiplies every branch before it is added to the stream
    # pre_norm: tensor names (below the prefix) of a gate on each sublayer's result, sigmoid(W x + b) element by
    # element with x the sublayer's input (`<name>` [hidden, hidden], `<name>.b`), or None
    residual_gates: Optional[tuple] = None
    token_input: Any = None        # a further branch fed by the token id (TokenInputSpec), or None
    # pre_norm: what each sublayer reads, u, is replaced by u + conv(u), a short causal convolution over time on each
    # channel: (taps, (tensor name for the mixer's input, for the feed-forward's)), tensors [hidden, taps] below the
    # prefix; the last taps - 1 inputs of a sequence are part of its state.  None: no convolution
    input_conv: Optional[tuple] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    layers: tuple
    final_norm: NormSpec
    embedding_name: str = "model.embed_tokens.weight"
    lm_head_name: Optional[str] = "lm_head.weight"   # None: the embedding table is the output matrix
    schedule: tuple = field(default=())
    max_position: int = 0
    # places in the run order (indices into `run_order()`) right before which the embedding output is added to the
    # stream once more
    reinject: tuple = field(default=())
    # a learned vector per position added to the embedding: tensor [max_position, hidden], or None
    position_table_name: Optional[str] = None
    # learned vectors added to every token's stream right before places of the run order: (tensor name [rows, hidden],
    # ((place, row), ...)), or None
    pass_vectors: Optional[tuple] = None
    logit_softcap: Optional[float] = None   # logits <- cap * tanh(logits / cap)
    logit_scale: Optional[float] = None     # logits <- logits * scale
    unused_tensors: tuple = ()    # names that a folder may hold without the model reading them

    def run_order(self) -> tuple:
        return self.schedule if self.schedule else tuple(range(len(self.layers)))

    def validate(self) -> None:
        n = len(self.layers)
        for i in self.run_order():
            if not 0 <= i < n:
                raise ValueError(f"schedule names layer {i}, the model has {n}")
        for k in self.reinject:
            if not 0 < k < len(self.run_order()):
                raise ValueError(f"the embedding cannot be added again before place {k} of the run order")
        for i, layer in enumerate(self.layers):
            j = layer.cache_from
            if j is not None:
                if not 0 <= j < n or j == i or self.layers[j].cache_from is not None:
                    raise ValueError(f"layer {i}: cache_from={j} must name another layer that owns a cache")
                order = list(self.run_order())
                if j not in order or (i in order and order.index(j) > order.index(i)):
                    raise ValueError(f"layer {i} reads the cache of layer {j}, which must run before it")
