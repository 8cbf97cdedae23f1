"""Architecture-neutral description of a model: what each layer is made of.

A model is a token embedding, a tuple of blocks, a schedule that says in which
order the blocks run, a final norm and an output head.  Every block names its
parts (mixer, feed-forward, norms) by a spec object; a spec carries every size
and constant the part needs and a ``kind`` string under which the part registry
(``parts/registry.py``) finds the class that builds it.  Blocks may differ from
one another, so one model can mix several mixers and feed-forwards.

The reference keeps the same facts in ``BnConfig`` plus per-layer kinds
(include/model_config.h:15-53, include/model_weights.h:9-17) and decides per
layer in its planner (src/transformer/plan.c:315-342).  Here they are plain
data so that an architecture module only has to translate its ``config.json``
into these records.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional, Tuple


@dataclass(frozen=True)
class RmsNormSpec:
    """Root-mean-square norm over the last axis with a learned gain."""

    width: int
    eps: float
    kind: str = "rmsnorm"
    optional: bool = False  # the file may lack the gain; the norm is then not applied by who owns it
    one_plus: bool = False  # the file holds the gain minus one: the factor is 1 + w


@dataclass(frozen=True)
class RotarySpec:
    """Rotary position encoding in the rotate-half pairing (i, i + rotary_dims/2)."""

    head_dim: int
    theta: float
    rotary_dims: int = 0  # 0 means the whole head
    kind: str = "rotary"

    @property
    def dims(self) -> int:
        return self.rotary_dims or self.head_dim


@dataclass(frozen=True)
class RotaryPairsSpec:
    """Rotary position encoding in the interleaved pairing (2i, 2i + 1): the pair i of the rotated part is turned
    by position * base^(-2i/dims).  ``scaling`` = (factor, low, high, original) slows long wavelengths down:
    beyond original / low by ``factor``, between original / high and original / low by a blend of both."""

    dims: int
    base: float
    scaling: Optional[Tuple[float, float, float, float]] = None
    kind: str = "rotary_pairs"


@dataclass(frozen=True)
class RotaryBlendSpec:
    """Rotary position encoding over a table of frequencies base^(-2i/dims) whose slow ones are divided by ``factor``:
    with turns(t) = dims * ln(original / (2 pi t)) / (2 ln base), lo = max(floor(turns(fast)), 0),
    hi = min(ceil(turns(slow)), dims - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1) the frequency
    is f_i / factor * ramp_i + f_i * (1 - ramp_i); cos and sin are both multiplied by
    ``magnitude_slope`` * ln(factor) + 1.  ``factor`` 1: the plain table.  ``pairing`` "halves": number i is turned
    with number i + dims / 2; "neighbours": number 2i with number 2i + 1."""

    dims: int
    base: float
    factor: float = 1.0
    original: float = 0.0
    fast: float = 32.0
    slow: float = 1.0
    magnitude_slope: float = 0.1
    pairing: str = "halves"
    kind: str = "rotary_blend"


@dataclass(frozen=True)
class NoPositionSpec:
    """No position encoding at all."""

    kind: str = "none"


@dataclass(frozen=True)
class AttentionSpec:
    """Causal softmax attention with grouped key/value heads over the paged cache."""

    width: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    position: Any  # a position spec (RotarySpec, NoPositionSpec, ...)
    scale: float = 0.0  # 0 means 1/sqrt(head_dim)
    window: int = 0  # 0 means every earlier key; w>0 means the last w keys
    kind: str = "attention"

    @property
    def q_dim(self) -> int:
        return self.n_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.n_kv_heads * self.head_dim

    @property
    def softmax_scale(self) -> float:
        return self.scale if self.scale > 0 else self.head_dim ** -0.5


@dataclass(frozen=True)
class BiasAttentionSpec:
    """Causal softmax attention with grouped key/value heads in its general form: value heads of a width
    of their own, queries and keys optionally divided by their root mean square per head, an optional
    learned bias by log-bucketed distance, a window that may keep the first tokens, an optional logistic
    gate per head on the output, and keys and values that may be another run's."""

    width: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    v_head_dim: int
    scale: float
    window: int = 0  # 0: every earlier key; w > 0: the last w keys ...
    keep_first: int = 0  # ... and the keys at positions below this
    unit_norm: bool = False  # q and k divided by their root mean square over the head (eps: norm_eps)
    norm_eps: float = 1e-6
    bias_buckets: int = 0  # rows of the distance-bias table; 0: no bias
    bias_max_distance: int = 0  # the distance from which on the last bucket is used
    head_gate: bool = False  # one gate per head from the mixer's input
    own_kv: bool = True  # False: no key/value projections; the run reads another run's cache
    chunk: int = 0  # c > 0 (in place of a window): a token sees the earlier keys of its own chunk of c positions
    position: Any = None  # a position spec whose encoding q and k get (after the unit norm, if any); None: none
    values_are_keys: bool = False  # no value projection: the values are the keys as projected, before any encoding
    kind: str = "bias_attention"


@dataclass(frozen=True)
class NormedAttentionSpec:
    """Causal softmax attention with grouped key/value heads whose queries and keys pass an RMS norm with a gain,
    per head (``qk_norm`` "head": one gain of ``head_dim`` numbers for all heads) or over the whole projection of
    a token (``qk_norm`` "whole": all heads at once, gains as wide as the projections); biases on the projections;
    a factor 1 + ``temp_coef`` * ln(floor((position + 1) / ``temp_every``) + 1) on the queries; a sink in the
    softmax's denominator (``sink`` "zero": a score of 0, "learned": a score per head); a logistic gate per head.
    ``maps`` 2: every head has two maps of scores (queries and keys twice as wide, [map 1 | map 2]) over the same
    values, combined as a1 - lambda a2 with lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + ``diff``, divided by its
    root mean square over the head's values and multiplied by 1 - ``diff``."""

    width: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    v_head_dim: int
    scale: float
    window: int = 0  # 0: every earlier key; w > 0: the last w keys
    qk_norm: str = "none"  # "none" | "head" | "whole"
    norm_eps: float = 1e-6
    proj_bias: bool = False  # biases on the query, key and value projections
    out_bias: bool = False  # a bias on the output projection
    temp_coef: float = 0.0
    temp_every: int = 0  # 0: no factor on the queries
    sink: str = "none"  # "none" | "zero" | "learned"
    head_gate: bool = False
    maps: int = 1
    diff: float = 0.0
    kind: str = "normed_attention"


@dataclass(frozen=True)
class SigmoidAttentionSpec:
    """Causal attention without a softmax: a visible key weighs sigmoid(q . k * scale + bias) and nothing is
    normalised over the keys.  Grouped key/value heads with value heads of a width of their own; optionally an
    RMS norm with a gain over the whole query projection and one over the whole key projection (all heads of a
    token at once); a learned bias by log-bucketed distance; a bias per head inside the logistic function; the
    heads' weights mixed by a learned matrix (weight_h <- sum_g M[h, g] weight_g, each head applying its mixed
    weights to the values of its own key/value head); values blended with those of another layer
    (``value_mix``: "source" keeps its values for later layers of the same ``value_group``, "blend" computes
    v <- (1 - l) v + l v_source with a learned l and caches that); a logistic gate on every output number."""

    width: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    v_head_dim: int
    scale: float
    window: int = 0  # 0: every earlier key; w > 0: the last w keys
    whole_norm: bool = True  # RMS norms over the whole query and key projections, each with a gain
    norm_eps: float = 1e-6
    bias_buckets: int = 0  # rows of the distance-bias table; 0: no bias
    bias_max_distance: int = 0  # the distance from which on the last bucket is used
    head_bias: bool = True  # a learned number per head added to the score
    head_mix: bool = True  # the heads' weights are mixed by a learned [heads, heads] matrix
    value_mix: str = "none"  # "none" | "source" | "blend"
    value_group: str = "v"  # layers that blend read the source of the same group
    output_gate: bool = True  # the heads' outputs times the logistic function of a projection of the mixer's input
    kind: str = "sigmoid_attention"


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Softmax attention through low-rank latents: queries from a normed latent of ``q_rank`` numbers (0: straight
    from the mixer's input); per token
    one normed latent of ``kv_rank`` numbers, from which every head's unrotated keys (``head_dim``) and values
    (``v_head_dim``) come, and one rotated key part of ``rot_dim`` numbers that all heads share.  Only the latent
    and the rotated part are cached.  ``window``: the last so many keys (0: all); a logistic gate per head
    (``head_gate``) or per output number (``element_gate``); ``sink``: a learned score per head in the softmax's
    denominator, without a key or a value."""

    width: int
    n_heads: int
    head_dim: int
    rot_dim: int
    v_head_dim: int
    q_rank: int
    kv_rank: int
    scale: float
    position: Any  # the encoding of the rotated parts (dims = rot_dim)
    norm_eps: float
    window: int = 0
    head_gate: bool = True
    element_gate: bool = False
    sink: bool = False
    kind: str = "latent_attention"


@dataclass(frozen=True)
class DeltaRuleSpec:
    """Gated delta rule with one decay per head and key channel: short causal convolutions and SiLU on q, k, v;
    unit q and k; beta and the decays from the mixer's input (the decays through ``decay_rank`` numbers); a
    per-head unit norm with a shared gain and a logistic gate (through ``gate_rank`` numbers) on the output."""

    width: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    v_head_dim: int
    conv_taps: int
    decay_rank: int
    gate_rank: int
    norm_eps: float
    kind: str = "delta_rule"


@dataclass(frozen=True)
class MlstmSpec:
    """mLSTM: a matrix memory per head with exponential gating, a soft cap on the gates' pre-activations,
    a unit norm per head, a gain over all heads and a logistic output gate."""

    width: int
    n_heads: int
    head_dim: int
    v_head_dim: int
    gate_cap: float
    norm_eps: float
    kind: str = "mlstm"


@dataclass(frozen=True)
class MoeSpec:
    """Mixture of clamped gated experts with logistic router scores, optionally with a shared expert."""

    width: int
    n_experts: int
    top: int
    expert_ff: int
    expert_limit: float
    shared_ff: int = 0  # 0: no shared expert
    shared_limit: float = 0.0
    slope: float = 1.702  # the activation is g * sigmoid(slope * g) * (u + 1)
    weight_on_input: bool = True  # the router weight multiplies the expert's input (False: its output)
    renormalise: bool = False  # divide the chosen experts' weights by their sum
    # the router's scores: "sigmoid" of each logit, or "softmax" over all experts; "table": no router, a table
    # [``table_rows``, top] of expert ids by token id chooses, and every chosen expert weighs 1 / top
    scores: str = "sigmoid"
    table_rows: int = 0
    weight_scale: float = 1.0  # factor on the (renormalised) weights
    renormalise_eps: float = 0.0  # added to the sum the weights are divided by
    activation: str = "limited"  # "limited": the clamped unit above; "silu" / "gelu_tanh": act(g) * u, no clamps
    kind: str = "moe"


@dataclass(frozen=True)
class GatedMlpSpec:
    """Dense feed-forward ``down(act(gate x) * up x)``."""

    width: int
    intermediate: int
    activation: str = "silu"  # or "gelu_tanh"
    wide_output: bool = False  # the delta leaves the last product in float32 instead of the compute type
    kind: str = "gated_mlp"


@dataclass(frozen=True)
class LimitedMlpSpec:
    """Dense feed-forward with the clamped gated unit: down(g * sigmoid(slope g) * (u + 1)) with
    g = min(gate x, limit), u = clamp(up x, -limit, limit)."""

    width: int
    intermediate: int
    limit: float
    slope: float = 1.702
    kind: str = "limited_mlp"


@dataclass(frozen=True)
class BlockSpec:
    """One block: which mixer, which feed-forward, which norms, and how they are arranged."""

    mixer: Any
    ffn: Any
    mixer_norm: Any
    ffn_norm: Any
    kind: str = "pre_norm"


@dataclass(frozen=True)
class PostNormBlockSpec:
    """A block whose norms follow the sums: x <- norm(alpha x + mixer(x)), x <- norm(alpha x + ffn(x)).
    ``ffn`` may be None (no feed-forward); ``ffn_norm`` is then applied to alpha x if it is given."""

    mixer: Any
    ffn: Any
    mixer_norm: Any
    ffn_norm: Any
    alpha: float = 1.0
    kind: str = "post_norm"


@dataclass(frozen=True)
class SandwichBlockSpec:
    """A block with a norm before and after each sublayer: x <- x + post(mixer(pre(x))), then
    x <- x + ffn_post(ffn(ffn_pre(x))).  ``ffn`` may be None (the second step is then left out).  ``label``: the
    name under which the block's parameters are listed (``blocks.<label>...``) when it is not its index."""

    mixer: Any
    ffn: Any
    mixer_norm: Any
    mixer_post_norm: Any
    ffn_norm: Any = None
    ffn_post_norm: Any = None
    label: Optional[str] = None
    kind: str = "sandwich"


@dataclass(frozen=True)
class TokenSideSpec:
    """A small input by token id at the end of a block: e = table[token, column : column + dim];
    y = proj (act(gate x) * e); x <- x + y / rms(y) * gain.  ``table_width``: the row of the table, which the
    blocks of a model share, each with its own columns."""

    width: int
    vocab_size: int
    dim: int
    column: int
    table_width: int
    eps: float
    activation: str = "gelu_tanh"
    kind: str = "token_side"


@dataclass(frozen=True)
class ParallelBlockSpec:
    """A block with one norm whose output both sublayers read: x <- x + (mixer(norm(x)) + ffn(norm(x))); then
    ``side`` (optional), which adds an input of its own.  ``ffn`` may be None.  With ``ffn_norm`` the feed-forward
    reads a second norm of the same x: x <- x + (mixer(norm(x)) + ffn(ffn_norm(x)))."""

    mixer: Any
    ffn: Any
    norm: Any
    side: Any = None
    ffn_norm: Any = None
    kind: str = "parallel"


@dataclass(frozen=True)
class LinearHeadSpec:
    """The output head: logits = scale * (W h), then optionally ``softcap * tanh(logits / softcap)``
    (the reference's final soft-cap, src/transformer/logits.c:325-333; 0 means none).  W is the
    head matrix, or the embedding table when the embeddings are tied."""

    scale: float = 1.0
    softcap: float = 0.0
    kind: str = "linear"


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a block.

    ``block`` indexes ``ModelSpec.blocks``; the same block may appear in several
    entries and then runs with the same weights more than once.  ``cache_of``
    names an *earlier schedule entry* whose cache this run reads instead of
    owning one (the reference's ``kv_reuse_layer``, src/transformer/cpu.c:496-498).
    """

    block: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    vocab_size: int
    width: int
    blocks: Tuple[BlockSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: Any
    max_positions: int
    tie_embeddings: bool = False
    embedding_scale: float = 1.0
    embedding_norm: Any = None  # a norm spec: the embedding rows are normed before the first block reads them
    stop_ids: Tuple[int, ...] = field(default_factory=tuple)
    head: Any = field(default_factory=LinearHeadSpec)  # a head spec; its part turns normed rows into logits

    def validate(self) -> None:
        if self.vocab_size <= 0 or self.width <= 0 or self.max_positions <= 0:
            raise ConfigError("vocab_size, width and max_positions must be positive")
        if not self.blocks or not self.schedule:
            raise ConfigError("a model needs at least one block and one schedule entry")
        for i, e in enumerate(self.schedule):
            if not 0 <= e.block < len(self.blocks):
                raise ConfigError(f"schedule entry {i} names block {e.block}, "
                                  f"but there are {len(self.blocks)} blocks")
            if e.cache_of is not None:
                if not 0 <= e.cache_of < i:
                    raise ConfigError(f"schedule entry {i} reads the cache of entry "
                                      f"{e.cache_of}, which does not run before it")
                if self.schedule[e.cache_of].cache_of is not None:
                    raise ConfigError(f"schedule entry {i} reads the cache of entry "
                                      f"{e.cache_of}, which owns none")


class ConfigError(ValueError):
    """A configuration that cannot be built; the message names the key and the value."""
