"""What a model is made of, as data.

A ``ModelSpec`` lists blocks (one per distinct set of weights) and a run order. Each block names its mixer,
feed-forward, norms and arrangement by a spec object whose ``kind`` selects the part class from the part
registries (``roost_b200.parts``); every size and constant a part needs is a field of its spec. Nothing
here knows an architecture: an architecture module (``roost_b200.config.qwen3``) turns its config.json into
these objects, as the reference's model definition turns attributes into a node list whose ops take their
constants as arguments (src/Starlings.Roost.Models.Tiny/RoostTiny.cs:14-57).
"""
from __future__ import annotations

from dataclasses import dataclass, field


@dataclass(frozen=True)
class NormSpec:
    """``rms_norm``: x / sqrt(mean(x^2) + eps) * w. ``layer_norm``: (x - mean) / sqrt(var + eps) * w + b, var the mean squared
    deviation; it reads a 32-bit stream and writes the activation dtype. ``rms_norm_wide``: the first over a 32-bit stream,
    written in the activation dtype. ``weight_offset``: what is added to the stored
    weight before it multiplies (1.0 for weights stored around zero)."""
    size: int
    eps: float
    kind: str = "rms_norm"
    weight_offset: float = 0.0


@dataclass(frozen=True)
class PositionSpec:
    """Position encoding applied inside a mixer. ``rope_neox``: rotation of the first ``rotary_dim``
    elements of each head, pairs (i, i + rotary_dim/2), frequencies theta^(-2i/rotary_dim). ``rope_interleaved``: the same
    angles with element 2i paired with element 2i + 1."""
    kind: str = "rope_neox"
    rotary_dim: int = 0
    theta: float = 10000.0
    max_positions: int = 0


@dataclass(frozen=True)
class MixerSpec:
    kind: str = ""


@dataclass(frozen=True)
class AttentionSpec(MixerSpec):
    """Grouped-query causal attention over a paged cache. ``window`` counts the keys a query sees, its own
    included (Hugging Face ``sliding_window``); None means every earlier key."""
    kind: str = "paged_attention"
    hidden: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    scale: float = 0.0
    window: int | None = None
    qk_norm: NormSpec | None = None
    position: PositionSpec | None = None


@dataclass(frozen=True)
class LatentAttentionSpec(MixerSpec):
    """Causal attention whose keys and values are made per head from one latent vector a token: the cache keeps the
    latent (``kv_rank`` numbers, unit root mean square times a weight) and one rotated key part of ``rope_dim`` numbers
    that all heads share. A head's key is [W_uk c | shared part] against a query of ``nope_dim`` plain and ``rope_dim``
    rotated numbers, its value W_uv c of ``v_dim`` numbers. ``window`` counts the keys a query sees, its own included
    (None: all). ``own_latent`` False: the run makes no latent and reads another run's; ``cache_window`` is then the
    window the shared cache is kept for (the widest of the runs that read it; None: everything is kept). ``rope_dim`` 0 (and no
    ``position``): keys have no rotated part and the cache entry is the latent alone. ``head_gate``: head h's output is multiplied
    by sigmoid((W_g x)_h), one number a token and head, from the mixer's own input."""
    kind: str = "latent_attention"
    hidden: int = 0
    num_heads: int = 0
    nope_dim: int = 0
    rope_dim: int = 0
    v_dim: int = 0
    kv_rank: int = 0
    scale: float = 0.0
    window: int | None = None
    cache_window: int | None = None
    own_latent: bool = True
    latent_eps: float = 1e-6
    position: PositionSpec | None = None
    head_gate: bool = False


@dataclass(frozen=True)
class SinkAttentionSpec(MixerSpec):
    """Grouped-query causal attention whose values have a size of their own (``v_dim``) and whose softmax may have a sink:
    with ``sink`` the denominator is 1 + sum exp(s_j), a key of score 0 that has no value. Queries and keys are rotated
    (``position``) and then, with ``unit_norm_eps`` set, divided by their root mean square over ``head_dim`` (eps inside the
    root, no weight). ``window`` counts the keys a query sees, its own included (None: every earlier key). With ``softcap``
    c > 0 a score s (already scaled) becomes c tanh(s / c). ``bias``: the q, k and v projections add a stored vector. The
    cache keeps one entry [key | value] a token and key/value head, or keys and values in two planes when their sizes agree."""
    kind: str = "sink_attention"
    hidden: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    v_dim: int = 0
    scale: float = 0.0
    sink: bool = True
    unit_norm_eps: float | None = None
    position: PositionSpec | None = None
    window: int | None = None
    softcap: float = 0.0
    bias: bool = False


@dataclass(frozen=True)
class Mamba1Spec(MixerSpec):
    """The Mamba selective scan. The input projection gives [x | z] of ``inner`` channels each; x passes a causal
    convolution of ``conv_taps`` taps a channel and SiLU; a projection of x gives [dt (``dt_rank``) | B (``state``) | C
    (``state``)]; dt = softplus(W_dt dt + bias), one a channel; per channel c and state n S[c, n] <- exp(dt_c A[c, n]) S[c, n] +
    dt_c x_c B_n with A = -exp(A_log), y_c = sum_n S[c, n] C_n + D_c x_c; y SiLU(z) is projected out. S and the last
    ``conv_taps`` - 1 inputs of the convolution are kept per request in 32-bit."""
    kind: str = "mamba1"
    hidden: int = 0
    inner: int = 0
    state: int = 0
    dt_rank: int = 0
    conv_taps: int = 4


@dataclass(frozen=True)
class Mamba2Spec(MixerSpec):
    """The Mamba-2 recurrence. The input projection gives [z | x | B | C | dt]; x, B and C pass a causal convolution of
    ``conv_taps`` taps a channel and SiLU; per head (``head_dim`` values, state ``state`` x ``head_dim``, B and C shared by
    the heads of one of ``groups`` groups) S <- exp(-exp(A_log) dt) S + dt B x^T, y = S^T C + D x with dt = softplus(dt +
    dt_bias); y SiLU(z) is divided by its root mean square in ``norm_groups`` equal parts, times a weight, and projected
    out. The state and the last ``conv_taps`` - 1 inputs of the convolution are kept per request in 32-bit."""
    kind: str = "mamba2"
    hidden: int = 0
    num_heads: int = 0
    head_dim: int = 0
    state: int = 0
    groups: int = 1
    conv_taps: int = 4
    norm_groups: int = 1
    eps: float = 1e-6


@dataclass(frozen=True)
class GatedRecurrenceSpec(MixerSpec):
    """A gated linear recurrence a channel (the real-gated linear recurrent unit) between two branches of ``width`` channels:
    y = gelu_tanh(W_y h + b_y); u = conv(W_x h + b_x), a causal convolution of ``conv_taps`` taps a channel with a bias and no
    activation. u is cut into ``blocks`` equal parts; in each, r = sigmoid(R_b u_b + b) and i = sigmoid(I_b u_b + b) with square
    matrices; a = exp(-``rate`` r softplus(lam)); S <- a S + sqrt(1 - a^2) i u from S = 0; the output is W_o (S y). S and the
    convolution's last ``conv_taps`` - 1 inputs are kept per request in 32-bit."""
    kind: str = "gated_recurrence"
    hidden: int = 0
    width: int = 0
    blocks: int = 1
    conv_taps: int = 4
    rate: float = 8.0


@dataclass(frozen=True)
class MatrixMemorySpec(MixerSpec):
    """A matrix memory a head with exponential gates (the mLSTM cell). q = W_q h / sqrt(head_dim), k = W_k h, v = W_v h; per
    head the logarithms of an input gate i = c tanh((W_i h + b) / c) and of a forget gate f = logsigmoid(c tanh((W_f h + b) / c)),
    c = ``gate_cap``; with a running maximum m (from 0): m' = max(f + m, i), S <- exp(f + m - m') S + exp(i - m') k v^T, n likewise
    with k alone, o = S^T q / (max(|n . q|, exp(-m')) + ``floor``). Each head's o is divided by its root mean square (``eps``),
    the heads side by side are multiplied by a weight and by sigmoid(W_g h), then projected out. S, n and m are kept per
    request in 32-bit."""
    kind: str = "matrix_memory"
    hidden: int = 0
    num_heads: int = 0
    head_dim: int = 0
    v_dim: int = 0
    gate_cap: float = 0.0
    eps: float = 1e-6
    floor: float = 1e-6


@dataclass(frozen=True)
class RetentionSpec(MixerSpec):
    """A matrix state a head that fades by a constant factor a token and is read by the query as it is: nothing is exponentiated and
    nothing divides. q = W_q h, k = W_k h (``num_heads`` x ``head_dim``),
    v = W_v h (``num_heads`` x ``v_dim``); q and k are rotated (``position``), k then multiplied by head_dim^(-1/2); per head
    S <- decay_h S + k v^T from S = 0, o = S^T q. Each head's o is divided by its root mean square (``eps``, no weight); the heads side
    by side are multiplied by silu(W_g h) and projected out. S is kept per request in 32-bit."""
    kind: str = "retention"
    hidden: int = 0
    num_heads: int = 0
    head_dim: int = 0
    v_dim: int = 0
    decay: tuple = ()
    eps: float = 1e-6
    position: PositionSpec | None = None


@dataclass(frozen=True)
class SigmoidAttentionSpec(MixerSpec):
    """Grouped-query causal attention without a softmax: a visible key j gets the weight sigmoid(s_ij + b_h) of its own, and the
    weights are used as they are: nothing divides by their sum. Queries and keys are divided by their root mean square over the head (``qk_norm_eps``)
    and multiplied by a weight of ``head_dim`` numbers shared by the heads (one for queries, one for keys). ``temp_coef`` c > 0: the
    query at position p is multiplied by 1 + c ln(floor((p + 1) / ``temp_every``) + 1). s_ij = (q_i . k_j) ``scale`` - slope_h (i - j)
    with one ``slopes`` entry a query head (empty: no distance bias); b_h is a stored number a head (``head_bias``). With
    ``output_gate`` the heads side by side are multiplied element by element by sigmoid(W_g h) before the output projection. No
    position encoding. The cache keeps one entry [key | value] a token and key/value head, or two planes when their sizes agree."""
    kind: str = "sigmoid_attention"
    hidden: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    v_dim: int = 0
    scale: float = 0.0
    qk_norm_eps: float = 1e-6
    temp_coef: float = 0.0
    temp_every: int = 1
    slopes: tuple = ()
    head_bias: bool = True
    output_gate: bool = True


@dataclass(frozen=True)
class ParallelMixerSpec(MixerSpec):
    """Several mixers side by side that read the same input; the result is the mean of their outputs, each first divided by
    its root mean square over the model width (``eps``) and multiplied by a weight of its own. Every branch keeps the cache
    or state its own kind asks for."""
    kind: str = "parallel"
    hidden: int = 0
    branches: tuple = ()
    eps: float = 1e-6


@dataclass(frozen=True)
class FeedForwardSpec:
    kind: str = ""


@dataclass(frozen=True)
class GatedMlpSpec(FeedForwardSpec):
    """down(act(x Wg^T) * (x Wu^T)); ``activation`` is the gate's function: "silu", "gelu_tanh" (0.5 g (1 + tanh(sqrt(2/pi)
    (g + 0.044715 g^3)))), or "clamped_swish": with g = min(gate, limit) and u = clamp(up, -limit, limit) the product is
    g sigmoid(1.702 g) (u + 1)."""
    kind: str = "gated_mlp"
    hidden: int = 0
    intermediate: int = 0
    activation: str = "silu"
    limit: float = 0.0


@dataclass(frozen=True)
class DenseMlpSpec(FeedForwardSpec):
    """down(act(x Wu^T)), no gate. ``activation`` "xielu": with two stored numbers (p, q), act(z) = softplus(p) z^2 + z / 2 for
    z > 0 and (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2 for z <= 0."""
    kind: str = "dense_mlp"
    hidden: int = 0
    intermediate: int = 0
    activation: str = "xielu"


@dataclass(frozen=True)
class RoutedMlpSpec(FeedForwardSpec):
    """``experts`` gated feed-forwards of ``expert_intermediate`` rows of which a token uses the ``top`` with the largest
    router scores, and a shared one of ``shared_intermediate`` rows (0: none) that every token uses. ``score``: the
    function that turns router logits into scores ("sigmoid"); ``renormalize``: whether the chosen scores are divided by
    their sum; ``weight_on``: "input" when a chosen expert is given score * x (the sum of expert(score x)), "output" when
    its output is multiplied. ``score`` "softmax": scores are the softmax of the logits over the experts and the
    ``identity_experts`` (router outputs beyond the experts, whose output is their input; they have no weights); with
    ``correction`` a stored vector is added to the scores for the choice only; the weights are the chosen scores times
    ``route_scale``. ``activation``, ``limit``: as in ``GatedMlpSpec``; ``shared_limit`` is the shared expert's limit;
    ``shared_gate``: the shared expert's output is multiplied by the sigmoid of one more router-like product a token."""
    kind: str = "routed_mlp"
    hidden: int = 0
    experts: int = 0
    top: int = 1
    expert_intermediate: int = 0
    shared_intermediate: int = 0
    activation: str = "silu"
    score: str = "sigmoid"
    renormalize: bool = False
    weight_on: str = "input"
    correction: bool = False
    route_scale: float = 1.0
    identity_experts: int = 0
    limit: float = 0.0
    shared_limit: float = 0.0
    shared_gate: bool = False


@dataclass(frozen=True)
class EmbeddingSpec:
    """How token ids become the first hidden states. ``table``: a row copy, no scaling
    (src/Starlings.Roost.Ops/CpuOps.cs:441-458)."""
    kind: str = "table"
    vocab: int = 0
    hidden: int = 0


@dataclass(frozen=True)
class HeadSpec:
    """How the final hidden states of the wanted rows become logits. ``linear``: a product with a [vocab, hidden] matrix
    into 32-bit logits, no soft cap (src/Starlings.Roost.Ops/CpuOps.cs:465-495)."""
    kind: str = "linear"
    vocab: int = 0
    hidden: int = 0


@dataclass(frozen=True)
class ScaledEmbeddingSpec(EmbeddingSpec):
    """h0[t, :] = table[ids[t], :] * scale, formed and kept in 32-bit (the stream of a ``pre_norm_wide`` model)."""
    kind: str = "scaled_table"
    scale: float = 1.0


@dataclass(frozen=True)
class CappedHeadSpec(HeadSpec):
    """logits = cap * tanh((final W^T) / cap) in 32-bit."""
    kind: str = "capped_linear"
    cap: float = 0.0


@dataclass(frozen=True)
class ScaledHeadSpec(HeadSpec):
    """logits = (final W^T) * scale in 32-bit."""
    kind: str = "scaled_linear"
    scale: float = 1.0


@dataclass(frozen=True)
class PairHashedEmbeddingSpec(EmbeddingSpec):
    """h0[t] = table[id_t] + pairs[(id_(t-1) * mul_prev + id_t * mul_cur) mod buckets] as a 32-bit stream; a request's first
    token takes row ``buckets`` of ``pairs`` (the row after the buckets). The previous token is kept per request."""
    kind: str = "pair_hashed_table"
    buckets: int = 0
    mul_prev: int = 0
    mul_cur: int = 0


@dataclass(frozen=True)
class TokenInputSpec:
    """What a layer adds to the stream at its end from the token itself: e = ``dim`` numbers of a second embedding table (the
    columns from ``column`` on of a table ``columns`` wide), g = gelu_tanh(W_gate x) * e, y = W_proj g, and the stream gains
    y / sqrt(mean(y^2) + eps) * w."""
    kind: str = "gated_token_input"
    hidden: int = 0
    vocab: int = 0
    dim: int = 0
    column: int = 0
    columns: int = 0
    eps: float = 1e-6


@dataclass(frozen=True)
class ConnectionSpec:
    """How a sublayer reads the residual and writes back to it. ``hyper_connection``: the residual is ``streams`` copies
    x_1 .. x_S in 32-bit, all equal to the embedding at the start; the sublayer reads u = sum_s in[s] x_s and its output y
    goes back as x_t <- sum_s mix[s, t] x_s + out[t] y, every stream at once from the old ones; the model's output is the sum
    of the streams. ``learned`` False: in, mix and out are ones (with one stream: the plain residual sum)."""
    kind: str = "hyper_connection"
    streams: int = 1
    learned: bool = True


@dataclass(frozen=True)
class GatedResidualSpec(ConnectionSpec):
    """A sublayer's output y is multiplied element by element by sigmoid(W h + b) before it is added to the residual, h being the
    sublayer's own (normed) input and W a square matrix of the model's width: x <- x + y sigmoid(W h + b)."""
    kind: str = "sigmoid_gate"
    hidden: int = 0


@dataclass(frozen=True)
class BlockSpec:
    """One layer's parts and their arrangement. ``pre_norm``: h += mixer(norm1(h)); h += ff(norm2(h)), the stream in the
    activation dtype. ``pre_norm_wide``: the same with the stream kept and summed in 32-bit whatever the activation dtype
    is; its ``feed_forward`` and ``post_mixer_norm`` may be None (a layer that is its mixer only). ``pre_norm_streams``:
    the same two sublayers over several 32-bit residual streams, read and written through ``connection``. ``pre_norm_gated``:
    ``pre_norm_wide`` with every sublayer's output scaled by a gate of its ``connection`` (``sigmoid_gate``) before the sum."""
    mixer: MixerSpec
    feed_forward: FeedForwardSpec | None
    input_norm: NormSpec
    post_mixer_norm: NormSpec | None
    kind: str = "pre_norm"
    connection: ConnectionSpec | None = None
    token_input: TokenInputSpec | None = None     # ``pre_norm_wide`` only: added after the last sublayer


@dataclass(frozen=True)
class RunEntry:
    """One run of a block. ``block`` indexes ``ModelSpec.blocks`` (the same block may run twice: it then has
    one set of weights and two caches). ``reads_cache_of`` is None when the run keeps a cache of its own, or
    the index of an earlier run whose cache it reads without writing. ``adds_embedding``: the embedding's output is added to
    the residual stream once more right before the run (a model that runs a range of blocks several times)."""
    block: int
    reads_cache_of: int | None = None
    adds_embedding: bool = False


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden: int
    vocab: int
    blocks: tuple[BlockSpec, ...]
    schedule: tuple[RunEntry, ...]
    final_norm: NormSpec
    tie_embeddings: bool
    max_positions: int
    stop_token_ids: tuple[int, ...] = ()
    stored_dtype: str = "bfloat16"
    # the two ends of the model as parts of their own kinds (None: a table embedding and a linear head of the model's
    # vocabulary and width)
    embedding: EmbeddingSpec | None = None
    head: HeadSpec | None = None
    # checkpoint tensors the model does not use and a checkpoint may hold all the same (the loader passes over them)
    ignorable_tensors: tuple = ()
    # checkpoint tensor names: scope -> {part-local parameter name -> tuple of checkpoint names whose rows
    # are concatenated in order}. Scopes: "embed", "final_norm", "lm_head", "blocks.<i>.<part>".
    weight_names: dict = field(default_factory=dict, compare=False, hash=False)

    def __post_init__(self):
        if self.embedding is None:
            object.__setattr__(self, "embedding", EmbeddingSpec(vocab=self.vocab, hidden=self.hidden))
        if self.head is None:
            object.__setattr__(self, "head", HeadSpec(vocab=self.vocab, hidden=self.hidden))
        for n, e in enumerate(self.schedule):
            if not 0 <= e.block < len(self.blocks):
                raise ValueError(f"schedule entry {n} names block {e.block}; the model has {len(self.blocks)}")
            if e.reads_cache_of is not None:
                if not 0 <= e.reads_cache_of < n:
                    raise ValueError(f"schedule entry {n} reads the cache of entry {e.reads_cache_of}, which does not run before it")
                if self.schedule[e.reads_cache_of].reads_cache_of is not None:
                    raise ValueError(f"schedule entry {n} reads the cache of entry {e.reads_cache_of}, which keeps none of its own")
