"""Descriptions of a model as data: parts, blocks, and the order they run in.

A ``ModelSpec`` is what an architecture's ``config.json`` is turned into.  It
names every size and constant and every weight tensor, layer by layer, so that
two layers of one model may use different mixers, feed-forwards, norms or
position encodings.  Nothing here computes; the classes under ``parts`` are
built from these records through the registries in ``parts.registry``.

A new kind of part adds a frozen dataclass with a ``kind`` string here or in its
own module (tests define toy ones) and registers a class for that ``kind``.
"""

from __future__ import annotations

from dataclasses import dataclass, field


@dataclass(frozen=True)
class RopeScaling:
    """Frequency scaling of rotary embeddings, read from ``rope_scaling``."""

    rope_type: str
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int


@dataclass(frozen=True)
class NormSpec:
    """A normalisation over the last axis."""

    kind: str          # "rmsnorm" | "layernorm"
    size: int
    eps: float
    weight: str        # tensor name of the gain
    bias: str | None = None   # tensor name of the additive term ("layernorm")
    unit_offset: bool = False  # "rmsnorm": the tensor is stored around zero and the multiplier is 1 + weight
    scalar: bool = False       # "rmsnorm": the tensor is ONE number (shape ()), the multiplier of every coordinate


@dataclass(frozen=True)
class YarnScaling:
    """Frequencies of a rotation blended for a context longer than the original one.  With ``dim(t) = dims *
    ln(original / (2 pi t)) / (2 ln base)``, ``lo = max(floor(dim(fast)), 0)``, ``hi = min(ceil(dim(slow)), dims - 1)``
    and ``ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)`` the frequency of pair i is ``f_i / factor * ramp_i +
    f_i * (1 - ramp_i)``, and cosine and sine are both multiplied by ``mult_slope * ln(factor) + 1``."""

    factor: float
    original: float
    fast: float
    slow: float
    mult_slope: float = 0.1


@dataclass(frozen=True)
class PositionSpec:
    """How positions enter a mixer."""

    kind: str                     # "rotary" | "none" | "bucketed_bias" | "rotary_pairs" | "rotary_partial"
    head_dim: int = 0
    theta: float = 0.0
    max_positions: int = 0
    scaling: RopeScaling | None = None
    # "rotary_pairs": neighbouring dimensions (2i, 2i + 1) of the first ``rot_dims`` dimensions of a head turn by
    # position * theta^(-2i / rot_dims); the rest of the head passes unchanged.  Angles are worked out from the
    # position inside the kernel, so there is no table and no limit on positions.
    rot_dims: int = 0
    # "rotary_partial": ``rot_dims`` dimensions of a head turn by position * theta^(-2i / rot_dims), paired in halves
    # (i with i + rot_dims / 2) or as neighbours (2i with 2i + 1); where in the head they start is the mixer's
    # business.  ``yarn`` blends the frequencies and multiplies cosine and sine.  No table, no limit on positions.
    layout: str = "halves"        # "halves" | "neighbours"
    yarn: YarnScaling | None = None
    # "bucketed_bias": a learned table [n_buckets, n_heads] added to the scores by distance; distances below half
    # the buckets have a row each, the rest share rows on a logarithmic scale that ends at ``max_distance``
    table: str = ""
    n_buckets: int = 0
    n_heads: int = 0
    max_distance: int = 0


@dataclass(frozen=True)
class HeadNormSpec:
    """RMS norm of every query head and key head before the scores, with gains of the head's size that all heads
    share (a name of None leaves that side alone)."""

    eps: float
    q_weight: str | None = None
    k_weight: str | None = None


@dataclass(frozen=True)
class MixerSpec:
    """Base of token mixers; ``kind`` selects the registered class."""

    kind: str


@dataclass(frozen=True)
class AttentionSpec(MixerSpec):
    """Causal grouped-query attention over a paged key/value cache."""

    hidden: int = 0
    n_heads: int = 0
    n_kv_heads: int = 0
    head_dim: int = 0
    window: int | None = None      # None: every earlier key; n: the last n keys, itself included
    position: PositionSpec = PositionSpec(kind="none")
    q_proj: str = ""
    k_proj: str = ""
    v_proj: str = ""
    o_proj: str = ""
    v_head_dim: int | None = None  # head size of values and output when it is not ``head_dim``
    scale: float | None = None     # multiplier of q . k; None: head_dim ** -0.5
    qk_norm: HeadNormSpec | None = None
    head_scale: str | None = None  # tensor [n_heads]: a learned multiplier of each head's scores beside ``scale``
    # beside a window: keys at positions below ``keep_first`` stay visible to every later query (and stay in the
    # cache), at their true positions
    keep_first: int = 0
    q_bias: str | None = None      # biases of the three projections ([heads * head size] each)
    k_bias: str | None = None
    v_bias: str | None = None
    # RMS norm over the WHOLE projection of q (and of k), all heads at once, with gains of that size, before the
    # heads are split and rotated (``HeadNormSpec`` above norms each head by itself)
    q_row_norm: str | None = None
    k_row_norm: str | None = None
    row_norm_eps: float = 1e-6
    out_scale: float = 1.0         # multiplier of the heads' outputs before the output projection

    @property
    def value_dim(self) -> int:
        return self.v_head_dim if self.v_head_dim is not None else self.head_dim


@dataclass(frozen=True)
class LatentAttentionSpec(MixerSpec):
    """Causal softmax attention whose keys and values are expanded from one compressed vector per token.

    ``q_proj`` gives ``n_heads`` query heads laid out [head_dim unrotated, rot_dim rotated].  ``down_proj`` gives
    ``kv_rank + rot_dim`` numbers a token: the first ``kv_rank``, RMS-normed with ``latent_norm`` (eps ``norm_eps``), are
    the compressed vector c; the last ``rot_dim`` (not normed) are a rotated key part that all heads share.  Per head the
    unrotated key is ``k_up`` c and the value ``v_up`` c (both laid out head by head); the score is (q_unrotated .
    k_unrotated + q_rotated . k_rotated) * scale.  The cache holds c and the rotated key part only.  ``position``
    (kind "rotary_partial" with rot_dims = rot_dim, or "none") turns the rotated parts.  ``chunk``: a query sees only
    the keys of its own chunk of that many positions (None: every earlier key)."""

    hidden: int = 0
    n_heads: int = 0
    head_dim: int = 0              # unrotated query/key dimensions of a head
    rot_dim: int = 0               # rotated ones
    v_head_dim: int = 0
    kv_rank: int = 0
    scale: float = 1.0
    norm_eps: float = 1e-6
    position: PositionSpec = PositionSpec(kind="none")
    chunk: int | None = None
    q_proj: str = ""
    down_proj: str = ""
    latent_norm: str = ""
    k_up: str = ""
    v_up: str = ""
    o_proj: str = ""
    # Queries through a compressed vector of their own: c_q = RMSnorm(q_down x) with the gain q_norm (eps norm_eps),
    # then q = q_proj c_q (q_proj is then [heads * (head_dim + rot_dim), q_rank]).  q_rank 0: q = q_proj x.
    q_rank: int = 0
    q_down: str = ""
    q_norm: str = ""
    window: int | None = None      # a query sees itself and the window - 1 keys before it (None: every earlier key)
    sink: str | None = None        # tensor [n_heads]: exp(sink_h) joins the softmax's denominator of head h: a learned
                                   # logit beside the keys' scores that ``scale`` does not multiply and that weighs nothing
    head_gate: str | None = None   # tensor [n_heads, hidden]: head h's output is multiplied by sigmoid(head_gate x)_h


@dataclass(frozen=True)
class TalkingAttentionSpec(MixerSpec):
    """Grouped-query softmax attention without positions whose weights are mixed across heads after the softmax.

    q, k, v = q_proj x, k_proj x, v_proj x (+ biases); with ``qk_norm`` every query and key head, with ``v_norm`` every
    value head (as it is cached), is divided by its root mean square (``norm_eps`` inside the root, no gain).
    score = q . k * scale under a causal mask (``window``: a query sees itself and the window - 1 keys before it);
    ordinary softmax per head; then weight_h(i, j) <- sum_g talk[h, g] weight_g(i, j) (``talk`` [heads, heads], None:
    no mixing) and head h applies its mixed weights to the values of its own key/value head h // (heads / kv heads).
    The concatenated heads are multiplied by sigmoid(gate_proj x) element by element (None: no gate), then ``o_proj``."""

    hidden: int = 0
    n_heads: int = 0
    n_kv_heads: int = 0
    head_dim: int = 0
    v_head_dim: int = 0
    scale: float = 1.0
    norm_eps: float = 1e-6
    qk_norm: bool = True
    v_norm: bool = True
    window: int | None = None
    q_proj: str = ""
    k_proj: str = ""
    v_proj: str = ""
    q_bias: str | None = None
    k_bias: str | None = None
    v_bias: str | None = None
    talk: str | None = None
    gate_proj: str | None = None
    o_proj: str = ""


@dataclass(frozen=True)
class MatrixMemorySpec(MixerSpec):
    """The matrix memory of xLSTM (mLSTM) with exponential gates and a running maximum.

    q = q_proj x * head_dim^-1/2 and k = k_proj x (heads x head_dim), v = v_proj x (heads x v_head_dim).  Per head the
    log input gate i = cap * tanh((i_proj x + i_bias) / cap) and the log forget gate f = logsigmoid(cap * tanh((f_proj x
    + f_bias) / cap)), cap = ``gate_cap``.  With S, n and the maximum m all zero at the start:
        m' = max(f + m, i);  S <- exp(f + m - m') S + exp(i - m') k v^T;  n likewise with k alone;  m <- m'
        o = S^T q / (max(|n . q|, exp(-m)) + denom_eps)
    Each head's o is divided by its root mean square (norm_eps); the heads, side by side, are multiplied by ``out_gain``
    (all heads' size) and by sigmoid(gate_proj x), then ``o_proj``."""

    hidden: int = 0
    n_heads: int = 0
    head_dim: int = 0
    v_head_dim: int = 0
    gate_cap: float = 15.0
    norm_eps: float = 1e-6
    q_proj: str = ""
    k_proj: str = ""
    v_proj: str = ""
    i_proj: str = ""
    i_bias: str = ""
    f_proj: str = ""
    f_bias: str = ""
    gate_proj: str = ""
    out_gain: str = ""
    o_proj: str = ""


@dataclass(frozen=True)
class DifferentialAttentionSpec(MixerSpec):
    """Grouped-query attention with two score maps a head over the same values.

    ``q_proj`` gives ``n_heads`` x 2 x ``head_dim`` and ``k_proj`` ``n_kv_heads`` x 2 x ``head_dim`` rows, laid out head by
    head as [map 1, map 2]; ``v_proj`` ``n_kv_heads`` x ``v_head_dim``.  Every map of every head is RMS-normed over
    ``head_dim`` with ``q_norm`` / ``k_norm`` (gains of that size, shared; eps ``norm_eps``; None: no norm), then
    ``position`` turns its first dimensions.  Each map is a softmax attention of its own (score = q . k * scale,
    causal, within a chunk of ``chunk`` positions when that is given).  With lambda = exp(sum(lq1 * lk1)) -
    exp(sum(lq2 * lk2)) + lambda_init:  o = a1 - lambda a2, divided by its root mean square over the head's values
    (``norm_eps``, no gain), times (1 - lambda_init), times sigmoid(``gate_proj`` x) if there is one, then
    ``o_proj``."""

    hidden: int = 0
    n_heads: int = 0
    n_kv_heads: int = 0
    head_dim: int = 0
    v_head_dim: int = 0
    scale: float = 1.0
    norm_eps: float = 1e-6
    lambda_init: float = 0.0
    position: PositionSpec = PositionSpec(kind="none")
    chunk: int | None = None
    q_proj: str = ""
    k_proj: str = ""
    v_proj: str = ""
    q_norm: str | None = None
    k_norm: str | None = None
    lambda_q1: str = ""
    lambda_k1: str = ""
    lambda_q2: str = ""
    lambda_k2: str = ""
    gate_proj: str | None = None
    o_proj: str = ""


@dataclass(frozen=True)
class MinGRUSpec(MixerSpec):
    """A gated recurrence whose gates read the current token only, ``width`` channels:
        z = sigmoid(z_proj x + z_bias);  u = x_proj x + x_bias;  candidate = u + 1/2 (u >= 0) | sigmoid(u) (u < 0)
        S <- (1 - z) S + z candidate;   out = o_proj (S * silu(gate_proj x))
    with S a float32 vector per request that starts at zero."""

    hidden: int = 0
    width: int = 0
    z_proj: str = ""
    z_bias: str = ""
    x_proj: str = ""
    x_bias: str = ""
    gate_proj: str = ""
    o_proj: str = ""


@dataclass(frozen=True)
class ShortConvSpec:
    """A causal convolution over time, one filter per channel: ``weight`` [channels, taps], whose last column
    multiplies the current token's input; zeros stand before a sequence's start.  The last ``taps - 1`` inputs of a
    sequence are state that a mixer carries from step to step."""

    taps: int
    weight: str
    bias: str | None = None


@dataclass(frozen=True)
class GatedDeltaSpec(MixerSpec):
    """The gated delta rule: a recurrent mixer with a ``head_dim x v_head_dim`` float32 state per head.

    q and k have ``n_kv_heads`` heads of ``head_dim`` (head h of the state reads q/k head h // (n_heads / n_kv_heads)),
    v has ``n_heads`` heads of ``v_head_dim``.  Each passes a short convolution and SiLU; q and k become unit vectors
    (``key_eps`` inside the root) and q takes head_dim^-1/2.  Per token and head, with beta = sigmoid(b x) and the
    decay g = exp(-exp(A_log) * softplus(a x + dt_bias)):
        S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q.
    o is divided by its root mean square over ``v_head_dim`` (norm_eps), multiplied by ``out_gain`` ([v_head_dim],
    shared by the heads) and by silu(gate x), and projected by ``o_proj``."""

    hidden: int = 0
    n_heads: int = 0
    n_kv_heads: int = 0
    head_dim: int = 0
    v_head_dim: int = 0
    key_eps: float = 1e-6
    norm_eps: float = 1e-6
    q_proj: str = ""
    k_proj: str = ""
    v_proj: str = ""
    q_conv: ShortConvSpec | None = None
    k_conv: ShortConvSpec | None = None
    v_conv: ShortConvSpec | None = None
    beta_proj: str = ""
    decay_proj: str = ""
    decay_log: str = ""            # A_log, [n_heads]
    decay_bias: str = ""           # dt_bias, [n_heads]
    gate_proj: str = ""
    out_gain: str = ""
    o_proj: str = ""


@dataclass(frozen=True)
class GatedLinearRecurrenceSpec(MixerSpec):
    """A recurrent block around a real-gated linear recurrent unit, ``width`` channels:
        y = gelu_tanh(y_proj x + y_bias);  u = conv(x_proj x + x_bias)
        r = sigmoid(A_b u_b + a_b), i = sigmoid(I_b u_b + i_b)     per block b of ``n_blocks`` equal parts of u
        a = exp(-decay_scale * r * softplus(lam));  S <- a S + sqrt(1 - a^2) (i * u);  out = o_proj (S * y)
    with S a float32 vector per request that starts at zero."""

    hidden: int = 0
    width: int = 0
    n_blocks: int = 1
    decay_scale: float = 8.0
    y_proj: str = ""
    y_bias: str = ""
    x_proj: str = ""
    x_bias: str = ""
    conv: ShortConvSpec | None = None
    a_gate: str = ""               # [n_blocks, width / n_blocks, width / n_blocks], rows are outputs
    a_gate_bias: str = ""          # [n_blocks, width / n_blocks]
    i_gate: str = ""
    i_gate_bias: str = ""
    lam: str = ""                  # [width]
    o_proj: str = ""
    out_scale: float = 1.0         # multiplier of S * y before the output projection


@dataclass(frozen=True)
class ParallelMixerSpec(MixerSpec):
    """Several mixers side by side that read the same input; the result is the sum of their outputs, each times its
    weight (a branch folds the weight into what it hands its output projection)."""

    hidden: int = 0
    branches: tuple[MixerSpec, ...] = ()


@dataclass(frozen=True)
class GeneralDeltaSpec(MixerSpec):
    """The generalized delta rule: a recurrent mixer with a head_dim x head_dim float32 state per head.

    Per token and head, with projections r, k, v, a gate g, a removal rate a = sigmoid(a_proj x + a_bias) and a
    decay w = exp(-decay_rate * sigmoid(w2 tanh(w1 x) + w0)) per key channel, and the unit key
    u = k / sqrt(sum(k^2) + key_eps):  S <- diag(w) S - (a * u)(u^T S) + k v^T,  o = S^T r.  Each head's o is
    divided by its root mean square (norm_eps), multiplied by ``out_gain`` and sigmoid(g), then projected by o_proj.
    """

    hidden: int = 0
    n_heads: int = 0
    head_dim: int = 0
    decay_rank: int = 0            # inner size of the low-rank pair w1, w2
    decay_rate: float = 0.0
    key_eps: float = 1e-6
    norm_eps: float = 1e-6
    r_proj: str = ""
    k_proj: str = ""
    v_proj: str = ""
    g_proj: str = ""
    a_proj: str = ""
    a_bias: str = ""
    w1: str = ""
    w2: str = ""
    w0: str = ""
    out_gain: str = ""
    o_proj: str = ""


@dataclass(frozen=True)
class FeedForwardSpec:
    kind: str


@dataclass(frozen=True)
class GatedMLPSpec(FeedForwardSpec):
    """``down(act(gate(x)) * (up(x) + up_offset))``.  ``activation`` "silu": g sigmoid(g).  "clamped_swish": with
    g' = min(g, act_limit) and up clamped to [-act_limit, act_limit], g' sigmoid(act_alpha g')."""

    hidden: int = 0
    intermediate: int = 0
    activation: str = "silu"
    act_alpha: float = 1.0
    act_limit: float = 0.0
    up_offset: float = 0.0
    gate_proj: str = ""
    up_proj: str = ""
    down_proj: str = ""


@dataclass(frozen=True)
class PolyNormMLPSpec(FeedForwardSpec):
    """``down(act(up(x) + up_bias)) + down_bias`` with the PolyNorm activation: c0 N(z) + c1 N(z^2) + c2 N(z^3) + c3,
    powers element by element, N(x) = x / sqrt(mean(x^2) + eps) over a token's ``intermediate`` values; ``coef`` names
    the tensor of the four numbers."""

    hidden: int = 0
    intermediate: int = 0
    eps: float = 1e-6
    up_proj: str = ""
    up_bias: str | None = None
    down_proj: str = ""
    down_bias: str | None = None
    coef: str = ""


@dataclass(frozen=True)
class RoutedExpertsSpec(FeedForwardSpec):
    """A mixture of gated feed-forward experts with a sigmoid router.

    Router scores s = sigmoid(router x) in float32; an expert's choice score is s + ``correction``.  The experts
    form ``n_groups`` groups of neighbours; a group's score is the sum of its two largest choice scores, and only
    experts of the ``keep_groups`` best groups can be chosen.  The ``top`` largest choice scores among them are
    taken; their weights are their s divided by the sum of those (+ ``weight_eps``), times ``route_scale``.  The
    output is the weighted sum of the chosen experts' ``down(silu(gate x) * up x)``.  ``shared`` (optional) is a
    dense expert that every token runs; it is added times sigmoid(shared_gate x), one number a token."""

    hidden: int = 0
    intermediate: int = 0
    n_experts: int = 0
    top: int = 1
    n_groups: int = 1
    keep_groups: int = 1
    route_scale: float = 1.0
    weight_eps: float = 1e-20
    router: str = ""
    correction: str | None = None
    expert_prefix: str = ""        # expert e's tensors are <prefix><e>.gate / .up / .down
    shared: GatedMLPSpec | None = None
    shared_gate: str | None = None
    # ``score`` "softmax_top": the logits are router x + ``router_bias`` (float32); the ``top`` largest are chosen (no
    # groups, no correction) and their weights are the softmax over the chosen logits alone, times ``route_scale``.
    score: str = "sigmoid"
    router_bias: str | None = None


@dataclass(frozen=True)
class BlockSpec:
    """One residual block: which norm, mixer and feed-forward, and how arranged.  A block without a feed-forward
    (``feedforward`` and ``ff_norm`` None) is its mixer half alone."""

    kind: str       # "prenorm": x += part(norm(x)) | "outnorm": x += norm(part(x)) | "gated_prenorm" (below)
    mixer_norm: NormSpec
    mixer: MixerSpec
    ff_norm: NormSpec | None
    feedforward: FeedForwardSpec | None
    # "gated_prenorm": x += sigmoid(W h + b) * part(h) with h = norm(x): a gate per coordinate that reads what the
    # sublayer reads.  Tensor names of W ([hidden, hidden]) and b ([hidden]) for the mixer and the feed-forward.
    mixer_gate: str | None = None
    mixer_gate_bias: str | None = None
    ff_gate: str | None = None
    ff_gate_bias: str | None = None
    # "sandwich": x += out_norm(part(norm(x))): a norm before and after each sublayer (``mixer_norm`` / ``ff_norm``
    # before, these two after).  ``token_shift`` names a tensor [hidden]: the mixer's input, h = mixer_norm(x), is
    # replaced by h + (h' - h) * token_shift with h' the h of the token before (zeros before the first); the last h of a
    # sequence is state of the run beside the mixer's own.
    mixer_out_norm: NormSpec | None = None
    ff_out_norm: NormSpec | None = None
    token_shift: str | None = None


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.

    ``layer`` indexes ``ModelSpec.layers`` and may occur in several entries
    (shared weights).  ``cache_from`` names an EARLIER entry of the schedule whose
    cache this run reads instead of writing one of its own.
    """

    layer: int
    cache_from: int | None = None


@dataclass(frozen=True)
class ModelSpec:
    """A whole decoder: embedding, layers, their order, final norm and head."""

    architecture: str
    vocab_size: int
    hidden: int
    max_positions: int
    embedding: str                           # tensor name of the token table
    layers: tuple[BlockSpec, ...]
    schedule: tuple[ScheduleEntry, ...]
    final_norm: NormSpec
    head: str | None                         # tensor name, or None: tied to the embedding
    optional_tensors: tuple[str, ...] = field(default_factory=tuple)  # present-but-unused names tolerated
    kind: str = "decoder"                    # which registered top level puts the parts together


@dataclass(frozen=True)
class BigramDecoderSpec(ModelSpec):
    """A decoder whose first residual is the token embedding plus a hashed bigram embedding: row
    ``(previous token * mul_prev + token * mul_cur) mod buckets`` of the tensor ``bigram`` ([buckets + 1, hidden]),
    and its last row for a sequence's first token."""

    bigram: str = ""
    bigram_buckets: int = 0
    bigram_mul_prev: int = 0
    bigram_mul_cur: int = 0
    kind: str = "bigram_decoder"


@dataclass(frozen=True)
class ReinjectDecoderSpec(ModelSpec):
    """A decoder whose token embedding is multiplied by ``embedding_scale`` and added to the residual stream again
    right before each schedule entry that ``reinject_before`` names (a group of layers run several times in a row takes
    the embedding anew at the start of every pass but the first)."""

    embedding_scale: float = 1.0
    reinject_before: tuple[int, ...] = ()
    kind: str = "reinject_decoder"


@dataclass(frozen=True)
class PassOffsetDecoderSpec(ModelSpec):
    """A decoder whose first residual is the token embedding times ``embedding_scale`` plus, with ``sinusoid_base`` > 0,
    a sinusoidal position vector (entry 2i: sin(p base^(-2i / hidden)), entry 2i + 1: the cosine of the same angle), and
    which adds a learned vector to the stream right before some schedule entries: ``offset_before`` lists (entry, row)
    pairs, and row r of the tensor ``pass_offsets`` ([rows, hidden]) is added before that entry runs (a group of layers
    run several times in a row takes the vector of its pass at the start of each pass, the first too)."""

    embedding_scale: float = 1.0
    sinusoid_base: float = 0.0
    pass_offsets: str | None = None
    offset_before: tuple[tuple[int, int], ...] = ()
    kind: str = "pass_offset_decoder"
