"""Typed description of a decoder model: which parts each layer is made of, and in which order
layers run.

A model is data: a tuple of ``LayerSpec`` (one per set of weights) and a tuple of ``LayerRun``
(the order in which those layers execute).  Every size and constant lives in a spec; the parts
under ``turingserve_b200.parts`` read them from there and nowhere else.

A spec is any frozen dataclass with a ``kind`` string; ``kind`` selects the implementation in
the part registries (``turingserve_b200.parts.registry``).  New kinds of mixer, feed-forward,
norm or position encoding bring their own spec class; nothing in this file lists them.

The reference keeps one flat ``Qwen2Config`` (turingserve/model/qwen2_config.py:10-63) and
hard-codes the layer recipe in ``Qwen2Model._run`` (turingserve/model/qwen2.py:38-61); here the
recipe itself is configuration so that layers of different kinds can alternate.
"""

from __future__ import annotations

from dataclasses import dataclass, fields, is_dataclass
from typing import Any


@dataclass(frozen=True)
class RMSNormSpec:
    """Root-mean-square norm over the last dimension with a learned scale."""

    eps: float
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class RotarySpec:
    """Rotate-half rotary position encoding over the first ``rotary_dim`` dims of a head."""

    theta: float
    rotary_dim: int
    max_positions: int
    kind: str = "rope"


@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query softmax attention over a paged key/value cache.

    ``window`` = None means every earlier key is visible; an integer w means the query at
    position p sees keys at positions p-w+1 .. p.
    """

    num_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float
    qkv_bias: bool
    out_bias: bool
    position: Any                       # a position-encoding spec, or None
    window: int | None = None
    kind: str = "attention"


@dataclass(frozen=True)
class GatedMLPSpec:
    """Dense gated feed-forward: down(act(gate(x)) * up(x)), act silu | gelu_tanh | gelu | relu2.  ``names``: the
    local tensor names of the gate, up and down weights."""

    intermediate_size: int
    activation: str = "silu"
    bias: bool = False
    names: tuple[str, str, str] = ("gate_proj.weight", "up_proj.weight", "down_proj.weight")
    kind: str = "gated_mlp"


@dataclass(frozen=True)
class StreamRMSNormSpec:
    """Root-mean-square norm of a residual stream that is kept in 32-bit whatever the engine's type:
    x / sqrt(mean(x^2) + eps) * scale, all in 32-bit, rounded once."""

    eps: float
    weight_name: str = "weight"         # local tensor name of the scale ('' = the norm's prefix itself)
    kind: str = "rmsnorm_stream"


@dataclass(frozen=True)
class StreamLayerNormSpec:
    """Layer norm of a residual stream that is kept in 32-bit whatever the engine's type:
    (x - mean) / sqrt(mean((x - mean)^2) + eps) * weight + bias, all in 32-bit, rounded once."""

    eps: float
    weight_name: str = "weight"         # local tensor names ('' = the norm's prefix itself)
    bias_name: str = "bias"
    kind: str = "layernorm_stream"


@dataclass(frozen=True)
class BranchJoinSpec:
    """How the outputs of a layer's branches enter the residual stream: x <- x + scale * (their sum)."""

    scale: float = 1.0
    kind: str = "branch_join"


@dataclass(frozen=True)
class HalfRotarySpec:
    """Rotary position encoding over the first ``dims`` dimensions of a head, dimension i paired with dimension
    i + dims/2: the pair (u, v) at position p becomes (u cos a - v sin a, v cos a + u sin a), a = p * f_i,
    f_i = base^(-2i/dims).  The angle is a 32-bit product of the position and the frequency, so no table over
    positions exists and no longest sequence has to be known."""

    base: float
    dims: int
    kind: str = "rope_half"


@dataclass(frozen=True)
class SinkAttentionSpec:
    """Grouped-query softmax attention over keys ``key_dim`` and values ``value_dim`` wide, no biases.
    ``position``: a rotation of q and k (not v).  ``qk_norm_eps`` not None: after the rotation every head of q
    and k is divided by its root mean square (eps inside the root, no learned weight).  ``chunk`` c: position i
    sees j <= i only inside its own block of c positions, floor(i / c) = floor(j / c), blocks counted from the
    sequence's position 0.  ``window`` w: only i - w < j.  ``sinks``: the softmax's denominator also holds
    exp(sink_h), a learned number per head without key or value, unscaled, counted once.  ``qkv_bias``: the q, k and v
    projections have biases (tensor name + '.b').  ``out_gate``: the heads side by side are multiplied by
    sigmoid(W_g h) ('g', a projection of the mixer's own input) before the output projection."""

    num_heads: int
    num_kv_heads: int
    key_dim: int
    value_dim: int
    scale: float
    position: Any = None
    qk_norm_eps: float | None = None
    chunk: int | None = None
    window: int | None = None
    sinks: bool = True
    qkv_bias: bool = False
    out_gate: bool = False
    kind: str = "sink_attention"


@dataclass(frozen=True)
class HyperRMSNormSpec:
    """RMS norm of what a sublayer reads from a residual stream kept as ``streams`` copies in 32-bit:
    u = sum_s in[s] x_s, then u / sqrt(mean(u^2) + eps) * (weight_offset + weight), all in 32-bit, rounded once.
    ``weight_offset`` 1: the weight is stored around zero.  The norm's kernel also carries out the write-back of the
    sublayer before it (see ``StreamLinkSpec``)."""

    eps: float
    streams: int = 1
    weight_offset: float = 0.0
    weight_name: str = "weight"         # local tensor name of the scale ('' = the norm's prefix itself)
    kind: str = "rmsnorm_hyper"


@dataclass(frozen=True)
class StreamLinkSpec:
    """How one sublayer hangs on a residual stream of ``streams`` copies (hyper-connections): it reads
    u = sum_s in[s] x_s and its output y comes back as x_t <- sum_s mix[s, t] x_s + out[t] y, all copies at once
    from the old ones (mix indexed [from, to]).  ``learned`` False: no tensors, in = out = 1 and mix the identity,
    which with one copy is the ordinary residual sum.  ``names``: local tensor names of in, out and mix."""

    streams: int = 1
    learned: bool = True
    names: tuple[str, str, str] = ("in", "out", "mix")
    kind: str = "stream_link"


@dataclass(frozen=True)
class BandScaledRotarySpec:
    """Rotary position encoding over pairs of neighbouring dimensions (2i, 2i+1) of the first ``dims`` dimensions of
    a head, angle = position * f_i, f_i = base^(-2i/dims), the frequencies rescaled by wavelength bands (the rule of
    Llama 3.1): with l = 2 pi / f, f stays where l < original / high, becomes f / factor where l > original / low,
    and between the two is (1 - s) f / factor + s f with s = (original / l - low) / (high - low).  ``factor`` None:
    the plain frequencies."""

    base: float
    dims: int
    factor: float | None = None
    low: float = 1.0
    high: float = 4.0
    original: float = 8192.0
    kind: str = "rope_pairs_banded"


@dataclass(frozen=True)
class PairedMixerSpec:
    """Two mixers side by side that read the same input: ``left_scale`` * left(h) + ``right_scale`` * right(h).
    ``names``: the prefixes of their tensors inside the mixer's own."""

    left: Any
    right: Any
    left_scale: float = 1.0
    right_scale: float = 1.0
    names: tuple[str, str] = ("left.", "right.")
    kind: str = "paired_mixer"


@dataclass(frozen=True)
class Mamba2Spec:
    """Selective state-space mixer with a scalar decay per head.  One projection gives
    [z (H P) | x (H P) | B (G N) | C (G N) | dt (H)]; x, B and C pass a causal filter of ``conv_taps`` taps per channel
    (with bias) and SiLU; dt <- softplus(dt + dt_bias); per head (head h reads group h // (H / G)), with S [N, P]:
    S <- exp(-exp(A_log_h) dt) S + dt B x^T,  y = S^T C + D_h x.  The heads side by side are multiplied by silu(z),
    RMS-normed in ``norm_groups`` equal parts (each by its own root mean square) times a weight, and projected."""

    num_heads: int
    head_dim: int
    state_size: int
    num_groups: int
    conv_taps: int
    norm_groups: int
    norm_eps: float
    kind: str = "mamba2"


@dataclass(frozen=True)
class LightningSpec:
    """Linear attention with a matrix state per head and a fixed decay per head:
    S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t with q, k, v = activation(projection); the heads'
    outputs are normed together (RMS, learned scale), gated by sigmoid(gate projection) and projected."""

    num_heads: int
    key_dim: int
    value_dim: int
    decays: tuple[float, ...]
    norm_eps: float
    activation: str = "silu"
    kind: str = "lightning"


@dataclass(frozen=True)
class DiffAttentionSpec:
    """Grouped-query softmax attention with two score maps a head over the same values
    (differential attention): o = a1 - lam * a2, lam = exp(lq1.lk1) - exp(lq2.lk2) + ``diff``;
    each head's o is divided by its root mean square and multiplied by 1 - ``diff``.  Queries and keys
    are ``key_dim`` wide per map, values ``value_dim``; no position encoding."""

    num_heads: int
    num_kv_heads: int
    key_dim: int
    value_dim: int
    scale: float
    diff: float
    norm_eps: float
    qkv_bias: bool = True
    out_bias: bool = False
    kind: str = "diff_attention"


@dataclass(frozen=True)
class YarnRotarySpec:
    """Rotary position encoding over pairs of neighbouring dimensions (2i, 2i+1) of the first ``dims``
    dimensions of a vector, angle = position * f_i with f_i = base^(-2i/dims).  With ``factor`` set the
    frequencies are blended (YaRN) between the plain ones and the ones slowed by ``factor``: a pair that turns
    ``fast`` times or more within ``original`` positions keeps f_i, one that turns ``slow`` times or fewer gets
    f_i / factor, and between them the share of the slowed frequency grows linearly with the pair's index.  The
    index at which a pair turns r times is idx(r) = dims * log(original / (2 * pi * r)) / (2 * log(base)); the
    blend starts at first = max(floor(idx(fast)), 0) and is complete at last = min(ceil(idx(slow)), dims - 1):
    share_i = min(max((i - first) / max(last - first, 0.001), 0), 1).  Cosine and sine are both scaled by
    1 + 0.1 * log(factor)."""

    base: float
    dims: int
    factor: float | None = None
    original: float = 0.0
    fast: float = 32.0
    slow: float = 1.0
    kind: str = "yarn_pairs"


@dataclass(frozen=True)
class DeltaRuleSpec:
    """Gated delta rule: a matrix memory M [key_dim, value_dim] per head that a token first fades, then corrects
    by what it gets wrong about the token's key, then reads:
        M <- d M;   e = w (v - M^T k);   M <- M + k e^T;   y = M^T q,
    with q, k, v = silu(short causal filter(projection)), q and k of unit length per head (``unit_eps`` inside
    the root), q also over sqrt(key_dim), write strength w = sigmoid(projection) and fade
    d = exp(-exp(A) * softplus(projection + dt)).  Heads are served by ``num_kv_heads`` query/key heads in equal
    groups.  Every head's y is normed by its own root mean square, scaled by a weight common to the heads and
    gated by silu(gate projection); then the output projection."""

    num_heads: int
    num_kv_heads: int
    key_dim: int
    value_dim: int
    conv_taps: int
    norm_eps: float
    unit_eps: float = 1e-6
    kind: str = "delta_rule"


@dataclass(frozen=True)
class CappedAttentionSpec:
    """Grouped-query softmax attention whose values are the key projection itself (before its norm), with
    queries and keys RMS-normed over the whole projection row (all heads at once, learned weights), and a
    score  cap tanh(q.k scale / cap) - slope_h (i - j)  (``softcap`` None: no cap; ``slope_power`` None: no
    distance bias, else slope_h = 2^(-slope_power (h + 1) / heads)).  ``window`` w: position i sees
    i - w < j <= i.  ``q_temp`` (coef, every): the query at position p is multiplied by
    1 + coef ln(floor((p + 1) / every) + 1).  No position encoding."""

    num_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float
    norm_eps: float
    softcap: float | None = None
    window: int | None = None
    q_temp: tuple[float, int] | None = None
    slope_power: float | None = 8.0
    kind: str = "capped_attention"


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Attention through low-rank latents: queries W_uq rms(W_dq h), per head [``nope_dim`` plain |
    ``rope_dim`` rotated]; per token one latent c = rms(first ``kv_rank`` rows of W_dkv h) and one rotated key
    part (the last ``rope_dim`` rows) that every head uses; head by head the keys are W_uk c and the values W_uv c.
    Causal softmax of (q_plain . k_plain + q_rot . k_rot) * scale.  The cache holds c and the rotated key part only."""

    num_heads: int
    nope_dim: int
    rope_dim: int
    value_dim: int
    q_rank: int
    kv_rank: int
    scale: float
    norm_eps: float
    position: Any = None                # a position-encoding spec for the rotated parts
    kind: str = "latent_attention"


@dataclass(frozen=True)
class MLPSpec:
    """Dense feed-forward without a gate: down(act(up(x)))."""

    intermediate_size: int
    activation: str = "gelu_tanh"       # gelu_tanh | relu2 | silu
    kind: str = "mlp"


@dataclass(frozen=True)
class RoutedMLPSpec:
    """Mixture of small feed-forwards down(act(up(.))) without biases: every token goes to the ``top_k``
    experts with the largest router scores.  ``scoring``: sigmoid | softmax of the router logits (32-bit);
    ``renormalize``: the chosen scores divided by their sum; ``weight_on``: "input" (the score multiplies
    what the expert reads) or "output" (what it returns).  ``gated``: the experts are
    down(act(gate(.)) * up(.)).  ``correction``: a learned vector added to the scores for the choice only (the
    weights stay the scores).  ``identity``: so many more router outputs, behind the ``num_experts`` with
    tensors, are experts that return their input.  ``shared_intermediate_size``: one more feed-forward of the same
    form ('shared.up', 'shared.down') that every token uses, added unweighted."""

    num_experts: int
    top_k: int
    intermediate_size: int
    activation: str = "relu2"
    scoring: str = "sigmoid"
    renormalize: bool = False
    weight_on: str = "input"
    gated: bool = False
    correction: bool = False
    identity: int = 0
    shared_intermediate_size: int | None = None
    kind: str = "routed_mlp"


class LayerSpec:
    """One decoder layer: the spec of each of its parts under a ROLE name, and the arrangement that
    wires them.

    The roles are whatever the arrangement asks for.  "pre_norm" wants ``mixer``, ``feed_forward``,
    ``mixer_norm`` and ``ffn_norm``: ``h += mixer(norm(h)); h += ffn(norm(h))`` with the residual add
    deferred into the next norm (turingserve/model/qwen2.py:44-57).  An arrangement registered
    elsewhere may name others (a third norm, a second feed-forward); the same role names key the
    checkpoint prefixes in ``LayerTensorNames``.  A role's spec reads as an attribute: ``spec.mixer``.
    """

    def __init__(self, arrangement: str = "pre_norm", **roles: Any) -> None:
        if not roles:
            raise ValueError("a layer needs at least one part")
        object.__setattr__(self, "arrangement", arrangement)
        object.__setattr__(self, "roles", dict(roles))

    def __getattr__(self, role: str) -> Any:
        try:
            return self.__dict__["roles"][role]
        except KeyError:
            raise AttributeError(f"this layer has no part in role {role!r} (it has: "
                                 f"{', '.join(self.__dict__.get('roles', {}))})") from None

    def __setattr__(self, name: str, value: Any) -> None:
        raise AttributeError("LayerSpec is immutable")

    def __eq__(self, other: object) -> bool:
        return (isinstance(other, LayerSpec) and self.arrangement == other.arrangement
                and self.roles == other.roles)

    def __hash__(self) -> int:
        return hash((self.arrangement, tuple(sorted(self.roles))))

    def __repr__(self) -> str:
        inner = ", ".join(f"{k}={v!r}" for k, v in self.roles.items())
        return f"LayerSpec(arrangement={self.arrangement!r}, {inner})"


@dataclass(frozen=True)
class LayerRun:
    """One entry of the execution order.

    ``layer`` indexes ``ModelConfig.layers`` (the weights to use).  ``cache_from`` is None when
    this run owns a cache of its own, or the index of an EARLIER entry of the schedule whose
    cache this run reads without writing.  Every run has its own cache and state: a layer that runs
    twice keeps two.
    """

    layer: int
    cache_from: int | None = None
    # the embedding rows of the step are added to the stream before this run (a model that runs a span of
    # layers several times re-injects its input at the start of every later pass)
    add_embedding: bool = False
    # this run opens pass number ``opens_pass`` of a span of layers that runs several times: the model adds
    # that pass's own vector to the stream before it (None: it opens none)
    opens_pass: int | None = None


@dataclass(frozen=True)
class ModelConfig:
    architecture: str
    hidden_size: int
    vocab_size: int
    layers: tuple[LayerSpec, ...]
    schedule: tuple[LayerRun, ...]
    final_norm: Any
    tie_word_embeddings: bool
    max_position_embeddings: int
    eos_token_ids: tuple[int, ...] = ()
    bos_token_id: int | None = None
    # constants of the architecture that no part's spec holds (what a model class registered with the
    # architecture reads: an embedding multiplier, a cap on the logits); plain data from config.json
    extras: tuple[tuple[str, Any], ...] = ()

    def extra(self, key: str, default: Any = None) -> Any:
        return dict(self.extras).get(key, default)

    def __post_init__(self) -> None:
        if not self.layers:
            raise ValueError("a model needs at least one layer")
        for r, run in enumerate(self.schedule):
            if not 0 <= run.layer < len(self.layers):
                raise ValueError(f"schedule[{r}] names layer {run.layer}, model has {len(self.layers)}")
            if run.cache_from is not None:
                if not 0 <= run.cache_from < r:
                    raise ValueError(f"schedule[{r}].cache_from={run.cache_from} must name an earlier run")
                if self.schedule[run.cache_from].cache_from is not None:
                    raise ValueError(f"schedule[{r}].cache_from={run.cache_from} names a run without a cache")

    @property
    def num_runs(self) -> int:
        return len(self.schedule)

    def run_layer(self, run_index: int) -> LayerSpec:
        return self.layers[self.schedule[run_index].layer]

    def with_schedule(self, schedule: list[LayerRun] | tuple[LayerRun, ...]) -> ModelConfig:
        kw = {f.name: getattr(self, f.name) for f in fields(self)}
        kw["schedule"] = tuple(schedule)
        return ModelConfig(**kw)


def spec_to_dict(spec: Any) -> Any:
    """Plain-data view of a spec tree (for logs and for the ``config`` key of the benchmark)."""
    if isinstance(spec, LayerSpec):
        return {"arrangement": spec.arrangement, **{k: spec_to_dict(v) for k, v in spec.roles.items()}}
    if is_dataclass(spec) and not isinstance(spec, type):
        return {f.name: spec_to_dict(getattr(spec, f.name)) for f in fields(spec)}
    if isinstance(spec, (tuple, list)):
        return [spec_to_dict(s) for s in spec]
    return spec
