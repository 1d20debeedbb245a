"""Descriptions of parts: plain data that an architecture's configuration produces.

A model is described without naming the architecture it came from: a list of
layers, each naming the kind and the constants of its mixer, feed-forward and
norms, and a schedule that says in which order layers run. The reference
passes the same constants as constructor arguments
(app/architectures/starcoder2_layers.py:34-43, app/architectures/qwen_layers.py:35-45,
app/architectures/rope.py:16); here they are data so that a layer list can mix kinds.

A spec class only needs a string attribute ``kind``; the class registered under
that kind (``parts.base.register_part``) is built from it. New kinds need no change here.

No tensor name is written in this file: what the tensors of a layer are called in a
checkpoint is the architecture's business, so every name is a field that the
architecture's configuration fills in (config/starcoder2.py for StarCoder2).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any


@dataclass(frozen=True)
class LayerNormSpec:
    """``(x - mean) / sqrt(var + eps) * weight (+ bias)`` over the last axis. The tensors are called
    ``<prefix><weight_name>`` and ``<prefix><bias_name>``; an empty ``weight_name`` makes the prefix itself the
    weight's name."""

    size: int
    eps: float
    bias: bool = True
    weight_name: str = "weight"
    bias_name: str = "bias"
    kind: str = "layernorm"


@dataclass(frozen=True)
class RotarySpec:
    """Rotary position encoding, halves paired as (i, i + rotary_dim/2)."""

    rotary_dim: int
    theta: float
    kind: str = "rotary_neox"


@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query attention over a paged cache.

    ``window`` is None for plain causal attention; otherwise the query at
    absolute position p sees key j iff ``j <= p and j > p - window``.
    """

    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    bias: bool
    window: int | None
    scale: float
    # tensor names under the mixer's prefix, without ".weight" / ".bias": either three names (the
    # query, key and value projections as separate tensors, packed into one at load) or one name
    # (a checkpoint that stores them fused: rows of q, then k, then v), and the output projection
    projection_names: tuple[str, ...]
    output_name: str
    position: Any | None = None
    kind: str = "attention"

    def __post_init__(self) -> None:
        if len(self.projection_names) not in (1, 3):
            raise ValueError("projection_names holds three names (q, k, v) or one (fused qkv), "
                             f"not {len(self.projection_names)}")
        if self.num_heads % self.num_kv_heads != 0:
            raise ValueError(f"{self.num_heads} attention heads are no multiple of "
                             f"{self.num_kv_heads} kv heads")
        if self.head_dim <= 0 or self.head_dim % 16 != 0 or self.head_dim > 256:
            raise ValueError(f"head_dim {self.head_dim} is not a multiple of 16 up to 256: "
                             "no attention kernel of this engine takes it")


@dataclass(frozen=True)
class MlpSpec:
    """``down(act(up(x)))`` without a gate."""

    hidden_size: int
    intermediate_size: int
    bias: bool
    activation: str
    up_name: str                 # tensor names under the feed-forward's prefix
    down_name: str
    kind: str = "mlp"


@dataclass(frozen=True)
class RmsNormSpec:
    """``x / sqrt(mean(x^2) + eps) * scale`` over the last axis, eps inside the root. ``unit_offset``:
    the checkpoint stores ``scale - 1`` (a weight around zero). The tensor is called
    ``<prefix><weight_name>``; an empty ``weight_name`` makes the prefix itself the tensor's name."""

    size: int
    eps: float
    unit_offset: bool = False
    weight_name: str = "weight"
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class InterpolatedRotarySpec:
    """Rotary encoding of the first ``rotary_dim`` entries of a vector, halves paired as
    (i, i + rotary_dim/2), whose frequencies are stretched for contexts longer than the ``original`` one:
    pair i keeps ``theta^(-2i/rotary_dim)`` when it turns more than ``fast`` times within the original
    context, is divided by ``factor`` when it turns fewer than ``slow`` times, and is blended linearly in
    between; cos and sin are multiplied by ``0.1 ln(factor) + 1``. ``factor`` None: plain frequencies."""

    rotary_dim: int
    theta: float
    factor: float | None = None
    original: float = 0.0
    fast: float = 32.0
    slow: float = 1.0
    kind: str = "rotary_interpolated"

    def __post_init__(self) -> None:
        if self.rotary_dim < 0 or self.rotary_dim % 2:
            raise ValueError(f"a rotary encoding pairs dimensions: {self.rotary_dim} is odd or negative")
        if self.factor is not None and not (self.factor > 0 and self.original > 0 and self.fast > 0 and self.slow > 0):
            raise ValueError("frequency interpolation needs positive factor, original, fast and slow")


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Attention whose keys and values are expanded per head from one cached latent vector per token.

    A query head is ``[head_dim plain | rot_dim rotated]``; the down projection gives ``latent_rank``
    entries (RMS-normalised with a plain weight: the latent) and ``rot_dim`` more (one rotated key
    part shared by all heads). Head h's plain key is ``Uk_h latent``, its value ``Uv_h latent``
    (``value_dim`` wide); scores are ``(q_plain . k_plain + q_rot . k_rot) * scale`` under the window
    rule of ``AttentionSpec``. Names are full tensor names under the mixer's prefix.

    ``query_rank`` set: the queries go through a latent of their own, ``q = Uq n(Dq h)`` with ``n`` an RMS norm
    with a plain weight (``query_down_name``, ``query_norm_name``; ``query_name`` is then Uq, [heads * (head_dim +
    rot_dim), query_rank]). ``sink_name``: a learned logit per head that joins the softmax's denominator without a
    value. ``gate_name``: the concatenated heads are multiplied entry by entry with ``sigmoid(G h)`` before the
    output projection. The rotation pairs entries as ``position`` says."""

    hidden_size: int
    num_heads: int
    head_dim: int
    rot_dim: int
    value_dim: int
    latent_rank: int
    window: int | None
    scale: float
    eps: float
    position: Any                      # how the rot_dim parts are rotated
    query_name: str
    down_name: str
    latent_norm_name: str
    key_up_name: str
    value_up_name: str
    output_name: str
    query_rank: int | None = None
    query_down_name: str | None = None
    query_norm_name: str | None = None
    sink_name: str | None = None
    gate_name: str | None = None
    kind: str = "latent_attention"

    def __post_init__(self) -> None:
        if min(self.num_heads, self.head_dim, self.value_dim, self.latent_rank) <= 0 or self.rot_dim < 0:
            raise ValueError("latent attention needs positive head count, head sizes and latent rank")
        if self.position is not None and self.position.rotary_dim > self.rot_dim:
            raise ValueError(f"{self.position.rotary_dim} rotated dimensions exceed the rotated part of {self.rot_dim}")
        if self.query_rank is not None and (self.query_rank <= 0 or self.query_down_name is None
                                            or self.query_norm_name is None):
            raise ValueError("queries through a latent need its positive rank and the names of its projection and norm")


@dataclass(frozen=True)
class GatedAttentionSpec:
    """Grouped-query attention without position encoding: queries and keys are RMS-normalised per head
    (one plain weight of ``head_dim`` entries for all query heads, one for all key heads; None: no norm),
    values are ``value_dim`` wide, and the concatenated heads are multiplied by ``sigmoid(gate(h))``
    before the output projection (``gate_name`` None: no gate). Window rule as ``AttentionSpec``."""

    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    value_dim: int
    window: int | None
    scale: float
    eps: float
    query_name: str
    key_name: str
    value_name: str
    output_name: str
    gate_name: str | None = None
    query_norm_name: str | None = None
    key_norm_name: str | None = None
    kind: str = "gated_attention"

    def __post_init__(self) -> None:
        if self.num_kv_heads <= 0 or self.num_heads % self.num_kv_heads != 0:
            raise ValueError(f"{self.num_heads} attention heads are no multiple of {self.num_kv_heads} kv heads")
        if self.head_dim <= 0 or self.value_dim <= 0 or max(self.head_dim, self.value_dim) > 256:
            raise ValueError(f"head sizes {self.head_dim} / {self.value_dim} are outside 1..256: "
                             "no attention kernel of this engine takes them")


@dataclass(frozen=True)
class UnitNormAttentionSpec:
    """Causal grouped-query attention without biases whose queries and keys are rotated over the first entries of
    every head (``position``; None: no rotation) and then divided, head by head, by their root mean square over
    ``head_dim`` (eps inside the root, no learned weight; ``unit_norm`` False leaves them as they are). Scores are
    ``q . k * scale`` under an ordinary softmax; values are ``value_dim`` wide.

    ``window`` None: every earlier key is seen. Otherwise the query at p sees key j iff ``j <= p`` and
    (``p - j < window`` or ``j < keep_first``): the sequence's first ``keep_first`` tokens stay in sight for good,
    at their true positions."""

    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    value_dim: int
    window: int | None
    keep_first: int
    scale: float
    eps: float
    position: Any | None
    query_name: str
    key_name: str
    value_name: str
    output_name: str
    unit_norm: bool = True
    kind: str = "unit_norm_attention"

    def __post_init__(self) -> None:
        if self.num_kv_heads <= 0 or self.num_heads % self.num_kv_heads != 0:
            raise ValueError(f"{self.num_heads} attention heads are no multiple of {self.num_kv_heads} kv heads")
        if self.head_dim <= 0 or self.value_dim <= 0 or max(self.head_dim, self.value_dim) > 256:
            raise ValueError(f"head sizes {self.head_dim} / {self.value_dim} are outside 1..256: "
                             "no attention kernel of this engine takes them")
        if self.window is not None and self.window <= 0:
            raise ValueError(f"a window holds at least the query's own position, got {self.window}")
        if self.keep_first < 0:
            raise ValueError(f"the number of first tokens kept in sight cannot be negative, got {self.keep_first}")
        if self.position is not None and self.position.rotary_dim > self.head_dim:
            raise ValueError(f"{self.position.rotary_dim} rotated entries exceed the head of {self.head_dim}")


@dataclass(frozen=True)
class TokenSideInputSpec:
    """What a layer adds to the stream from the token itself. A table shared by all layers (``table_name``, a full
    tensor name, [vocab, table_width]) holds for every token a vector per layer; this layer reads the columns
    ``[column, column + dim)``: ``g = gelu_tanh(G x) * e``, ``y = P g``, ``x <- x + y / rms(y) * norm`` with
    ``rms(y) = sqrt(mean(y^2) + eps)``. G, P and the norm's weight lie under the part's prefix."""

    hidden_size: int
    vocab_size: int
    dim: int
    column: int
    table_width: int
    eps: float
    table_name: str
    gate_name: str
    proj_name: str
    norm_name: str
    kind: str = "token_side_input"

    def __post_init__(self) -> None:
        if self.dim <= 0 or self.column < 0 or self.column + self.dim > self.table_width:
            raise ValueError(f"columns {self.column}..{self.column + self.dim} lie outside a table of {self.table_width}")


@dataclass(frozen=True)
class RglruSpec:
    """A gated linear recurrence behind a short causal convolution, times a GELU branch.

    ``y = gelu_tanh(Wy h + by)``, ``u = conv(Wx h + bx)`` (``taps`` per channel, the last tap on the
    current token); per block b of ``width / blocks`` channels ``r = sigmoid(Ra_b u_b + ba_b)`` and
    ``i = sigmoid(Ri_b u_b + bi_b)``; ``a = exp(-decay * r * softplus(lambda))``,
    ``S <- a S + sqrt(1 - a^2) i u`` from S = 0; the mixer's output is ``Wo (S * y)``."""

    hidden_size: int
    width: int
    blocks: int
    taps: int
    decay: float
    gate_branch_name: str              # y
    recurrent_branch_name: str         # x
    conv_name: str
    recurrence_gate_name: str
    input_gate_name: str
    lambda_name: str
    output_name: str
    bias_suffix: str = ".b"
    kind: str = "rglru"

    def __post_init__(self) -> None:
        if self.blocks <= 0 or self.width <= 0 or self.width % self.blocks:
            raise ValueError(f"a recurrence of {self.width} channels cannot be cut into {self.blocks} equal blocks")
        if self.taps < 1:
            raise ValueError("the convolution needs at least one tap")


@dataclass(frozen=True)
class ClampedGluSpec:
    """``down(g * sigmoid(slope * g) * (u + shift))`` with ``g = min(gate(h), limit)`` and
    ``u = clamp(up(h), -limit, limit)``; ``limit`` None leaves both unclamped. No biases."""

    hidden_size: int
    intermediate_size: int
    limit: float | None
    gate_name: str
    up_name: str
    down_name: str
    slope: float = 1.702
    shift: float = 1.0
    kind: str = "clamped_glu"


@dataclass(frozen=True)
class DynamicTanhSpec:
    """A norm without statistics: ``tanh(alpha * x) * weight + shift``, entry by entry, with one learned scalar
    ``alpha``. The three tensors are ``<prefix><weight_name>``, ``<prefix><shift_name>`` and ``<prefix><alpha_name>``."""

    size: int
    weight_name: str = "weight"
    shift_name: str = "bias"
    alpha_name: str = "alpha"
    kind: str = "dynamic_tanh"


@dataclass(frozen=True)
class WavelengthRotarySpec:
    """Rotary encoding of the first ``rotary_dim`` entries of a head, halves paired as (i, i + rotary_dim/2), with
    frequencies ``f_i = theta^(-2i/rotary_dim)`` rescaled by wavelength ``l = 2 pi / f`` for contexts longer than the
    ``original`` one: kept where ``l < original / high``, divided by ``factor`` where ``l > original / low``, and
    blended between, ``(1 - s) f / factor + s f`` with ``s = (original / l - low) / (high - low)``. ``factor`` None:
    plain frequencies."""

    rotary_dim: int
    theta: float
    factor: float | None = None
    original: float = 0.0
    low: float = 0.0
    high: float = 0.0
    kind: str = "rotary_wavelength"

    def __post_init__(self) -> None:
        if self.rotary_dim < 0 or self.rotary_dim % 2:
            raise ValueError(f"a rotary encoding pairs dimensions: {self.rotary_dim} is odd or negative")
        if self.factor is not None and not (self.factor > 0 and self.original > 0 and self.high > self.low > 0):
            raise ValueError("wavelength scaling needs positive factor and original and 0 < low < high")


@dataclass(frozen=True)
class SinkAttentionSpec:
    """Causal grouped-query attention with biased projections, a rotation of the first entries of every query and
    key head (``position``; None: none), scores ``softcap * tanh(q . k * scale / softcap)`` (``softcap`` None: plain
    scores), a learned logit per head that joins the softmax's denominator without a value (``sink_name`` None: no
    sink), values of a width of their own, and one sigmoid gate per head on the output (``gate_name`` None: no gate).

    ``value_mix`` ties layers together: a layer that says ``"source"`` publishes its values for the step's
    tokens; a layer that says ``"blend"`` stores and attends over ``(1 - m) v + m v_source`` with its
    learned scalar ``m`` (``value_mix_name``). Window rule as ``AttentionSpec``."""

    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    value_dim: int
    window: int | None
    scale: float
    softcap: float | None
    bias: bool
    position: Any | None
    query_name: str
    key_name: str
    value_name: str
    output_name: str
    gate_name: str | None = None
    sink_name: str | None = None
    value_mix: str | None = None              # None | "source" | "blend"
    value_mix_name: str | None = None         # the scalar's tensor; declared (and read) where it is named
    value_mix_key: str = "value_mix"
    bias_suffix: str = ".b"
    kind: str = "sink_attention"

    def __post_init__(self) -> None:
        if self.num_kv_heads <= 0 or self.num_heads % self.num_kv_heads != 0:
            raise ValueError(f"{self.num_heads} attention heads are no multiple of {self.num_kv_heads} kv heads")
        if self.head_dim <= 0 or self.value_dim <= 0 or max(self.head_dim, self.value_dim) > 256:
            raise ValueError(f"head sizes {self.head_dim} / {self.value_dim} are outside 1..256: "
                             "no attention kernel of this engine takes them")
        if self.value_mix not in (None, "source", "blend"):
            raise ValueError(f"value_mix is None, 'source' or 'blend', not {self.value_mix!r}")
        if self.value_mix == "blend" and self.value_mix_name is None:
            raise ValueError("a layer that blends values needs the name of its mixing scalar")
        if self.position is not None and self.position.rotary_dim > self.head_dim:
            raise ValueError(f"{self.position.rotary_dim} rotated entries exceed the head of {self.head_dim}")
        if self.softcap is not None and not self.softcap > 0:
            raise ValueError(f"a score cap must be positive, got {self.softcap}")


@dataclass(frozen=True)
class PairedRotarySpec:
    """Rotary encoding of the first ``rotary_dim`` entries of a head with plain frequencies
    ``f_i = theta^(-2i/rotary_dim)``. ``pairing`` says which entries turn together: ``"half"`` pairs entry i with
    entry i + rotary_dim/2, ``"interleaved"`` pairs entry 2i with entry 2i + 1 (i < rotary_dim/2). The pair
    ``(u, v)`` at position p becomes ``(u cos a - v sin a, v cos a + u sin a)`` with ``a = p f_i``."""

    rotary_dim: int
    theta: float
    pairing: str = "half"
    kind: str = "rotary_paired"

    def __post_init__(self) -> None:
        if self.rotary_dim < 0 or self.rotary_dim % 2:
            raise ValueError(f"a rotary encoding pairs dimensions: {self.rotary_dim} is odd or negative")
        if self.pairing not in ("half", "interleaved"):
            raise ValueError(f"pairing is 'half' or 'interleaved', not {self.pairing!r}")
        if not self.theta > 0:
            raise ValueError(f"the rotary base must be positive, got {self.theta}")


@dataclass(frozen=True)
class NormedRotaryAttentionSpec:
    """Grouped-query attention without biases whose queries and keys are RMS-normalised head by head (one plain
    weight of ``head_dim`` entries for all query heads, one for all key heads; a name of None: no norm) and THEN
    rotated over their first entries (``position``, a ``PairedRotarySpec``; None: no rotation). Scores are
    ``q . k * scale``, optionally capped to ``softcap * tanh(score / softcap)``; values are ``value_dim`` wide.

    ``mask`` names the rule beside ``j <= p``: ``"causal"`` (nothing more), ``"window"`` (``p - j < mask_size``) or
    ``"chunk"`` (``p // mask_size == j // mask_size``: the sequence is cut into blocks of ``mask_size`` positions
    counted from its start, and a query sees its own block only). ``sink``: ``None`` for the ordinary softmax,
    ``"zero"`` for a denominator with one added (a logit of 0 without a value), ``"learned"`` for a learned logit
    per head (``sink_name``). ``gate``: ``None``, ``"head"`` (head h times ``sigmoid(G h)_h``, G has one row per head)
    or ``"entry"`` (the concatenated heads times ``sigmoid(G h)`` entry by entry); the gate reads the mixer's input."""

    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    value_dim: int
    scale: float
    eps: float
    position: Any | None
    query_name: str
    key_name: str
    value_name: str
    output_name: str
    mask: str = "causal"
    mask_size: int = 0
    softcap: float | None = None
    sink: str | None = None
    sink_name: str | None = None
    gate: str | None = None
    gate_name: str | None = None
    query_norm_name: str | None = None
    key_norm_name: str | None = None
    kind: str = "normed_rotary_attention"

    def __post_init__(self) -> None:
        if self.num_kv_heads <= 0 or self.num_heads % self.num_kv_heads != 0:
            raise ValueError(f"{self.num_heads} attention heads are no multiple of {self.num_kv_heads} kv heads")
        if self.head_dim <= 0 or self.value_dim <= 0 or max(self.head_dim, self.value_dim) > 256:
            raise ValueError(f"head sizes {self.head_dim} / {self.value_dim} are outside 1..256: "
                             "no attention kernel of this engine takes them")
        if self.mask not in ("causal", "window", "chunk"):
            raise ValueError(f"mask is 'causal', 'window' or 'chunk', not {self.mask!r}")
        if self.mask != "causal" and self.mask_size <= 0:
            raise ValueError(f"a {self.mask} mask needs a positive size, got {self.mask_size}")
        if self.sink not in (None, "zero", "learned") or (self.sink == "learned" and self.sink_name is None):
            raise ValueError("sink is None, 'zero' or 'learned' (with the tensor's name)")
        if self.gate not in (None, "head", "entry") or (self.gate is not None and self.gate_name is None):
            raise ValueError("gate is None, 'head' or 'entry' (with the tensor's name)")
        if self.position is not None and self.position.rotary_dim > self.head_dim:
            raise ValueError(f"{self.position.rotary_dim} rotated entries exceed the head of {self.head_dim}")
        if self.softcap is not None and not self.softcap > 0:
            raise ValueError(f"a score cap must be positive, got {self.softcap}")


@dataclass(frozen=True)
class ReinjectionSpec:
    """What a model does to the stream before every pass of a repeated run of layers: with x0 the embedding output
    of the step's tokens, ``x <- M [x; x0] + s_t`` for pass t, where M is ``[hidden, 2 hidden]`` (the stream's columns
    first) and s is ``[passes, hidden]``. Full tensor names."""

    hidden_size: int
    passes: int
    matrix_name: str
    step_name: str
    kind: str = "reinjection"

    def __post_init__(self) -> None:
        if self.passes <= 0:
            raise ValueError(f"a repeated run has at least one pass, got {self.passes}")


@dataclass(frozen=True)
class GlaSpec:
    """Gated linear attention: per head a state ``S <- diag(a_t) S + k_t v_t^T`` from S = 0 and ``o_t = S^T q_t``
    with ``q = Wq h * query_scale``, ``k = Wk h`` (``head_dim`` wide), ``v = Wv h`` (``value_dim`` wide) and a decay
    per key channel ``a = sigmoid(A2 (A1 h) + b)^(1/tau)``; every head's o is RMS-normalised over ``value_dim`` with
    one plain weight shared by the heads, the heads are multiplied by ``silu(Wg h)`` and projected by Wo."""

    hidden_size: int
    num_heads: int
    head_dim: int
    value_dim: int
    decay_rank: int
    tau: float
    query_scale: float
    eps: float
    query_name: str
    key_name: str
    value_name: str
    gate_name: str
    output_name: str
    norm_name: str
    decay_down_name: str                # A1 [rank, hidden]
    decay_up_name: str                  # A2 [heads * head_dim, rank]
    bias_suffix: str = ".b"
    kind: str = "gla"

    def __post_init__(self) -> None:
        if min(self.num_heads, self.head_dim, self.value_dim, self.decay_rank) <= 0:
            raise ValueError("gated linear attention needs positive head count, head sizes and decay rank")
        if self.head_dim > 256:
            raise ValueError(f"{self.head_dim} key channels per head: the recurrence kernel takes up to 256")
        if self.decay_rank > 768:
            raise ValueError(f"a decay rank of {self.decay_rank}: the decay kernel takes up to 768")
        if not self.tau > 0:
            raise ValueError(f"tau must be positive, got {self.tau}")


@dataclass(frozen=True)
class GatedMlpSpec:
    """``down(act(gate(h)) * up(h))`` without biases; ``activation`` is ``gelu_tanh`` or ``silu``."""

    hidden_size: int
    intermediate_size: int
    activation: str
    gate_name: str
    up_name: str
    down_name: str
    kind: str = "gated_mlp"


@dataclass(frozen=True)
class RoutedExpertsSpec:
    """A mixture of ``num_experts`` gated feed-forwards (``GatedMlpSpec`` each, tensors under
    ``<prefix><expert_format.format(index=e)>``), of which a token runs ``top``. Router logits ``R h`` and scores
    ``sigmoid`` are float. The experts form ``num_groups`` equal runs of neighbours; a run is worth the sum of its
    ``group_best`` largest scores and only the ``groups_kept`` best runs may supply experts. The output is the sum
    of the chosen experts' outputs weighted by ``score / (sum of chosen scores + norm_eps) * route_scale``.

    ``score="softmax"`` is another rule: scores are the softmax over all router rows, the ``top`` rows with the
    largest ``score + correction`` win (``correction_name``: a float per row, None: none) and the weights use the
    plain scores; there are no groups and no ``route_scale``. The router then has ``num_experts + num_identity``
    rows, the last ``num_identity`` of which stand for experts without tensors whose output is their input.
    ``expert`` may be a ``GatedMlpSpec`` or a ``ClampedGluSpec``. ``shared`` (a feed-forward spec, tensors under
    ``<prefix><shared_name>``) runs for every token and is added. With ``bias_name`` the logits are ``R h + b``; the
    softmax rule with such a bias and without a correction is the same as choosing the ``top`` largest logits and
    weighting them by the softmax over the chosen logits alone."""

    hidden_size: int
    num_experts: int
    top: int
    num_groups: int
    groups_kept: int
    route_scale: float
    expert: Any                          # GatedMlpSpec
    router_name: str
    expert_format: str = "e{index}."
    group_best: int = 2
    norm_eps: float = 1e-20
    score: str = "sigmoid"
    correction_name: str | None = None
    bias_name: str | None = None          # softmax rule: a float per router row added to the logits themselves
    num_identity: int = 0
    shared: Any | None = None
    shared_name: str = "shared."
    kind: str = "routed_experts"

    def __post_init__(self) -> None:
        if self.score not in ("sigmoid", "softmax"):
            raise ValueError(f"router scores are 'sigmoid' or 'softmax', not {self.score!r}")
        if self.num_identity < 0 or self.num_experts < 0:
            raise ValueError("expert counts cannot be negative")
        if self.score == "sigmoid" and (self.num_identity or self.correction_name is not None
                                        or self.bias_name is not None):
            raise ValueError("experts without tensors, a correction of the choice and a bias on the logits belong "
                             "to the softmax rule")
        if self.score == "softmax" and (self.num_groups != 1 or self.route_scale != 1.0):
            raise ValueError("the softmax rule has neither groups nor a scale of its weights")
        if not 0 < self.top <= self.num_experts + self.num_identity:
            raise ValueError(f"a token cannot run {self.top} of {self.num_experts + self.num_identity} experts")
        if self.score == "softmax":
            if self.norm_eps != 1e-20:
                raise ValueError("the routing kernel adds 1e-20 to the sum")
            return
        if self.num_groups <= 0 or self.num_experts % self.num_groups:
            raise ValueError(f"{self.num_experts} experts cannot form {self.num_groups} equal groups")
        if not 0 < self.groups_kept <= self.num_groups:
            raise ValueError(f"{self.groups_kept} of {self.num_groups} groups cannot be kept")
        if self.groups_kept * (self.num_experts // self.num_groups) < self.top:
            raise ValueError(f"{self.groups_kept} kept groups hold fewer than {self.top} experts")
        if self.group_best != 2 or self.norm_eps != 1e-20:
            raise ValueError("the routing kernel ranks groups by their two best scores and adds 1e-20 to the sum")


@dataclass(frozen=True)
class LayerSpec:
    """One decoder layer: which block arrangement holds which parts. ``feed_forward`` (with its norm)
    may be None for blocks that can do without; ``skip_scale`` is the weight of the skip path in blocks
    that have one (``norm(skip_scale * x + sublayer(x))``)."""

    mixer: Any
    feed_forward: Any
    mixer_norm: Any
    ffn_norm: Any
    # weight-name fragments under the layer's prefix ("<layer_prefix>.<index>.")
    mixer_name: str
    feed_forward_name: str
    mixer_norm_name: str
    ffn_norm_name: str
    block: str = "pre_norm_sequential"
    skip_scale: float = 1.0
    # blocks that scale a branch entry by entry before it joins the stream: the tensors' name fragments under the
    # layer's prefix for the mixer's and the feed-forward's branch (None: no scale)
    branch_scale_names: tuple[str | None, str | None] = (None, None)
    # what the layer adds to the stream after its sublayers (``TokenSideInputSpec``; None: nothing) and its fragment
    side_input: Any | None = None
    side_input_name: str = ""
    # blocks that normalise a sublayer's output as well as its input: the norms behind the mixer and behind the
    # feed-forward and their name fragments
    mixer_out_norm: Any | None = None
    ffn_out_norm: Any | None = None
    mixer_out_norm_name: str = ""
    ffn_out_norm_name: str = ""
    # what the pre-norm block puts behind a part's name fragment to make its prefix ("" for checkpoints whose
    # fragments carry their own separators, as the post-norm block expects them)
    part_separator: str = "."


@dataclass(frozen=True)
class ScheduleEntry:
    """One execution of a layer.

    ``layer`` indexes ``ModelSpec.layers`` (a layer may be named by several
    entries: its weights are then shared, each execution keeps a cache of its
    own). ``cache_of`` names an earlier schedule entry whose cache this
    execution reads instead of owning one; it then writes nothing.
    """

    layer: int
    cache_of: int | None = None
    # the entry opens pass number ``pass_index`` of a repeated run of layers: the model's ``pass_input`` part
    # transforms the stream right before it (None: nothing happens before the entry)
    pass_index: int | None = None


@dataclass(frozen=True)
class ModelSpec:
    hidden_size: int
    vocab_size: int
    layers: tuple[LayerSpec, ...]
    schedule: tuple[ScheduleEntry, ...]
    final_norm: Any
    tie_word_embeddings: bool
    max_position_embeddings: int
    # tensor names: "<embedding_name>.weight", "<layer_prefix>.<index>.", "<final_norm_name>.",
    # "<head_name>.weight" (read only when the head is not tied to the embedding)
    embedding_name: str
    layer_prefix: str
    final_norm_name: str
    head_name: str
    # what some architectures do around the layers (StarCoder2 does none of it): the looked-up
    # embeddings times a constant, a bias on the output head ("<head_name>.bias"), and scores
    # squashed to cap * tanh(score / cap)
    embedding_scale: float = 1.0
    head_bias: bool = False
    logit_softcap: float | None = None
    logit_scale: float = 1.0             # logits times a constant
    # what happens to the stream before the schedule entries that open a pass (``ReinjectionSpec``; None: nothing)
    pass_input: Any | None = None
    # how names are put together: "<embedding_name><weight_suffix>", a layer's prefix from
    # ``layer_prefix_format`` (fields {prefix} and {index}), the final norm's prefix (None:
    # "<final_norm_name>.")
    weight_suffix: str = ".weight"
    layer_prefix_format: str = "{prefix}.{index}."
    final_norm_prefix: str | None = None
    extra: dict = field(default_factory=dict, compare=False, hash=False)

    def __post_init__(self) -> None:
        for position, entry in enumerate(self.schedule):
            if entry.pass_index is not None and self.pass_input is None:
                raise ValueError(f"schedule entry {position} opens a pass, but the model describes no pass input")
            if not 0 <= entry.layer < len(self.layers):
                raise ValueError(f"schedule entry {position} names layer {entry.layer}, "
                                 f"but the model has {len(self.layers)} layers")
            if entry.cache_of is not None:
                if not 0 <= entry.cache_of < position:
                    raise ValueError(f"schedule entry {position} reads the cache of entry "
                                     f"{entry.cache_of}, which does not run before it")
                if self.schedule[entry.cache_of].cache_of is not None:
                    raise ValueError(f"schedule entry {position} reads the cache of entry "
                                     f"{entry.cache_of}, which owns no cache itself")


    def layer_prefix_of(self, index: int) -> str:
        return self.layer_prefix_format.format(prefix=self.layer_prefix, index=index)

    @property
    def norm_prefix(self) -> str:
        return f"{self.final_norm_name}." if self.final_norm_prefix is None else self.final_norm_prefix


def sequential_schedule(num_layers: int) -> tuple[ScheduleEntry, ...]:
    return tuple(ScheduleEntry(layer=i) for i in range(num_layers))
