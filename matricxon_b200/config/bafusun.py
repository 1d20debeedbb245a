"""Bafusun configuration: a decoder whose sublayers read the stream itself and are normalised on their way out.

``config.json`` holds ``architecture: "Bafusun"``, ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``,
``logit_scale``, ``token_side.dim`` (absent: no per-layer token input) and a list ``layers``; every entry gives
``type`` (``attention``), the mixer's sizes under ``mixer`` (``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``,
``rot`` with ``dims`` and ``base``, ``mask`` with ``size`` and ``keep_first``) and its feed-forward under ``mlp``
(``kind: moe`` with ``expert`` (``ff``, ``limit``), ``router`` (``experts``, ``identity``, ``top``) and an optional
``shared`` expert, or null for a layer that has only the mixer sublayer).

A layer computes ``x += ls1 * norm1(mixer(x))``, then ``x += ls2 * norm2(ff(x))``, then adds what the token itself
brings (``parts.side_input``). Norms are layer norms with a weight and no bias. The logits come from the embedding
table itself (without the embedding's scale) times ``logit_scale``.

Tensor names: ``embed``, ``side.embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.ls1``, ``l<i>.ls2``,
``l<i>.mix.{q,k,v,o}``, ``l<i>.mlp.e<j>.{gate,up,down}``, ``l<i>.mlp.router``, ``l<i>.mlp.correction``,
``l<i>.mlp.shared.{gate,up,down}``, ``l<i>.side.{gate,proj,norm}``, ``final.norm`` (no ``.weight`` suffix). This
file is the only place that knows those names and keys; the parts are generic.
"""

from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Any

from matricxon_b200.config.base import ConfigError, ConfigReader
from matricxon_b200.parts.spec import (
    ClampedGluSpec,
    LayerNormSpec,
    LayerSpec,
    ModelSpec,
    RoutedExpertsSpec,
    TokenSideInputSpec,
    UnitNormAttentionSpec,
    WavelengthRotarySpec,
    sequential_schedule,
)

# what the design fixes
GATE_SLOPE = 1.702                   # an expert's gate is g * sigmoid(1.702 g)
UP_SHIFT = 1.0                       # ... times (u + 1)
ROUTE_NORM_EPS = 1e-20               # added to the sum of the chosen scores
SIDE_TABLE_NAME = "side.embed"       # one table for all layers, a layer's columns side by side
# no key of config.json limits a sequence's length; this sizes the block tables of captured steps
# (longer sequences run uncaptured)
DEFAULT_MAX_POSITIONS = 32768


def _object(raw: Any, key: str, where: str) -> dict:
    value = raw.get(key) if isinstance(raw, dict) else None
    if not isinstance(value, dict):
        raise ConfigError(f"{where}: {key!r} must be an object")
    return value


@dataclass(frozen=True)
class BafusunExpert:
    ff: int
    limit: float

    @classmethod
    def from_dict(cls, raw: Any, where: str) -> "BafusunExpert":
        r = ConfigReader(raw, where)
        return cls(ff=r.integer("ff", minimum=1), limit=r.number("limit", positive=True))

    def to_dict(self) -> dict:
        return {"ff": self.ff, "limit": self.limit}


@dataclass(frozen=True)
class BafusunFeedForward:
    expert: BafusunExpert
    experts: int                  # experts with matrices
    identity: int                 # router rows beyond them: experts that return their input
    top: int
    shared: BafusunExpert | None = None

    @classmethod
    def from_dict(cls, raw: Any, where: str) -> "BafusunFeedForward":
        r = ConfigReader(raw, where)
        kind = r.string("kind")
        if kind != "moe":
            raise ConfigError(f"{where}: unknown feed-forward kind {kind!r}; Bafusun has 'moe'")
        router = ConfigReader(_object(raw, "router", where), where + ".router")
        experts, identity = router.integer("experts", minimum=1), router.integer("identity", 0, minimum=0)
        top = router.integer("top", minimum=1)
        if top > experts + identity:
            raise ConfigError(f"{where}.router: 'top' ({top}) exceeds the {experts + identity} router outputs")
        expert = BafusunExpert.from_dict(_object(raw, "expert", where), where + ".expert")
        shared = None
        if raw.get("shared") is not None:
            shared = BafusunExpert.from_dict(raw["shared"], where + ".shared")
        return cls(expert=expert, experts=experts, identity=identity, top=top, shared=shared)

    def to_dict(self) -> dict:
        out: dict[str, Any] = {"expert": self.expert.to_dict(), "kind": "moe",
                               "router": {"experts": self.experts, "identity": self.identity, "top": self.top}}
        if self.shared is not None:
            out["shared"] = self.shared.to_dict()
        return out


@dataclass(frozen=True)
class BafusunLayer:
    type: str                     # "attention"
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_dims: int = 0             # 0: no rotation
    rot_base: float = 10000.0
    window: int | None = None     # None: every earlier token is seen
    keep_first: int = 0
    feed_forward: BafusunFeedForward | None = None

    @classmethod
    def from_dict(cls, raw: Any, where: str) -> "BafusunLayer":
        r = ConfigReader(raw, where)
        kind = r.string("type")
        if kind != "attention":
            raise ConfigError(f"{where}: unknown layer type {kind!r}; Bafusun has 'attention'")
        mixer = _object(raw, "mixer", where)
        m = ConfigReader(mixer, where + ".mixer")
        heads, dim = m.integer("heads", minimum=1), m.integer("dim", minimum=1)
        kv_heads, vdim = m.integer("kv_heads", heads, minimum=1), m.integer("vdim", dim, minimum=1)
        if heads % kv_heads:
            raise ConfigError(f"{where}.mixer: heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
        if max(dim, vdim) > 256:
            raise ConfigError(f"{where}.mixer: head sizes above 256 have no attention kernel")
        fields: dict[str, Any] = {"type": kind, "heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
                                  "scale": m.number("scale", positive=True)}
        if mixer.get("rot") is not None:
            rot = ConfigReader(mixer["rot"], where + ".mixer.rot")
            dims = rot.integer("dims", minimum=0)
            if dims % 2 or dims > dim:
                raise ConfigError(f"{where}.mixer.rot: 'dims' must be even and at most dim ({dim}), got {dims}")
            fields["rot_dims"], fields["rot_base"] = dims, rot.number("base", positive=True)
        if mixer.get("mask") is not None:
            mask = ConfigReader(mixer["mask"], where + ".mixer.mask")
            fields["window"] = mask.integer("size", minimum=1)
            fields["keep_first"] = mask.integer("keep_first", 0, minimum=0)
        if raw.get("mlp") is not None:
            fields["feed_forward"] = BafusunFeedForward.from_dict(raw["mlp"], where + ".mlp")
        return cls(**fields)

    def to_dict(self) -> dict:
        mixer: dict[str, Any] = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads,
                                 "scale": self.scale, "vdim": self.vdim}
        if self.rot_dims:
            mixer["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
        if self.window is not None:
            mixer["mask"] = {"keep_first": self.keep_first, "size": self.window}
        return {"mixer": mixer, "mlp": self.feed_forward.to_dict() if self.feed_forward else None, "type": self.type}


@dataclass(frozen=True)
class BafusunConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    logit_scale: float
    side_dim: int                 # 0: layers take nothing from the token itself
    layers: tuple[BafusunLayer, ...]
    max_positions: int = DEFAULT_MAX_POSITIONS
    # tensors a model folder holds although the model does not use them (the second norm and scale of a layer
    # without a feed-forward): (name, shape), found by ``with_tensor_shapes``; expected at the weight check and
    # never fetched
    unused_tensors: tuple[tuple[str, tuple[int, ...]], ...] = ()

    architecture = "Bafusun"
    model_type = "bafusun"

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @classmethod
    def from_dict(cls, raw: dict[str, Any], where: str = "config.json") -> "BafusunConfig":
        r = ConfigReader(raw, where)
        eps = ConfigReader(_object(raw, "norm", where), where + ".norm").number("eps", positive=True)
        scale = 1.0
        if raw.get("embedding") is not None:
            scale = ConfigReader(_object(raw, "embedding", where), where + ".embedding").number("scale", 1.0)
        side_dim = 0
        if raw.get("token_side") is not None:
            side_dim = ConfigReader(_object(raw, "token_side", where), where + ".token_side").integer("dim", minimum=1)
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError(f"{where}: 'layers' must be a non-empty list")
        parsed = tuple(BafusunLayer.from_dict(layer, f"{where}.layers[{i}]") for i, layer in enumerate(layers))
        return cls(vocab=r.integer("vocab", minimum=1), width=r.integer("width", minimum=1), eps=eps,
                   embedding_scale=scale, logit_scale=r.number("logit_scale", 1.0), side_dim=side_dim, layers=parsed,
                   max_positions=r.integer("max_positions", DEFAULT_MAX_POSITIONS, minimum=1))

    def with_tensor_shapes(self, shape_of) -> "BafusunConfig":
        """The configuration with the tensors noted that a folder holds for sublayers a layer does not have:
        ``shape_of(name)`` gives a tensor's shape or None."""
        unused = []
        for index, layer in enumerate(self.layers):
            if layer.feed_forward is not None:
                continue
            for name in (f"l{index}.norm2", f"l{index}.ls2"):
                shape = shape_of(name)
                if shape is not None:
                    unused.append((name, tuple(int(extent) for extent in shape)))
        return replace(self, unused_tensors=tuple(unused))

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"architecture": self.architecture, "embedding": {"scale": self.embedding_scale},
                               "layers": [layer.to_dict() for layer in self.layers], "logit_scale": self.logit_scale,
                               "norm": {"eps": self.eps}, "vocab": self.vocab, "width": self.width}
        if self.side_dim:
            out["token_side"] = {"dim": self.side_dim}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        return out

    # ------------------------------------------------------------------ description
    def _mixer_spec(self, layer: BafusunLayer):
        position = None
        if layer.rot_dims > 0:
            position = WavelengthRotarySpec(rotary_dim=layer.rot_dims, theta=layer.rot_base)
        return UnitNormAttentionSpec(
            hidden_size=self.width, num_heads=layer.heads, num_kv_heads=layer.kv_heads, head_dim=layer.dim,
            value_dim=layer.vdim, window=layer.window, keep_first=layer.keep_first if layer.window is not None else 0,
            scale=layer.scale, eps=self.eps, position=position, query_name="q", key_name="k", value_name="v",
            output_name="o")

    def _expert_spec(self, expert: BafusunExpert):
        return ClampedGluSpec(hidden_size=self.width, intermediate_size=expert.ff, limit=expert.limit,
                              gate_name="gate", up_name="up", down_name="down", slope=GATE_SLOPE, shift=UP_SHIFT)

    def _feed_forward_spec(self, f: BafusunFeedForward | None):
        if f is None:
            return None
        return RoutedExpertsSpec(
            hidden_size=self.width, num_experts=f.experts, top=f.top, num_groups=1, groups_kept=1, route_scale=1.0,
            expert=self._expert_spec(f.expert), router_name="router", expert_format="e{index}.",
            norm_eps=ROUTE_NORM_EPS, score="softmax", correction_name="correction", num_identity=f.identity,
            shared=self._expert_spec(f.shared) if f.shared is not None else None, shared_name="shared.")

    def model_spec(self) -> ModelSpec:
        norm = LayerNormSpec(size=self.width, eps=self.eps, bias=False, weight_name="")
        layers = []
        for index, layer in enumerate(self.layers):
            feed_forward = self._feed_forward_spec(layer.feed_forward)
            side = None
            if self.side_dim:
                side = TokenSideInputSpec(
                    hidden_size=self.width, vocab_size=self.vocab, dim=self.side_dim, column=index * self.side_dim,
                    table_width=len(self.layers) * self.side_dim, eps=self.eps, table_name=SIDE_TABLE_NAME,
                    gate_name="gate", proj_name="proj", norm_name="norm")
            layers.append(LayerSpec(
                mixer=self._mixer_spec(layer), feed_forward=feed_forward, mixer_norm=norm,
                ffn_norm=norm if feed_forward is not None else None, mixer_name="mix.", feed_forward_name="mlp.",
                mixer_norm_name="norm1", ffn_norm_name="norm2", block="branch_norm_sequential",
                branch_scale_names=("ls1", "ls2"), side_input=side, side_input_name="side.", part_separator=""))
        return ModelSpec(
            hidden_size=self.width, vocab_size=self.vocab, layers=tuple(layers),
            schedule=sequential_schedule(len(layers)), final_norm=norm, tie_word_embeddings=True,
            max_position_embeddings=self.max_positions, embedding_name="embed", layer_prefix="l",
            final_norm_name="final.norm", head_name="head", embedding_scale=self.embedding_scale,
            logit_scale=self.logit_scale, weight_suffix="", layer_prefix_format="{prefix}{index}.",
            final_norm_prefix="final.norm", extra={"unused_tensors": self.unused_tensors})
