"""Kefasun configuration: a decoder with a norm on both sides of every sublayer, three kinds of attention, routed
experts, and a run of layers that is repeated with the embedding fed in again before every pass.

``config.json`` holds ``architecture: "Kefasun"``, ``vocab``, ``width``, ``norm.eps``, ``logit_scale``, ``loop``
(``start``, ``stop``, ``times``; absent: every layer runs once) and a list ``layers``; every entry gives ``type``,
the mixer's sizes under ``mixer`` and its feed-forward under ``mlp`` (``kind: dense`` with ``ff``; ``kind: moe`` with
``expert.ff`` and ``router.experts`` / ``router.top``; null for a layer that has only the mixer sublayer).

Layer types (all without biases, all with a sigmoid gate that reads the mixer's input):

* ``attention``: grouped queries (``heads``, ``kv_heads``, ``dim``, ``vdim``), q and k RMS-normalised per head with a
  weight, then rotated over their first ``rot.dims`` entries with neighbouring entries paired; a query sees the keys
  of its own block of ``mask.size`` positions; the softmax's denominator has one added; one gate per head.
* ``latent_attention``: queries through a latent of ``q_rank`` entries, keys and values expanded from a cached
  latent of ``kv_rank`` entries plus one rotated key part of ``rot_dim`` entries shared by the heads (neighbouring
  entries paired); a window of ``mask.size`` positions; a learned sink logit per head; a gate per entry.
* ``attention_2``: as ``attention`` but rotated with entry i paired with entry i + dims/2, scores capped at
  ``softcap``, every earlier key in sight, an ordinary softmax, a gate per entry.

A layer computes ``x += norm1b(mixer(norm1(x)))``, ``x += norm2b(ff(norm2(x)))``. Layers ``start .. stop-1`` run
``times`` times in a row (same weights, a cache per pass); before the first layer of pass t the stream becomes
``loop.in [x; x0] + loop.step[t]`` with x0 the embedding output. The logits come from the embedding table itself
times ``logit_scale``.

Tensor names: ``embed``, ``loop.in``, ``loop.step``, ``l<i>.norm1|norm1b|norm2|norm2b``,
``l<i>.mix.{q,k,v,q.norm,k.norm,g,o}``, ``l<i>.mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,sink,g,o}``,
``l<i>.mlp.{gate,up,down}``, ``l<i>.mlp.e<j>.{gate,up,down}``, ``l<i>.mlp.router``, ``l<i>.mlp.router.b``,
``final.norm`` (no ``.weight`` suffix). This file is the only place that knows those names and keys; the parts are
generic.
"""

from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Any

from matricxon_b200.config.base import ConfigError, ConfigReader
from matricxon_b200.parts.spec import (
    GatedMlpSpec,
    LatentAttentionSpec,
    LayerSpec,
    ModelSpec,
    NormedRotaryAttentionSpec,
    PairedRotarySpec,
    ReinjectionSpec,
    RmsNormSpec,
    RoutedExpertsSpec,
    ScheduleEntry,
)

# what the design fixes
ACTIVATION = "silu"                  # dense feed-forward and experts: down(silu(gate h) * up h)
LAYER_TYPES = ("attention", "latent_attention", "attention_2")
LOOP_MATRIX_NAME = "loop.in"
LOOP_STEP_NAME = "loop.step"
# no key of config.json limits a sequence's length; this sizes the block tables of captured steps
# (longer sequences run uncaptured)
DEFAULT_MAX_POSITIONS = 32768


def _object(raw: Any, key: str, where: str) -> dict:
    value = raw.get(key) if isinstance(raw, dict) else None
    if not isinstance(value, dict):
        raise ConfigError(f"{where}: {key!r} must be an object")
    return value


@dataclass(frozen=True)
class KefasunFeedForward:
    kind: str                     # "dense" | "moe"
    ff: int                       # width of the dense feed-forward or of one expert
    experts: int = 0
    top: int = 0

    @classmethod
    def from_dict(cls, raw: Any, where: str) -> "KefasunFeedForward":
        r = ConfigReader(raw, where)
        kind = r.string("kind")
        if kind == "dense":
            return cls(kind=kind, ff=r.integer("ff", minimum=1))
        if kind != "moe":
            raise ConfigError(f"{where}: unknown feed-forward kind {kind!r}; Kefasun has 'dense' and 'moe'")
        router = ConfigReader(_object(raw, "router", where), where + ".router")
        experts, top = router.integer("experts", minimum=1), router.integer("top", minimum=1)
        if top > experts:
            raise ConfigError(f"{where}.router: 'top' ({top}) exceeds the {experts} experts")
        ff = ConfigReader(_object(raw, "expert", where), where + ".expert").integer("ff", minimum=1)
        return cls(kind=kind, ff=ff, experts=experts, top=top)

    def to_dict(self) -> dict:
        if self.kind == "dense":
            return {"ff": self.ff, "kind": "dense"}
        return {"expert": {"ff": self.ff}, "kind": "moe", "router": {"experts": self.experts, "top": self.top}}


@dataclass(frozen=True)
class KefasunLayer:
    type: str
    heads: int
    dim: int
    vdim: int
    scale: float
    rot_dims: int
    rot_base: float
    kv_heads: int = 0             # the two grouped kinds
    mask_size: int = 0            # block (attention) or window (latent_attention); 0: attention_2 has no mask
    softcap: float | None = None  # attention_2
    q_rank: int = 0               # latent_attention (0 while config.json leaves it to the tensors)
    kv_rank: int = 0
    rot_dim: int = 0
    feed_forward: KefasunFeedForward | None = None

    @classmethod
    def from_dict(cls, raw: Any, where: str) -> "KefasunLayer":
        r = ConfigReader(raw, where)
        kind = r.string("type")
        if kind not in LAYER_TYPES:
            raise ConfigError(f"{where}: unknown layer type {kind!r}; Kefasun has {list(LAYER_TYPES)}")
        mixer = _object(raw, "mixer", where)
        m = ConfigReader(mixer, where + ".mixer")
        heads, dim = m.integer("heads", minimum=1), m.integer("dim", minimum=1)
        fields: dict[str, Any] = {"type": kind, "heads": heads, "dim": dim, "vdim": m.integer("vdim", dim, minimum=1),
                                  "scale": m.number("scale", positive=True)}
        fields["rot_dims"], fields["rot_base"] = 0, 10000.0             # no 'rot': nothing is rotated
        if mixer.get("rot") is not None:
            rot = ConfigReader(_object(mixer, "rot", where + ".mixer"), where + ".mixer.rot")
            fields["rot_dims"], fields["rot_base"] = rot.integer("dims", minimum=0), rot.number("base", positive=True)
        if fields["rot_dims"] % 2:
            raise ConfigError(f"{where}.mixer.rot: 'dims' must be even, got {fields['rot_dims']}")
        if kind == "latent_attention":
            fields["rot_dim"] = m.integer("rot_dim", minimum=0)
            fields["q_rank"], fields["kv_rank"] = m.integer("q_rank", 0, minimum=0), m.integer("kv_rank", 0, minimum=0)
            if fields["rot_dims"] > fields["rot_dim"]:
                raise ConfigError(f"{where}.mixer.rot: 'dims' ({fields['rot_dims']}) exceeds rot_dim ({fields['rot_dim']})")
        else:
            kv_heads = m.integer("kv_heads", heads, minimum=1)
            if heads % kv_heads:
                raise ConfigError(f"{where}.mixer: heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
            if fields["rot_dims"] > dim:
                raise ConfigError(f"{where}.mixer.rot: 'dims' ({fields['rot_dims']}) exceeds dim ({dim})")
            if max(dim, fields["vdim"]) > 256:
                raise ConfigError(f"{where}.mixer: head sizes above 256 have no attention kernel")
            fields["kv_heads"] = kv_heads
        if kind != "attention_2" and mixer.get("mask") is not None:    # no 'mask': every earlier key is seen
            mask = ConfigReader(_object(mixer, "mask", where + ".mixer"), where + ".mixer.mask")
            fields["mask_size"] = mask.integer("size", minimum=1)
        if kind == "attention_2":
            fields["softcap"] = m.number("softcap", positive=True)
        if raw.get("mlp") is not None:
            fields["feed_forward"] = KefasunFeedForward.from_dict(raw["mlp"], where + ".mlp")
        return cls(**fields)

    def to_dict(self) -> dict:
        mixer: dict[str, Any] = {"dim": self.dim, "heads": self.heads, "scale": self.scale, "vdim": self.vdim}
        if self.rot_dims:
            mixer["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
        if self.type == "latent_attention":
            mixer.update({"kv_rank": self.kv_rank, "q_rank": self.q_rank, "rot_dim": self.rot_dim})
        else:
            mixer["kv_heads"] = self.kv_heads
        if self.type == "attention_2":
            mixer["softcap"] = self.softcap
        elif self.mask_size:
            mixer["mask"] = {"size": self.mask_size}
        return {"mixer": mixer, "mlp": self.feed_forward.to_dict() if self.feed_forward else None, "type": self.type}


@dataclass(frozen=True)
class KefasunLoop:
    start: int
    stop: int
    times: int

    def to_dict(self) -> dict:
        return {"start": self.start, "stop": self.stop, "times": self.times}


@dataclass(frozen=True)
class KefasunConfig:
    vocab: int
    width: int
    eps: float
    logit_scale: float
    layers: tuple[KefasunLayer, ...]
    loop: KefasunLoop | None = None
    max_positions: int = DEFAULT_MAX_POSITIONS
    # tensors a model folder holds although the model does not use them (the second pair of norms of a layer
    # without a feed-forward, the loop's tensors of a model that repeats nothing): (name, shape), found by
    # ``with_tensor_shapes``; expected at the weight check and never fetched
    unused_tensors: tuple[tuple[str, tuple[int, ...]], ...] = ()

    architecture = "Kefasun"
    model_type = "kefasun"

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @classmethod
    def from_dict(cls, raw: dict[str, Any], where: str = "config.json") -> "KefasunConfig":
        r = ConfigReader(raw, where)
        eps = ConfigReader(_object(raw, "norm", where), where + ".norm").number("eps", positive=True)
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError(f"{where}: 'layers' must be a non-empty list")
        parsed = tuple(KefasunLayer.from_dict(layer, f"{where}.layers[{i}]") for i, layer in enumerate(layers))
        loop = None
        if raw.get("loop") is not None:
            lr = ConfigReader(_object(raw, "loop", where), where + ".loop")
            start, stop = lr.integer("start", minimum=0), lr.integer("stop", minimum=0)
            times = lr.integer("times", minimum=1)
            if not start <= stop <= len(parsed):
                raise ConfigError(f"{where}.loop: layers {start} .. {stop} - 1 do not lie within the {len(parsed)} layers")
            loop = KefasunLoop(start=start, stop=stop, times=times)
        return cls(vocab=r.integer("vocab", minimum=1), width=r.integer("width", minimum=1), eps=eps,
                   logit_scale=r.number("logit_scale", 1.0), layers=parsed, loop=loop,
                   max_positions=r.integer("max_positions", DEFAULT_MAX_POSITIONS, minimum=1))

    @property
    def repeats(self) -> bool:
        return self.loop is not None and self.loop.stop > self.loop.start

    def with_tensor_shapes(self, shape_of) -> "KefasunConfig":
        """The configuration completed from the tensors: ``shape_of(name)`` gives a tensor's shape or None. Latent
        ranks that ``config.json`` leaves out are the row counts of the down projections; norms of a sublayer that
        a layer does not have, and the loop's tensors of a model that repeats nothing, are noted as held unused."""
        unused, layers = [], []
        for index, layer in enumerate(self.layers):
            if layer.type == "latent_attention" and not (layer.q_rank and layer.kv_rank):
                dq, dkv = shape_of(f"l{index}.mix.dq"), shape_of(f"l{index}.mix.dkv")
                if dq is None or dkv is None:
                    raise ConfigError(f"config.json.layers[{index}].mixer: q_rank / kv_rank are given neither by "
                                      "config.json nor by the tensors")
                layer = replace(layer, q_rank=layer.q_rank or int(dq[0]),
                                kv_rank=layer.kv_rank or int(dkv[0]) - layer.rot_dim)
            layers.append(layer)
            if layer.feed_forward is None:
                for name in (f"l{index}.norm2", f"l{index}.norm2b"):
                    shape = shape_of(name)
                    if shape is not None:
                        unused.append((name, tuple(int(extent) for extent in shape)))
        if not self.repeats:
            for name in (LOOP_MATRIX_NAME, LOOP_STEP_NAME):
                shape = shape_of(name)
                if shape is not None:
                    unused.append((name, tuple(int(extent) for extent in shape)))
        return replace(self, layers=tuple(layers), unused_tensors=tuple(unused))

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"architecture": self.architecture, "layers": [layer.to_dict() for layer in self.layers],
                               "logit_scale": self.logit_scale, "norm": {"eps": self.eps}, "vocab": self.vocab,
                               "width": self.width}
        if self.loop is not None:
            out["loop"] = self.loop.to_dict()
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        return out

    # ------------------------------------------------------------------ description
    def _mixer_spec(self, layer: KefasunLayer, where: str):
        if layer.type == "latent_attention":
            if not (layer.q_rank and layer.kv_rank):
                raise ConfigError(f"{where}.mixer: 'q_rank' and 'kv_rank' are needed (config.json or the tensors give them)")
            return LatentAttentionSpec(
                hidden_size=self.width, num_heads=layer.heads, head_dim=layer.dim, rot_dim=layer.rot_dim,
                value_dim=layer.vdim, latent_rank=layer.kv_rank, window=layer.mask_size or None, scale=layer.scale,
                eps=self.eps, position=PairedRotarySpec(rotary_dim=layer.rot_dims, theta=layer.rot_base,
                                                        pairing="interleaved"),
                query_name="uq", down_name="dkv", latent_norm_name="dkv.norm", key_up_name="uk", value_up_name="uv",
                output_name="o", query_rank=layer.q_rank, query_down_name="dq", query_norm_name="dq.norm",
                sink_name="sink", gate_name="g")
        first = layer.type == "attention"
        blocks = first and layer.mask_size > 0
        position = None
        if layer.rot_dims > 0:
            position = PairedRotarySpec(rotary_dim=layer.rot_dims, theta=layer.rot_base,
                                        pairing="interleaved" if first else "half")
        return NormedRotaryAttentionSpec(
            hidden_size=self.width, num_heads=layer.heads, num_kv_heads=layer.kv_heads, head_dim=layer.dim,
            value_dim=layer.vdim, scale=layer.scale, eps=self.eps, position=position, query_name="q", key_name="k",
            value_name="v", output_name="o", mask="chunk" if blocks else "causal",
            mask_size=layer.mask_size if blocks else 0, softcap=None if first else layer.softcap,
            sink="zero" if first else None, gate="head" if first else "entry", gate_name="g",
            query_norm_name="q.norm", key_norm_name="k.norm")

    def _feed_forward_spec(self, f: KefasunFeedForward | None):
        if f is None:
            return None
        gated = GatedMlpSpec(hidden_size=self.width, intermediate_size=f.ff, activation=ACTIVATION, gate_name="gate",
                             up_name="up", down_name="down")
        if f.kind == "dense":
            return gated
        # the `top` largest logits (bias included), weighted by the softmax over the chosen logits alone: the
        # softmax rule with a bias on the logits and no correction
        return RoutedExpertsSpec(
            hidden_size=self.width, num_experts=f.experts, top=f.top, num_groups=1, groups_kept=1, route_scale=1.0,
            expert=gated, router_name="router", expert_format="e{index}.", score="softmax", bias_name="router.b")

    def schedule(self) -> tuple[ScheduleEntry, ...]:
        n = len(self.layers)
        if not self.repeats:
            return tuple(ScheduleEntry(layer=i) for i in range(n))
        start, stop, times = self.loop.start, self.loop.stop, self.loop.times
        entries = [ScheduleEntry(layer=i) for i in range(start)]
        for t in range(times):
            entries += [ScheduleEntry(layer=i, pass_index=t if i == start else None) for i in range(start, stop)]
        return tuple(entries + [ScheduleEntry(layer=i) for i in range(stop, n)])

    def model_spec(self) -> ModelSpec:
        norm = RmsNormSpec(size=self.width, eps=self.eps, weight_name="")
        layers = []
        for index, layer in enumerate(self.layers):
            feed_forward = self._feed_forward_spec(layer.feed_forward)
            layers.append(LayerSpec(
                mixer=self._mixer_spec(layer, f"config.json.layers[{index}]"), feed_forward=feed_forward,
                mixer_norm=norm, ffn_norm=norm if feed_forward is not None else None, mixer_name="mix.",
                feed_forward_name="mlp.", mixer_norm_name="norm1", ffn_norm_name="norm2",
                block="sandwich_norm_sequential", part_separator="", mixer_out_norm=norm,
                ffn_out_norm=norm if feed_forward is not None else None, mixer_out_norm_name="norm1b",
                ffn_out_norm_name="norm2b"))
        pass_input = None
        if self.repeats:
            pass_input = ReinjectionSpec(hidden_size=self.width, passes=self.loop.times, matrix_name=LOOP_MATRIX_NAME,
                                         step_name=LOOP_STEP_NAME)
        return ModelSpec(
            hidden_size=self.width, vocab_size=self.vocab, layers=tuple(layers), schedule=self.schedule(),
            final_norm=norm, tie_word_embeddings=True, max_position_embeddings=self.max_positions,
            embedding_name="embed", layer_prefix="l", final_norm_name="final.norm", head_name="head",
            logit_scale=self.logit_scale, pass_input=pass_input, weight_suffix="", layer_prefix_format="{prefix}{index}.",
            final_norm_prefix="final.norm", extra={"unused_tensors": self.unused_tensors})
