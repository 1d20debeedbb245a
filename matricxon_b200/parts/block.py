"""Arrangements of a mixer, a feed-forward and their norms inside one layer.

``pre_norm_sequential``: ``x = x + mixer(norm1(x)); x = x + ffn(norm2(x))``
(app/architectures/starcoder2_layers.py:67-68); a layer without a feed-forward has only the first sublayer. The residual stream ``x`` is float32
and each sub-layer adds into it in float.

``post_norm_sequential``: ``x = norm1(a x + mixer(x)); x = norm2(a x + ffn(x))``.

``branch_norm_sequential``: ``x = x + s1 * norm1(mixer(x)); x = x + s2 * norm2(ffn(x))`` with learned vectors
``s1``, ``s2`` (optional), then whatever the layer adds from outside the stream (``LayerSpec.side_input``).

``sandwich_norm_sequential``: ``x = x + norm1b(mixer(norm1(x))); x = x + norm2b(ffn(norm2(x)))``: a norm before and
one after each sublayer.
"""

from __future__ import annotations

import torch

from matricxon_b200.ops.linear import PendingSum
from matricxon_b200.parts.base import Block, build_part, register_part


@register_part("block", "pre_norm_sequential")
class PreNormSequentialBlock(Block):
    takes_pending_sum = True

    def __init__(self, spec, runtime, prefix):
        super().__init__(spec, runtime, prefix)
        sep = spec.part_separator
        self.mixer_norm = build_part("norm", spec.mixer_norm, runtime, f"{prefix}{spec.mixer_norm_name}{sep}")
        self.mixer = build_part("mixer", spec.mixer, runtime, f"{prefix}{spec.mixer_name}{sep}")
        # a layer may have only the mixer sublayer
        self.ffn_norm = self.feed_forward = None
        if spec.feed_forward is not None:
            self.ffn_norm = build_part("norm", spec.ffn_norm, runtime, f"{prefix}{spec.ffn_norm_name}{sep}")
            self.feed_forward = build_part("feed_forward", spec.feed_forward, runtime,
                                           f"{prefix}{spec.feed_forward_name}{sep}")
        self.capturable = all(part.capturable for part in self.parts())

    @classmethod
    def weight_specs(cls, spec, prefix):
        from matricxon_b200.parts.base import part_class

        groups = [("norm", spec.mixer_norm, spec.mixer_norm_name), ("mixer", spec.mixer, spec.mixer_name)]
        if spec.feed_forward is not None:
            groups += [("norm", spec.ffn_norm, spec.ffn_norm_name),
                       ("feed_forward", spec.feed_forward, spec.feed_forward_name)]
        out = []
        for category, sub, name in groups:
            out.extend(part_class(category, sub.kind).weight_specs(sub, f"{prefix}{name}{spec.part_separator}"))
        return out

    def parts(self):
        return tuple(part for part in (self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward)
                     if part is not None)

    def load(self, fetch):
        for part in self.parts():
            part.load(fetch)

    @staticmethod
    def _normed(norm, x):
        """(x, norm(x)); ``x`` may arrive as a sum that the part before left to the norm to add up."""
        if isinstance(x, PendingSum):
            if norm.adds_pending_sum:
                return norm.forward_sum(x)
            x = x.tensor()
        return x, norm.forward(x)

    def forward(self, x, ctx, binding):
        """``x`` is the float residual stream or a ``PendingSum`` that stands for it; so is the result when
        the caller has said (``ctx.pending_sum_wanted``) that it takes one, else the result is the stream."""
        # this block knows what to do with a sum that one of its parts leaves pending; the parts only do so
        # on this say-so, which is withdrawn when the block is done
        ctx.sums_may_pend = True
        try:
            x, h = self._normed(self.mixer_norm, x)
            x = self.mixer.forward(h, x, ctx, binding)
            if self.feed_forward is not None:
                x, h = self._normed(self.ffn_norm, x)
                x = self.feed_forward.forward(h, x, ctx)
        finally:
            ctx.sums_may_pend = False
        if isinstance(x, PendingSum) and not getattr(ctx, "pending_sum_wanted", False):
            return x.tensor()
        return x


@register_part("block", "post_norm_sequential")
class PostNormSequentialBlock(Block):
    """Norm after the sum: ``x = norm1(a x + mixer(x)); x = norm2(a x + ffn(x))`` with ``a`` the layer's
    ``skip_scale``; a layer without a feed-forward has only the first sublayer. The sublayers read ``x``
    itself: in the runtime dtype, which the norm that ends a sublayer writes beside the float stream
    (``Norm.forward_scaled_sum``) and which a block hands to the next one through the step's memo; only
    the model's first block has to round the embedding rows itself. On the 32-bit path the stream is
    its own activation."""

    def __init__(self, spec, runtime, prefix):
        super().__init__(spec, runtime, prefix)
        self.mixer = build_part("mixer", spec.mixer, runtime, f"{prefix}{spec.mixer_name}")
        self.mixer_norm = build_part("norm", spec.mixer_norm, runtime, f"{prefix}{spec.mixer_norm_name}")
        self.feed_forward = self.ffn_norm = None
        if spec.feed_forward is not None:
            self.feed_forward = build_part("feed_forward", spec.feed_forward, runtime,
                                           f"{prefix}{spec.feed_forward_name}")
            self.ffn_norm = build_part("norm", spec.ffn_norm, runtime, f"{prefix}{spec.ffn_norm_name}")
        self.capturable = all(part.capturable for part in self.parts())

    @classmethod
    def weight_specs(cls, spec, prefix):
        from matricxon_b200.parts.base import part_class

        groups = [("mixer", spec.mixer, spec.mixer_name), ("norm", spec.mixer_norm, spec.mixer_norm_name)]
        if spec.feed_forward is not None:
            groups += [("feed_forward", spec.feed_forward, spec.feed_forward_name),
                       ("norm", spec.ffn_norm, spec.ffn_norm_name)]
        out = []
        for category, sub, name in groups:
            out.extend(part_class(category, sub.kind).weight_specs(sub, f"{prefix}{name}"))
        return out

    def parts(self):
        return tuple(part for part in (self.mixer, self.mixer_norm, self.feed_forward, self.ffn_norm)
                     if part is not None)

    def load(self, fetch):
        for part in self.parts():
            part.load(fetch)

    def _activations(self, x, ctx):
        """The stream's rows in the runtime dtype: what the block before left, or a rounding pass."""
        if self.runtime.dtype == torch.float32:
            return x
        handed = ctx.memo.get("stream_activations")
        if handed is not None and handed[0] is x:
            return handed[1]
        from matricxon_b200.ops import kernels

        act = torch.empty(tuple(x.shape), dtype=self.runtime.dtype, device=x.device)
        kernels.cast_rows(x, act)
        return act

    def forward(self, x, ctx, binding):
        if isinstance(x, PendingSum):
            x = x.tensor()
        h = self._activations(x, ctx)
        mixed = self.mixer.forward(h, None, ctx, binding)
        x, h = self.mixer_norm.forward_scaled_sum(x, mixed, self.spec.skip_scale)
        if self.feed_forward is not None:
            fed = self.feed_forward.forward(h, None, ctx)
            x, h = self.ffn_norm.forward_scaled_sum(x, fed, self.spec.skip_scale)
        ctx.memo["stream_activations"] = (x, h)
        return x


@register_part("block", "branch_norm_sequential")
class BranchNormSequentialBlock(Block):
    """Norm on the branch only: ``x = x + s1 * norm1(mixer(x)); x = x + s2 * norm2(ffn(x))``. The sublayers read
    ``x`` itself (in the runtime dtype, which the kernel that ends a sublayer writes beside the float stream); only
    a sublayer's own output is normalised, then scaled entry by entry by a learned vector
    (``LayerSpec.branch_scale_names``; None: no scale) and added in float. A layer without a feed-forward has only
    the first sublayer. After the sublayers the layer's ``side_input`` part, if it has one, adds its own term."""

    def __init__(self, spec, runtime, prefix):
        super().__init__(spec, runtime, prefix)
        if not hasattr(part_class_of("norm", spec.mixer_norm), "forward_scaled_add"):
            raise ValueError(f"norm {spec.mixer_norm.kind!r} cannot end a branch (no forward_scaled_add)")
        self.mixer = build_part("mixer", spec.mixer, runtime, f"{prefix}{spec.mixer_name}")
        self.mixer_norm = build_part("norm", spec.mixer_norm, runtime, f"{prefix}{spec.mixer_norm_name}")
        self.feed_forward = self.ffn_norm = None
        if spec.feed_forward is not None:
            self.feed_forward = build_part("feed_forward", spec.feed_forward, runtime,
                                           f"{prefix}{spec.feed_forward_name}")
            self.ffn_norm = build_part("norm", spec.ffn_norm, runtime, f"{prefix}{spec.ffn_norm_name}")
        self.side_input = (build_part("side_input", spec.side_input, runtime, f"{prefix}{spec.side_input_name}")
                           if spec.side_input is not None else None)
        self.mixer_scale = self.ffn_scale = None
        self.capturable = all(part.capturable for part in self.parts())

    @classmethod
    def _scale_names(cls, spec, prefix):
        mixer_scale, ffn_scale = spec.branch_scale_names
        if spec.feed_forward is None:
            ffn_scale = None
        return (prefix + mixer_scale if mixer_scale is not None else None,
                prefix + ffn_scale if ffn_scale is not None else None)

    @classmethod
    def weight_specs(cls, spec, prefix):
        from matricxon_b200.parts.base import part_class
        from matricxon_b200.weights.loader import WeightSpec

        groups = [("mixer", spec.mixer, spec.mixer_name), ("norm", spec.mixer_norm, spec.mixer_norm_name)]
        if spec.feed_forward is not None:
            groups += [("feed_forward", spec.feed_forward, spec.feed_forward_name),
                       ("norm", spec.ffn_norm, spec.ffn_norm_name)]
        if spec.side_input is not None:
            groups.append(("side_input", spec.side_input, spec.side_input_name))
        out = []
        for category, sub, name in groups:
            out.extend(part_class(category, sub.kind).weight_specs(sub, f"{prefix}{name}"))
        width = spec.mixer_norm.size
        for name in cls._scale_names(spec, prefix):
            if name is not None:
                out.append(WeightSpec(name, (width,), role="vector", init="norm_weight"))
        return out

    def parts(self):
        return tuple(part for part in (self.mixer, self.mixer_norm, self.feed_forward, self.ffn_norm, self.side_input)
                     if part is not None)

    def load(self, fetch):
        for part in self.parts():
            part.load(fetch)
        mixer_scale, ffn_scale = self._scale_names(self.spec, self.prefix)
        self.mixer_scale = fetch(mixer_scale) if mixer_scale is not None else None
        self.ffn_scale = fetch(ffn_scale) if ffn_scale is not None else None

    _activations = PostNormSequentialBlock._activations

    def forward(self, x, ctx, binding):
        if isinstance(x, PendingSum):
            x = x.tensor()
        h = self._activations(x, ctx)
        mixed = self.mixer.forward(h, None, ctx, binding)
        x, h = self.mixer_norm.forward_scaled_add(x, mixed, self.mixer_scale)
        if self.feed_forward is not None:
            fed = self.feed_forward.forward(h, None, ctx)
            x, h = self.ffn_norm.forward_scaled_add(x, fed, self.ffn_scale)
        if self.side_input is not None:
            x, h = self.side_input.forward(x, h, ctx)
        ctx.memo["stream_activations"] = (x, h)
        return x


@register_part("block", "sandwich_norm_sequential")
class SandwichNormSequentialBlock(Block):
    """A norm on both sides of each sublayer: ``x = x + out_norm1(mixer(in_norm1(x)))``, then
    ``x = x + out_norm2(ffn(in_norm2(x)))``; a layer without a feed-forward has only the first. The stream is float
    and the sums are formed in float. The kernel that ends a sublayer (``Norm.forward_branch_add``) also forms the
    next norm's output when that norm is known: the second sublayer's inside the block, and the next block's first
    norm when the model names it (``ctx.next_input_norm``; the next block finds the rows in the step's memo under
    ``normed_input``). Where nothing is known to follow, the new rows are left in the runtime dtype under
    ``stream_activations`` for whoever reads the stream itself next."""

    def __init__(self, spec, runtime, prefix):
        super().__init__(spec, runtime, prefix)
        if spec.mixer_out_norm is None or (spec.feed_forward is not None and spec.ffn_out_norm is None):
            raise ValueError("a sandwich block needs a norm behind every sublayer")
        for norm in (spec.mixer_out_norm, spec.ffn_out_norm):
            if norm is not None and not hasattr(part_class_of("norm", norm), "forward_branch_add"):
                raise ValueError(f"norm {norm.kind!r} cannot end a branch (no forward_branch_add)")
        sep = spec.part_separator
        self.mixer_norm = build_part("norm", spec.mixer_norm, runtime, f"{prefix}{spec.mixer_norm_name}{sep}")
        self.mixer = build_part("mixer", spec.mixer, runtime, f"{prefix}{spec.mixer_name}{sep}")
        self.mixer_out_norm = build_part("norm", spec.mixer_out_norm, runtime, f"{prefix}{spec.mixer_out_norm_name}{sep}")
        self.ffn_norm = self.feed_forward = self.ffn_out_norm = None
        if spec.feed_forward is not None:
            self.ffn_norm = build_part("norm", spec.ffn_norm, runtime, f"{prefix}{spec.ffn_norm_name}{sep}")
            self.feed_forward = build_part("feed_forward", spec.feed_forward, runtime,
                                           f"{prefix}{spec.feed_forward_name}{sep}")
            self.ffn_out_norm = build_part("norm", spec.ffn_out_norm, runtime, f"{prefix}{spec.ffn_out_norm_name}{sep}")
        self.capturable = all(part.capturable for part in self.parts())

    @property
    def input_norm(self):
        """The norm this block applies to the stream first (a block before it may apply it on its way out)."""
        return self.mixer_norm

    @classmethod
    def weight_specs(cls, spec, prefix):
        from matricxon_b200.parts.base import part_class

        groups = [("norm", spec.mixer_norm, spec.mixer_norm_name), ("mixer", spec.mixer, spec.mixer_name),
                  ("norm", spec.mixer_out_norm, spec.mixer_out_norm_name)]
        if spec.feed_forward is not None:
            groups += [("norm", spec.ffn_norm, spec.ffn_norm_name),
                       ("feed_forward", spec.feed_forward, spec.feed_forward_name),
                       ("norm", spec.ffn_out_norm, spec.ffn_out_norm_name)]
        out = []
        for category, sub, name in groups:
            out.extend(part_class(category, sub.kind).weight_specs(sub, f"{prefix}{name}{spec.part_separator}"))
        return out

    def parts(self):
        return tuple(part for part in (self.mixer_norm, self.mixer, self.mixer_out_norm, self.ffn_norm,
                                       self.feed_forward, self.ffn_out_norm) if part is not None)

    def load(self, fetch):
        for part in self.parts():
            part.load(fetch)

    def forward(self, x, ctx, binding):
        if isinstance(x, PendingSum):
            x = x.tensor()
        handed = ctx.memo.pop("normed_input", None)
        if handed is not None and handed[0] is x and handed[1] is self.mixer_norm:
            h = handed[2]                           # the block before applied this block's first norm on its way out
        else:
            h = self.mixer_norm.forward(x)
        follower = getattr(ctx, "next_input_norm", None)
        mixed = self.mixer.forward(h, None, ctx, binding)
        last = self.mixer_out_norm
        if self.feed_forward is not None:
            x, h = self.mixer_out_norm.forward_branch_add(x, mixed, next_norm=self.ffn_norm)
            mixed = self.feed_forward.forward(h, None, ctx)
            last = self.ffn_out_norm
        if follower is not None:
            x, h = last.forward_branch_add(x, mixed, next_norm=follower)
            ctx.memo["normed_input"] = (x, follower, h)
        else:
            x, h = last.forward_branch_add(x, mixed, want_activations=True)
            ctx.memo["stream_activations"] = (x, h)
        return x


def part_class_of(category, spec):
    from matricxon_b200.parts.base import part_class

    return part_class(category, spec.kind)
