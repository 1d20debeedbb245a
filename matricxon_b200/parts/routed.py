"""A routed feed-forward: every token runs a few of many small gated feed-forwards.

``RoutedExpertsSpec``: scores ``sigmoid(R h)`` in float, the experts in equal runs of neighbours, a run worth its
two best scores, the best runs' experts eligible, the ``top`` best of them chosen; the output is
``sum_e w_e down_e(act(gate_e h) * up_e h)`` with ``w = score / (sum of chosen scores + 1e-20) * route_scale``.

The step never leaves the device and is stream-ordered: one kernel routes and counts every expert's (token, slot)
pairs, two sort the pairs by expert and list the row tiles, two grouped products walk those tiles, and one kernel
adds a token's weighted pairs to the residual stream in slot order, so that a token's result depends on nothing else
in the batch. In bfloat16 the grouped products are the engine's tcgen05 product with a tile list (rows copied into
sorted order first, the gated activation a kernel of its own, as in the dense feed-forward); in float32, and for sizes
that TMA does not take, they run on the FP32 cores (the first gathers rows itself and applies the activation, the
second weighs every pair's row). The experts' matrices are stacked at load: ``[experts, 2 ff, hidden]`` (gate rows, then up rows) and
``[experts, hidden, ff]``. The router's matrix is held in float.

``score="softmax"`` routes by another rule (softmax over all router rows, a correction that moves the choice and not
the weights; optionally a bias on the logits themselves, which makes the rule "the largest logits, weighted by the
softmax over the chosen ones") and may name experts without matrices that return their input: such a pair takes no row of the grouped
products, and the combining kernel adds ``weight * h`` for it. An expert may be a ``GatedMlpSpec`` or a
``ClampedGluSpec`` (the activation differs). A ``shared`` feed-forward runs for every token; the routed sum is added
onto its output.
"""

from __future__ import annotations

import torch

from matricxon_b200.ops import kernels
from matricxon_b200.parts.base import FeedForward, build_part, part_class, register_part
from matricxon_b200.weights.loader import WeightSpec


@register_part("feed_forward", "routed_experts")
class RoutedExperts(FeedForward):
    capturable = True

    def __init__(self, spec, runtime, prefix):
        super().__init__(spec, runtime, prefix)
        e = spec.expert
        if e.kind == "clamped_glu":
            # (limit, slope, shift) of ``min(g, limit) * sigmoid(slope g) * (clamp(u) + shift)``; limit 0: unclamped
            self.clamped = (float(e.limit) if e.limit is not None else 0.0, float(e.slope), float(e.shift))
        else:
            self.clamped = None
            if e.activation not in kernels.GLU_ACTIVATIONS:
                raise ValueError(f"expert activation {e.activation!r} has no kernel")
        self.shared = (build_part("feed_forward", spec.shared, runtime, prefix + spec.shared_name)
                       if spec.shared is not None else None)
        if self.shared is not None:
            self.capturable = bool(self.shared.capturable)

    @classmethod
    def weight_specs(cls, spec, prefix):
        e = spec.expert
        wide, narrow = (e.intermediate_size, spec.hidden_size), (spec.hidden_size, e.intermediate_size)
        specs = []
        for index in range(spec.num_experts):
            q = prefix + spec.expert_format.format(index=index)
            specs += [WeightSpec(q + e.gate_name, wide, role="matrix", init="weight"),
                      WeightSpec(q + e.up_name, wide, role="matrix", init="weight"),
                      WeightSpec(q + e.down_name, narrow, role="matrix", init="weight")]
        # router logits are float: the matrix is held like a vector
        rows = spec.num_experts + spec.num_identity
        specs.append(WeightSpec(prefix + spec.router_name, (rows, spec.hidden_size), role="vector", init="weight"))
        if spec.correction_name is not None:
            specs.append(WeightSpec(prefix + spec.correction_name, (rows,), role="vector", init="bias"))
        if spec.bias_name is not None:
            specs.append(WeightSpec(prefix + spec.bias_name, (rows,), role="vector", init="bias"))
        if spec.shared is not None:
            specs += part_class("feed_forward", spec.shared.kind).weight_specs(spec.shared, prefix + spec.shared_name)
        return specs

    def load(self, fetch):
        s, e = self.spec, self.spec.expert
        names = [self.prefix + s.expert_format.format(index=index) for index in range(s.num_experts)]
        self.gate_up = torch.stack([torch.cat([fetch(q + e.gate_name), fetch(q + e.up_name)]) for q in names])
        self.down = torch.stack([fetch(q + e.down_name) for q in names])
        self.router = fetch(self.prefix + s.router_name)
        self.correction = fetch(self.prefix + s.correction_name) if s.correction_name is not None else None
        self.bias = fetch(self.prefix + s.bias_name) if s.bias_name is not None else None
        if self.shared is not None:
            self.shared.load(fetch)

    def forward(self, h, residual, ctx):
        s, e = self.spec, self.spec.expert
        n, device = h.shape[0], h.device
        n_pairs = n * s.top
        # bfloat16 with TMA-friendly sizes: the grouped products run on tcgen05 over rows copied into sorted order
        on_tc = (self.runtime.gemm_backend == "auto" and kernels.grouped_tcgen05_supported(h, self.gate_up)
                 and e.intermediate_size % 8 == 0 and s.hidden_size % 4 == 0)
        tile_rows = kernels.GROUPED_TILE_ROWS if on_tc else kernels.moe_tile_rows()
        max_tiles = kernels.moe_max_tiles(n_pairs, s.num_experts, tile_rows)
        # one int32 block for everything the routing leaves on the device
        sizes = [s.num_experts, n_pairs, n_pairs, n_pairs, s.num_experts + 1, 3 * max_tiles, 1]
        ints = torch.empty(sum(sizes), dtype=torch.int32, device=device)
        counts, ids, place, order, first, tile_map, n_tiles = torch.split(ints, sizes)
        if s.num_identity:
            ints.zero_()        # pairs of experts without matrices take no sorted row: the rows behind the last one read token 0
        else:
            counts.zero_()
        weights = torch.empty(n_pairs, dtype=torch.float32, device=device)
        if s.score == "softmax":
            kernels.moe_route_softmax(h, self.router, s.top, s.num_identity, self.correction, ids, weights, counts, place,
                                      bias=self.bias)
        else:
            kernels.moe_route(h, self.router, s.top, s.num_groups, s.groups_kept, s.route_scale, ids, weights, counts,
                              place)
        choices = ctx.memo.get("expert_choices") if hasattr(ctx, "memo") else None
        if choices is not None:            # a caller listens (``StepRunner.taps``)
            choices.append(ids.view(n, s.top).clone())
        kernels.moe_plan(counts, ids, place, first, tile_map, n_tiles, order, tile_rows)
        if self.shared is not None:
            # the shared feed-forward's float output is the sum's first term (added to the stream if there is one)
            residual = self.shared.forward(h, residual, ctx)
            if not isinstance(residual, torch.Tensor):
                residual = residual.tensor()
        elif residual is None:
            residual = torch.zeros((n, s.hidden_size), dtype=torch.float32, device=device)
        identity = (h, s.num_experts) if s.num_identity else None
        if on_tc:
            status = getattr(ctx, "status", None)
            rows = torch.empty((n_pairs, s.hidden_size), dtype=h.dtype, device=device)
            kernels.moe_gather(h, order, s.top, rows)
            gate_up = torch.empty((n_pairs, 2 * e.intermediate_size), dtype=h.dtype, device=device)
            kernels.gemm_tcgen05_grouped(rows, self.gate_up, tile_map, n_tiles, max_tiles, gate_up, status)
            mid = torch.empty((n_pairs, e.intermediate_size), dtype=h.dtype, device=device)
            if self.clamped is not None:
                kernels.clamped_glu(gate_up, mid, *self.clamped)
            else:
                kernels.glu(gate_up, mid, e.activation)
            down = torch.empty((n_pairs, s.hidden_size), dtype=torch.float32, device=device)
            kernels.gemm_tcgen05_grouped(mid, self.down, tile_map, n_tiles, max_tiles, down, status)
            kernels.moe_combine_sorted(down, ids, place, first, weights, residual, s.top, identity=identity)
            return residual
        mid = torch.empty((n_pairs, e.intermediate_size), dtype=h.dtype, device=device)
        activation = ("clamped", *self.clamped) if self.clamped is not None else e.activation
        kernels.moe_gemm(h, order, s.top, self.gate_up, tile_map, n_tiles, max_tiles, mid, None, activation)
        pairs = torch.empty((n_pairs, s.hidden_size), dtype=torch.float32, device=device)
        kernels.moe_gemm(mid, order, 1, self.down, tile_map, n_tiles, max_tiles, pairs, weights, None)
        kernels.moe_combine(pairs, residual, s.top,
                            identity=(ids, weights, h, s.num_experts) if s.num_identity else None)
        return residual
