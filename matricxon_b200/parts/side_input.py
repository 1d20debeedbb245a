"""What a layer adds to the residual stream from the token itself.

``TokenSideInputSpec``: a second embedding table, shared by all layers, holds a short vector per token and
layer. With ``e`` this layer's columns of the token's row, ``g = gelu_tanh(G x) * e``, ``y = P g`` and
``x <- x + y / sqrt(mean(y^2) + eps) * w``: the stream gates what the token brings, and the result joins the
stream at unit root mean square times a learned weight. Everything is float arithmetic in one kernel
(``kernels.token_side_input``), which also writes the new rows in the runtime dtype for the next sublayer.

The table is one tensor whatever the number of layers: the parts that name it fetch it once and share it
(``weights.loader`` hands out the same device tensor for the same name).
"""

from __future__ import annotations

import torch

from matricxon_b200.ops import kernels
from matricxon_b200.parts.base import SideInput, register_part
from matricxon_b200.weights.loader import WeightSpec


@register_part("side_input", "token_side_input")
class TokenSideInput(SideInput):
    capturable = True

    @classmethod
    def weight_specs(cls, spec, prefix):
        return [WeightSpec(spec.table_name, (spec.vocab_size, spec.table_width), role="matrix", init="weight"),
                WeightSpec(prefix + spec.gate_name, (spec.dim, spec.hidden_size), role="matrix", init="weight"),
                WeightSpec(prefix + spec.proj_name, (spec.hidden_size, spec.dim), role="matrix", init="weight"),
                WeightSpec(prefix + spec.norm_name, (spec.hidden_size,), role="vector", init="norm_weight")]

    def load(self, fetch):
        s = self.spec
        self.table = fetch(s.table_name)
        self.gate = fetch(self.prefix + s.gate_name)
        self.proj = fetch(self.prefix + s.proj_name)
        self.norm = fetch(self.prefix + s.norm_name)

    def forward(self, x, ctx):
        s = self.spec
        act = None
        if self.runtime.dtype != torch.float32:
            act = torch.empty(tuple(x.shape), dtype=self.runtime.dtype, device=x.device)
        kernels.token_side_input(x, ctx.token_ids, self.table, s.column, self.gate, self.proj, self.norm, s.eps,
                                 ctx.status, act)
        return x, (x if act is None else act)
