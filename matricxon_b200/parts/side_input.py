"""What a layer adds to the residual stream from the token itself.

``TokenSideInputSpec``: a second embedding table, shared by all layers, holds a short vector per token and
layer. With ``e`` this layer's columns of the token's row, ``g = gelu_tanh(G x) * e``, ``y = P g`` and
``x <- x + y / sqrt(mean(y^2) + eps) * w``: the stream gates what the token brings, and the result joins the
stream at unit root mean square times a learned weight. In narrow layers everything is float arithmetic in one
kernel (``kernels.token_side_input``); in wide ones the two products are matrix products of the runtime dtype with
float results, with a gate kernel between them and the root-mean-square form of the branch norm's kernel after
them. Either way the new rows are also written in the runtime dtype for the next sublayer. Which way a layer
goes depends on its sizes alone, never on the step.

The table is one tensor whatever the number of layers: the parts that name it fetch it once and share it
(``weights.loader`` hands out the same device tensor for the same name).
"""

from __future__ import annotations

import torch

from matricxon_b200.ops import kernels
from matricxon_b200.ops.linear import EPILOGUE_F32, linear
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

    # up to this many entries in each of the two matrices, one kernel does everything on the FP32 cores (every
    # block of four tokens reads both matrices); wider layers run the two products as matrix products
    FUSED_MAX_WEIGHTS = 16384

    def forward(self, x, h, ctx):
        s = self.spec
        act = None
        if self.runtime.dtype != torch.float32:
            act = torch.empty(tuple(x.shape), dtype=self.runtime.dtype, device=x.device)
        if s.dim * s.hidden_size <= self.FUSED_MAX_WEIGHTS:
            kernels.token_side_input(x, ctx.token_ids, self.table, s.column, self.gate, self.proj, self.norm, s.eps,
                                     ctx.status, act)
            return x, (x if act is None else act)
        backend = self.runtime.gemm_backend
        z = linear(h, self.gate, None, EPILOGUE_F32, backend=backend)
        gated = torch.empty((x.shape[0], s.dim), dtype=self.runtime.dtype, device=x.device)
        kernels.gelu_gate_rows(z, ctx.token_ids, self.table, s.column, gated, ctx.status)
        y = linear(gated, self.proj, None, EPILOGUE_F32, backend=backend)
        kernels.layernorm_scaled_add(x, y, self.norm, None, None, s.eps, act, centre=False)
        return x, (x if act is None else act)
