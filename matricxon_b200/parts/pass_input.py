"""What a model does to the stream before every pass of a repeated run of layers.

``ReinjectionSpec``: with x0 the embedding output of the step's tokens and t the number of the pass,
``x <- M [x; x0] + s_t``. M is split by columns at load, ``M = [A | B]``: ``B x0`` is the same for every pass and is
formed once per step, right after the embedding lookup (``begin``), so the stream's buffer may be overwritten by the
layers before the run; a pass then costs one product, ``A x`` with ``s_t`` as its bias and ``B x0`` as the sum's
other term, in float.
"""

from __future__ import annotations

import torch

from matricxon_b200.ops import kernels
from matricxon_b200.ops.linear import EPILOGUE_F32, EPILOGUE_RESIDUAL, linear
from matricxon_b200.parts.base import Part, register_part
from matricxon_b200.weights.loader import WeightSpec


class PassInput(Part):
    """``begin(x0, ctx)`` sees the embedding output before any layer runs; ``forward(x, pass_index, ctx) -> x`` runs
    before the schedule entry that opens a pass (the result may be a new buffer)."""

    def begin(self, x0, ctx):
        return None

    def forward(self, x, pass_index, ctx):
        raise NotImplementedError


@register_part("pass_input", "reinjection")
class Reinjection(PassInput):
    capturable = True

    @classmethod
    def weight_specs(cls, spec, prefix):
        return [WeightSpec(prefix + spec.matrix_name, (spec.hidden_size, 2 * spec.hidden_size), role="matrix",
                           init="weight"),
                WeightSpec(prefix + spec.step_name, (spec.passes, spec.hidden_size), role="vector", init="bias")]

    def load(self, fetch):
        s = self.spec
        matrix = fetch(self.prefix + s.matrix_name)
        self.stream_weight = matrix[:, :s.hidden_size].contiguous()
        self.embedding_weight = matrix[:, s.hidden_size:].contiguous()
        self.steps = fetch(self.prefix + s.step_name)

    def _activations(self, x, ctx):
        if self.runtime.dtype == torch.float32:
            return x
        handed = ctx.memo.get("stream_activations")
        if handed is not None and handed[0] is x:
            return handed[1]
        act = torch.empty(tuple(x.shape), dtype=self.runtime.dtype, device=x.device)
        kernels.cast_rows(x, act)
        return act

    def begin(self, x0, ctx):
        act = self._activations(x0, ctx)
        ctx.memo["stream_activations"] = (x0, act)       # the first layer may read the same rows
        ctx.memo["reinjection_base"] = linear(act, self.embedding_weight, None, EPILOGUE_F32,
                                              backend=self.runtime.gemm_backend)

    def forward(self, x, pass_index, ctx):
        if not 0 <= pass_index < self.spec.passes:
            raise ValueError(f"pass {pass_index} of a run of {self.spec.passes}")
        base = ctx.memo.get("reinjection_base")
        if base is None:
            raise RuntimeError("a pass opens, but the step's embedding output was never seen")
        out = torch.empty_like(base)
        return linear(self._activations(x, ctx), self.stream_weight, self.steps[pass_index], EPILOGUE_RESIDUAL,
                      residual=base, out=out, backend=self.runtime.gemm_backend)
