"""LayerNorm with float statistics.

``(x - mean) / sqrt(var + eps) * weight + bias`` with the biased variance, as
nn.LayerNorm computes it in the reference (app/architectures/starcoder2_layers.py:45,56;
app/architectures/starcoder2.py:97). The input is the float32 residual stream; mean,
variance and the affine step stay float, and the result is rounded once to the runtime dtype.
"""

from __future__ import annotations

import torch

from matricxon_b200.ops import kernels
from matricxon_b200.parts.base import Norm, register_part
from matricxon_b200.weights.loader import WeightSpec


@register_part("norm", "layernorm")
class LayerNorm(Norm):
    capturable = True
    adds_pending_sum = True

    @classmethod
    def weight_specs(cls, spec, prefix):
        specs = [WeightSpec(prefix + spec.weight_name, (spec.size,), role="vector", init="norm_weight")]
        if spec.bias:
            specs.append(WeightSpec(prefix + spec.bias_name, (spec.size,), role="vector", init="norm_bias"))
        return specs

    def load(self, fetch):
        self.weight = fetch(self.prefix + self.spec.weight_name)
        self.bias = fetch(self.prefix + self.spec.bias_name) if self.spec.bias else None

    def forward(self, x, out=None, rows=None):
        n_rows = x.shape[0] if rows is None else rows.numel()
        if out is None:
            out = torch.empty((n_rows, self.spec.size), dtype=self.runtime.dtype, device=x.device)
        kernels.layernorm(x, self.weight, self.bias, self.spec.eps, out, rows)
        return out

    def forward_sum(self, pending):
        """The norm of a residual sum that has not been added up yet (``ops.linear.PendingSum``): one
        kernel forms the sum, writes it to the residual stream and normalises it. Returns (x, norm(x))."""
        x = pending.added_by_kernel()
        out = torch.empty(tuple(x.shape), dtype=self.runtime.dtype, device=x.device)
        kernels.layernorm_sum(x, pending.acc, pending.bias, self.weight, self.bias, self.spec.eps, out)
        return x, out


    def forward_scaled_add(self, x, branch, scale=None):
        """``x <- x + norm(branch) * scale`` in place (both float32; ``scale`` a float32 vector or None): the
        end of a sublayer whose own output is normalised. Returns (x, activations): the new rows in the runtime
        dtype, which is ``x`` itself on the 32-bit path."""
        if self.runtime.dtype == torch.float32:
            kernels.layernorm_scaled_add(x, branch, self.weight, self.bias, scale, self.spec.eps)
            return x, x
        act = torch.empty(tuple(x.shape), dtype=self.runtime.dtype, device=x.device)
        kernels.layernorm_scaled_add(x, branch, self.weight, self.bias, scale, self.spec.eps, act)
        return x, act


@register_part("norm", "rmsnorm")
class RmsNorm(Norm):
    """``x / sqrt(mean(x^2) + eps) * scale`` with float statistics; the stored weight is the scale or,
    with ``unit_offset``, the scale minus one. Beside the plain form it ends a post-norm sublayer in one
    kernel: ``forward_scaled_sum`` forms ``skip_scale * x + sublayer``, normalises it into the residual
    stream and hands the next sublayer its input in the runtime dtype."""

    capturable = True

    @classmethod
    def weight_specs(cls, spec, prefix):
        # a weight stored around zero is drawn like a norm's shift when random weights are asked for
        init = "norm_bias" if spec.unit_offset else "norm_weight"
        return [WeightSpec(prefix + spec.weight_name, (spec.size,), role="vector", init=init)]

    def load(self, fetch):
        self.weight = fetch(self.prefix + self.spec.weight_name)
        self.offset = 1.0 if self.spec.unit_offset else 0.0
        self.scale = self.weight + 1.0 if self.spec.unit_offset else self.weight      # what a row is multiplied with

    def forward(self, x, out=None, rows=None):
        n_rows = x.shape[0] if rows is None else rows.numel()
        if out is None:
            out = torch.empty((n_rows, self.spec.size), dtype=self.runtime.dtype, device=x.device)
        kernels.rmsnorm(x, self.weight, self.offset, self.spec.eps, out, rows)
        return out

    def forward_scaled_sum(self, x, sublayer, skip_scale):
        """``x <- norm(skip_scale * x + sublayer)`` in place (both float32). Returns (x, activations): the
        same rows in the runtime dtype, which is ``x`` itself on the 32-bit path."""
        if self.runtime.dtype == torch.float32:
            kernels.rmsnorm_sum(x, sublayer, skip_scale, self.weight, self.offset, self.spec.eps)
            return x, x
        act = torch.empty(tuple(x.shape), dtype=self.runtime.dtype, device=x.device)
        kernels.rmsnorm_sum(x, sublayer, skip_scale, self.weight, self.offset, self.spec.eps, act)
        return x, act


    def forward_branch_add(self, x, branch, next_norm=None, want_activations=False):
        """``x <- x + norm(branch)`` in place (both float32): the end of a sublayer whose own output is normalised
        before it joins the stream. Returns (x, activations): with ``next_norm`` (another ``RmsNorm`` of the same
        size) the rows ``next_norm(x)`` in the runtime dtype, formed by the same kernel; else, with
        ``want_activations``, the new rows of ``x`` in the runtime dtype (``x`` itself on the 32-bit path); else
        None."""
        dtype = self.runtime.dtype
        if next_norm is not None and (not isinstance(next_norm, RmsNorm) or next_norm.spec.eps != self.spec.eps
                                      or next_norm.spec.size != self.spec.size):
            kernels.rmsnorm_branch_add(x, branch, self.scale, None, None, self.spec.eps)
            return x, next_norm.forward(x)
        if next_norm is not None:
            out = torch.empty(tuple(x.shape), dtype=dtype, device=x.device)
            kernels.rmsnorm_branch_add(x, branch, self.scale, next_norm.scale, out, self.spec.eps)
            return x, out
        if want_activations and dtype != torch.float32:
            out = torch.empty(tuple(x.shape), dtype=dtype, device=x.device)
            kernels.rmsnorm_branch_add(x, branch, self.scale, None, out, self.spec.eps)
            return x, out
        kernels.rmsnorm_branch_add(x, branch, self.scale, None, None, self.spec.eps)
        return x, (x if want_activations else None)


@register_part("norm", "dynamic_tanh")
class DynamicTanh(Norm):
    """``tanh(alpha * x) * weight + shift`` on the float residual stream (``DynamicTanhSpec``): no mean, no
    variance, one learned scalar. Float arithmetic, one rounding to the runtime dtype. Like LayerNorm it can form
    a residual sum that a library product left unadded on its way through the rows."""

    capturable = True
    adds_pending_sum = True

    @classmethod
    def weight_specs(cls, spec, prefix):
        return [WeightSpec(prefix + spec.weight_name, (spec.size,), role="vector", init="norm_weight"),
                WeightSpec(prefix + spec.shift_name, (spec.size,), role="vector", init="norm_bias"),
                WeightSpec(prefix + spec.alpha_name, (), role="vector", init="norm_weight")]

    def load(self, fetch):
        self.weight = fetch(self.prefix + self.spec.weight_name)
        self.shift = fetch(self.prefix + self.spec.shift_name)
        self.alpha = fetch(self.prefix + self.spec.alpha_name).reshape(1)

    def forward(self, x, out=None, rows=None):
        n_rows = x.shape[0] if rows is None else rows.numel()
        if out is None:
            out = torch.empty((n_rows, self.spec.size), dtype=self.runtime.dtype, device=x.device)
        kernels.dyt(x, self.weight, self.shift, self.alpha, out, rows)
        return out

    def forward_sum(self, pending):
        x = pending.added_by_kernel()
        out = torch.empty(tuple(x.shape), dtype=self.runtime.dtype, device=x.device)
        kernels.dyt(x, self.weight, self.shift, self.alpha, out, acc=pending.acc, col_bias=pending.bias)
        return x, out
