"""Rotary position encoding over whole heads, halves paired NeoX-style.

``inv_freq[i] = 1 / theta^(2i/dim)``; the angle of position p is ``p * inv_freq[i]``
in float32; ``o[i] = x[i] cos - x[i+dim/2] sin`` and ``o[i+dim/2] = x[i+dim/2] cos + x[i] sin``
(app/architectures/rope.py:16-29,152-169; app/native/src/mx_fused_ops.c:20-34). The
reference rounds cos and sin to the activation dtype before multiplying (rope.py:168);
here the rotation itself is float and the result is rounded once.

The table of inverse frequencies is built on the host exactly as the reference builds it,
so that angles at large positions agree to the last bit of the table.
"""

from __future__ import annotations

import torch

from matricxon_b200.ops import kernels
from matricxon_b200.parts.base import PositionEncoding, register_part


def inverse_frequencies(rotary_dim: int, theta: float) -> torch.Tensor:
    exponent = torch.arange(0, rotary_dim, 2, dtype=torch.float32) / rotary_dim
    return 1.0 / (theta ** exponent)


@register_part("position", "rotary_neox")
class RotaryNeox(PositionEncoding):
    capturable = True
    adds_bias = True

    def __init__(self, spec, runtime, prefix):
        super().__init__(spec, runtime, prefix)
        self.inv_freq = inverse_frequencies(spec.rotary_dim, spec.theta).to(runtime.device)

    def project_rotate_store(self, h, weight, bias, ctx, binding, n_heads, n_kv_heads, head_dim):
        rt = self.runtime
        if (rt.dtype != torch.bfloat16 or rt.gemm_backend != "auto" or self.spec.rotary_dim != head_dim
                or head_dim % 16 != 0 or not kernels.skinny_gemm_supported(h, weight)):
            return None
        writes = binding.writes and binding.kv is not None
        qkv = torch.empty((h.shape[0], weight.shape[0]), dtype=rt.dtype, device=h.device)
        kernels.gemm_skinny_rope(h, weight, bias, qkv, ctx.positions, self.inv_freq,
                                 ctx.groups[binding.group].slots if writes else None,
                                 binding.kv if writes else None, n_heads, n_kv_heads, head_dim,
                                 rt.page_size, ctx.status)
        return qkv

    def rotate_and_store(self, qkv, ctx, binding, n_heads, n_kv_heads, head_dim, bias=None):
        group = ctx.groups[binding.group] if binding.group is not None else None
        writes = binding.writes and binding.kv is not None
        kernels.rope_kv_write(
            qkv, ctx.positions, self.inv_freq,
            group.slots if writes else None, binding.kv if writes else None,
            n_heads, n_kv_heads, head_dim, self.spec.rotary_dim, self.runtime.page_size, ctx.status, bias=bias)


def store_without_rotation(qkv, ctx, binding, n_heads, n_kv_heads, head_dim, page_size):
    """Stores k and v as they are: what an attention layer without a position encoding needs,
    and what a position encoding written outside this package can call after its own rotation."""
    if not (binding.writes and binding.kv is not None):
        return
    empty = torch.empty(0, dtype=torch.float32, device=qkv.device)
    kernels.rope_kv_write(qkv, ctx.positions, empty, ctx.groups[binding.group].slots, binding.kv,
                          n_heads, n_kv_heads, head_dim, 0, page_size, ctx.status)


def interpolated_frequencies(spec) -> tuple[torch.Tensor, float]:
    """(frequency per pair, factor on cos and sin) of an ``InterpolatedRotarySpec``, in float64 on the host.

    With D = rotary_dim and base theta, pair i turns ``f_i = theta^(-2i/D)`` radians a position. The pair
    that makes t turns within the original context has index ``d(t) = D ln(original / (2 pi t)) / (2 ln theta)``.
    Pairs below ``lo = max(floor(d(fast)), 0)`` keep f_i, pairs above ``hi = min(ceil(d(slow)), D - 1)`` get
    ``f_i / factor``, and those between are blended with ``ramp = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)``."""
    import math

    dims, half = spec.rotary_dim, spec.rotary_dim // 2
    freq = [spec.theta ** (-2.0 * i / dims) for i in range(half)]
    if spec.factor is None:
        return torch.tensor(freq, dtype=torch.float64), 1.0

    def pair_of(turns: float) -> float:
        return dims * math.log(spec.original / (2.0 * math.pi * turns)) / (2.0 * math.log(spec.theta))

    lo = max(math.floor(pair_of(spec.fast)), 0)
    hi = min(math.ceil(pair_of(spec.slow)), dims - 1)
    out = []
    for i, f in enumerate(freq):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / spec.factor * ramp + f * (1.0 - ramp))
    return torch.tensor(out, dtype=torch.float64), 0.1 * math.log(spec.factor) + 1.0


@register_part("position", "rotary_interpolated")
class InterpolatedRotary(PositionEncoding):
    """Rotary encoding with stretched frequencies and an amplitude on cos and sin. It holds the table
    (``frequencies`` float32 on the device, ``amplitude``) for mixers whose own kernels rotate (latent
    attention rotates a part of each query head and one shared key part); the whole-head
    ``rotate_and_store`` of the stock attention part knows no amplitude and is not offered."""

    capturable = True

    def __init__(self, spec, runtime, prefix):
        super().__init__(spec, runtime, prefix)
        table, self.amplitude = interpolated_frequencies(spec)
        self.frequencies = table.to(torch.float32).to(runtime.device)

    def rotate_and_store(self, qkv, ctx, binding, n_heads, n_kv_heads, head_dim):
        raise NotImplementedError("an interpolated rotary table serves mixers that rotate in their own kernels")


def wavelength_scaled_frequencies(spec) -> torch.Tensor:
    """Radians per position of every pair of a ``WavelengthRotarySpec``, in float64 on the host: ``theta^(-2i/D)``,
    kept for wavelengths below ``original / high``, divided by ``factor`` above ``original / low``, blended
    linearly in ``original / wavelength`` between the two."""
    import math

    dims = spec.rotary_dim
    out = []
    for i in range(dims // 2):
        f = spec.theta ** (-2.0 * i / dims)
        if spec.factor is not None:
            wavelength = 2.0 * math.pi / f
            if wavelength > spec.original / spec.low:
                f = f / spec.factor
            elif wavelength >= spec.original / spec.high:
                s = (spec.original / wavelength - spec.low) / (spec.high - spec.low)
                f = (1.0 - s) * f / spec.factor + s * f
        out.append(f)
    return torch.tensor(out, dtype=torch.float64)


@register_part("position", "rotary_wavelength")
class WavelengthScaledRotary(PositionEncoding):
    """Holds the frequency table (``frequencies``, float32 on the device) of a ``WavelengthRotarySpec`` for mixers
    whose own kernels rotate a part of each head; angles are ``position * frequency`` in float there."""

    capturable = True

    def __init__(self, spec, runtime, prefix):
        super().__init__(spec, runtime, prefix)
        self.frequencies = wavelength_scaled_frequencies(spec).to(torch.float32).to(runtime.device)

    def rotate_and_store(self, qkv, ctx, binding, n_heads, n_kv_heads, head_dim):
        raise NotImplementedError("a wavelength-scaled table serves mixers that rotate in their own kernels")


def paired_frequencies(spec) -> torch.Tensor:
    """Radians per position of every pair of a ``PairedRotarySpec``: ``theta^(-2i/D)``, in float64 on the host."""
    dims = spec.rotary_dim
    return torch.tensor([spec.theta ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64)


@register_part("position", "rotary_paired")
class PairedRotary(PositionEncoding):
    """Holds the frequency table (``frequencies``, float32 on the device) and the pairing (``interleaved``) of a
    ``PairedRotarySpec`` for mixers whose own kernels rotate a part of each head; angles are
    ``position * frequency`` in float there. ``amplitude`` is 1: cos and sin are used as they are."""

    capturable = True
    amplitude = 1.0

    def __init__(self, spec, runtime, prefix):
        super().__init__(spec, runtime, prefix)
        self.frequencies = paired_frequencies(spec).to(torch.float32).to(runtime.device)
        self.interleaved = spec.pairing == "interleaved"

    def rotate_and_store(self, qkv, ctx, binding, n_heads, n_kv_heads, head_dim):
        raise NotImplementedError("a paired rotary table serves mixers that rotate in their own kernels")
