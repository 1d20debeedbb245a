"""Grouped-query attention over the paged cache.

``q, k, v = h Wq^T + bq, h Wk^T + bk, h Wv^T + bv`` (three Linear modules in the reference,
app/architectures/qwen_layers.py:50-52,71; packed here into one product), heads split as
feature ``head * head_dim + d`` (qwen_layers.py:72-74), position encoding on q and k
(qwen_layers.py:80), k and v stored (k already rotated, qwen_layers.py:83-86), scores scaled by
``scale`` with the causal rule ``j <= p`` (qwen_layers.py:12-17) and, when ``window`` is set,
``j > p - window`` (app/architectures/gemma4_layers.py:17-34, app/native/src/mx_attention.c:36-39);
query head h uses KV head ``h // (heads / kv heads)`` (qwen_layers.py:90-100); then
``residual + o Wo^T + bo`` (qwen_layers.py:101-102, app/architectures/starcoder2_layers.py:67).

Which kernel runs a step's rows, how the rows are cut into tiles and into how many pieces the
keys of a tile are split is decided here, beside the kernels' wrappers: the step context only
says what the step looks like (``host.q_lens``, ``max_kv_len``, ``sm_count``) and hands out
scratch memory (``ctx.scratch``) and a per-step memo (``ctx.memo``) so that layers with the same
geometry build their tile lists once.
"""

from __future__ import annotations

import os

import torch

from matricxon_b200.ops import kernels
from matricxon_b200.ops.linear import EPILOGUE_F32, EPILOGUE_NONE, EPILOGUE_RESIDUAL, chosen_backend, linear
from matricxon_b200.parts.base import KVCacheRequest, Mixer, build_part, register_part
from matricxon_b200.parts.rotary import store_without_rotation
from matricxon_b200.weights.loader import WeightSpec


# MATRICXON_TC_ATTENTION=0 keeps prompt portions on the mma.sync kernel (for comparisons)
_TC_ATTENTION = os.environ.get("MATRICXON_TC_ATTENTION", "1") != "0"


# ---------------------------------------------------------------------- tiling and key splits
def attention_tiles(ctx, group: int, token_tiles: bool = False):
    """Tile lists of the tensor-core attention for query groups of ``group`` heads:
    (narrow tiles, their count, wide tiles, their count); built once per step, group and
    kind of wide tile (64 rows, or ``token_tiles``: 128 // group tokens for the tcgen05 kernel)."""
    key = ("attention_tiles", group, token_tiles)
    cached = ctx.memo.get(key)
    if cached is not None:
        return cached
    q_lens = [1] * ctx.n_seqs if ctx.padded else ctx.host.q_lens
    narrow, wide = kernels.attention_tile_lists(q_lens, group, token_tiles)
    both = torch.tensor(narrow + wide + [0, 0], dtype=torch.int32).to(ctx.device, non_blocking=True)
    ctx.memo[key] = (both[:len(narrow)], len(narrow) // 2,
                     both[len(narrow):len(narrow) + len(wide)], len(wide) // 2)
    return ctx.memo[key]


def _key_span(ctx, window: int | None) -> int:
    return ctx.max_kv_len if window is None else min(ctx.max_kv_len, window)


class _SpanLimited:
    """A step context whose longest key range is capped (a mask that never shows a query more than ``limit`` keys):
    what sizes the key splits. Everything else is the context's own."""

    def __init__(self, ctx, limit: int) -> None:
        self._ctx, self._limit = ctx, limit

    @property
    def max_kv_len(self) -> int:
        return min(self._ctx.max_kv_len, self._limit)

    def __getattr__(self, name):
        return getattr(self._ctx, name)


def mma_tile_splits(ctx, n_tiles: int, narrow: bool, alone: bool, n_heads: int, n_kv_heads: int,
                    head_dim: int, window: int | None):
    """Key splits for one launch of the mma.sync attention (a block per tile, KV head and
    split). Splits only pay when the tiles alone leave SMs idle, and only a launch that covers
    every token of the step may use them (the merge runs over all tokens)."""
    if not alone:
        return 1, None
    items = max(n_tiles * n_kv_heads, 1)
    chunks = _key_span(ctx, window) // 32 + 1
    # a narrow block fills an SM's shared memory with its eight private stages: one per SM. A share of at
    # least eight chunks gives every warp of a narrow block one (a lone request at 3,100 tokens: 12 shares
    # of 8 chunks decode at 585 tok/s, 24 of 4 at 570, 48 of 2 at 520: more blocks, more to merge)
    target = ctx.sm_count * (1 if narrow else 2)
    n_splits = max(1, min(target // items, chunks // 8, 128))
    while n_splits > 1 and kernels.attention_scratch_bytes(
            ctx.n_tokens, n_heads, head_dim, n_splits) > (256 << 20):
        n_splits //= 2
    if n_splits == 1:
        return 1, None
    return n_splits, ctx.scratch(kernels.attention_scratch_bytes(ctx.n_tokens, n_heads, head_dim, n_splits))


def tc_tile_splits(ctx, n_tiles: int, alone: bool, n_heads: int, n_kv_heads: int, head_dim: int,
                   window: int | None):
    """Key splits for the tcgen05 attention (one block per SM, chunks of 128 keys): a short
    portion after a long context has few tiles with many chunks each."""
    items = max(n_tiles * n_kv_heads, 1)
    n_splits = min(ctx.sm_count // items, (_key_span(ctx, window) // 128 + 1) // 3, 8) if alone else 1
    if n_splits < 2:
        return 1, None
    return n_splits, ctx.scratch(kernels.attention_scratch_bytes(ctx.n_tokens, n_heads, head_dim, n_splits))


def simt_splits(ctx, n_heads: int, n_kv_heads: int, head_dim: int, window: int | None):
    """Key splits of the generic kernel: few query tokens (decoding) leave most SMs idle unless
    the keys are split; many tokens fill the GPU by themselves."""
    group = n_heads // n_kv_heads
    blocks = ctx.n_tokens * n_kv_heads * ((group + 15) // 16)
    chunks = _key_span(ctx, window) // 32 + 2
    n_splits = max(1, min(ctx.sm_count * 4 // max(blocks, 1), chunks // 2, 64))
    if n_splits == 1:
        return 1, None
    return n_splits, ctx.scratch(kernels.attention_scratch_bytes(ctx.n_tokens, n_heads, head_dim, n_splits))


def paged_attend(q, q_stride, ctx, binding, rt, n_heads, n_kv_heads, head_dim, window, scale, softcap=None,
                 sink=None, keep_first=0, chunk=None):
    """Attention of the step's query rows (``q``: query head h of a row at column ``h * head_dim``, rows
    ``q_stride`` apart) over the keys and values already stored in ``binding.kv``: picks the kernel, the
    tiles and the key splits for this step. Returns [tokens, heads * head_dim] in the runtime dtype.
    ``softcap`` caps the scaled scores at ``softcap * tanh(score / softcap)``; ``sink`` (float32, one logit per
    head) joins the softmax's denominator without a value. ``keep_first``: under a window, the keys of the
    sequence's first ``keep_first`` positions stay visible at any distance. ``chunk`` (instead of a window): the
    sequence is cut into blocks of ``chunk`` positions counted from its start and a query sees the keys of its own
    block only; the kernels take this rule as a negative ``window``. Every kernel takes cap, sink, kept tokens and
    blocks."""
    if chunk is not None:
        if window is not None:
            raise ValueError("attention is masked by a window or by blocks, not both")
        if int(chunk) <= 0:
            raise ValueError(f"blocks hold at least one position, got {chunk}")
        # a query walks at most the keys of one block
        attn = paged_attend(q, q_stride, _SpanLimited(ctx, int(chunk)), binding, rt, n_heads, n_kv_heads, head_dim,
                            -int(chunk), scale, softcap=softcap, sink=sink)
        return attn
    keep_first = int(keep_first) if window is not None and window > 0 else 0
    extras = {"softcap": softcap, "sink": sink}
    kept = {"keep_first": keep_first}
    # the kept keys are walked beside the window's: the span that sizes the key splits grows by them
    span = None if window is None or window < 0 else window + keep_first
    group = ctx.groups[binding.group]
    attn = torch.empty((ctx.n_tokens, n_heads * head_dim), dtype=rt.dtype, device=q.device)
    if kernels.mma_attention_supported(rt.dtype, head_dim, rt.page_size, q_stride):
        group_size = n_heads // n_kv_heads
        # prompt portions on tcgen05 when the kernel takes the geometry, else on mma.sync
        on_tc = _TC_ATTENTION and kernels.tc_attention_supported(rt.dtype, head_dim, rt.page_size, q_stride, group_size)
        narrow, n_narrow, wide, n_wide = attention_tiles(ctx, group_size, token_tiles=on_tc)
        for tiles, n_tiles, is_narrow in ((narrow, n_narrow, True), (wide, n_wide, False)):
            if n_tiles == 0:
                continue
            if on_tc and not is_narrow:
                n_splits, scratch = tc_tile_splits(ctx, n_tiles, n_narrow == 0, n_heads,
                                                       n_kv_heads, head_dim, span)
                kernels.paged_attention_tc(q, q_stride, binding.kv, group.block_tables, ctx.cu_q,
                                           ctx.context_lens, tiles, n_tiles, ctx.n_tokens,
                                           n_heads, n_kv_heads, head_dim,
                                           window, scale, attn, ctx.status,
                                           n_splits=n_splits, scratch=scratch, **extras, **kept)
                continue
            alone = (n_wide == 0) if is_narrow else (n_narrow == 0)
            if is_narrow and ctx.padded:
                tiles, n_tiles = None, ctx.n_seqs      # a batch of decoding requests: tile i is sequence i
            n_splits, scratch = mma_tile_splits(ctx, n_tiles, is_narrow, alone, n_heads,
                                                n_kv_heads, head_dim, span)
            kernels.paged_attention_mma(q, q_stride, binding.kv, group.block_tables,
                                        ctx.cu_q, ctx.context_lens, tiles, n_tiles, is_narrow,
                                        ctx.n_tokens, n_heads, n_kv_heads,
                                        head_dim, window, scale, attn, ctx.status,
                                        n_splits=n_splits, scratch=scratch, **extras, **kept)
    else:
        n_splits, scratch = simt_splits(ctx, n_heads, n_kv_heads,
                                                 head_dim, span)
        kernels.paged_attention(q, q_stride, binding.kv, group.block_tables, ctx.tok_seq,
                                ctx.positions, ctx.n_tokens, n_heads, n_kv_heads,
                                head_dim, window, scale, attn, ctx.status,
                                n_splits=n_splits, scratch=scratch, **extras, **kept)
    return attn


@register_part("mixer", "attention")
class PagedAttention(Mixer):
    def __init__(self, spec, runtime, prefix):
        super().__init__(spec, runtime, prefix)
        self.q_size = spec.num_heads * spec.head_dim
        self.kv_size = spec.num_kv_heads * spec.head_dim
        self.position = (build_part("position", spec.position, runtime, prefix)
                         if spec.position is not None else None)
        # the kernels here are stream-ordered; a position encoding from elsewhere decides for itself
        self.capturable = self.position is None or self.position.capturable

    @classmethod
    def weight_specs(cls, spec, prefix):
        q_size, kv_size = spec.num_heads * spec.head_dim, spec.num_kv_heads * spec.head_dim
        if len(spec.projection_names) == 3:
            shapes = dict(zip(spec.projection_names, ((q_size, spec.hidden_size), (kv_size, spec.hidden_size),
                                                      (kv_size, spec.hidden_size))))
        else:
            shapes = {spec.projection_names[0]: (q_size + 2 * kv_size, spec.hidden_size)}
        shapes[spec.output_name] = (spec.hidden_size, q_size)
        specs = []
        for name, shape in shapes.items():
            specs.append(WeightSpec(f"{prefix}{name}.weight", shape, role="matrix", init="weight"))
            if spec.bias:
                specs.append(WeightSpec(f"{prefix}{name}.bias", (shape[0],), role="vector", init="bias"))
        return specs

    @classmethod
    def cache_request(cls, spec):
        return KVCacheRequest(num_kv_heads=spec.num_kv_heads, head_dim=spec.head_dim,
                              window=spec.window)

    def load(self, fetch):
        p, names = self.prefix, self.spec.projection_names

        def packed(kind: str) -> torch.Tensor:
            parts = [fetch(f"{p}{n}.{kind}") for n in names]
            return parts[0] if len(parts) == 1 else torch.cat(parts)

        self.qkv_weight = packed("weight")
        self.o_weight = fetch(f"{p}{self.spec.output_name}.weight")
        if self.spec.bias:
            self.qkv_bias = packed("bias")
            self.o_bias = fetch(f"{p}{self.spec.output_name}.bias")
        else:
            self.qkv_bias = self.o_bias = None

    def forward(self, h, residual, ctx, binding):
        spec, rt = self.spec, self.runtime
        if binding.kv is None:
            raise RuntimeError("attention needs cache pages bound to it")
        qkv = None
        if self.position is not None:
            qkv = self.position.project_rotate_store(h, self.qkv_weight, self.qkv_bias, ctx, binding,
                                                     spec.num_heads, spec.num_kv_heads, spec.head_dim)
        if qkv is not None:
            pass                                        # product, rotation and cache write were one kernel
        elif (self.position is not None and self.position.adds_bias and self.qkv_bias is not None
              and chosen_backend(h, self.qkv_weight, rt.gemm_backend) == "library"):
            # the library's product has no epilogue of its own: the rotation kernel adds the bias on its way
            qkv = linear(h, self.qkv_weight, None, EPILOGUE_NONE, backend=rt.gemm_backend)
            self.position.rotate_and_store(qkv, ctx, binding, spec.num_heads, spec.num_kv_heads,
                                           spec.head_dim, bias=self.qkv_bias)
        elif self.position is not None:
            qkv = linear(h, self.qkv_weight, self.qkv_bias, EPILOGUE_NONE, backend=rt.gemm_backend)
            self.position.rotate_and_store(qkv, ctx, binding, spec.num_heads, spec.num_kv_heads,
                                           spec.head_dim)
        else:
            qkv = linear(h, self.qkv_weight, self.qkv_bias, EPILOGUE_NONE, backend=rt.gemm_backend)
            store_without_rotation(qkv, ctx, binding, spec.num_heads, spec.num_kv_heads,
                                   spec.head_dim, rt.page_size)
        attn = paged_attend(qkv, qkv.stride(0), ctx, binding, rt, spec.num_heads, spec.num_kv_heads, spec.head_dim,
                            spec.window, spec.scale)
        return linear(attn, self.o_weight, self.o_bias, EPILOGUE_RESIDUAL, residual=residual,
                      out=residual, backend=rt.gemm_backend, defer_sum=getattr(ctx, "sums_may_pend", False))


@register_part("mixer", "gated_attention")
class GatedAttention(Mixer):
    """Grouped-query attention with per-head RMS-normalised queries and keys, no position encoding,
    values of a width of their own and a sigmoid gate on the concatenated heads (``GatedAttentionSpec``).

    One fused product gives float rows ``[q | k | v | gate]``; one kernel normalises q and k per head in
    float and stores k and v in the paged cache in the layout the stock attention kernels read
    (``paged_attend``), every head padded with zeros to a common size of a multiple of 16 when the query
    and value widths differ or are no such multiple; one kernel applies the gate and drops the padding.
    ``forward(h, None, ...)`` returns the mixer's float output without a residual."""

    capturable = True

    def __init__(self, spec, runtime, prefix):
        super().__init__(spec, runtime, prefix)
        self.padded_dim = self.cache_head_dim(spec)

    @staticmethod
    def cache_head_dim(spec) -> int:
        return -(-max(spec.head_dim, spec.value_dim) // 16) * 16

    @classmethod
    def _matrices(cls, spec):
        q, kv = spec.num_heads * spec.head_dim, spec.num_kv_heads * spec.head_dim
        shapes = [(spec.query_name, (q, spec.hidden_size)), (spec.key_name, (kv, spec.hidden_size)),
                  (spec.value_name, (spec.num_kv_heads * spec.value_dim, spec.hidden_size))]
        if spec.gate_name is not None:
            shapes.append((spec.gate_name, (spec.num_heads * spec.value_dim, spec.hidden_size)))
        return shapes

    @classmethod
    def weight_specs(cls, spec, prefix):
        specs = [WeightSpec(prefix + name, shape, role="matrix", init="weight") for name, shape in cls._matrices(spec)]
        specs.append(WeightSpec(prefix + spec.output_name, (spec.hidden_size, spec.num_heads * spec.value_dim),
                                role="matrix", init="weight"))
        for name in (spec.query_norm_name, spec.key_norm_name):
            if name is not None:
                specs.append(WeightSpec(prefix + name, (spec.head_dim,), role="vector", init="norm_weight"))
        return specs

    @classmethod
    def cache_request(cls, spec):
        return KVCacheRequest(num_kv_heads=spec.num_kv_heads, head_dim=cls.cache_head_dim(spec), window=spec.window)

    def load(self, fetch):
        p, s = self.prefix, self.spec
        self.proj_weight = torch.cat([fetch(p + name) for name, _ in self._matrices(s)])
        self.o_weight = fetch(p + s.output_name)
        self.q_norm = fetch(p + s.query_norm_name) if s.query_norm_name is not None else None
        self.k_norm = fetch(p + s.key_norm_name) if s.key_norm_name is not None else None

    def forward(self, h, residual, ctx, binding):
        s, rt, hd = self.spec, self.runtime, self.padded_dim
        if binding.kv is None:
            raise RuntimeError("attention needs cache pages bound to it")
        n = h.shape[0]
        proj = linear(h, self.proj_weight, None, EPILOGUE_F32, backend=rt.gemm_backend)
        q = torch.empty((n, s.num_heads * hd), dtype=rt.dtype, device=h.device)
        writes = binding.writes
        kernels.qk_norm_kv_write(proj, self.q_norm, self.k_norm, s.eps,
                                 ctx.groups[binding.group].slots if writes else None,
                                 binding.kv if writes else None, q, s.num_heads, s.num_kv_heads,
                                 s.head_dim, s.value_dim, ctx.status)
        attn = paged_attend(q, q.stride(0), ctx, binding, rt, s.num_heads, s.num_kv_heads, hd, s.window, s.scale)
        if s.gate_name is not None:
            gate_col = (s.num_heads + s.num_kv_heads) * s.head_dim + s.num_kv_heads * s.value_dim
            gated = torch.empty((n, s.num_heads * s.value_dim), dtype=rt.dtype, device=h.device)
            kernels.sigmoid_gate(attn, proj[:, gate_col:], gated, s.num_heads, s.value_dim)
            attn = gated
        elif hd != s.value_dim:
            attn = attn.view(n, s.num_heads, hd)[:, :, :s.value_dim].reshape(n, -1)
        if residual is None:
            return linear(attn, self.o_weight, None, EPILOGUE_F32, backend=rt.gemm_backend)
        return linear(attn, self.o_weight, None, EPILOGUE_RESIDUAL, residual=residual, out=residual,
                      backend=rt.gemm_backend)


@register_part("mixer", "sink_attention")
class SinkAttention(Mixer):
    """Grouped-query attention with biased projections, a rotation of the first entries of every head, capped
    scores, a sink logit per head in the softmax's denominator, values that may be blended with an earlier
    layer's values of the same token, and one sigmoid gate per head (``SinkAttentionSpec``).

    One fused product gives float rows ``[q | k | v | gate]`` with the biases added; one kernel rotates q and k in
    float, blends the values and stores k and v in the paged cache in the layout the stock attention kernels
    read (``paged_attend``, which caps the scores and counts the sink), every head padded with zeros to a common
    size of a multiple of 16 when the key and value widths differ or are no such multiple; one kernel applies
    the gate and drops the padding. A layer whose ``value_mix`` is ``"source"`` leaves its float values in the
    step's memo under ``value_mix_key``; a ``"blend"`` layer reads them there."""

    capturable = True

    def __init__(self, spec, runtime, prefix):
        super().__init__(spec, runtime, prefix)
        self.padded_dim = self.cache_head_dim(spec)
        self.position = (build_part("position", spec.position, runtime, prefix)
                         if spec.position is not None else None)

    @staticmethod
    def cache_head_dim(spec) -> int:
        return -(-max(spec.head_dim, spec.value_dim) // 16) * 16

    @classmethod
    def _matrices(cls, spec):
        """(name, shape, has a bias) of the projections, in the order of the fused product's rows."""
        shapes = [(spec.query_name, (spec.num_heads * spec.head_dim, spec.hidden_size), spec.bias),
                  (spec.key_name, (spec.num_kv_heads * spec.head_dim, spec.hidden_size), spec.bias),
                  (spec.value_name, (spec.num_kv_heads * spec.value_dim, spec.hidden_size), spec.bias)]
        if spec.gate_name is not None:
            shapes.append((spec.gate_name, (spec.num_heads, spec.hidden_size), False))
        return shapes

    @classmethod
    def weight_specs(cls, spec, prefix):
        specs = []
        for name, shape, biased in cls._matrices(spec):
            specs.append(WeightSpec(prefix + name, shape, role="matrix", init="weight"))
            if biased:
                specs.append(WeightSpec(prefix + name + spec.bias_suffix, (shape[0],), role="vector", init="bias"))
        specs.append(WeightSpec(prefix + spec.output_name, (spec.hidden_size, spec.num_heads * spec.value_dim),
                                role="matrix", init="weight"))
        if spec.sink_name is not None:
            specs.append(WeightSpec(prefix + spec.sink_name, (spec.num_heads,), role="vector", init="bias"))
        if spec.value_mix_name is not None:
            specs.append(WeightSpec(prefix + spec.value_mix_name, (), role="vector", init="bias"))
        return specs

    @classmethod
    def cache_request(cls, spec):
        return KVCacheRequest(num_kv_heads=spec.num_kv_heads, head_dim=cls.cache_head_dim(spec), window=spec.window)

    def load(self, fetch):
        p, s = self.prefix, self.spec
        matrices = self._matrices(s)
        self.proj_weight = torch.cat([fetch(p + name) for name, _, _ in matrices])
        self.proj_bias = None
        if s.bias:
            self.proj_bias = torch.cat([fetch(p + name + s.bias_suffix) if biased else
                                        torch.zeros(shape[0], dtype=torch.float32, device=self.runtime.device)
                                        for name, shape, biased in matrices])
        self.o_weight = fetch(p + s.output_name)
        self.sink = fetch(p + s.sink_name) if s.sink_name is not None else None
        # the scalar is read even where the layer does not blend (a source layer's is unused)
        self.value_mix = fetch(p + s.value_mix_name).reshape(1) if s.value_mix_name is not None else None

    def forward(self, h, residual, ctx, binding):
        s, rt, hd = self.spec, self.runtime, self.padded_dim
        if binding.kv is None:
            raise RuntimeError("attention needs cache pages bound to it")
        n = h.shape[0]
        proj = linear(h, self.proj_weight, self.proj_bias, EPILOGUE_F32, backend=rt.gemm_backend)
        v_col = (s.num_heads + s.num_kv_heads) * s.head_dim
        v_width = s.num_kv_heads * s.value_dim
        other = None
        if s.value_mix is not None:
            if s.value_mix == "blend":
                other = ctx.memo.get(s.value_mix_key)
                if other is None:
                    raise RuntimeError("a layer blends values, but no earlier layer of this step published any")
            else:
                # every run of the step publishes anew: a captured run must not read what its warm-up run left
                ctx.memo[s.value_mix_key] = proj[:, v_col:v_col + v_width]
        if other is not None and other.shape[1] != v_width:
            raise RuntimeError(f"cannot blend values of width {v_width} with published values of width {other.shape[1]}")
        q = torch.empty((n, s.num_heads * hd), dtype=rt.dtype, device=h.device)
        writes = binding.writes
        if self.position is not None:
            freq, rot = self.position.frequencies, s.position.rotary_dim
        else:
            freq, rot = torch.empty(0, dtype=torch.float32, device=h.device), 0
        kernels.rotate_mix_kv_write(proj, ctx.positions, freq, rot, other, self.value_mix if other is not None else None,
                                    ctx.groups[binding.group].slots if writes else None,
                                    binding.kv if writes else None, q, s.num_heads, s.num_kv_heads, s.head_dim,
                                    s.value_dim, ctx.status)
        attn = paged_attend(q, q.stride(0), ctx, binding, rt, s.num_heads, s.num_kv_heads, hd, s.window, s.scale,
                            softcap=s.softcap, sink=self.sink)
        if s.gate_name is not None:
            gate_col = v_col + v_width
            gated = torch.empty((n, s.num_heads * s.value_dim), dtype=rt.dtype, device=h.device)
            kernels.head_gate(attn, proj[:, gate_col:gate_col + s.num_heads], gated, s.num_heads, s.value_dim)
            attn = gated
        elif hd != s.value_dim:
            attn = attn.view(n, s.num_heads, hd)[:, :, :s.value_dim].reshape(n, -1)
        if residual is None:
            return linear(attn, self.o_weight, None, EPILOGUE_F32, backend=rt.gemm_backend)
        return linear(attn, self.o_weight, None, EPILOGUE_RESIDUAL, residual=residual, out=residual,
                      backend=rt.gemm_backend, defer_sum=getattr(ctx, "sums_may_pend", False))


@register_part("mixer", "unit_norm_attention")
class UnitNormAttention(Mixer):
    """Grouped-query attention without biases whose queries and keys are rotated over the first entries of every
    head and then divided by their root mean square, head by head, with no learned weight; a window that keeps
    the sequence's first tokens in sight; values of a width of their own (``UnitNormAttentionSpec``).

    One fused product gives float rows ``[q | k | v]``; one kernel rotates and normalises q and k in float and
    stores k and v in the paged cache in the layout the stock attention kernels read (``paged_attend``, which
    knows the window's kept first tokens), every head padded with zeros to a common size of a multiple of 16
    when the key and value widths differ or are no such multiple. ``forward(h, None, ...)`` returns the mixer's
    float output without a residual."""

    capturable = True

    def __init__(self, spec, runtime, prefix):
        super().__init__(spec, runtime, prefix)
        self.padded_dim = self.cache_head_dim(spec)
        self.position = (build_part("position", spec.position, runtime, prefix)
                         if spec.position is not None and spec.position.rotary_dim > 0 else None)

    @staticmethod
    def cache_head_dim(spec) -> int:
        return -(-max(spec.head_dim, spec.value_dim) // 16) * 16

    @classmethod
    def _matrices(cls, spec):
        return [(spec.query_name, (spec.num_heads * spec.head_dim, spec.hidden_size)),
                (spec.key_name, (spec.num_kv_heads * spec.head_dim, spec.hidden_size)),
                (spec.value_name, (spec.num_kv_heads * spec.value_dim, spec.hidden_size))]

    @classmethod
    def weight_specs(cls, spec, prefix):
        specs = [WeightSpec(prefix + name, shape, role="matrix", init="weight") for name, shape in cls._matrices(spec)]
        specs.append(WeightSpec(prefix + spec.output_name, (spec.hidden_size, spec.num_heads * spec.value_dim),
                                role="matrix", init="weight"))
        return specs

    @classmethod
    def cache_request(cls, spec):
        return KVCacheRequest(num_kv_heads=spec.num_kv_heads, head_dim=cls.cache_head_dim(spec), window=spec.window,
                              keep_first=spec.keep_first if spec.window is not None else 0)

    def load(self, fetch):
        p, s = self.prefix, self.spec
        self.proj_weight = torch.cat([fetch(p + name) for name, _ in self._matrices(s)])
        self.o_weight = fetch(p + s.output_name)

    def forward(self, h, residual, ctx, binding):
        s, rt, hd = self.spec, self.runtime, self.padded_dim
        if binding.kv is None:
            raise RuntimeError("attention needs cache pages bound to it")
        n = h.shape[0]
        proj = linear(h, self.proj_weight, None, EPILOGUE_F32, backend=rt.gemm_backend)
        q = torch.empty((n, s.num_heads * hd), dtype=rt.dtype, device=h.device)
        writes = binding.writes
        if self.position is not None:
            freq, rot = self.position.frequencies, s.position.rotary_dim
        else:
            freq, rot = torch.empty(0, dtype=torch.float32, device=h.device), 0
        kernels.rotate_norm_kv_write(proj, ctx.positions, freq, rot, s.eps if s.unit_norm else None,
                                     ctx.groups[binding.group].slots if writes else None,
                                     binding.kv if writes else None, q, s.num_heads, s.num_kv_heads, s.head_dim,
                                     s.value_dim, ctx.status)
        attn = paged_attend(q, q.stride(0), ctx, binding, rt, s.num_heads, s.num_kv_heads, hd, s.window, s.scale,
                            keep_first=s.keep_first)
        if hd != s.value_dim:
            attn = attn.view(n, s.num_heads, hd)[:, :, :s.value_dim].reshape(n, -1)
        if residual is None:
            return linear(attn, self.o_weight, None, EPILOGUE_F32, backend=rt.gemm_backend)
        return linear(attn, self.o_weight, None, EPILOGUE_RESIDUAL, residual=residual, out=residual,
                      backend=rt.gemm_backend, defer_sum=getattr(ctx, "sums_may_pend", False))


@register_part("mixer", "normed_rotary_attention")
class NormedRotaryAttention(Mixer):
    """Grouped-query attention without biases whose queries and keys are RMS-normalised head by head with a learned
    weight and then rotated over their first entries; causal, windowed or cut into blocks; with an ordinary softmax,
    one added to its denominator, or a learned sink; optionally capped scores; a sigmoid gate per head or per entry
    that reads the mixer's input (``NormedRotaryAttentionSpec``).

    One fused product gives float rows ``[q | k | v | gate]``; one kernel normalises and rotates q and k in float and
    stores k and v in the paged cache in the layout the stock attention kernels read (``paged_attend``, which knows
    every mask, the cap and the sink), every head padded with zeros to a common size of a multiple of 16 when the key
    and value widths differ or are no such multiple; one kernel applies the gate and drops the padding.
    ``forward(h, None, ...)`` returns the mixer's float output without a residual."""

    capturable = True

    def __init__(self, spec, runtime, prefix):
        super().__init__(spec, runtime, prefix)
        self.padded_dim = self.cache_head_dim(spec)
        self.position = (build_part("position", spec.position, runtime, prefix)
                         if spec.position is not None and spec.position.rotary_dim > 0 else None)
        if self.position is not None and not hasattr(self.position, "frequencies"):
            raise ValueError(f"position encoding {spec.position.kind!r} offers no frequency table")
        self.gate_rows = {None: 0, "head": spec.num_heads, "entry": spec.num_heads * spec.value_dim}[spec.gate]

    @staticmethod
    def cache_head_dim(spec) -> int:
        return -(-max(spec.head_dim, spec.value_dim) // 16) * 16

    @classmethod
    def _matrices(cls, spec):
        shapes = [(spec.query_name, (spec.num_heads * spec.head_dim, spec.hidden_size)),
                  (spec.key_name, (spec.num_kv_heads * spec.head_dim, spec.hidden_size)),
                  (spec.value_name, (spec.num_kv_heads * spec.value_dim, spec.hidden_size))]
        if spec.gate == "head":
            shapes.append((spec.gate_name, (spec.num_heads, spec.hidden_size)))
        elif spec.gate == "entry":
            shapes.append((spec.gate_name, (spec.num_heads * spec.value_dim, spec.hidden_size)))
        return shapes

    @classmethod
    def weight_specs(cls, spec, prefix):
        specs = [WeightSpec(prefix + name, shape, role="matrix", init="weight") for name, shape in cls._matrices(spec)]
        specs.append(WeightSpec(prefix + spec.output_name, (spec.hidden_size, spec.num_heads * spec.value_dim),
                                role="matrix", init="weight"))
        for name in (spec.query_norm_name, spec.key_norm_name):
            if name is not None:
                specs.append(WeightSpec(prefix + name, (spec.head_dim,), role="vector", init="norm_weight"))
        if spec.sink == "learned":
            specs.append(WeightSpec(prefix + spec.sink_name, (spec.num_heads,), role="vector", init="bias"))
        return specs

    @classmethod
    def cache_request(cls, spec):
        # pages live by the mask: a window's rule, or whole blocks until the sequence has left them
        return KVCacheRequest(num_kv_heads=spec.num_kv_heads, head_dim=cls.cache_head_dim(spec),
                              window=spec.mask_size if spec.mask == "window" else None,
                              block=spec.mask_size if spec.mask == "chunk" else None)

    def load(self, fetch):
        p, s = self.prefix, self.spec
        self.proj_weight = torch.cat([fetch(p + name) for name, _ in self._matrices(s)])
        self.o_weight = fetch(p + s.output_name)
        self.q_norm = fetch(p + s.query_norm_name) if s.query_norm_name is not None else None
        self.k_norm = fetch(p + s.key_norm_name) if s.key_norm_name is not None else None
        if s.sink == "learned":
            self.sink = fetch(p + s.sink_name)
        elif s.sink == "zero":
            self.sink = torch.zeros(s.num_heads, dtype=torch.float32, device=self.runtime.device)
        else:
            self.sink = None

    def forward(self, h, residual, ctx, binding):
        s, rt, hd = self.spec, self.runtime, self.padded_dim
        if binding.kv is None:
            raise RuntimeError("attention needs cache pages bound to it")
        n = h.shape[0]
        proj = linear(h, self.proj_weight, None, EPILOGUE_F32, backend=rt.gemm_backend)
        q = torch.empty((n, s.num_heads * hd), dtype=rt.dtype, device=h.device)
        writes = binding.writes
        if self.position is not None:
            freq, rot = self.position.frequencies, s.position.rotary_dim
            interleaved = bool(getattr(self.position, "interleaved", False))
        else:
            freq, rot, interleaved = torch.empty(0, dtype=torch.float32, device=h.device), 0, False
        kernels.norm_rotate_kv_write(proj, ctx.positions, freq, rot, interleaved, self.q_norm, self.k_norm, s.eps,
                                     ctx.groups[binding.group].slots if writes else None,
                                     binding.kv if writes else None, q, s.num_heads, s.num_kv_heads, s.head_dim,
                                     s.value_dim, ctx.status)
        attn = paged_attend(q, q.stride(0), ctx, binding, rt, s.num_heads, s.num_kv_heads, hd,
                            s.mask_size if s.mask == "window" else None, s.scale, softcap=s.softcap, sink=self.sink,
                            chunk=s.mask_size if s.mask == "chunk" else None)
        if s.gate is not None:
            gate_col = (s.num_heads + s.num_kv_heads) * s.head_dim + s.num_kv_heads * s.value_dim
            gated = torch.empty((n, s.num_heads * s.value_dim), dtype=rt.dtype, device=h.device)
            gate = proj[:, gate_col:gate_col + self.gate_rows]
            if s.gate == "head":
                kernels.head_gate(attn, gate, gated, s.num_heads, s.value_dim)
            else:
                kernels.sigmoid_gate(attn, gate, gated, s.num_heads, s.value_dim)
            attn = gated
        elif hd != s.value_dim:
            attn = attn.view(n, s.num_heads, hd)[:, :, :s.value_dim].reshape(n, -1)
        if residual is None:
            return linear(attn, self.o_weight, None, EPILOGUE_F32, backend=rt.gemm_backend)
        return linear(attn, self.o_weight, None, EPILOGUE_RESIDUAL, residual=residual, out=residual,
                      backend=rt.gemm_backend, defer_sum=getattr(ctx, "sums_may_pend", False))
