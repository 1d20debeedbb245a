"""Attention over one cached latent vector per token, with the per-head expansions folded around it.

With c_j the normalised latent of token j and r_j its rotated shared key part, head h's score is
``(q_plain_h . Uk_h c_j + q_rot_h . r_j) * scale = ((Uk_h^T q_plain_h) . c_j + q_rot_h . r_j) * scale``
and its output ``Uv_h sum_j p_j c_j``: so the cache holds only ``[c_j | r_j]`` (one plane, one "head"),
the key expansion becomes a per-head product on the query side and the value expansion a per-head
product after the softmax. A step is: one fused product (queries and the down projection, float
result), one kernel that normalises the latent, rotates the rotated parts and stores the token's cache
vector, the query-side per-head product, the attention kernel over the paged latent cache, the
value-side per-head product, and the output projection. Scores, softmax, norm and angles are float.

Optional, by the spec: queries through a latent of their own (the first product then gives the query latent, the
down projection and the gate; an RMS norm and a second product give the queries), a learned sink logit per head in
the softmax's denominator, a sigmoid gate on the concatenated heads that reads the mixer's input, and either
pairing of the rotated entries.
"""

from __future__ import annotations

import os

import torch

from matricxon_b200.ops import kernels
from matricxon_b200.ops.linear import EPILOGUE_F32, EPILOGUE_RESIDUAL, batched_linear, linear
from matricxon_b200.parts.base import KVCacheRequest, Mixer, build_part, register_part
from matricxon_b200.weights.loader import WeightSpec


# fewest chunks of 32 keys a key split is given (MATRICXON_LATENT_SPLIT_CHUNKS, for measurements)
_SPLIT_CHUNKS = max(1, int(os.environ.get("MATRICXON_LATENT_SPLIT_CHUNKS", "4")))


@register_part("mixer", "latent_attention")
class LatentAttention(Mixer):
    def __init__(self, spec, runtime, prefix):
        super().__init__(spec, runtime, prefix)
        self.position = build_part("position", spec.position, runtime, prefix)
        self.capturable = self.position.capturable
        self.key_width = spec.latent_rank + spec.rot_dim

    @classmethod
    def weight_specs(cls, spec, prefix):
        s = spec
        q_rows = s.num_heads * (s.head_dim + s.rot_dim)
        matrices = {s.query_name: (q_rows, s.hidden_size if s.query_rank is None else s.query_rank),
                    s.down_name: (s.latent_rank + s.rot_dim, s.hidden_size),
                    s.key_up_name: (s.num_heads * s.head_dim, s.latent_rank),
                    s.value_up_name: (s.num_heads * s.value_dim, s.latent_rank),
                    s.output_name: (s.hidden_size, s.num_heads * s.value_dim)}
        specs = [WeightSpec(prefix + name, shape, role="matrix", init="weight") for name, shape in matrices.items()]
        specs.append(WeightSpec(prefix + s.latent_norm_name, (s.latent_rank,), role="vector", init="norm_weight"))
        if s.query_rank is not None:
            specs.append(WeightSpec(prefix + s.query_down_name, (s.query_rank, s.hidden_size), role="matrix", init="weight"))
            specs.append(WeightSpec(prefix + s.query_norm_name, (s.query_rank,), role="vector", init="norm_weight"))
        if s.gate_name is not None:
            specs.append(WeightSpec(prefix + s.gate_name, (s.num_heads * s.value_dim, s.hidden_size), role="matrix",
                                    init="weight"))
        if s.sink_name is not None:
            specs.append(WeightSpec(prefix + s.sink_name, (s.num_heads,), role="vector", init="bias"))
        return specs

    @classmethod
    def cache_request(cls, spec):
        # one vector per token for all heads: the latent, then the rotated shared key part
        return KVCacheRequest(num_kv_heads=1, head_dim=spec.latent_rank + spec.rot_dim, window=spec.window,
                              planes=1)

    def load(self, fetch):
        p, s = self.prefix, self.spec
        # rows of the product that reads the mixer's input: [queries or their latent | down projection | gate]
        first = [fetch(p + (s.query_name if s.query_rank is None else s.query_down_name)), fetch(p + s.down_name)]
        if s.gate_name is not None:
            first.append(fetch(p + s.gate_name))
        self.proj_weight = torch.cat(first)
        self.query_up = self.query_norm = None
        if s.query_rank is not None:
            self.query_up = fetch(p + s.query_name)
            self.query_norm = fetch(p + s.query_norm_name)
        self.sink = fetch(p + s.sink_name) if s.sink_name is not None else None
        self.latent_norm = fetch(p + s.latent_norm_name)
        # Uk as [head][rank][dim]: the query-side product is q_plain_h @ Uk_h, i.e. "weight" Uk_h^T
        self.key_up_t = fetch(p + s.key_up_name).view(s.num_heads, s.head_dim, s.latent_rank) \
                                                .transpose(1, 2).contiguous()
        self.value_up = fetch(p + s.value_up_name).view(s.num_heads, s.value_dim, s.latent_rank).contiguous()
        self.o_weight = fetch(p + s.output_name)

    def _tiles(self, ctx):
        """(tile list on the device or None, number of tiles) for the tensor-core kernel, built once per
        step and head count. A fixed-size batch of decoding requests needs no list: tile i is sequence i."""
        heads = self.spec.num_heads
        if ctx.padded:
            return None, ctx.n_seqs
        key = ("latent_tiles", heads)
        if key not in ctx.memo:
            flat = kernels.latent_tile_list(ctx.host.q_lens, heads)
            ctx.memo[key] = (torch.tensor(flat + [0, 0], dtype=torch.int32).to(ctx.device, non_blocking=True),
                             len(flat) // 2)
        return ctx.memo[key]

    def _splits(self, ctx, n_tiles: int):
        """Key splits: a block fills an SM's shared memory, so few tiles (decoding) leave SMs idle unless
        each tile's keys are shared out; a split keeps at least ``_SPLIT_CHUNKS`` chunks of 32 keys."""
        span = ctx.max_kv_len if self.spec.window is None else min(ctx.max_kv_len, self.spec.window)
        blocks = n_tiles * (-(-self.spec.num_heads // 64) if ctx.padded else 1)
        n_splits = max(1, min(ctx.sm_count // max(blocks, 1), (span // 32 + 1) // _SPLIT_CHUNKS, 64))
        if n_splits == 1:
            return 1, None
        return n_splits, ctx.scratch(kernels.attention_scratch_bytes(ctx.n_tokens, self.spec.num_heads,
                                                                     self.spec.latent_rank, n_splits))

    def forward(self, h, residual, ctx, binding):
        s, rt = self.spec, self.runtime
        if binding.kv is None:
            raise RuntimeError("latent attention needs cache pages bound to it")
        n, heads, rank = h.shape[0], s.num_heads, s.latent_rank
        proj = linear(h, self.proj_weight, None, EPILOGUE_F32, backend=rt.gemm_backend)
        interleaved = bool(getattr(self.position, "interleaved", False))
        down = None
        first_width = heads * (s.head_dim + s.rot_dim) if s.query_rank is None else s.query_rank
        if s.query_rank is not None:
            # the queries' own latent: normalised in float, then expanded to the heads (float result)
            latent_q = torch.empty((n, s.query_rank), dtype=rt.dtype, device=h.device)
            kernels.rmsnorm(proj, self.query_norm, 0.0, s.eps, latent_q)
            down = proj[:, first_width:]
            queries = linear(latent_q, self.query_up, None, EPILOGUE_F32, backend=rt.gemm_backend)
        else:
            queries = proj
        q_plain = torch.empty((n, heads * s.head_dim), dtype=rt.dtype, device=h.device)
        q_lat = torch.empty((n, heads, self.key_width), dtype=rt.dtype, device=h.device)
        writes = binding.writes
        kernels.latent_prepare(queries, ctx.positions, self.position.frequencies, self.position.amplitude,
                               self.latent_norm, s.eps, ctx.groups[binding.group].slots if writes else None,
                               binding.kv if writes else None, q_plain, q_lat, heads, s.head_dim, s.rot_dim,
                               s.position.rotary_dim, rank, ctx.status, down=down, interleaved=interleaved)
        batched_linear(q_plain.view(n, heads, s.head_dim), self.key_up_t, None, q_lat[:, :, :rank])
        mixed = torch.empty((n, heads, rank), dtype=rt.dtype, device=h.device)
        tables = ctx.groups[binding.group].block_tables
        if kernels.latent_attention_mma_supported(rt.dtype, rank, self.key_width):
            tiles, n_tiles = self._tiles(ctx)
            n_splits, scratch = self._splits(ctx, n_tiles)
            few_rows = heads <= 16 and (ctx.padded or max(ctx.host.q_lens) * heads <= 16)
            kernels.latent_attention_mma(q_lat, binding.kv, tables, ctx.cu_q, ctx.context_lens, tiles, n_tiles, rank,
                                         s.window, s.scale, mixed, ctx.status, n_splits=n_splits, scratch=scratch,
                                         few_rows=few_rows, sink=self.sink)
        else:       # the 32-bit path, and sizes the tensor-core kernel does not take
            kernels.latent_attention(q_lat, binding.kv, tables, ctx.tok_seq, ctx.positions, rank, s.window,
                                     s.scale, mixed, ctx.status, sink=self.sink)
        attn = torch.empty((n, heads * s.value_dim), dtype=rt.dtype, device=h.device)
        batched_linear(mixed, self.value_up, None, attn.view(n, heads, s.value_dim))
        if s.gate_name is not None:
            gate_col = first_width + rank + s.rot_dim
            gated = torch.empty_like(attn)
            kernels.sigmoid_gate(attn, proj[:, gate_col:gate_col + heads * s.value_dim], gated, heads, s.value_dim)
            attn = gated
        if residual is None:
            return linear(attn, self.o_weight, None, EPILOGUE_F32, backend=rt.gemm_backend)
        return linear(attn, self.o_weight, None, EPILOGUE_RESIDUAL, residual=residual, out=residual,
                      backend=rt.gemm_backend)
