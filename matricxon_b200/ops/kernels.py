"""Tensor-level faces of the CUDA kernels.

Each function checks device, dtype and layout, then launches on torch's current
stream. Nothing here computes with torch: a tensor that is not on a CUDA device
is an error, not a cue to fall back.
"""

from __future__ import annotations

import torch

from matricxon_b200.ops.library import KernelLibraryError, check, library

F32, BF16 = 0, 1
EPILOGUE_NONE, EPILOGUE_GELU, EPILOGUE_RESIDUAL, EPILOGUE_F32 = 0, 1, 2, 3

launch_count = 0      # kernels of this library launched so far in this process


def _launched(n: int = 1) -> None:
    global launch_count
    launch_count += n


STATUS_BITS = {1: "a token id outside the vocabulary", 2: "a cache slot outside the pool",
               4: "a block-table entry that names no page", 8: "a device-side wait ran out"}


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelLibraryError(f"kernels take float32 or bfloat16, not {dtype}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_device_index: int | None = None


def _stream() -> int:
    """The current stream's handle. ``torch.cuda.current_stream()`` builds a Python object and looks the
    device up through several layers on every call (a third of a prompt step's host time when asked
    once per launch); the raw query is one C call. One device per process."""
    global _device_index
    if _raw_stream is None:
        return torch.cuda.current_stream().cuda_stream
    if _device_index is None:
        _device_index = torch.cuda.current_device()
    return _raw_stream(_device_index)


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, name: str, dtype: torch.dtype | None = None, contiguous: bool = True):
    if not t.is_cuda:
        raise KernelLibraryError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise KernelLibraryError(f"{name} must be {dtype}, got {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelLibraryError(f"{name} must be contiguous")


def set_chained_launch(on: bool) -> None:
    """Programmatic dependent launch for the kernels launched from here on (decode kernels only
    take part): what a graph captures stays with the graph."""
    library().mx_set_chained_launch(1 if on else 0)


def describe_status(word: int) -> str:
    return "; ".join(text for bit, text in STATUS_BITS.items() if word & bit) or "no error"


def embed(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, status: torch.Tensor,
          scale: float = 1.0) -> None:
    _need(ids, "ids", torch.int32)
    _need(table, "table")
    _need(out, "out", torch.float32)
    _need(status, "status", torch.int32)
    n, hidden = out.shape
    assert ids.numel() == n and table.shape[1] == hidden
    check(library().mx_embed(_ptr(ids), _ptr(table), dtype_code(table.dtype), _ptr(out), n, hidden,
                             table.shape[0], float(scale), _ptr(status), _stream()), "embed")
    _launched()


def softcap(logits: torch.Tensor, cap: float) -> None:
    """logits <- cap * tanh(logits / cap) in place (float32)."""
    _need(logits, "logits", torch.float32)
    check(library().mx_softcap(_ptr(logits), logits.numel(), float(cap), _stream()), "softcap")
    _launched()


def layernorm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, eps: float,
              out: torch.Tensor, rows: torch.Tensor | None = None) -> None:
    """out[r] = LayerNorm(x[rows[r]] if rows is given else x[r]); x is the float residual stream."""
    _need(x, "x", torch.float32)
    _need(weight, "weight", torch.float32)
    if bias is not None:
        _need(bias, "bias", torch.float32)
    if rows is not None:
        _need(rows, "rows", torch.int32)
    _need(out, "out")
    n_rows, hidden = out.shape
    assert x.shape[1] == hidden and weight.numel() == hidden
    assert rows is None or rows.numel() == n_rows
    assert rows is not None or x.shape[0] == n_rows
    check(library().mx_layernorm(_ptr(x), _ptr(rows), _ptr(weight), _ptr(bias), _ptr(out),
                                 dtype_code(out.dtype), n_rows, hidden, float(eps), _stream()),
          "layernorm")
    _launched()


def layernorm_sum(x: torch.Tensor, acc: torch.Tensor, col_bias: torch.Tensor | None, weight: torch.Tensor,
                  bias: torch.Tensor | None, eps: float, out: torch.Tensor) -> None:
    """``x += acc + col_bias`` (the residual epilogue of a product whose float accumulator is ``acc``),
    then ``out = LayerNorm(x)``, in one pass over the rows."""
    _need(x, "x", torch.float32)
    _need(acc, "acc", torch.float32)
    _need(weight, "weight", torch.float32)
    _need(out, "out")
    assert acc.shape == x.shape and out.shape == x.shape, (x.shape, acc.shape, out.shape)
    if col_bias is not None:
        _need(col_bias, "col_bias", torch.float32)
        assert col_bias.numel() == x.shape[1]
    if bias is not None:
        _need(bias, "bias", torch.float32)
    check(library().mx_layernorm_sum(_ptr(x), _ptr(acc), _ptr(col_bias), _ptr(weight), _ptr(bias), _ptr(out),
                                     dtype_code(out.dtype), x.shape[0], x.shape[1], float(eps), _stream()),
          "layernorm_sum")
    _launched()


def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor,
                  slots: torch.Tensor | None, cache: torch.Tensor | None, n_heads: int,
                  n_kv_heads: int, head_dim: int, rotary_dim: int, page_size: int,
                  status: torch.Tensor, bias: torch.Tensor | None = None) -> None:
    """Rotates q (and k) of each row of ``qkv`` in float; writes k and v to the cache pages.

    ``cache`` is [pages, 2, kv heads, page_size, head_dim]; None rotates q only. ``bias`` (float32,
    one per column of ``qkv``): the bias of the product that made ``qkv``, still to be added; each
    sum is rounded to the dtype of ``qkv`` before it is used, as a separate epilogue would."""
    _need(qkv, "qkv")
    _need(positions, "positions", torch.int32)
    _need(inv_freq, "inv_freq", torch.float32)
    _need(status, "status", torch.int32)
    n = qkv.shape[0]
    assert qkv.shape[1] == (n_heads + 2 * n_kv_heads) * head_dim
    assert inv_freq.numel() == rotary_dim // 2
    write = cache is not None
    n_pages = 0
    if write:
        _need(cache, "cache", qkv.dtype)
        _need(slots, "slots", torch.int32)
        assert tuple(cache.shape[1:]) == (2, n_kv_heads, page_size, head_dim), cache.shape
        n_pages = cache.shape[0]
    if bias is not None:
        _need(bias, "bias", torch.float32)
        assert bias.numel() == qkv.shape[1]
    check(library().mx_rope_kv_write_bias(_ptr(qkv), dtype_code(qkv.dtype), qkv.stride(0),
                                          _ptr(positions), _ptr(inv_freq), _ptr(slots), _ptr(cache), n,
                                          n_heads, n_kv_heads, head_dim, rotary_dim, page_size, n_pages,
                                          1 if write else 0, _ptr(status), _ptr(bias), _stream()),
          "rope_kv_write")
    _launched()


def epilogue(acc: torch.Tensor, bias: torch.Tensor | None, residual: torch.Tensor | None,
             out: torch.Tensor, mode: int) -> None:
    _need(acc, "acc")
    _need(out, "out")
    n_rows, n_cols = acc.shape
    check(library().mx_epilogue(_ptr(acc), dtype_code(acc.dtype), _ptr(bias), _ptr(residual),
                                _ptr(out), dtype_code(out.dtype), n_rows, n_cols, mode, _stream()),
          "epilogue")
    _launched()


def gemm_simt(a: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None,
              residual: torch.Tensor | None, out: torch.Tensor, mode: int) -> None:
    """out = epilogue(a @ w.T + bias) with float accumulation on the FP32 cores."""
    _need(a, "a", contiguous=False)
    _need(w, "w")
    _need(out, "out")
    if a.stride(1) != 1:
        raise KernelLibraryError("a must have unit stride along K")
    m, k = a.shape
    n = w.shape[0]
    assert w.shape[1] == k and tuple(out.shape) == (m, n), (a.shape, w.shape, out.shape)
    assert w.dtype == a.dtype
    if bias is not None:
        _need(bias, "bias", torch.float32)
        assert bias.numel() == n
    if residual is not None:
        _need(residual, "residual", torch.float32)
        assert tuple(residual.shape) == (m, n)
    check(library().mx_gemm_simt(_ptr(a), _ptr(w), dtype_code(a.dtype), _ptr(bias), _ptr(residual),
                                 _ptr(out), dtype_code(out.dtype), m, n, k, a.stride(0), w.stride(0),
                                 out.stride(0), mode, _stream()), "gemm_simt")
    _launched()


_default_status: dict[int, torch.Tensor] = {}


def default_status(device: torch.device) -> torch.Tensor:
    """The status word kernels with bounded waits report to when the caller names none; a step
    runner registers its own with ``set_default_status`` so that one read covers everything."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    if index not in _default_status:
        _default_status[index] = torch.zeros(1, dtype=torch.int32, device=device)
    return _default_status[index]


def set_default_status(status: torch.Tensor) -> None:
    _default_status[status.device.index if status.device.index is not None
                    else torch.cuda.current_device()] = status


def tcgen05_gemm_supported(a: torch.Tensor, w: torch.Tensor) -> bool:
    return (a.dtype == torch.bfloat16 and a.shape[1] % 8 == 0 and a.stride(1) == 1
            and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tcgen05(a: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None,
                 residual: torch.Tensor | None, out: torch.Tensor, mode: int,
                 status: torch.Tensor | None = None) -> None:
    """The prompt-sized product on the tcgen05 tensor cores: TMA-fed, accumulator in tensor
    memory, epilogue fused."""
    _need(a, "a", torch.bfloat16, contiguous=False)
    _need(w, "w", torch.bfloat16)
    _need(out, "out")
    m, k = a.shape
    n = w.shape[0]
    assert w.shape[1] == k and tuple(out.shape) == (m, n), (a.shape, w.shape, out.shape)
    if bias is not None:
        _need(bias, "bias", torch.float32)
        assert bias.numel() == n
    if residual is not None:
        _need(residual, "residual", torch.float32)
        assert tuple(residual.shape) == (m, n) and residual.stride(0) == out.stride(0)
    if status is None:
        status = default_status(a.device)
    check(library().mx_gemm_tcgen05(_ptr(a), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out),
                                    dtype_code(out.dtype), m, n, k, a.stride(0), w.stride(0),
                                    out.stride(0), mode, _ptr(status), _stream()), "gemm_tcgen05")
    _launched()


def gemm_tcgen05_force_tiles(rows: int) -> None:
    """Makes ``gemm_tcgen05`` use its 128-, 256- or 512-row kernel wherever the shape allows it; 0
    gives the choice back to the shape. For tests that run all three on the same product."""
    check(library().mx_gemm_tcgen05_force_tiles(int(rows)), "gemm_tcgen05_force_tiles")


_sm_counts: dict[int, int] = {}


def sm_count(device: torch.device) -> int:
    index = device.index if device.index is not None else torch.cuda.current_device()
    if index not in _sm_counts:
        _sm_counts[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return _sm_counts[index]


def stream_gemm_supported(a: torch.Tensor, w: torch.Tensor) -> bool:
    return (a.dtype == torch.bfloat16 and 0 < a.shape[0] <= 128 and a.shape[1] % 8 == 0 and a.stride(1) == 1
            and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_stream(a: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None,
                residual: torch.Tensor | None, out: torch.Tensor, mode: int,
                status: torch.Tensor | None = None) -> None:
    """The product for up to 128 rows (decoding, short prompt portions): the weight matrix is streamed
    from HBM once, dealt out evenly over the SMs, through TMA into tcgen05 products with the tokens
    as the narrow side; the epilogue is fused. A row's result does not depend on the other rows."""
    _need(a, "a", torch.bfloat16, contiguous=False)
    _need(w, "w", torch.bfloat16)
    _need(out, "out")
    m, k = a.shape
    n = w.shape[0]
    assert w.shape[1] == k and tuple(out.shape) == (m, n), (a.shape, w.shape, out.shape)
    if bias is not None:
        _need(bias, "bias", torch.float32)
        assert bias.numel() == n
    if residual is not None:
        _need(residual, "residual", torch.float32)
        assert tuple(residual.shape) == (m, n) and residual.stride(0) == out.stride(0)
    if status is None:
        status = default_status(a.device)
    check(library().mx_gemm_stream(_ptr(a), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out),
                                   dtype_code(out.dtype), m, n, k, a.stride(0), w.stride(0),
                                   out.stride(0), mode, _ptr(status), _stream()), "gemm_stream")
    _launched()


def skinny_gemm_supported(a: torch.Tensor, w: torch.Tensor) -> bool:
    return (a.dtype == torch.bfloat16 and a.shape[0] <= 16 and a.shape[1] % 32 == 0
            and a.stride(1) == 1 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_skinny(a: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None,
                residual: torch.Tensor | None, out: torch.Tensor, mode: int) -> None:
    """The decode product: at most 16 rows of bfloat16 ``a`` against all of ``w``, streamed once,
    with the epilogue fused."""
    _need(a, "a", torch.bfloat16, contiguous=False)
    _need(w, "w", torch.bfloat16)
    _need(out, "out")
    m, k = a.shape
    n = w.shape[0]
    assert w.shape[1] == k and tuple(out.shape) == (m, n), (a.shape, w.shape, out.shape)
    if bias is not None:
        _need(bias, "bias", torch.float32)
        assert bias.numel() == n
    if residual is not None:
        _need(residual, "residual", torch.float32)
        assert tuple(residual.shape) == (m, n) and residual.stride(0) == out.stride(0)
    check(library().mx_gemm_skinny(_ptr(a), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out),
                                   dtype_code(out.dtype), m, n, k, a.stride(0), w.stride(0),
                                   out.stride(0), mode, _stream()), "gemm_skinny")
    _launched()


def gemm_skinny_rope(a: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, qkv: torch.Tensor,
                     positions: torch.Tensor, inv_freq: torch.Tensor, slots: torch.Tensor | None,
                     cache: torch.Tensor | None, n_heads: int, n_kv_heads: int, head_dim: int,
                     page_size: int, status: torch.Tensor) -> None:
    """The decode QKV product with the rotation and the cache write in its epilogue: rotated
    queries go to the query columns of ``qkv``, rotated keys and the values to ``slots`` of
    ``cache`` (both None: nothing stored). The rotation spans the whole head."""
    _need(a, "a", torch.bfloat16, contiguous=False)
    _need(w, "w", torch.bfloat16)
    _need(qkv, "qkv", torch.bfloat16)
    _need(positions, "positions", torch.int32)
    _need(inv_freq, "inv_freq", torch.float32)
    _need(status, "status", torch.int32)
    m, k = a.shape
    n = (n_heads + 2 * n_kv_heads) * head_dim
    assert tuple(w.shape) == (n, k) and tuple(qkv.shape) == (m, n), (a.shape, w.shape, qkv.shape)
    assert inv_freq.numel() == head_dim // 2 and positions.numel() >= m
    if bias is not None:
        _need(bias, "bias", torch.float32)
        assert bias.numel() == n
    n_pages = 0
    if cache is not None:
        _need(cache, "cache", torch.bfloat16)
        _need(slots, "slots", torch.int32)
        assert tuple(cache.shape[1:]) == (2, n_kv_heads, page_size, head_dim), cache.shape
        n_pages = cache.shape[0]
    check(library().mx_gemm_skinny_rope(_ptr(a), _ptr(w), _ptr(bias), _ptr(qkv), m, k, a.stride(0),
                                        w.stride(0), qkv.stride(0), _ptr(positions), _ptr(inv_freq),
                                        _ptr(slots) if cache is not None else None, _ptr(cache), n_pages,
                                        n_heads, n_kv_heads, head_dim, page_size, _ptr(status), _stream()),
          "gemm_skinny_rope")
    _launched()


def _sink_ptr(sink: torch.Tensor | None, n_heads: int) -> int | None:
    if sink is None:
        return None
    _need(sink, "sink", torch.float32)
    assert sink.numel() == n_heads, (sink.shape, n_heads)
    return sink.data_ptr()


def attention_scratch_bytes(n_tokens: int, n_heads: int, head_dim: int, n_splits: int) -> int:
    return int(library().mx_attention_scratch_bytes(n_tokens, n_heads, head_dim, n_splits))


def paged_attention(q: torch.Tensor, q_stride: int, cache: torch.Tensor, block_tables: torch.Tensor,
                    tok_seq: torch.Tensor, positions: torch.Tensor, n_tokens: int, n_heads: int,
                    n_kv_heads: int, head_dim: int, window: int | None, scale: float,
                    out: torch.Tensor, status: torch.Tensor, n_splits: int = 1,
                    scratch: torch.Tensor | None = None, softcap: float | None = None,
                    sink: torch.Tensor | None = None, keep_first: int = 0) -> None:
    """Attention of ``n_tokens`` query rows over the paged cache.

    ``q`` points at the first query head of row 0 and rows are ``q_stride`` elements apart
    (so the q part of a fused qkv buffer can be used in place). ``out`` is [tokens, heads * dim].
    ``softcap``: scaled scores become ``softcap * tanh(score / softcap)``. ``sink`` (float32, one per
    head): ``exp(sink[h])`` joins the softmax's denominator and brings no value. ``keep_first``: with a
    window, the keys at positions below it stay visible at any distance.
    """
    _need(q, "q", contiguous=False)
    _need(cache, "cache", q.dtype)
    _need(block_tables, "block_tables", torch.int32)
    _need(tok_seq, "tok_seq", torch.int32)
    _need(positions, "positions", torch.int32)
    _need(out, "out", q.dtype)
    _need(status, "status", torch.int32)
    page_size = cache.shape[3]
    assert tuple(cache.shape[1:]) == (2, n_kv_heads, page_size, head_dim), cache.shape
    assert out.shape[1] == n_heads * head_dim and out.shape[0] >= n_tokens
    if n_splits > 1:
        need = attention_scratch_bytes(n_tokens, n_heads, head_dim, n_splits)
        if scratch is None or scratch.numel() * scratch.element_size() < need:
            raise KernelLibraryError(f"attention with {n_splits} splits needs {need} bytes of scratch")
        _need(scratch, "scratch", torch.float32)
    check(library().mx_paged_attention(
        _ptr(q), dtype_code(q.dtype), q_stride, _ptr(cache), cache.shape[0], page_size,
        _ptr(block_tables), block_tables.stride(0), _ptr(tok_seq), _ptr(positions), n_tokens,
        n_heads, n_kv_heads, head_dim, int(window or 0), float(scale), _ptr(out), out.stride(0),
        n_splits, _ptr(scratch), _ptr(status), float(softcap or 0.0), _sink_ptr(sink, n_heads), int(keep_first),
        _stream()), "paged_attention")
    _launched(2 if n_splits > 1 else 1)


def attention_tile_lists(q_lens: list[int], group: int,
                         token_tiles: bool = False) -> tuple[list[int], list[int]]:
    """Row tiles of the tensor-core attention for sequences that bring ``q_lens`` tokens and
    ``group`` query heads per KV head. Sequences with at most 16 rows (decode tokens) go to the
    narrow list, one (sequence, 0) tile each. The others go to the wide list: cut into 64-row
    tiles as (sequence, first row) pairs, or, with ``token_tiles`` (the tcgen05 kernel), into
    tiles of 128 // group tokens as (sequence, first token) pairs, the latest tokens first
    because they have the most keys to walk."""
    narrow: list[int] = []
    wide: list[int] = []
    per_tile = max(1, 128 // group)
    for seq, q_len in enumerate(q_lens):
        rows = q_len * group
        if rows <= 0:
            continue
        if rows <= 16:
            narrow.extend((seq, 0))
        elif token_tiles:
            for token in range((q_len - 1) // per_tile * per_tile, -1, -per_tile):
                wide.extend((seq, token))
        else:
            for row in range(0, rows, 64):
                wide.extend((seq, row))
    return narrow, wide


def tc_attention_supported(dtype: torch.dtype, head_dim: int, page_size: int, q_stride: int,
                           group: int) -> bool:
    """Whether prompt portions can run on the tcgen05 attention kernel."""
    return (dtype == torch.bfloat16 and head_dim == 128 and page_size in (16, 32)
            and q_stride % 8 == 0 and 1 <= group <= 128)


def paged_attention_tc(q: torch.Tensor, q_stride: int, cache: torch.Tensor, block_tables: torch.Tensor,
                       cu_q: torch.Tensor, context_lens: torch.Tensor, tiles: torch.Tensor, n_tiles: int,
                       n_tokens: int, n_heads: int, n_kv_heads: int, head_dim: int, window: int | None,
                       scale: float, out: torch.Tensor, status: torch.Tensor, n_splits: int = 1,
                       scratch: torch.Tensor | None = None, softcap: float | None = None,
                       sink: torch.Tensor | None = None, keep_first: int = 0) -> None:
    """Attention of prompt portions on tcgen05 (bfloat16, head_dim 128, pages of 16 or 32). Under a window the
    sequence's first ``keep_first`` keys stay visible.
    ``tiles`` is int32 [n_tiles, 2]: (sequence, first token) of tiles of 128 // group tokens
    (``attention_tile_lists(..., token_tiles=True)``); ``q`` holds the step's rows, query head h
    at column h * head_dim. ``n_splits`` > 1 shares every tile's keys out between that many blocks
    (few tiles, long contexts); ``scratch`` (float32, ``attention_scratch_bytes``) takes their parts."""
    _need(q, "q", torch.bfloat16, contiguous=False)
    _need(cache, "cache", torch.bfloat16)
    for name, tensor in (("block_tables", block_tables), ("cu_q", cu_q),
                         ("context_lens", context_lens), ("tiles", tiles), ("status", status)):
        _need(tensor, name, torch.int32)
    _need(out, "out", torch.bfloat16)
    page_size = cache.shape[3]
    assert tuple(cache.shape[1:]) == (2, n_kv_heads, page_size, head_dim), cache.shape
    assert out.shape[1] == n_heads * head_dim and out.shape[0] >= n_tokens and q.shape[0] >= n_tokens
    assert tiles.numel() >= 2 * n_tiles
    if n_splits > 1:
        _need(scratch, "scratch", torch.float32)
        assert scratch.numel() * 4 >= attention_scratch_bytes(n_tokens, n_heads, head_dim, n_splits)
    check(library().mx_paged_attention_tc_split(
        _ptr(q), q_stride, _ptr(cache), cache.shape[0], page_size, _ptr(block_tables),
        block_tables.stride(0), _ptr(cu_q), _ptr(context_lens), _ptr(tiles), n_tiles, n_tokens,
        n_heads, n_kv_heads, head_dim, int(window or 0), float(scale), _ptr(out), out.stride(0),
        int(n_splits), _ptr(scratch) if n_splits > 1 else None, _ptr(status), float(softcap or 0.0),
        _sink_ptr(sink, n_heads), int(keep_first) if window else 0, _stream()), "paged_attention_tc")
    _launched()


def paged_attention_mma(q: torch.Tensor, q_stride: int, cache: torch.Tensor,
                        block_tables: torch.Tensor, cu_q: torch.Tensor, context_lens: torch.Tensor,
                        tiles: torch.Tensor, n_tiles: int, narrow: bool, n_tokens: int, n_heads: int,
                        n_kv_heads: int, head_dim: int, window: int | None, scale: float,
                        out: torch.Tensor, status: torch.Tensor, n_splits: int = 1,
                        scratch: torch.Tensor | None = None, softcap: float | None = None,
                        sink: torch.Tensor | None = None, keep_first: int = 0) -> None:
    """Tensor-core attention (bfloat16, head_dim 64 or 128). ``tiles`` is int32 [n_tiles, 2]:
    (sequence, first row) of each tile of the (token, head-in-group) rows; ``narrow`` tiles
    hold at most 16 rows, the others 64 (see ``attention_tile_lists``)."""
    _need(q, "q", torch.bfloat16, contiguous=False)
    _need(cache, "cache", torch.bfloat16)
    for name, tensor in (("block_tables", block_tables), ("cu_q", cu_q),
                         ("context_lens", context_lens), ("status", status)):
        _need(tensor, name, torch.int32)
    _need(out, "out", torch.bfloat16)
    page_size = cache.shape[3]
    assert tuple(cache.shape[1:]) == (2, n_kv_heads, page_size, head_dim), cache.shape
    assert out.shape[1] == n_heads * head_dim and out.shape[0] >= n_tokens
    if tiles is None:
        # no list: tile i is the whole of sequence i (narrow tiles only: every sequence brings at most 16 rows)
        assert narrow and n_tiles <= context_lens.numel()
    else:
        _need(tiles, "tiles", torch.int32)
        assert tiles.numel() >= 2 * n_tiles
    if n_splits > 1:
        need = attention_scratch_bytes(n_tokens, n_heads, head_dim, n_splits)
        if scratch is None or scratch.numel() * scratch.element_size() < need:
            raise KernelLibraryError(f"attention with {n_splits} splits needs {need} bytes of scratch")
        _need(scratch, "scratch", torch.float32)
    check(library().mx_paged_attention_mma(
        _ptr(q), q_stride, _ptr(cache), cache.shape[0], page_size, _ptr(block_tables),
        block_tables.stride(0), _ptr(cu_q), _ptr(context_lens), _ptr(tiles) if tiles is not None else None, n_tiles,
        1 if narrow else 0, n_tokens, n_heads, n_kv_heads, head_dim, int(window or 0), float(scale),
        _ptr(out), out.stride(0), n_splits, _ptr(scratch), _ptr(status), float(softcap or 0.0),
        _sink_ptr(sink, n_heads), int(keep_first), _stream()), "paged_attention_mma")
    _launched(2 if n_splits > 1 else 1)


def mma_attention_supported(dtype: torch.dtype, head_dim: int, page_size: int, q_stride: int) -> bool:
    return (dtype == torch.bfloat16 and head_dim in (64, 128) and page_size in (8, 16, 32)
            and q_stride % 8 == 0)


# ---------------------------------------------------------------------- RMS norm, post-norm sums
def rmsnorm(x: torch.Tensor, weight: torch.Tensor, offset: float, eps: float, out: torch.Tensor,
            rows: torch.Tensor | None = None) -> None:
    """out[r] = x[row] / sqrt(mean(x[row]^2) + eps) * (offset + weight), row = rows[r] if given else r. ``x`` may be
    the first columns of wider rows (a view with a row stride)."""
    _need(x, "x", torch.float32, contiguous=False)
    assert x.stride(1) == 1
    _need(weight, "weight", torch.float32)
    _need(out, "out")
    if rows is not None:
        _need(rows, "rows", torch.int32)
    n_rows, hidden = out.shape
    assert x.shape[1] >= hidden and weight.numel() == hidden
    assert (rows.numel() if rows is not None else x.shape[0]) == n_rows
    check(library().mx_rmsnorm(_ptr(x), _ptr(rows), _ptr(weight), float(offset), _ptr(out),
                               dtype_code(out.dtype), n_rows, hidden, float(eps), x.stride(0), _stream()), "rmsnorm")
    _launched()


def rmsnorm_sum(x: torch.Tensor, acc: torch.Tensor, alpha: float, weight: torch.Tensor, offset: float,
                eps: float, act: torch.Tensor | None = None) -> None:
    """``x <- unit(alpha * x + acc) * (offset + weight)`` in place (float32); ``act``, when given, gets the
    same rows in its own dtype."""
    _need(x, "x", torch.float32)
    _need(acc, "acc", torch.float32)
    _need(weight, "weight", torch.float32)
    assert acc.shape == x.shape and weight.numel() == x.shape[1]
    if act is not None:
        _need(act, "act")
        assert act.shape == x.shape
    check(library().mx_rmsnorm_sum(_ptr(x), _ptr(acc), float(alpha), _ptr(weight), float(offset), _ptr(act),
                                   dtype_code(act.dtype) if act is not None else F32, x.shape[0], x.shape[1],
                                   float(eps), _stream()), "rmsnorm_sum")
    _launched()


def rmsnorm_branch_add(x: torch.Tensor, branch: torch.Tensor, branch_weight: torch.Tensor,
                       next_weight: torch.Tensor | None, out: torch.Tensor | None, eps: float) -> None:
    """``x <- x + unit(branch) * branch_weight`` in place (float32, ``unit(v) = v / sqrt(mean(v^2) + eps)``); then
    ``out`` (any activation dtype, or None) gets ``unit(x) * next_weight``, or the new ``x`` itself when
    ``next_weight`` is None."""
    _need(x, "x", torch.float32)
    _need(branch, "branch", torch.float32)
    _need(branch_weight, "branch_weight", torch.float32)
    n, hidden = x.shape
    assert tuple(branch.shape) == (n, hidden) and branch_weight.numel() == hidden
    if next_weight is not None:
        _need(next_weight, "next_weight", torch.float32)
        assert next_weight.numel() == hidden and out is not None
    if out is not None:
        _need(out, "out")
        assert tuple(out.shape) == (n, hidden)
    check(library().mx_rmsnorm_branch_add(_ptr(x), _ptr(branch), _ptr(branch_weight), _ptr(next_weight), _ptr(out),
                                          dtype_code(out.dtype) if out is not None else F32, n, hidden, float(eps),
                                          _stream()), "rmsnorm_branch_add")
    _launched()


def cast_rows(x: torch.Tensor, out: torch.Tensor) -> None:
    """out (bfloat16) = x (float32), element by element."""
    _need(x, "x", torch.float32)
    _need(out, "out", torch.bfloat16)
    assert out.numel() == x.numel()
    check(library().mx_cast_rows(_ptr(x), _ptr(out), x.numel(), _stream()), "cast_rows")
    _launched()


# ---------------------------------------------------------------------- batched products
def gemm_batched_simt(a: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, out: torch.Tensor) -> None:
    """``out[:, b] = a[:, b] @ w[b].T (+ bias[b])`` for every b on the FP32 cores: a [M, B, K] and out
    [M, B, N] may be views with any row and batch strides (unit stride along K and N), w [B, N, K],
    bias float32 [B, N]. ``out`` is in the dtype of ``a`` or float32."""
    _need(a, "a", contiguous=False)
    _need(w, "w", a.dtype)
    _need(out, "out", contiguous=False)
    m, batch, k = a.shape
    n = w.shape[1]
    assert tuple(w.shape) == (batch, n, k) and tuple(out.shape) == (m, batch, n), (a.shape, w.shape, out.shape)
    if a.stride(2) != 1 or out.stride(2) != 1:
        raise KernelLibraryError("batched operands must have unit stride along their last axis")
    if out.dtype not in (a.dtype, torch.float32):
        raise KernelLibraryError(f"a batched product of {a.dtype} writes {a.dtype} or float32, not {out.dtype}")
    if bias is not None:
        _need(bias, "bias", torch.float32)
        assert tuple(bias.shape) == (batch, n)
    mode = EPILOGUE_F32 if out.dtype == torch.float32 and a.dtype != torch.float32 else EPILOGUE_NONE
    check(library().mx_gemm_batched_simt(_ptr(a), _ptr(w), dtype_code(a.dtype), _ptr(bias), _ptr(out),
                                         dtype_code(out.dtype), m, n, k, a.stride(0), w.stride(1), out.stride(0),
                                         batch, a.stride(1), w.stride(0), out.stride(1), n, mode, _stream()),
          "gemm_batched_simt")
    _launched()


def batched_skinny_supported(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
    return (a.dtype == torch.bfloat16 and a.shape[0] <= 16 and a.shape[2] % 8 == 0 and a.stride(2) == 1
            and a.stride(0) % 8 == 0 and a.stride(1) % 8 == 0 and w.is_contiguous() and out.stride(2) == 1
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_batched_skinny(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """``gemm_batched_simt`` without a bias for at most 16 rows of bfloat16: a warp per output column, the
    weights read once with 16-byte loads."""
    _need(a, "a", torch.bfloat16, contiguous=False)
    _need(w, "w", torch.bfloat16)
    _need(out, "out", contiguous=False)
    m, batch, k = a.shape
    n = w.shape[1]
    assert tuple(w.shape) == (batch, n, k) and tuple(out.shape) == (m, batch, n), (a.shape, w.shape, out.shape)
    if out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelLibraryError(f"a batched product writes bfloat16 or float32, not {out.dtype}")
    check(library().mx_gemm_batched_skinny(_ptr(a), _ptr(w), _ptr(out), dtype_code(out.dtype), m, n, k, a.stride(0),
                                           w.stride(1), out.stride(0), batch, a.stride(1), w.stride(0),
                                           out.stride(1), _stream()), "gemm_batched_skinny")
    _launched()


# ---------------------------------------------------------------------- latent attention
def latent_prepare(proj: torch.Tensor, positions: torch.Tensor, freq: torch.Tensor, amplitude: float,
                   latent_weight: torch.Tensor, eps: float, slots: torch.Tensor | None,
                   cache: torch.Tensor | None, q_plain: torch.Tensor, q_lat: torch.Tensor, n_heads: int,
                   dim: int, rot: int, rot_dims: int, rank: int, status: torch.Tensor,
                   down: torch.Tensor | None = None, interleaved: bool = False) -> None:
    """From the float rows ``[heads x (dim | rot) | rank | rot]`` of the fused query / down projection:
    the plain query parts, the rotated query parts (at offset ``rank`` of each head of ``q_lat``) and the
    token's cache vector ``[unit(latent) * latent_weight | rotated shared part]`` at ``slots``.
    ``cache`` is [pages, 1, 1, page_size, rank + rot]; None stores nothing. ``down`` (float rows ``[rank | rot]``,
    rows may be strided): the latent and the shared part come from there and ``proj`` holds the query heads only.
    ``interleaved`` pairs entry 2i with 2i + 1 in the rotation instead of i with i + rot_dims/2."""
    _need(proj, "proj", torch.float32, contiguous=False)
    if down is not None:
        _need(down, "down", torch.float32, contiguous=False)
        assert down.stride(1) == 1 and down.shape[0] >= proj.shape[0] and down.shape[1] >= rank + rot
    assert proj.stride(1) == 1
    _need(positions, "positions", torch.int32)
    _need(freq, "freq", torch.float32)
    _need(latent_weight, "latent_weight", torch.float32)
    _need(q_plain, "q_plain")
    _need(q_lat, "q_lat", q_plain.dtype)
    n = proj.shape[0]
    assert freq.numel() == rot_dims // 2 and latent_weight.numel() == rank
    assert tuple(q_plain.shape) == (n, n_heads * dim) and tuple(q_lat.shape) == (n, n_heads, rank + rot)
    n_pages = page_size = 0
    if cache is not None:
        _need(cache, "cache", q_plain.dtype)
        _need(slots, "slots", torch.int32)
        assert tuple(cache.shape[1:3]) == (1, 1) and cache.shape[4] == rank + rot, cache.shape
        n_pages, page_size = cache.shape[0], cache.shape[3]
    check(library().mx_latent_prepare(_ptr(proj), proj.stride(0), _ptr(down), down.stride(0) if down is not None else 0,
                                      1 if interleaved else 0, _ptr(positions), _ptr(freq), float(amplitude),
                                      _ptr(latent_weight), float(eps), _ptr(slots), _ptr(cache), n_pages,
                                      page_size, _ptr(q_plain), _ptr(q_lat), dtype_code(q_plain.dtype), n,
                                      n_heads, dim, rot, rot_dims, rank, _ptr(status), _stream()),
          "latent_prepare")
    _launched()


def latent_attention(q_lat: torch.Tensor, cache: torch.Tensor, block_tables: torch.Tensor,
                     tok_seq: torch.Tensor, positions: torch.Tensor, rank: int, window: int | None,
                     scale: float, out: torch.Tensor, status: torch.Tensor, sink: torch.Tensor | None = None) -> None:
    """Attention of ``q_lat`` [tokens, heads, dk] over the one-vector-per-token cache
    [pages, 1, 1, page_size, dk]; ``out`` [tokens, heads, rank] is the softmax-weighted sum of the first
    ``rank`` elements of the visible vectors. ``sink`` (float32, one logit per head) joins the denominator."""
    _need(q_lat, "q_lat")
    _need(cache, "cache", q_lat.dtype)
    _need(out, "out", q_lat.dtype)
    for name, tensor in (("block_tables", block_tables), ("tok_seq", tok_seq), ("positions", positions),
                         ("status", status)):
        _need(tensor, name, torch.int32)
    n, n_heads, dk = q_lat.shape
    assert tuple(cache.shape[1:3]) == (1, 1) and cache.shape[4] == dk, cache.shape
    assert tuple(out.shape) == (n, n_heads, rank)
    check(library().mx_latent_attention(_ptr(q_lat), _ptr(cache), dtype_code(q_lat.dtype), cache.shape[0],
                                        cache.shape[3], _ptr(block_tables), block_tables.stride(0),
                                        _ptr(tok_seq), _ptr(positions), n, n_heads, rank, dk, int(window or 0),
                                        float(scale), _ptr(out), _sink_ptr(sink, n_heads), _ptr(status), _stream()),
          "latent_attention")
    _launched()


def latent_attention_mma_supported(dtype: torch.dtype, rank: int, dk: int) -> bool:
    """Whether the tensor-core latent attention takes this geometry (bfloat16, rank a multiple of 32 up to
    512, key width a multiple of 16 that fits in shared memory)."""
    return dtype == torch.bfloat16 and bool(library().mx_latent_attention_mma_supported(rank, dk))


def latent_tile_list(q_lens: list[int], n_heads: int) -> list[int]:
    """(sequence, first row) of the 64-row tiles of the (token, head) rows of sequences that bring
    ``q_lens`` tokens, flattened; the tiles of a sequence's latest tokens first (they walk the most keys)."""
    tiles: list[int] = []
    for seq, q_len in enumerate(q_lens):
        rows = q_len * n_heads
        for row in range((rows - 1) // 64 * 64, -1, -64):
            tiles.extend((seq, row))
    return tiles


def latent_attention_mma(q_lat: torch.Tensor, cache: torch.Tensor, block_tables: torch.Tensor,
                         cu_q: torch.Tensor, context_lens: torch.Tensor, tiles: torch.Tensor | None,
                         n_tiles: int, rank: int, window: int | None, scale: float, out: torch.Tensor,
                         status: torch.Tensor, n_splits: int = 1, scratch: torch.Tensor | None = None,
                         few_rows: bool = False, sink: torch.Tensor | None = None) -> None:
    """``latent_attention`` on the tensor cores (bfloat16). ``few_rows``: the caller vouches that every
    sequence brings at most 16 (token, head) rows, which lets the kernel keep more keys in flight. ``tiles`` is int32 [n_tiles, 2] from
    ``latent_tile_list``; None means that tile i is sequence i (a fixed-size batch of decoding requests,
    ``n_tiles`` sequences). ``n_splits`` > 1 shares every tile's keys out between that many blocks;
    ``scratch`` (float32, ``attention_scratch_bytes(tokens, heads, rank, n_splits)``) takes their parts."""
    _need(q_lat, "q_lat", torch.bfloat16)
    _need(cache, "cache", torch.bfloat16)
    _need(out, "out", torch.bfloat16)
    for name, tensor in (("block_tables", block_tables), ("cu_q", cu_q), ("context_lens", context_lens),
                         ("status", status)):
        _need(tensor, name, torch.int32)
    n, n_heads, dk = q_lat.shape
    assert tuple(cache.shape[1:3]) == (1, 1) and cache.shape[4] == dk, cache.shape
    assert tuple(out.shape) == (n, n_heads, rank)
    if tiles is not None:
        _need(tiles, "tiles", torch.int32)
        assert tiles.numel() >= 2 * n_tiles
    else:
        assert n_tiles <= context_lens.numel()
    if n_splits > 1:
        need = attention_scratch_bytes(n, n_heads, rank, n_splits)
        if scratch is None or scratch.numel() * scratch.element_size() < need:
            raise KernelLibraryError(f"latent attention with {n_splits} splits needs {need} bytes of scratch")
        _need(scratch, "scratch", torch.float32)
    check(library().mx_latent_attention_mma(
        _ptr(q_lat), _ptr(cache), cache.shape[0], cache.shape[3], _ptr(block_tables), block_tables.stride(0),
        _ptr(cu_q), _ptr(context_lens), _ptr(tiles), n_tiles, (n_heads + 63) // 64, n, n_heads, rank, dk,
        int(window or 0), float(scale), _ptr(out), int(n_splits), _ptr(scratch) if n_splits > 1 else None,
        1 if few_rows else 0, _sink_ptr(sink, n_heads), _ptr(status), _stream()), "latent_attention_mma")
    _launched(2 if n_splits > 1 else 1)


# ---------------------------------------------------------------------- normalised, gated attention
def qk_norm_kv_write(proj: torch.Tensor, q_weight: torch.Tensor | None, k_weight: torch.Tensor | None,
                     eps: float, slots: torch.Tensor | None, cache: torch.Tensor | None, q_out: torch.Tensor,
                     n_heads: int, n_kv_heads: int, dim: int, vdim: int, status: torch.Tensor) -> None:
    """From the float rows ``[heads x dim | kv heads x dim | kv heads x vdim | ...]`` of a fused projection:
    per-head RMS-normalised queries to ``q_out`` [tokens, heads * hd] and normalised keys and plain values
    to ``slots`` of ``cache`` [pages, 2, kv heads, page_size, hd]; hd >= dim, vdim, tails are zero."""
    _need(proj, "proj", torch.float32)
    _need(q_out, "q_out")
    n = proj.shape[0]
    hd = q_out.shape[1] // n_heads
    assert tuple(q_out.shape) == (n, n_heads * hd)
    for weight in (q_weight, k_weight):
        if weight is not None:
            _need(weight, "norm weight", torch.float32)
            assert weight.numel() == dim
    n_pages = page_size = 0
    if cache is not None:
        _need(cache, "cache", q_out.dtype)
        _need(slots, "slots", torch.int32)
        assert tuple(cache.shape[1:3]) == (2, n_kv_heads) and cache.shape[4] == hd, cache.shape
        n_pages, page_size = cache.shape[0], cache.shape[3]
    check(library().mx_qk_norm_kv_write(_ptr(proj), proj.stride(0), _ptr(q_weight), _ptr(k_weight), float(eps),
                                        _ptr(slots), _ptr(cache), n_pages, page_size, _ptr(q_out),
                                        dtype_code(q_out.dtype), n, n_heads, n_kv_heads, dim, vdim, hd,
                                        _ptr(status), _stream()), "qk_norm_kv_write")
    _launched()


def sigmoid_gate(attn: torch.Tensor, gate: torch.Tensor, out: torch.Tensor, n_heads: int, vdim: int) -> None:
    """out[t, h * vdim + e] = attn[t, h * hd + e] * sigmoid(gate[t, h * vdim + e]); ``gate`` is a float32
    view with any row stride."""
    _need(attn, "attn")
    _need(gate, "gate", torch.float32, contiguous=False)
    _need(out, "out", attn.dtype)
    n = attn.shape[0]
    hd = attn.shape[1] // n_heads
    assert tuple(out.shape) == (n, n_heads * vdim) and tuple(gate.shape) == (n, n_heads * vdim)
    assert gate.stride(1) == 1
    check(library().mx_sigmoid_gate(_ptr(attn), _ptr(gate), gate.stride(0), _ptr(out), dtype_code(attn.dtype), n,
                                    n_heads, vdim, hd, _stream()), "sigmoid_gate")
    _launched()


def clamped_glu(gate_up: torch.Tensor, out: torch.Tensor, limit: float, slope: float, shift: float) -> None:
    """Rows ``[gate | up]`` -> ``min(gate, limit) * sigmoid(slope * min(gate, limit)) * (clamp(up) + shift)``."""
    _need(gate_up, "gate_up")
    _need(out, "out", gate_up.dtype)
    n, ff = out.shape
    assert tuple(gate_up.shape) == (n, 2 * ff)
    check(library().mx_clamped_glu(_ptr(gate_up), gate_up.stride(0), _ptr(out), dtype_code(out.dtype), n, ff,
                                   float(limit), float(slope), float(shift), _stream()), "clamped_glu")
    _launched()


# ---------------------------------------------------------------------- gated linear recurrence
def causal_conv(xy: torch.Tensor, x_col: int, conv_weight: torch.Tensor, conv_bias: torch.Tensor | None,
                state: torch.Tensor, tok_seq: torch.Tensor, cu_q: torch.Tensor, state_slots: torch.Tensor,
                u: torch.Tensor, u_act: torch.Tensor | None) -> None:
    """The per-channel causal convolution of columns ``x_col ..`` of ``xy`` (float32), continuing from the
    inputs kept in ``state`` [slots, taps, width]; ``u`` float32, ``u_act`` an optional rounded copy."""
    _need(xy, "xy", torch.float32)
    _need(conv_weight, "conv_weight", torch.float32)
    _need(state, "state", torch.float32)
    _need(u, "u", torch.float32)
    n, width = u.shape
    taps = conv_weight.shape[1]
    assert tuple(conv_weight.shape) == (width, taps) and tuple(state.shape[1:]) == (taps, width)
    if u_act is not None:
        _need(u_act, "u_act")
        assert u_act.shape == u.shape
    check(library().mx_causal_conv(_ptr(xy), xy.stride(0), x_col, _ptr(conv_weight), _ptr(conv_bias), _ptr(state),
                                   _ptr(tok_seq), _ptr(cu_q), _ptr(state_slots), _ptr(u), _ptr(u_act),
                                   dtype_code(u_act.dtype) if u_act is not None else F32, n, width, taps,
                                   _stream()), "causal_conv")
    _launched()


def rglru_scan(xy: torch.Tensor, x_col: int, y_col: int, u: torch.Tensor, gates: torch.Tensor,
               gate_bias: torch.Tensor | None, lam: torch.Tensor, decay: float, state: torch.Tensor,
               cu_q: torch.Tensor, state_slots: torch.Tensor, n_seqs: int, block_width: int,
               out: torch.Tensor) -> None:
    """The gated recurrence over every sequence's tokens in order, from and to ``state``; ``gates`` is
    float32 [tokens, blocks, 2 * block_width] (recurrence gate, then input gate, before their sigmoids and,
    when ``gate_bias`` [blocks, 2 * block_width] is given, before their biases)."""
    for name, tensor in (("xy", xy), ("u", u), ("gates", gates), ("lambda", lam), ("state", state)):
        _need(tensor, name, torch.float32)
    if gate_bias is not None:
        _need(gate_bias, "gate_bias", torch.float32)
        assert gate_bias.numel() == 2 * u.shape[1]
    _need(out, "out")
    n, width = u.shape
    taps = state.shape[1]
    assert gates.numel() == n * 2 * width and tuple(out.shape) == (n, width) and lam.numel() == width
    check(library().mx_rglru_scan(_ptr(xy), xy.stride(0), x_col, y_col, _ptr(u), _ptr(gates), _ptr(gate_bias), _ptr(lam),
                                  float(decay), _ptr(state), _ptr(cu_q), _ptr(state_slots), _ptr(out),
                                  dtype_code(out.dtype), n_seqs, width, block_width, taps, _stream()),
          "rglru_scan")
    _launched()


SCAN_CHUNK = 32     # tokens per chunk of the three-launch recurrence


def scan_chunk_lists(q_lens: list[int]) -> tuple[list[int], list[int]]:
    """For ``rglru_scan_chunked``: (sequence, first token) of every chunk of ``SCAN_CHUNK`` tokens,
    flattened, sequence by sequence, and the index of each sequence's first chunk (one more entry than
    sequences)."""
    chunks: list[int] = []
    first = [0]
    for seq, q_len in enumerate(q_lens):
        for start in range(0, q_len, SCAN_CHUNK):
            chunks.extend((seq, start))
        first.append(len(chunks) // 2)
    return chunks, first


def rglru_scan_chunked(xy: torch.Tensor, x_col: int, y_col: int, u: torch.Tensor, gates: torch.Tensor,
                       gate_bias: torch.Tensor | None, lam: torch.Tensor, decay: float, state: torch.Tensor,
                       cu_q: torch.Tensor, state_slots: torch.Tensor, n_seqs: int, block_width: int,
                       chunks: torch.Tensor, seq_chunk0: torch.Tensor, n_chunks: int, scratch: torch.Tensor,
                       out: torch.Tensor) -> None:
    """``rglru_scan`` for long portions: chunk maps, the chunks' start states in order, then the tokens
    (three launches, every token of every chunk in parallel). ``chunks`` / ``seq_chunk0`` are
    ``scan_chunk_lists`` on the device; ``scratch`` is float32 with 3 * n_chunks * width elements."""
    for name, tensor in (("xy", xy), ("u", u), ("gates", gates), ("lambda", lam), ("state", state),
                         ("scratch", scratch)):
        _need(tensor, name, torch.float32)
    _need(chunks, "chunks", torch.int32)
    _need(seq_chunk0, "seq_chunk0", torch.int32)
    _need(out, "out")
    n, width = u.shape
    taps = state.shape[1]
    assert gates.numel() == n * 2 * width and tuple(out.shape) == (n, width) and lam.numel() == width
    assert chunks.numel() >= 2 * n_chunks and seq_chunk0.numel() >= n_seqs + 1
    assert scratch.numel() >= 3 * n_chunks * width
    check(library().mx_rglru_scan_chunked(_ptr(xy), xy.stride(0), x_col, y_col, _ptr(u), _ptr(gates),
                                          _ptr(gate_bias), _ptr(lam), float(decay), _ptr(state), _ptr(cu_q),
                                          _ptr(state_slots), _ptr(chunks), _ptr(seq_chunk0), n_chunks, SCAN_CHUNK,
                                          _ptr(scratch), _ptr(out), dtype_code(out.dtype), n_seqs, width,
                                          block_width, taps, _stream()), "rglru_scan_chunked")
    _launched(3)


# ---------------------------------------------------------------------- dynamic tanh
def dyt(x: torch.Tensor, weight: torch.Tensor, shift: torch.Tensor | None, alpha: torch.Tensor, out: torch.Tensor,
        rows: torch.Tensor | None = None, acc: torch.Tensor | None = None,
        col_bias: torch.Tensor | None = None) -> None:
    """out[r] = tanh(alpha * x[row]) * weight + shift, row = rows[r] if given else r; ``alpha`` is a float32
    scalar on the device. With ``acc`` (float32, the shape of x): ``x += acc + col_bias`` first, written back."""
    _need(x, "x", torch.float32)
    _need(weight, "weight", torch.float32)
    _need(alpha, "alpha", torch.float32)
    _need(out, "out")
    n_rows, hidden = out.shape
    assert x.shape[1] == hidden and weight.numel() == hidden and alpha.numel() == 1
    assert (rows.numel() if rows is not None else x.shape[0]) == n_rows
    if shift is not None:
        _need(shift, "shift", torch.float32)
        assert shift.numel() == hidden
    if rows is not None:
        _need(rows, "rows", torch.int32)
    if acc is not None:
        _need(acc, "acc", torch.float32)
        assert acc.shape == x.shape and rows is None
        if col_bias is not None:
            _need(col_bias, "col_bias", torch.float32)
    check(library().mx_dyt(_ptr(x), _ptr(rows), _ptr(acc), _ptr(col_bias) if acc is not None else None, _ptr(weight),
                           _ptr(shift), _ptr(alpha), _ptr(out), dtype_code(out.dtype), n_rows, hidden, _stream()), "dyt")
    _launched()


# ---------------------------------------------------------------------- partly rotated, blended, head-gated attention
def rotate_mix_kv_write(proj: torch.Tensor, positions: torch.Tensor, freq: torch.Tensor, rot: int,
                        other: torch.Tensor | None, mix: torch.Tensor | None, slots: torch.Tensor | None,
                        cache: torch.Tensor | None, q_out: torch.Tensor, n_heads: int, n_kv_heads: int, dim: int,
                        vdim: int, status: torch.Tensor) -> None:
    """From the float rows ``[heads x dim | kv heads x dim | kv heads x vdim | ...]`` of a fused projection: queries
    with their first ``rot`` entries rotated (pairs (i, i + rot/2), angle ``position * freq[i]``) to ``q_out``
    [tokens, heads * hd], keys rotated the same way and values to ``slots`` of ``cache``
    [pages, 2, kv heads, page_size, hd]; hd >= dim, vdim, tails are zero. ``other`` (a float32 view
    [tokens, kv heads * vdim], any row stride) and ``mix`` (a float32 scalar on the device): the stored values are
    ``(1 - mix) * v + mix * other``."""
    _need(proj, "proj", torch.float32)
    _need(positions, "positions", torch.int32)
    _need(freq, "freq", torch.float32)
    _need(q_out, "q_out")
    n = proj.shape[0]
    hd = q_out.shape[1] // n_heads
    assert tuple(q_out.shape) == (n, n_heads * hd) and freq.numel() == rot // 2
    other_ld = 0
    if other is not None:
        _need(other, "other", torch.float32, contiguous=False)
        _need(mix, "mix", torch.float32)
        assert tuple(other.shape) == (n, n_kv_heads * vdim) and other.stride(1) == 1 and mix.numel() == 1
        other_ld = other.stride(0)
    n_pages = page_size = 0
    if cache is not None:
        _need(cache, "cache", q_out.dtype)
        _need(slots, "slots", torch.int32)
        assert tuple(cache.shape[1:3]) == (2, n_kv_heads) and cache.shape[4] == hd, cache.shape
        n_pages, page_size = cache.shape[0], cache.shape[3]
    check(library().mx_rotate_mix_kv_write(_ptr(proj), proj.stride(0), _ptr(positions), _ptr(freq), rot, _ptr(other),
                                           other_ld, _ptr(mix) if other is not None else None, _ptr(slots), _ptr(cache),
                                           n_pages, page_size, _ptr(q_out), dtype_code(q_out.dtype), n, n_heads,
                                           n_kv_heads, dim, vdim, hd, _ptr(status), _stream()), "rotate_mix_kv_write")
    _launched()


def head_gate(attn: torch.Tensor, gate: torch.Tensor, out: torch.Tensor, n_heads: int, vdim: int) -> None:
    """out[t, h * vdim + e] = attn[t, h * hd + e] * sigmoid(gate[t, h]); ``gate`` is a float32 view [tokens, heads]
    with any row stride."""
    _need(attn, "attn")
    _need(gate, "gate", torch.float32, contiguous=False)
    _need(out, "out", attn.dtype)
    n = attn.shape[0]
    hd = attn.shape[1] // n_heads
    assert tuple(out.shape) == (n, n_heads * vdim) and tuple(gate.shape) == (n, n_heads) and gate.stride(1) == 1
    check(library().mx_head_gate(_ptr(attn), _ptr(gate), gate.stride(0), _ptr(out), dtype_code(attn.dtype), n, n_heads,
                                 vdim, hd, _stream()), "head_gate")
    _launched()


# ---------------------------------------------------------------------- gated linear attention
def gla_decay(low: torch.Tensor, a2: torch.Tensor, bias: torch.Tensor | None, tau: float, decay: torch.Tensor) -> None:
    """decay[t, c] = sigmoid(a2[c] . low[t] + bias[c]) ** (1 / tau), all float32; ``low`` [tokens, rank] may be a
    column range of wider rows."""
    _need(low, "low", torch.float32, contiguous=False)
    _need(a2, "a2", torch.float32)
    _need(decay, "decay", torch.float32)
    n, rank = low.shape
    channels = a2.shape[0]
    assert tuple(a2.shape) == (channels, rank) and tuple(decay.shape) == (n, channels) and low.stride(1) == 1
    if bias is not None:
        _need(bias, "bias", torch.float32)
        assert bias.numel() == channels
    check(library().mx_gla_decay(_ptr(low), low.stride(0), _ptr(a2), _ptr(bias), float(tau), _ptr(decay), n, channels,
                                 rank, _stream()), "gla_decay")
    _launched()


def gla_scan(proj: torch.Tensor, q_col: int, k_col: int, v_col: int, decay: torch.Tensor, q_scale: float,
             state: torch.Tensor, cu_q: torch.Tensor, state_slots: torch.Tensor, n_seqs: int, out: torch.Tensor,
             n_heads: int, dim: int, vdim: int) -> None:
    """``S <- diag(decay_t) S + k_t v_t^T; out_t = S^T (q_scale * q_t)`` over every sequence's tokens in order, from
    and to ``state`` [slots, heads, dim, vdim] (float32); q, k and v are column ranges of the float rows ``proj``."""
    for name, tensor in (("proj", proj), ("decay", decay), ("state", state), ("out", out)):
        _need(tensor, name, torch.float32)
    n = proj.shape[0]
    assert tuple(state.shape[1:]) == (n_heads, dim, vdim), state.shape
    assert tuple(decay.shape) == (n, n_heads * dim) and tuple(out.shape) == (n, n_heads * vdim)
    check(library().mx_gla_scan(_ptr(proj), proj.stride(0), q_col, k_col, v_col, _ptr(decay), float(q_scale),
                                _ptr(state), _ptr(cu_q), _ptr(state_slots), _ptr(out), n_seqs, n_heads, dim, vdim,
                                _stream()), "gla_scan")
    _launched()


def gla_norm_gate(o: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
                  n_heads: int, vdim: int) -> None:
    """out[t, h, e] = unit(o[t, h])[e] * weight[e] * silu(gate[t, h, e]); unit is the RMS norm over one head's
    ``vdim`` entries with eps inside the root; ``gate`` a float32 view with any row stride."""
    _need(o, "o", torch.float32)
    _need(gate, "gate", torch.float32, contiguous=False)
    _need(weight, "weight", torch.float32)
    _need(out, "out")
    n = o.shape[0]
    assert tuple(o.shape) == (n, n_heads * vdim) and tuple(gate.shape) == (n, n_heads * vdim) and gate.stride(1) == 1
    assert tuple(out.shape) == (n, n_heads * vdim) and weight.numel() == vdim
    check(library().mx_gla_norm_gate(_ptr(o), _ptr(gate), gate.stride(0), _ptr(weight), float(eps), _ptr(out),
                                     dtype_code(out.dtype), n, n_heads, vdim, _stream()), "gla_norm_gate")
    _launched()


# ---------------------------------------------------------------------- gated and routed feed-forwards
GLU_ACTIVATIONS = {"gelu_tanh": 0, "silu": 1}
CLAMPED_ACTIVATION = 2       # the grouped product's code for ``min(g, limit) * sigmoid(slope g) * (clamp(u) + shift)``


def glu(gate_up: torch.Tensor, out: torch.Tensor, activation: str) -> None:
    """Rows ``[gate | up]`` -> ``act(gate) * up``."""
    _need(gate_up, "gate_up")
    _need(out, "out", gate_up.dtype)
    n, ff = out.shape
    assert tuple(gate_up.shape) == (n, 2 * ff)
    check(library().mx_glu(_ptr(gate_up), gate_up.stride(0), _ptr(out), dtype_code(out.dtype), n, ff,
                           GLU_ACTIVATIONS[activation], _stream()), "glu")
    _launched()


def moe_tile_rows() -> int:
    return int(library().mx_moe_tile_rows())


def moe_route(h: torch.Tensor, router: torch.Tensor, top: int, n_groups: int, keep: int, scale: float,
              ids: torch.Tensor, weights: torch.Tensor, counts: torch.Tensor, place: torch.Tensor) -> None:
    """Per token: sigmoid scores of the float32 router [experts, K], the ``top`` best experts of the ``keep`` best
    of ``n_groups`` runs of neighbours (a run is worth its two best scores), weights = scores / their sum * scale.
    ``counts`` [experts] must be zero; afterwards it holds every expert's pairs and ``place`` each pair's index
    among them."""
    _need(h, "h")
    _need(router, "router", torch.float32)
    for name, tensor in (("ids", ids), ("counts", counts), ("place", place)):
        _need(tensor, name, torch.int32)
    _need(weights, "weights", torch.float32)
    n, k = h.shape
    n_experts = router.shape[0]
    assert router.shape[1] == k and ids.numel() == n * top == weights.numel() == place.numel()
    assert counts.numel() == n_experts
    check(library().mx_moe_route(_ptr(h), dtype_code(h.dtype), h.stride(0), _ptr(router), k, n_experts, top, n_groups,
                                 keep, float(scale), _ptr(ids), _ptr(weights), _ptr(counts), _ptr(place), n, _stream()),
          "moe_route")
    _launched()


def moe_plan(counts: torch.Tensor, ids: torch.Tensor, place: torch.Tensor, first: torch.Tensor, tile_map: torch.Tensor,
             n_tiles: torch.Tensor, order: torch.Tensor, tile_rows: int | None = None) -> None:
    """From the routing's counts: ``first`` [experts + 1] (first sorted row of every expert), the row tiles
    ``tile_map`` [tiles, 3] = (expert, first sorted row, rows) of at most ``tile_rows`` rows (default: the FP32-core
    product's) with their number in ``n_tiles`` [1], and ``order`` [pairs]: the pairs sorted by expert."""
    tile_rows = tile_rows or moe_tile_rows()
    for name, tensor in (("counts", counts), ("ids", ids), ("place", place), ("first", first), ("tile_map", tile_map),
                         ("n_tiles", n_tiles), ("order", order)):
        _need(tensor, name, torch.int32)
    n_experts, n_pairs = counts.numel(), ids.numel()
    assert first.numel() == n_experts + 1 and order.numel() == n_pairs
    assert tile_map.numel() >= 3 * moe_max_tiles(n_pairs, n_experts, tile_rows)
    check(library().mx_moe_plan(_ptr(counts), _ptr(ids), _ptr(place), n_experts, n_pairs, tile_rows, _ptr(first),
                                _ptr(tile_map), _ptr(n_tiles), _ptr(order), _stream()), "moe_plan")
    _launched(2)


def moe_max_tiles(n_pairs: int, n_experts: int, tile_rows: int | None = None) -> int:
    """The most row tiles that ``n_pairs`` pairs shared out between ``n_experts`` experts can make."""
    rows = tile_rows or moe_tile_rows()
    return min(n_pairs, n_pairs // rows + n_experts)


def moe_gemm(a: torch.Tensor, order: torch.Tensor, a_div: int, w: torch.Tensor, tile_map: torch.Tensor,
             n_tiles: torch.Tensor, max_tiles: int, out: torch.Tensor, pair_weight: torch.Tensor | None,
             activation: str | tuple | None) -> None:
    """The grouped product over the pairs sorted by expert. With ``activation``: ``a`` holds the tokens' rows (pair
    p reads row ``p // a_div``), ``w`` [experts, 2 N, K] stacks gate and up rows, ``out`` [pairs, N] (sorted order,
    dtype of a) = act(gate) * up. Without: ``a`` [pairs, K] is in sorted order, ``w`` [experts, N, K], ``out``
    float32 [pairs, N] in pair order = ``pair_weight[pair] *`` product. ``activation`` is a name of
    ``GLU_ACTIVATIONS`` or ``("clamped", limit, slope, shift)``: ``g = min(gate, limit)``,
    ``u = clamp(up, -limit, limit)`` (limit <= 0: neither), ``g * sigmoid(slope g) * (u + shift)``."""
    _need(a, "a")
    _need(w, "w", a.dtype)
    _need(out, "out")
    for name, tensor in (("order", order), ("tile_map", tile_map), ("n_tiles", n_tiles)):
        _need(tensor, name, torch.int32)
    glu_form = activation is not None
    k = a.shape[1]
    n = out.shape[1]
    assert w.shape[2] == k and w.shape[1] == (2 * n if glu_form else n), (a.shape, w.shape, out.shape)
    if glu_form:
        assert out.dtype == a.dtype
    else:
        _need(pair_weight, "pair_weight", torch.float32)
        assert out.dtype == torch.float32
    code, constants = 0, (0.0, 0.0, 0.0)
    if isinstance(activation, tuple):
        code, constants = CLAMPED_ACTIVATION, tuple(float(c) for c in activation[1:4])
    elif glu_form:
        code = GLU_ACTIVATIONS[activation]
    check(library().mx_moe_gemm(_ptr(a), dtype_code(a.dtype), a.stride(0), _ptr(order), a_div, _ptr(w), w.stride(0), n, k,
                                _ptr(tile_map), _ptr(n_tiles), max_tiles, _ptr(out), _ptr(pair_weight),
                                1 if glu_form else 0, code, *constants, _stream()),
          "moe_gemm")
    _launched()


def _identity_arguments(identity, n: int, width: int):
    """(ids, weights, input, its dtype code, its row stride, experts with rows) of pairs that stand for their
    token's input (float32 or bfloat16 rows)."""
    if identity is None:
        return None, None, None, F32, 0, 0
    ids, weights, rows, n_experts = identity
    _need(ids, "ids", torch.int32)
    _need(weights, "weights", torch.float32)
    _need(rows, "identity input", contiguous=False)
    assert tuple(rows.shape) == (n, width) and rows.stride(1) == 1
    return ids, weights, rows, dtype_code(rows.dtype), rows.stride(0), int(n_experts)


def moe_combine(pairs: torch.Tensor, residual: torch.Tensor, top: int, identity=None) -> None:
    """residual[t] += the sum of the token's ``top`` rows of ``pairs`` [tokens * top, width], first slot first.
    ``identity`` = (ids, weights, input [tokens, width], n_experts): a pair whose id is ``>= n_experts``
    has no row; ``weights[pair] * input[t]`` stands for it."""
    _need(pairs, "pairs", torch.float32)
    _need(residual, "residual", torch.float32)
    n, width = residual.shape
    assert tuple(pairs.shape) == (n * top, width)
    ids, weights, rows, code, ld, n_experts = _identity_arguments(identity, n, width)
    check(library().mx_moe_combine(_ptr(pairs), _ptr(residual), n, top, width, _ptr(ids), _ptr(weights), _ptr(rows), code,
                                   ld, n_experts, _stream()), "moe_combine")
    _launched()


def moe_route_softmax(h: torch.Tensor, router: torch.Tensor, top: int, n_identity: int, correction: torch.Tensor | None,
                      ids: torch.Tensor, weights: torch.Tensor, counts: torch.Tensor, place: torch.Tensor,
                      bias: torch.Tensor | None = None) -> None:
    """Per token: softmax scores over the rows of the float32 router [experts + n_identity, K] (``bias``, float32 per
    row or None, is added to the logits first: with a bias and no correction the rule reads "the ``top`` largest
    logits, weighted by the softmax over those alone"); the ``top`` rows
    with the largest ``score + correction`` (float32 per row or None; ties to the lower index); weights = the
    chosen rows' plain scores / their sum. ``counts`` [experts] must be zero; afterwards it holds every expert's
    pairs and ``place`` each pair's index among them. A pair of one of the last ``n_identity`` rows keeps its id,
    is counted nowhere and has place 0."""
    _need(h, "h")
    _need(router, "router", torch.float32)
    for name, tensor in (("ids", ids), ("counts", counts), ("place", place)):
        _need(tensor, name, torch.int32)
    _need(weights, "weights", torch.float32)
    n, k = h.shape
    n_experts = router.shape[0] - n_identity
    assert router.shape[1] == k and ids.numel() == n * top == weights.numel() == place.numel()
    assert n_experts >= 0 and counts.numel() == n_experts
    if correction is not None:
        _need(correction, "correction", torch.float32)
        assert correction.numel() == router.shape[0]
    if bias is not None:
        _need(bias, "bias", torch.float32)
        assert bias.numel() == router.shape[0]
    check(library().mx_moe_route_softmax(_ptr(h), dtype_code(h.dtype), h.stride(0), _ptr(router), k, n_experts, n_identity,
                                         top, _ptr(correction), _ptr(bias), _ptr(ids), _ptr(weights), _ptr(counts), _ptr(place), n,
                                         _stream()), "moe_route_softmax")
    _launched()


GROUPED_TILE_ROWS = 128      # row tiles of the grouped tcgen05 product


def grouped_tcgen05_supported(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether ``gemm_tcgen05_grouped`` takes rows ``a`` [rows, K] and stacked matrices ``w`` [groups, N, K]."""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[1] % 8 == 0 and a.stride(1) == 1
            and a.stride(0) % 8 == 0 and w.is_contiguous() and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and w.shape[0] * w.shape[1] < 2 ** 31)


def moe_gather(h: torch.Tensor, order: torch.Tensor, top: int, out: torch.Tensor) -> None:
    """out[r] = h[order[r] // top]: the tokens' rows (bfloat16) in the order of the sorted pairs."""
    _need(h, "h", torch.bfloat16, contiguous=False)
    _need(order, "order", torch.int32)
    _need(out, "out", torch.bfloat16)
    n_pairs, k = out.shape
    assert h.shape[1] == k and order.numel() == n_pairs and h.stride(1) == 1
    check(library().mx_moe_gather(_ptr(h), h.stride(0), _ptr(order), top, _ptr(out), n_pairs, k, _stream()), "moe_gather")
    _launched()


def gemm_tcgen05_grouped(a: torch.Tensor, w: torch.Tensor, tile_map: torch.Tensor, n_tiles: torch.Tensor,
                         max_tiles: int, out: torch.Tensor, status: torch.Tensor | None = None) -> None:
    """out[r] = a[r] @ w[group of r].T on tcgen05: ``a`` [rows, K] bfloat16 sorted by group, ``w`` [groups, N, K],
    ``tile_map`` / ``n_tiles`` from ``moe_plan(..., tile_rows=GROUPED_TILE_ROWS)``; ``out`` [rows, N] bfloat16 or
    float32."""
    _need(a, "a", torch.bfloat16, contiguous=False)
    _need(w, "w", torch.bfloat16)
    _need(out, "out")
    _need(tile_map, "tile_map", torch.int32)
    _need(n_tiles, "n_tiles", torch.int32)
    rows, k = a.shape
    groups, n = w.shape[0], w.shape[1]
    assert w.shape[2] == k and tuple(out.shape) == (rows, n), (a.shape, w.shape, out.shape)
    if out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelLibraryError(f"a grouped product writes bfloat16 or float32, not {out.dtype}")
    if status is None:
        status = default_status(a.device)
    check(library().mx_gemm_tcgen05_grouped(_ptr(a), _ptr(w), _ptr(out), dtype_code(out.dtype), rows, groups, n, k,
                                            a.stride(0), w.stride(1), out.stride(0), _ptr(tile_map), _ptr(n_tiles),
                                            max_tiles, EPILOGUE_F32 if out.dtype == torch.float32 else EPILOGUE_NONE,
                                            _ptr(status), _stream()), "gemm_tcgen05_grouped")
    _launched()


def moe_combine_sorted(rows: torch.Tensor, ids: torch.Tensor, place: torch.Tensor, first: torch.Tensor,
                       weights: torch.Tensor, residual: torch.Tensor, top: int, identity=None) -> None:
    """residual[t] += sum over the token's ``top`` pairs of ``weights[pair] * rows[first[ids[pair]] + place[pair]]``
    (``rows`` float32 [pairs, width] in sorted order), first slot first. ``identity`` = (input [tokens, width],
    n_experts): a pair whose id is ``>= n_experts`` has no row; its token's input stands for it."""
    _need(rows, "rows", torch.float32)
    _need(residual, "residual", torch.float32)
    _need(weights, "weights", torch.float32)
    for name, tensor in (("ids", ids), ("place", place), ("first", first)):
        _need(tensor, name, torch.int32)
    n, width = residual.shape
    assert tuple(rows.shape) == (n * top, width) and ids.numel() == n * top == place.numel() == weights.numel()
    _, _, source, code, ld, n_experts = _identity_arguments(
        None if identity is None else (ids, weights, identity[0], identity[1]), n, width)
    check(library().mx_moe_combine_sorted(_ptr(rows), _ptr(ids), _ptr(place), _ptr(first), _ptr(weights), _ptr(residual),
                                          n, top, width, _ptr(source), code, ld, n_experts, _stream()), "moe_combine_sorted")
    _launched()


# ---------------------------------------------------------------------- branches normalised on their way out
def layernorm_scaled_add(x: torch.Tensor, branch: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None,
                         scale: torch.Tensor | None, eps: float, act: torch.Tensor | None = None,
                         centre: bool = True) -> None:
    """x[r] += LayerNorm(branch[r]) * weight (+ bias), times ``scale`` entry by entry (a float32 vector or None); float
    statistics. ``act`` (bfloat16 or float32, same shape) receives the new rows. ``centre`` False leaves the mean in:
    the branch is divided by its root mean square."""
    _need(x, "x", torch.float32)
    _need(branch, "branch", torch.float32)
    _need(weight, "weight", torch.float32)
    n, hidden = x.shape
    assert tuple(branch.shape) == (n, hidden) and weight.numel() == hidden
    for name, tensor in (("bias", bias), ("scale", scale)):
        if tensor is not None:
            _need(tensor, name, torch.float32)
            assert tensor.numel() == hidden
    if act is not None:
        _need(act, "act")
        assert tuple(act.shape) == (n, hidden)
    check(library().mx_layernorm_scaled_add(_ptr(x), _ptr(branch), _ptr(weight), _ptr(bias), _ptr(scale), _ptr(act),
                                            dtype_code(act.dtype) if act is not None else F32, n, hidden, float(eps),
                                            1 if centre else 0, _stream()), "layernorm_scaled_add")
    _launched()


def scale_rows(x: torch.Tensor, factor: float) -> None:
    """x *= factor (float32, in place)."""
    _need(x, "x", torch.float32)
    check(library().mx_scale_rows(_ptr(x), x.numel(), float(factor), _stream()), "scale_rows")
    _launched()


def token_side_input(x: torch.Tensor, token_ids: torch.Tensor, table: torch.Tensor, column: int, gate: torch.Tensor,
                     proj: torch.Tensor, norm: torch.Tensor, eps: float, status: torch.Tensor,
                     act: torch.Tensor | None = None) -> None:
    """x[t] += y / sqrt(mean(y^2) + eps) * norm with y = proj (gelu_tanh(gate x[t]) * table[id_t, column:column + dim]),
    in float, in place. ``table`` [vocab, width], ``gate`` [dim, hidden], ``proj`` [hidden, dim] share a dtype, which
    ``act`` (the new rows, optional) has too."""
    _need(x, "x", torch.float32)
    _need(token_ids, "token_ids", torch.int32)
    _need(table, "table")
    _need(gate, "gate", table.dtype)
    _need(proj, "proj", table.dtype)
    _need(norm, "norm", torch.float32)
    _need(status, "status", torch.int32)
    n, hidden = x.shape
    dim = gate.shape[0]
    assert tuple(gate.shape) == (dim, hidden) and tuple(proj.shape) == (hidden, dim) and norm.numel() == hidden
    assert token_ids.numel() >= n
    if act is not None:
        _need(act, "act", table.dtype)
        assert tuple(act.shape) == (n, hidden)
    check(library().mx_token_side_input(_ptr(x), _ptr(act), _ptr(token_ids), _ptr(table), table.shape[1], int(column),
                                        table.shape[0], _ptr(gate), _ptr(proj), _ptr(norm), dtype_code(table.dtype), n,
                                        hidden, dim, float(eps), _ptr(status), _stream()), "token_side_input")
    _launched()


def gelu_gate_rows(z: torch.Tensor, token_ids: torch.Tensor, table: torch.Tensor, column: int, out: torch.Tensor,
                   status: torch.Tensor) -> None:
    """out[t] = gelu_tanh(z[t]) * table[id_t, column:column + dim]: ``z`` float32 [tokens, dim], ``out`` [tokens, dim]
    in the table's dtype."""
    _need(z, "z", torch.float32, contiguous=False)
    _need(token_ids, "token_ids", torch.int32)
    _need(table, "table")
    _need(out, "out", table.dtype)
    _need(status, "status", torch.int32)
    n, dim = out.shape
    assert tuple(z.shape) == (n, dim) and z.stride(1) == 1 and token_ids.numel() >= n
    check(library().mx_gelu_gate_rows(_ptr(z), z.stride(0), _ptr(token_ids), _ptr(table), table.shape[1], int(column),
                                      table.shape[0], _ptr(out), dtype_code(table.dtype), n, dim, _ptr(status), _stream()),
          "gelu_gate_rows")
    _launched()


def rotate_norm_kv_write(proj: torch.Tensor, positions: torch.Tensor, freq: torch.Tensor, rot: int, eps: float | None,
                         slots: torch.Tensor | None, cache: torch.Tensor | None, q_out: torch.Tensor, n_heads: int,
                         n_kv_heads: int, dim: int, vdim: int, status: torch.Tensor) -> None:
    """From float rows ``[q | k | v | ...]`` of a fused projection: q and k heads rotated over their first ``rot``
    entries (pairs (i, i + rot/2), angle ``position * freq[i]``) and then divided by their root mean square over
    ``dim`` (``eps`` inside the root; None: not divided); q into ``q_out`` [tokens, heads * hd], k and v into the
    paged ``cache`` [pages, 2, kv heads, page_size, hd] at ``slots`` (both None: nothing is stored). ``hd`` is the
    padded head size of ``q_out``; tails are zero."""
    _need(proj, "proj", torch.float32, contiguous=False)
    _need(positions, "positions", torch.int32)
    _need(freq, "freq", torch.float32)
    _need(q_out, "q_out")
    _need(status, "status", torch.int32)
    n = q_out.shape[0]
    hd = q_out.shape[1] // n_heads
    assert q_out.shape[1] == n_heads * hd and proj.stride(1) == 1 and proj.shape[0] >= n
    assert freq.numel() >= rot // 2
    n_pages, page_size = 0, 1
    if cache is not None:
        _need(cache, "cache", q_out.dtype)
        _need(slots, "slots", torch.int32)
        n_pages, page_size = cache.shape[0], cache.shape[3]
        assert tuple(cache.shape[1:]) == (2, n_kv_heads, page_size, hd), cache.shape
    check(library().mx_rotate_norm_kv_write(_ptr(proj), proj.stride(0), _ptr(positions), _ptr(freq), int(rot),
                                            -1.0 if eps is None else float(eps), _ptr(slots) if cache is not None else None,
                                            _ptr(cache), n_pages, page_size, _ptr(q_out), dtype_code(q_out.dtype), n,
                                            n_heads, n_kv_heads, dim, vdim, hd, _ptr(status), _stream()),
          "rotate_norm_kv_write")
    _launched()


def norm_rotate_kv_write(proj: torch.Tensor, positions: torch.Tensor, freq: torch.Tensor, rot: int, interleaved: bool,
                         q_weight: torch.Tensor | None, k_weight: torch.Tensor | None, eps: float,
                         slots: torch.Tensor | None, cache: torch.Tensor | None, q_out: torch.Tensor, n_heads: int,
                         n_kv_heads: int, dim: int, vdim: int, status: torch.Tensor) -> None:
    """From float rows ``[q | k | v | ...]`` of a fused projection: q and k heads RMS-normalised over ``dim`` with the
    weights ``q_weight`` / ``k_weight`` (float32 [dim]; None: left as they are; ``eps`` inside the root) and then
    rotated over their first ``rot`` entries (pairs (i, i + rot/2) or, ``interleaved``, (2i, 2i + 1); angle
    ``position * freq[i]``); q into ``q_out`` [tokens, heads * hd], k and v into the paged ``cache``
    [pages, 2, kv heads, page_size, hd] at ``slots`` (both None: nothing is stored). ``hd`` is the padded head size of
    ``q_out``; tails are zero."""
    _need(proj, "proj", torch.float32, contiguous=False)
    _need(positions, "positions", torch.int32)
    _need(freq, "freq", torch.float32)
    _need(q_out, "q_out")
    _need(status, "status", torch.int32)
    n = q_out.shape[0]
    hd = q_out.shape[1] // n_heads
    assert q_out.shape[1] == n_heads * hd and proj.stride(1) == 1 and proj.shape[0] >= n
    assert freq.numel() >= rot // 2
    for name, weight in (("q_weight", q_weight), ("k_weight", k_weight)):
        if weight is not None:
            _need(weight, name, torch.float32)
            assert weight.numel() == dim
    n_pages, page_size = 0, 1
    if cache is not None:
        _need(cache, "cache", q_out.dtype)
        _need(slots, "slots", torch.int32)
        n_pages, page_size = cache.shape[0], cache.shape[3]
        assert tuple(cache.shape[1:]) == (2, n_kv_heads, page_size, hd), cache.shape
    check(library().mx_norm_rotate_kv_write(_ptr(proj), proj.stride(0), _ptr(positions), _ptr(freq), int(rot),
                                            1 if interleaved else 0, _ptr(q_weight), _ptr(k_weight), float(eps),
                                            _ptr(slots) if cache is not None else None, _ptr(cache), n_pages, page_size,
                                            _ptr(q_out), dtype_code(q_out.dtype), n, n_heads, n_kv_heads, dim, vdim, hd,
                                            _ptr(status), _stream()), "norm_rotate_kv_write")
    _launched()
