"""Bafusun through the engine against the plain implementation (tests/plain_bafusun.py): every mechanism alone,
then whole models cut and batched every way, in float32 and bfloat16, with pools so small that pages and slots
are used again. Sizes, orders and constants are the tests' own."""

import copy
import json
import math
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_bafusun as plain
from bafusun_configs import MODELS, attention, draw, ids, moe, single_layer
from matricxon_b200.config.registry import config_from_dict
from matricxon_b200.engine.core import model_from_tensors
from matricxon_b200.engine.replay import TraceReplayer
from matricxon_b200.ops import kernels
from trace_utils import ROOT

pytestmark = pytest.mark.gpu

DEVICE = "cuda:0"
CHUNKS = [7, 2, 5, 3, 11, 2, 4, 13, 2, 9]
F64 = torch.float64


def limit_for(dtype: str, reference: np.ndarray) -> float:
    scale = max(1.0, float(np.abs(reference).max()))
    return (2e-4 if dtype == "float32" else 0.06) * scale


def rounded(tensors: dict, dtype: str) -> dict:
    """What the engine holds: a bfloat16 engine reads bfloat16 matrices, so the plain side gets the same."""
    if dtype == "float32":
        return tensors
    return {name: value.to(torch.bfloat16).float() for name, value in tensors.items()}


class Run:
    """One engine over one model: requests fed in portions, logits kept per (request, position).

    A bfloat16 engine may send a token to another expert than the plain model does when two choice scores lie
    closer than 16-bit rounding resolves, and in a model of several layers the positions that attend to such a
    token differ then too. That is no fault, so the bfloat16 runs listen to the engine's choices
    (``StepRunner.taps``; such steps run launch by launch) and hand them to the plain model, which is then
    compared at every position; where the plain model's own choice is clear, the engine's is the same but for
    one in fifty.
    float32 runs listen to nothing, replay captured steps and are compared with the plain model's own routing."""

    def __init__(self, raw: dict, tensors: dict, dtype: str, max_tokens: int, max_requests: int = 4,
                 page_size: int = 16) -> None:
        self.raw, self.dtype = raw, dtype
        self.weights = rounded(tensors, dtype)
        config = config_from_dict(copy.deepcopy(raw))
        model = model_from_tensors(config, self.weights, dtype=dtype, device=DEVICE, page_size=page_size)
        self.replayer = TraceReplayer(None, dtype, max_tokens, page_size=page_size, device=DEVICE,
                                      max_requests=max_requests, model=model, poison_cache=True)
        self.listens = dtype == "bfloat16" and any(layer.get("mlp") for layer in raw["layers"])
        if self.listens:
            self.replayer.core.runner.taps = ("expert_choices",)
        self.logits: dict[tuple[str, int], np.ndarray] = {}
        self.choices: dict[tuple[str, int], list] = {}
        self.progress: dict[str, int] = {}
        self.slots_seen: dict[str, int] = {}
        self.reference_cache: dict[tuple, np.ndarray] = {}

    def step(self, portions: list[tuple[str, list[int]]], end=()) -> None:
        entries, keys = [], []
        for request, tokens in portions:
            start = self.progress.get(request, 0)
            entries.append({"id": request, "tokens": tokens, "want": list(range(len(tokens)))})
            keys.extend((request, start + i) for i in range(len(tokens)))
            self.progress[request] = start + len(tokens)
        out = self.replayer.step(entries, [])
        rows = list(self.replayer.last_rows)
        if self.listens:
            heard = [layer.cpu() for layer in self.replayer.core.runner.last_taps["expert_choices"]]
            for row, key in enumerate(keys):
                self.choices[key] = [layer[row].tolist() for layer in heard]
        for request, _ in portions:
            self.slots_seen[request] = self.replayer.core.cache.record(request).state_slot
        if end:
            self.replayer.step([], list(end))
            for request in end:
                self.progress.pop(request, None)
        assert rows == keys
        for key, row in zip(keys, out.numpy()):
            self.logits[key] = row
        self.replayer.core.cache.check_invariants()

    def feed(self, request: str, tokens: list[int], sizes, end: bool = True) -> None:
        """One request alone, cut into portions of the given sizes (a list, then one by one; or a function of
        the turn)."""
        start, turn = 0, 0
        while start < len(tokens):
            if isinstance(sizes, list):
                size = sizes[turn] if turn < len(sizes) else 1
            else:
                size = sizes(turn)
            size = min(size, len(tokens) - start)
            turn += 1
            last = start + size == len(tokens)
            self.step([(request, tokens[start:start + size])], end=[request] if last and end else [])
            start += size

    def reference(self, tokens: list[int], forced=None):
        """(logits, every routed layer's margins, every routed layer's own choice) of the plain model."""
        key = (tuple(tokens), None if forced is None else tuple(tuple(sum(layer, [])) for layer in forced))
        if key not in self.reference_cache:
            margins, choices = [], []
            logits = plain.forward(self.raw, self.weights, tokens, margins=margins, forced=forced, choices=choices)
            self.reference_cache[key] = (logits.numpy(), [m.numpy() for m in margins], [c.tolist() for c in choices])
        return self.reference_cache[key]

    def check(self, request: str, tokens: list[int], first: int = 0, allowed_over: int = 0) -> None:
        forced = None
        if self.listens:
            n_routed = len(self.choices[(request, 0)])
            forced = [[self.choices[(request, i)][layer] for i in range(len(tokens))] for layer in range(n_routed)]
        want, margins, own = self.reference(tokens, forced)
        if self.listens:
            # under the engine's routing the plain model's stream is the engine's: where its own choice there
            # is clear, it is the engine's
            for layer, margin in enumerate(margins):
                clear = np.nonzero(margin > 0.6)[0]        # a router logit would have to move by more than one
                self.clear += len(clear)
                self.unclear += len(tokens) - len(clear)
                same = sum(sorted(own[layer][t]) == sorted(forced[layer][t]) for t in clear)
                # 16-bit rounding of a router's input moves its logits by some tenths here; a rare token differs
                assert same >= len(clear) - max(1, len(clear) // 50), (request, layer, same, len(clear))
        got = np.stack([self.logits[(request, i)] for i in range(first, len(tokens))])
        worst = np.abs(got - want[first:]).max(axis=1)
        limit = limit_for(self.dtype, want)
        bad = np.nonzero(~(worst <= limit))[0]
        assert bad.size <= allowed_over, (f"{request}: first wrong position {first + bad[0]} of {len(tokens)}, "
                                          f"error {worst[bad[0]]:.3e} > {limit:.1e}; {bad.size} positions over")

    clear = unclear = 0


def cycle(turn: int) -> int:
    return CHUNKS[turn % len(CHUNKS)]


# ---------------------------------------------------------------------- kernels alone
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden", [40, 96, 1002, 4100])
def test_branch_norm_kernel(dtype, hidden):
    """x += scale * LayerNorm(branch) * weight with float statistics; a branch with a large mean shows whether
    the variance is of the deviations."""
    torch.manual_seed(hidden)
    x = torch.randn(9, hidden, device=DEVICE) * 3
    branch = torch.randn(9, hidden, device=DEVICE) * 0.3 + 50.0
    weight, scale = torch.randn(hidden, device=DEVICE), torch.randn(hidden, device=DEVICE)
    for with_scale in (True, False):
        stream = x.clone()
        act = None if dtype == torch.float32 else torch.empty(9, hidden, dtype=dtype, device=DEVICE)
        kernels.layernorm_scaled_add(stream, branch, weight, None, scale if with_scale else None, 1e-3, act)
        want = x.double() + plain.layer_norm(branch.double(), weight.double(), 1e-3) * (scale.double() if with_scale else 1.0)
        assert torch.allclose(stream.double(), want, rtol=1e-4, atol=2e-4), (stream.double() - want).abs().max()
        if act is not None:
            assert torch.equal(act, stream.to(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden, dim, layers", [(96, 10, 4), (64, 1, 1), (1000, 24, 3), (256, 130, 2)])
def test_token_input_kernel(dtype, hidden, dim, layers):
    gen = torch.Generator().manual_seed(hidden + dim)
    n, vocab, layer = 13, 37, layers - 1
    w = {"side.embed": torch.randn(vocab, layers * dim, generator=gen) * 2, "l%d.side.gate" % layer: torch.randn(dim, hidden, generator=gen) * 0.2,
         "l%d.side.proj" % layer: torch.randn(hidden, dim, generator=gen) * 0.3, "l%d.side.norm" % layer: torch.randn(hidden, generator=gen)}
    w = {k: (v if k.endswith("norm") else v.to(dtype).float()) for k, v in w.items()}
    x = torch.randn(n, hidden, generator=gen)
    tokens = torch.randint(0, vocab, (n,), generator=gen)
    stream = x.clone().to(DEVICE)
    act = None if dtype == torch.float32 else torch.empty(n, hidden, dtype=dtype, device=DEVICE)
    status = torch.zeros(1, dtype=torch.int32, device=DEVICE)
    p = f"l{layer}.side."
    kernels.token_side_input(stream, tokens.to(torch.int32).to(DEVICE), w["side.embed"].to(dtype).to(DEVICE), layer * dim,
                             w[p + "gate"].to(dtype).to(DEVICE), w[p + "proj"].to(dtype).to(DEVICE),
                             w[p + "norm"].to(DEVICE), 1e-4, status, act)
    want = x.double() + plain.token_input(x.double(), tokens, {k: v.double() for k, v in w.items()}, layer, dim, 1e-4)
    assert int(status.item()) == 0
    assert torch.allclose(stream.cpu().double(), want, rtol=2e-4, atol=2e-4), (stream.cpu().double() - want).abs().max()
    if act is not None:
        assert torch.equal(act, stream.to(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads, kv, dim, vdim, rot", [(6, 3, 24, 40, 12), (4, 1, 40, 8, 40), (3, 3, 16, 16, 0),
                                                       (2, 2, 64, 64, 64), (2, 1, 128, 64, 32), (5, 5, 12, 20, 6)])
def test_rotation_unit_norm_and_cache_write_kernel(dtype, heads, kv, dim, vdim, rot):
    """q and k rotated over their first entries, then brought to unit root mean square; k and v land in the
    pages their slots name, padded with zeros to the common head size; large positions keep their angles."""
    gen = torch.Generator().manual_seed(dim * 3 + vdim)
    n, page = 11, 4
    hd = -(-max(dim, vdim) // 16) * 16
    width = heads * dim + kv * dim + kv * vdim
    proj = torch.randn(n, width + 5, generator=gen) * 2
    positions = torch.tensor([0, 1, 2, 3, 77, 78, 1000, 2001, 5, 6, 7], dtype=torch.int32)
    freq = torch.tensor([300.0 ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float32)
    slots = torch.randperm(6 * page, generator=gen)[:n].to(torch.int32)
    cache = torch.full((6, 2, kv, page, hd), 7.0, dtype=dtype, device=DEVICE)
    q_out = torch.full((n, heads * hd), 7.0, dtype=dtype, device=DEVICE)
    status = torch.zeros(1, dtype=torch.int32, device=DEVICE)
    kernels.rotate_norm_kv_write(proj.to(DEVICE), positions.to(DEVICE), freq.to(DEVICE), rot, 1e-5, slots.to(DEVICE), cache,
                                 q_out, heads, kv, dim, vdim, status)
    assert int(status.item()) == 0
    p64 = proj.double()
    q = p64[:, :heads * dim].view(n, heads, dim)
    k = p64[:, heads * dim:(heads + kv) * dim].view(n, kv, dim)
    v = p64[:, (heads + kv) * dim:width].view(n, kv, vdim)
    if rot:
        spec = {"dims": rot, "base": 300.0}
        q, k = plain.rotate(q, positions, spec), plain.rotate(k, positions, spec)
    q, k = plain.rms_unit(q, 1e-5), plain.rms_unit(k, 1e-5)
    tol = 5e-4 if dtype == torch.float32 else 0.02          # float angles of positions in the thousands
    got_q = q_out.cpu().double().view(n, heads, hd)
    assert torch.allclose(got_q[..., :dim], q, rtol=tol, atol=tol), (got_q[..., :dim] - q).abs().max()
    assert hd == dim or float(got_q[..., dim:].abs().max()) == 0.0
    held = cache.cpu().double()
    for t in range(n):
        page_id, offset = int(slots[t]) // page, int(slots[t]) % page
        got_k = held[page_id, 0, :, offset]
        got_v = held[page_id, 1].reshape(kv, hd, page)[:, :, offset]          # values lie transposed in a page
        assert torch.allclose(got_k[:, :dim], k[t], rtol=tol, atol=tol), t
        assert torch.allclose(got_v[:, :vdim], v[t], rtol=tol, atol=tol * 4), t
        assert float(got_k[:, dim:].abs().sum()) == 0.0 and float(got_v[:, vdim:].abs().sum()) == 0.0
    untouched = sorted(set(range(6 * page)) - set(slots.tolist()))
    for slot in untouched:
        assert float(held[slot // page, 0, :, slot % page].min()) == 7.0


def _paged_case(dtype, n_heads, n_kv, hd, page_size, contexts, q_lens, seed, spikes=()):
    """Unit-norm queries and keys, a paged cache with shuffled pages in which only the pages a window still needs
    are mapped when ``drop`` says so. ``spikes`` = (sequence, key position): that key equals the direction of the
    sequence's last query's first head of each group."""
    gen = torch.Generator().manual_seed(seed)
    n_seqs, n_tok = len(contexts), sum(q_lens)
    totals = [c + q for c, q in zip(contexts, q_lens)]
    pages_of = [-(-t // page_size) for t in totals]
    n_pages = sum(pages_of) + 3
    order = torch.randperm(n_pages, generator=gen).tolist()
    tables = torch.full((n_seqs, max(pages_of)), -1, dtype=torch.int32)
    cache = torch.zeros((n_pages, 2, n_kv, page_size, hd))
    unit = lambda x: x / x.pow(2).mean(-1, keepdim=True).sqrt()
    q = unit(torch.randn(n_tok, n_heads, hd, generator=gen)).reshape(n_tok, n_heads * hd)
    keys, values, group, row = [], [], n_heads // n_kv, 0
    for s in range(n_seqs):
        k = unit(torch.randn(totals[s], n_kv, hd, generator=gen))
        v = torch.randn(totals[s], n_kv, hd, generator=gen)
        last = row + q_lens[s] - 1
        for seq, where in spikes:
            if seq == s:
                for g in range(n_kv):
                    k[where, g] = q[last].view(n_heads, hd)[g * group]
        keys.append(k)
        values.append(v)
        for lp in range(pages_of[s]):
            page = order.pop()
            tables[s, lp] = page
            lo, hi = lp * page_size, min((lp + 1) * page_size, totals[s])
            cache[page, 0, :, :hi - lo] = k[lo:hi].transpose(0, 1)
            cache[page, 1].view(n_kv, hd, page_size)[:, :, :hi - lo] = v[lo:hi].permute(1, 2, 0)
        row += q_lens[s]
    tok_seq = torch.tensor([s for s in range(n_seqs) for _ in range(q_lens[s])], dtype=torch.int32)
    positions = torch.tensor([contexts[s] + i for s in range(n_seqs) for i in range(q_lens[s])], dtype=torch.int32)
    cu_q = torch.tensor([0] + list(np.cumsum(q_lens)), dtype=torch.int32)
    meta = {"tables": tables, "tok_seq": tok_seq.to(DEVICE), "positions": positions.to(DEVICE),
            "cu_q": cu_q.to(DEVICE), "contexts": torch.tensor(contexts, dtype=torch.int32, device=DEVICE)}
    return q.to(dtype).to(DEVICE), cache.to(dtype), meta, keys, values


def _plain_attend(q, keys, values, contexts, q_lens, n_heads, n_kv, hd, scale, mask):
    out = torch.zeros(q.shape[0], n_heads, hd, dtype=F64)
    group, row = n_heads // n_kv, 0
    for s, (c, n) in enumerate(zip(contexts, q_lens)):
        k, v = keys[s].double(), values[s].double()
        for i in range(n):
            seen = torch.tensor([plain.visible(c + i, j, mask) for j in range(c + n)])
            qi = q[row].double().view(n_heads, hd)
            for h in range(n_heads):
                score = ((k[:, h // group] @ qi[h]) * scale).masked_fill(~seen, -math.inf)
                out[row, h] = torch.softmax(score, dim=0) @ v[:, h // group]
            row += 1
    return out.view(q.shape[0], n_heads * hd)


@pytest.mark.parametrize("kernel, dtype, hd, group", [
    ("simt", torch.float32, 48, 3), ("simt", torch.float32, 128, 2), ("simt", torch.bfloat16, 32, 1),
    ("simt", torch.float32, 64, 8), ("mma", torch.bfloat16, 64, 4), ("mma", torch.bfloat16, 128, 2),
    ("mma", torch.bfloat16, 64, 1), ("mma", torch.bfloat16, 128, 8), ("tc", torch.bfloat16, 128, 2),
    ("tc", torch.bfloat16, 128, 4), ("tc", torch.bfloat16, 128, 1)])
@pytest.mark.parametrize("window, keep", [(44, 12), (21, 3), (16, 16), (7, 50), (64, 0), (33, 1), (150, 130), (40, 300)])
def test_attention_kernels_under_a_window_that_keeps_the_first_tokens(kernel, dtype, hd, group, window, keep):
    """Prompt portions and single tokens in one launch, shuffled pages, key splits. The pages that neither the
    window nor the kept tokens need are unmapped and poisoned, as the cache manager leaves them. The last query
    of every sequence meets a key equal to itself just inside the window, just outside it, at the last kept
    position and at the first one not kept: with a sharp scale each of them would take the softmax."""
    n_kv, n_heads, page = 2, 2 * group, 16
    contexts, q_lens = [70, 5, 300, 0, 131], [1, 37, 1, 45, 2]
    if kernel == "tc":                     # prompt portions only; windows that end in the first, a middle and the last chunk
        contexts, q_lens = [70, 5, 130, 600, 0], [40, 37, 64, 150, 300]
    spikes = []
    for s, (c, n) in enumerate(zip(contexts, q_lens)):
        last = c + n - 1
        spikes += [(s, j) for j in (last - window, last - window + 1, keep - 1, keep) if 0 <= j < last]
    q, cache, meta, keys, values = _paged_case(dtype, n_heads, n_kv, hd, page, contexts, q_lens, seed=hd + group + window,
                                               spikes=spikes)
    # what the cache manager would have given back before this step: pages wholly older than the window of the
    # step's first query, except those of the kept tokens
    tables = meta["tables"].clone()
    for s, c in enumerate(contexts):
        first_needed, kept_pages = max(0, c - window + 1) // page, -(-keep // page)
        for lp in range(kept_pages, min(first_needed, tables.shape[1])):
            if tables[s, lp] >= 0:
                cache[tables[s, lp]] = float("nan") if dtype == torch.float32 else 1e4
                tables[s, lp] = -1
    cache, tables = cache.to(DEVICE), tables.to(DEVICE)
    mask = {"size": window, "keep_first": keep}
    scale = 12.0 / hd                                       # a key equal to the query scores 12, the others about 0
    n_tok = sum(q_lens)
    status = torch.zeros(1, dtype=torch.int32, device=DEVICE)
    want = _plain_attend(q.cpu().float(), [k.to(dtype).float() for k in keys], [v.to(dtype).float() for v in values],
                         contexts, q_lens, n_heads, n_kv, hd, scale, mask)
    for n_splits in (1, 3):
        out = torch.zeros(n_tok, n_heads * hd, dtype=dtype, device=DEVICE)
        scratch = None
        if n_splits > 1:
            scratch = torch.empty(kernels.attention_scratch_bytes(n_tok, n_heads, hd, n_splits) // 4 + 4,
                                  dtype=torch.float32, device=DEVICE)
        if kernel == "simt":
            kernels.paged_attention(q, q.stride(0), cache, tables, meta["tok_seq"], meta["positions"], n_tok,
                                    n_heads, n_kv, hd, window, scale, out, status, n_splits=n_splits, scratch=scratch,
                                    keep_first=keep)
        elif kernel == "tc":
            _, wide = kernels.attention_tile_lists([max(n, 17) for n in q_lens], group, True)
            tiles = torch.tensor(wide, dtype=torch.int32, device=DEVICE)
            kernels.paged_attention_tc(q, q.stride(0), cache, tables, meta["cu_q"], meta["contexts"], tiles,
                                       len(wide) // 2, n_tok, n_heads, n_kv, hd, window, scale, out, status,
                                       n_splits=n_splits, scratch=scratch, keep_first=keep)
        else:
            narrow, wide = kernels.attention_tile_lists(q_lens, group, False)
            if n_splits > 1:        # key splits need a launch that covers every token: all tiles wide
                narrow, wide = [], [x for s, n in enumerate(q_lens) for r in range(0, n * group, 64) for x in (s, r)]
            for tiles, is_narrow in ((narrow, True), (wide, False)):
                if tiles:
                    t = torch.tensor(tiles, dtype=torch.int32, device=DEVICE)
                    kernels.paged_attention_mma(q, q.stride(0), cache, tables, meta["cu_q"], meta["contexts"], t,
                                                len(tiles) // 2, is_narrow, n_tok, n_heads, n_kv, hd, window, scale, out,
                                                status, n_splits=n_splits, scratch=scratch, keep_first=keep)
        tol = 2e-5 if dtype == torch.float32 else 0.03
        got = out.double().cpu()
        assert torch.allclose(got, want, rtol=tol, atol=tol), (n_splits, (got - want).abs().max())
        assert int(status.item()) == 0
    # the planted keys matter: seen through a window one longer, the last rows come out differently
    wider = _plain_attend(q.cpu().float(), keys, values, contexts, q_lens, n_heads, n_kv, hd, scale,
                          {"size": window + 1, "keep_first": keep})
    last_rows = [int(x) - 1 for x in np.cumsum(q_lens)]
    moved = [float((wider[r] - want[r]).abs().max()) for r, (c, n) in zip(last_rows, zip(contexts, q_lens))
             if c + n - 1 - window >= keep]
    assert (moved or keep >= 300) and min(moved, default=1.0) > 0.05


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts, identity, top", [(5, 2, 2), (3, 0, 1), (2, 3, 4), (14, 3, 5), (1, 1, 2),
                                                    (60, 4, 8), (9, 0, 9)])
def test_softmax_router_kernel_against_the_plain_choice(dtype, experts, identity, top):
    gen = torch.Generator().manual_seed(experts * 7 + top)
    n, width, rows = 50, 72, experts + identity
    h = torch.randn(n, width, generator=gen).to(dtype)
    w = {"r.router": torch.randn(rows, width, generator=gen) * 0.5, "r.correction": torch.randn(rows, generator=gen) * 0.2}
    chosen, weights = plain.route(h.double(), {k: v.double() for k, v in w.items()}, "r.",
                                  {"experts": experts, "identity": identity, "top": top})
    ints = torch.zeros(experts + 3 * n * top, dtype=torch.int32, device=DEVICE)
    counts, got_ids, place, _ = torch.split(ints, [experts, n * top, n * top, n * top])
    got_w = torch.empty(n * top, dtype=torch.float32, device=DEVICE)
    for correction in (w["r.correction"], None):
        ints.zero_()
        if correction is None:
            chosen, weights = plain.route(h.double(), {"r.router": w["r.router"].double(), "r.correction": torch.zeros(rows, dtype=F64)},
                                          "r.", {"experts": experts, "identity": identity, "top": top})
        kernels.moe_route_softmax(h.to(DEVICE), w["r.router"].to(DEVICE), top, identity,
                                  None if correction is None else correction.to(DEVICE), got_ids, got_w, counts, place)
        ids_, w_ = got_ids.view(n, top).cpu().long(), got_w.view(n, top).cpu().double()
        assert torch.equal(ids_, chosen), "the experts, in the order of their corrected scores"
        assert torch.allclose(w_, weights, rtol=1e-5, atol=1e-7)
        real = chosen.flatten()[chosen.flatten() < experts]
        assert torch.equal(counts.cpu().long(), torch.bincount(real, minlength=experts)[:experts])
        seen = {(int(e), int(p)) for e, p in zip(ids_.flatten(), place.cpu()) if e < experts}
        assert len(seen) == real.numel() and all(p < counts[e] for e, p in seen)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_clamped_gate_kernel(dtype):
    gen = torch.Generator().manual_seed(1)
    gate_up = (torch.randn(33, 2 * 52, generator=gen) * 3).to(dtype)
    for limit, slope, shift in ((1.0, 1.702, 1.0), (2.5, 1.0, 0.0), (0.3, 1.702, 1.0)):
        out = torch.empty(33, 52, dtype=dtype, device=DEVICE)
        kernels.clamped_glu(gate_up.to(DEVICE), out, limit, slope, shift)
        g = gate_up.double()[:, :52].clamp(max=limit)
        u = gate_up.double()[:, 52:].clamp(-limit, limit)
        want = g * torch.sigmoid(slope * g) * (u + shift)
        tol = 1e-5 if dtype == torch.float32 else 0.02
        assert torch.allclose(out.cpu().double(), want, rtol=tol, atol=tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n, experts, identity, top, width, ff, shared", [
    (1, 4, 1, 2, 64, 40, 24), (70, 5, 2, 3, 96, 52, None), (300, 3, 0, 1, 40, 136, 64), (45, 2, 3, 4, 128, 64, 128),
    (17, 1, 2, 3, 64, 8, 16), (260, 12, 3, 4, 192, 80, None)])
def test_routed_feed_forward_part_against_the_plain_one(dtype, n, experts, identity, top, width, ff, shared):
    """The part as the layer calls it (no residual: the branch's float output), on both product paths: few rows
    run on the FP32 cores, many on the grouped tensor-core product."""
    from matricxon_b200.parts.base import Runtime, build_part
    from matricxon_b200.parts.spec import ClampedGluSpec, RoutedExpertsSpec

    gen = torch.Generator().manual_seed(n + experts)
    glu = lambda size, limit: ClampedGluSpec(hidden_size=width, intermediate_size=size, limit=limit, gate_name="gate",
                                             up_name="up", down_name="down", slope=1.702, shift=1.0)
    spec = RoutedExpertsSpec(hidden_size=width, num_experts=experts, top=top, num_groups=1, groups_kept=1, route_scale=1.0,
                             expert=glu(ff, 0.9), router_name="router", expert_format="e{index}.", norm_eps=1e-20,
                             score="softmax", correction_name="correction", num_identity=identity,
                             shared=glu(shared, 1.4) if shared else None, shared_name="shared.")
    part = build_part("feed_forward", spec, Runtime(DEVICE, dtype), "f.")
    w = {"f.router": torch.randn(experts + identity, width, generator=gen), "f.correction": torch.randn(experts + identity, generator=gen) * 0.1}
    for q, size in [(f"f.e{e}.", ff) for e in range(experts)] + ([("f.shared.", shared)] if shared else []):
        w[q + "gate"] = torch.randn(size, width, generator=gen) * 0.3
        w[q + "up"] = torch.randn(size, width, generator=gen) * 0.3
        w[q + "down"] = torch.randn(width, size, generator=gen) * 0.2
    floats = ("f.router", "f.correction")
    w = {k: (v if k in floats else v.to(dtype).float()) for k, v in w.items()}
    part.load(lambda name: w[name].to(DEVICE).to(torch.float32 if name in floats else dtype))
    h = torch.randn(n, width, generator=gen).to(dtype)

    class Ctx:
        status = torch.zeros(1, dtype=torch.int32, device=DEVICE)
        memo = {}

    got = part.forward(h.to(DEVICE), None, Ctx())
    got = (got if isinstance(got, torch.Tensor) else got.tensor()).cpu().double()
    f = {"expert": {"ff": ff, "limit": 0.9}, "router": {"experts": experts, "identity": identity, "top": top}}
    if shared:
        f["shared"] = {"ff": shared, "limit": 1.4}
    want = plain.mixture(h.double(), {k: v.double() for k, v in w.items()}, "f.", f)
    tol = 2e-4 if dtype == torch.float32 else 0.06
    assert torch.allclose(got, want, rtol=tol, atol=tol), (got - want).abs().max()
    assert int(Ctx.status.item()) == 0


# ---------------------------------------------------------------------- each mechanism alone, as a model of one layer
LAYERS_ALONE = {
    "window_with_kept_tokens": (attention(4, 2, 24, 8, 0.6, rot=(12, 1000.0), mask=(9, 3)), 0),
    "kept_tokens_beyond_a_page": (attention(3, 1, 8, 24, 0.9, rot=(8, 50.0), mask=(5, 21)), 0),
    "window_of_one": (attention(2, 2, 16, 16, 0.5, rot=(16, 100.0), mask=(1, 2)), 0),
    "window_without_kept_tokens": (attention(4, 4, 16, 16, 0.5, rot=(4, 30.0), mask=(17, 0)), 0),
    "no_window_no_rotation": (attention(4, 1, 32, 32, 0.3), 0),
    "tensor_core_head": (attention(4, 1, 64, 64, 0.2, rot=(64, 10000.0), mask=(20, 6)), 0),
    "tensor_core_head_128": (attention(2, 2, 128, 128, 0.12, rot=(32, 10000.0), mask=(24, 16)), 0),
    "keys_wider_than_values_64": (attention(2, 1, 64, 24, 0.2, rot=(16, 10000.0), mask=(33, 5)), 0),
    "experts_with_identity_and_shared": (attention(2, 2, 16, 16, 0.4, mlp=moe(40, 0.8, 5, 2, 2, shared=(56, 1.2))), 0),
    "experts_top_one_no_shared": (attention(2, 2, 16, 16, 0.4, mlp=moe(24, 2.0, 3, 0, 1)), 0),
    "experts_mostly_identity": (attention(2, 2, 16, 16, 0.4, mlp=moe(32, 0.5, 2, 3, 4, shared=(16, 3.0))), 0),
    "token_input": (attention(2, 2, 16, 16, 0.4), 10),
    "token_input_of_one": (attention(2, 2, 16, 16, 0.4, mlp=moe(24, 1.0, 2, 1, 2)), 1),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(LAYERS_ALONE))
def test_one_layer_models(name, dtype):
    """Whole, then one token at a time, then in portions: the three must agree with the plain model."""
    layer, side = LAYERS_ALONE[name]
    raw = single_layer(layer, width=64, vocab=120, side_dim=side)
    tensors = draw(raw, seed=len(name))
    run = Run(raw, tensors, dtype, max_tokens=256)
    tokens = ids(75, raw["vocab"], seed=1)
    run.feed("whole", tokens, [75])
    run.check("whole", tokens)
    run.feed("single", tokens[:60], [])
    run.check("single", tokens[:60])
    run.feed("cut", tokens, cycle)
    run.check("cut", tokens)


def _planted(window, keep, length, scale=0.8):
    """A one-layer model without rotation whose last token's query equals the key of one token that occurs
    nowhere else: where that token stands decides the last logits if and only if the last query sees it."""
    raw = single_layer(attention(2, 1, 32, 32, scale, mask=(window, keep)), width=64, vocab=90)
    tensors = draw(raw, seed=9)
    x88, x89 = tensors["embed"][88] * 2.5, tensors["embed"][89] * 2.5
    k88 = tensors["l0.mix.k"] @ x88
    tensors["l0.mix.q"] = (torch.outer(k88.repeat(2), x89) / (x89 @ x89)).contiguous()
    tensors["l0.ls1"] = torch.ones(64)
    tokens = [t % 86 for t in ids(length, 86, seed=2)]
    tokens[-1] = 89
    return raw, tensors, tokens


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("decode", [0, 50])
@pytest.mark.parametrize("window, keep, length", [(45, 12, 180), (16, 16, 100), (33, 3, 430), (64, 0, 200), (7, 50, 120)])
def test_a_token_decides_exactly_where_the_last_query_sees_it(window, keep, length, decode, dtype):
    """The asked-for token far back, at the window's two edges, at the kept tokens' two edges and at page
    borders, in a whole prompt and with the tail decoded token by token across page borders."""
    raw, tensors, tokens = _planted(window, keep, length)
    run = Run(raw, tensors, dtype, max_tokens=2 * (length + 64))
    last = length - 1
    places = {0, keep - 1, keep, keep + 1, 15, 16, 17, last - window - 20, last - window, last - window + 1,
              last - window + 2, last - 1}
    base = None
    for turn, place in enumerate([None] + sorted(p for p in places if 0 <= p < last)):
        planted = list(tokens)
        if place is not None:
            planted[place] = 88
        name = f"p{turn}"
        run.feed(name, planted, [length - decode] if decode else [length])
        run.check(name, planted)
        row = run.logits[(name, last)]
        if place is None:
            base = row
            continue
        moved = float(np.abs(row - base).max())
        if plain.visible(last, place, {"size": window, "keep_first": keep}):
            assert moved > 0.3, (place, moved)
        else:
            assert moved <= (1e-4 if dtype == "float32" else 0.02), (place, moved)


# ---------------------------------------------------------------------- whole models
@pytest.fixture(scope="module", params=[(n, d) for n in ("A", "B", "C") for d in ("float32", "bfloat16")],
                ids=lambda p: f"{p[0]}-{p[1]}")
def run(request):
    name, dtype = request.param
    raw = MODELS[name]
    # four live requests of at most 128 tokens: pages and slots must come back to be used again
    made = Run(raw, draw(raw, seed=11 + ord(name)), dtype, max_tokens=4 * 128, max_requests=4)
    yield made
    assert made.clear >= 2 * made.unclear, "most choices must have been clear enough to be compared"


LENGTHS = [1, 2, 17, 40, 65, 100, 128]


def prompts_of(run):
    return {f"r{n}": ids(n, run.raw["vocab"], seed=100 + n) for n in LENGTHS}


def test_whole_prompts(run):
    for request, tokens in prompts_of(run).items():
        run.feed(request + "w", tokens, [len(tokens)])
        run.check(request + "w", tokens)


def test_prefill_then_token_by_token(run):
    for request, tokens in prompts_of(run).items():
        head = max(len(tokens) - 70, 0)
        run.feed(request + "d", tokens, [head] if head else [])
        run.check(request + "d", tokens)


def test_portions_down_to_two_tokens(run):
    for shift, (request, tokens) in enumerate(prompts_of(run).items()):
        run.feed(request + "c", tokens, lambda turn: cycle(turn + shift))
        run.check(request + "c", tokens)
    tokens = prompts_of(run)["r65"]
    run.feed("pairs", tokens, lambda turn: 2)
    run.check("pairs", tokens)


def test_unequal_requests_batched_with_pages_and_slots_used_again(run):
    prompts = prompts_of(run)
    waiting = [(f"{request}m{again}", tokens) for again in range(2) for request, tokens in prompts.items()]
    tokens_of = dict(waiting)
    live: dict[str, int] = {}
    cache = run.replayer.core.cache
    turn = 0
    while waiting or live:
        while waiting and len(live) < 4:
            live[waiting.pop(0)[0]] = 0
        portions, ended = [], []
        for place, (request, done) in enumerate(list(live.items())):
            tokens = tokens_of[request]
            if (turn + place) % 5 == 4 and len(live) > 1:
                continue                                          # sits this step out
            remaining = len(tokens) - done
            size = 1 if (turn + place) % 3 == 0 else min(cycle(turn + place), remaining)
            portions.append((request, tokens[done:done + size]))
            live[request] = done + size
            if done + size == len(tokens):
                ended.append(request)
        turn += 1
        if portions:
            run.step(portions, end=ended)
        for request in ended:
            del live[request]
    for request, tokens in tokens_of.items():
        run.check(request, tokens)
    assert cache.pages_reused > 0
    assert len(set(run.slots_seen[r] for r in tokens_of)) <= 4 < len(tokens_of)


def test_long_decoding(run):
    """Hundreds of single-token steps (the captured decode step replayed) after a short prompt, two requests
    side by side, one of them starting later: every window passes over decoded tokens many times."""
    a = ids(260, run.raw["vocab"], seed=7)
    b = ids(150, run.raw["vocab"], seed=8)
    run.step([("la", a[:6])])
    for i in range(6, len(a)):
        portions = [("la", a[i:i + 1])]
        j = i - 100
        if 0 <= j < len(b):
            portions.append(("lb", b[j:j + 1]))
        ended = [name for name, k, seq in (("la", i, a), ("lb", j, b)) if k == len(seq) - 1]
        run.step(portions, end=ended)
    run.check("la", a)
    run.check("lb", b)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_prompts(dtype):
    """A prompt long enough for the prompt-sized product kernels and many attention tiles, windows of many
    chunks with kept tokens of more than one: whole, then in uneven portions with the tail decoded."""
    raw, length = MODELS["L"], 1100
    run = Run(raw, draw(raw, seed=21), dtype, max_tokens=2 * (length + 64))
    tokens = ids(length, raw["vocab"], seed=5)
    run.feed("whole", tokens, [length])
    slack = 0
    run.check("whole", tokens, allowed_over=slack)
    run.feed("cut", tokens, [length // 3 + 1, 2, length // 2, length - 40 - (length // 3 + 3 + length // 2)])
    run.check("cut", tokens, allowed_over=slack)


def test_greedy_generation_through_the_engine_entry_point():
    from matricxon_b200 import ChatEngine, GenerationRequest, SamplingConfig

    raw = MODELS["A"]
    tensors = draw(raw, seed=11)
    config = config_from_dict(copy.deepcopy(raw))
    model = model_from_tensors(config, tensors, dtype="float32", device=DEVICE)
    engine = ChatEngine(model, max_cache_tokens=4 * 128, max_active=3, max_batched_tokens=64, prefill_chunk=24,
                        max_model_len=128)
    prompts = [ids(n, raw["vocab"], seed=40 + n) for n in (5, 33, 70, 12, 50)]
    sampling = SamplingConfig(temperature=0.0, repeat_penalty=1.0, num_predict=24, num_ctx=128, seed=0)
    results = engine.generate_batch([GenerationRequest(input_ids=p, sampling=sampling) for p in prompts])
    for prompt, result in zip(prompts, results):
        assert result.finish_reason == "length" and len(result.token_ids) == 24
        logits = plain.forward(raw, tensors, prompt + result.token_ids[:-1]).numpy()
        for k, token in enumerate(result.token_ids):
            row = logits[len(prompt) - 1 + k]
            assert row[token] >= row.max() - 2e-3, (k, token, int(row.argmax()))


def test_trace_program_and_command_line(tmp_path):
    """The replay program itself on a model folder (bfloat16 file, both dtypes), and the generation command."""
    from matricxon_b200.weights.safetensors_io import write_safetensors

    raw = copy.deepcopy(MODELS["C"])
    tensors = draw(raw, seed=12, store_dtype=torch.bfloat16)
    folder = tmp_path / "model"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(raw))
    write_safetensors(folder / "model.safetensors", tensors.items())
    tokens = ids(50, raw["vocab"], seed=3)
    want = plain.forward(raw, {k: v.float() for k, v in tensors.items()}, tokens).numpy()
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": tokens[:31], "want": [0, 30]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": tokens[31:33], "want": []},
                                     {"id": "b", "tokens": tokens[:9], "want": [8]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": tokens[33:], "want": [16]}], "end": ["a"]}]
    for dtype in ("float32", "bfloat16"):
        out = tmp_path / dtype
        done = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype",
                               dtype, "--out", str(out), "--max-tokens", "128"],
                              input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True,
                              timeout=600)
        assert done.returncode == 0, done.stderr[-2000:]
        assert [line for line in done.stdout.splitlines() if line.startswith("done")] == ["done 0", "done 1", "done 2"]
        got = {s: np.fromfile(out / f"{s}.f32", dtype="<f4").reshape(-1, raw["vocab"]) for s in (0, 1, 2)}
        limit = limit_for(dtype, want)
        assert np.abs(got[0] - want[[0, 30]]).max() <= limit
        assert np.abs(got[1] - want[[8]]).max() <= limit
        assert np.abs(got[2] - want[[49]]).max() <= limit
    config_path = tmp_path / "config.json"
    config_path.write_text(json.dumps(MODELS["B"]))
    done = subprocess.run([sys.executable, "-m", "matricxon_b200.generate", "--random-config", str(config_path),
                           "--prompt-len", "20", "--num-predict", "12"], capture_output=True, text=True,
                          timeout=600, cwd=str(ROOT))
    assert done.returncode == 0, done.stderr[-2000:]
    assert "finish_reason:  length" in done.stdout and "Bafusun" in done.stdout


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden, dim, n", [(1000, 24, 13), (256, 130, 300), (2048, 8, 1), (96, 10, 40)])
def test_token_input_part_on_both_of_its_paths(dtype, hidden, dim, n):
    """The part as a layer calls it: narrow layers in one kernel, wide ones as two matrix products around a gate
    kernel; the same sums either way."""
    from matricxon_b200.parts.base import Runtime, build_part
    from matricxon_b200.parts.spec import TokenSideInputSpec

    gen = torch.Generator().manual_seed(hidden + dim)
    vocab, layers, layer = 37, 3, 1
    spec = TokenSideInputSpec(hidden_size=hidden, vocab_size=vocab, dim=dim, column=layer * dim, table_width=layers * dim,
                              eps=1e-4, table_name="side.embed", gate_name="gate", proj_name="proj", norm_name="norm")
    part = build_part("side_input", spec, Runtime(DEVICE, dtype), "l1.side.")
    w = {"side.embed": torch.randn(vocab, layers * dim, generator=gen) * 2, "l1.side.gate": torch.randn(dim, hidden, generator=gen) * 0.2,
         "l1.side.proj": torch.randn(hidden, dim, generator=gen) * 0.3, "l1.side.norm": torch.randn(hidden, generator=gen)}
    w = {k: (v if k.endswith("norm") else v.to(dtype).float()) for k, v in w.items()}
    part.load(lambda name: w[name].to(DEVICE).to(torch.float32 if name.endswith("norm") else dtype))
    x = torch.randn(n, hidden, generator=gen).to(dtype).float()          # the stream's rows are exact in both dtypes
    tokens = torch.randint(0, vocab, (n,), generator=gen)

    class Ctx:
        status = torch.zeros(1, dtype=torch.int32, device=DEVICE)
        token_ids = tokens.to(torch.int32).to(DEVICE)

    stream = x.clone().to(DEVICE)
    got, act = part.forward(stream, stream.to(dtype), Ctx())
    want = x.double() + plain.token_input(x.double(), tokens, {k: v.double() for k, v in w.items()}, layer, dim, 1e-4)
    tol = 3e-4 if dtype == torch.float32 else 0.03
    assert got is stream and int(Ctx.status.item()) == 0
    assert torch.allclose(stream.cpu().double(), want, rtol=tol, atol=tol), (stream.cpu().double() - want).abs().max()
    assert torch.equal(act, stream.to(dtype))
