"""Kefasun written out plainly: every mechanism as one float64 function, no cache, no batching, no kernels.

The yardstick of the Kefasun tests. A model is (config dict as in ``config.json``, dict of float64 tensors by
checkpoint name); ``forward`` runs one whole sequence and returns logits at every position (and, on request, the
stream after every layer run). Nothing here is shared with the engine.

Notation: T tokens, positions p = 0 .. T-1; a matrix W is stored [out, in] and applied as ``x @ W.T``.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * weight over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * weight


def rotate(x, positions, dims, base, layout):
    """Rotates the first ``dims`` entries of the last axis of x [T, ..., D]; pair i is (2i, 2i+1) for
    ``interleaved`` and (i, i + dims/2) for ``half``; its angle at position p is p * base^(-2i/dims)."""
    if dims == 0:
        return x
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    angle = positions.to(F64)[:, None] * freq[None, :]                    # [T, half]
    while angle.dim() < x.dim():
        angle = angle.unsqueeze(1)
    cos, sin = torch.cos(angle), torch.sin(angle)
    out = x.clone()
    if layout == "interleaved":
        a, b = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = a * cos - b * sin
        out[..., 1:dims:2] = b * cos + a * sin
    elif layout == "half":
        a, b = x[..., :half], x[..., half:dims]
        out[..., :half] = a * cos - b * sin
        out[..., half:dims] = b * cos + a * sin
    else:
        raise ValueError(layout)
    return out


def visible(n, rule, size):
    """[n, n] bool: may the query at row i see the key at column j. ``causal``: j <= i; ``window``: also
    i - j < size; ``chunk``: also i // size == j // size."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    seen = j <= i
    if rule == "window":
        seen = seen & (i - j < size)
    elif rule == "chunk":
        seen = seen & (i // size == j // size)
    elif rule != "causal":
        raise ValueError(rule)
    return seen


def attention_weights(scores, seen, sink=None):
    """Softmax of scores [H, T, T] over the visible keys; ``sink`` [H] (or None) is a logit per head that joins
    the denominator and carries no value."""
    s = scores.masked_fill(~seen[None], -math.inf)
    m = s.max(dim=-1, keepdim=True).values
    if sink is not None:
        m = torch.maximum(m, sink.to(F64)[:, None, None])
    e = torch.exp(s - m)
    denom = e.sum(dim=-1, keepdim=True)
    if sink is not None:
        denom = denom + torch.exp(sink.to(F64)[:, None, None] - m)
    return e / denom


def grouped_attention(h, w, p, m, eps, *, layout, rule, sink_zero, softcap, gate_per_head):
    """The two grouped-query mixers. ``w``: tensors under prefix p; ``m``: the mixer's config."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = (h @ w[p + "q"].T).view(T, H, D)
    k = (h @ w[p + "k"].T).view(T, G, D)
    v = (h @ w[p + "v"].T).view(T, G, V)
    q = rms_norm(q, w[p + "q.norm"], eps)
    k = rms_norm(k, w[p + "k.norm"], eps)
    rot = m.get("rot")
    if rot:
        q = rotate(q, pos, rot["dims"], rot["base"], layout)
        k = rotate(k, pos, rot["dims"], rot["base"], layout)
    kv_of = torch.arange(H) // (H // G)
    scores = torch.einsum("ihd,jhd->hij", q, k[:, kv_of]) * m["scale"]
    if softcap is not None:
        scores = softcap * torch.tanh(scores / softcap)
    seen = visible(T, rule, m["mask"]["size"] if rule != "causal" else 0)
    sink = torch.zeros(H, dtype=F64) if sink_zero else None
    a = attention_weights(scores, seen, sink)
    o = torch.einsum("hij,jhv->ihv", a, v[:, kv_of])                      # [T, H, V]
    g = torch.sigmoid(h @ w[p + "g"].T)
    o = o * g[:, :, None] if gate_per_head else o * g.view(T, H, V)
    return o.reshape(T, H * V) @ w[p + "o"].T


def latent_attention(h, w, p, m, eps):
    T = h.shape[0]
    H, D, R, V, L = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    cq = rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].T).view(T, H, D + R)
    down = h @ w[p + "dkv"].T
    c = rms_norm(down[:, :L], w[p + "dkv.norm"], eps)
    base = m["rot"]["base"]
    kr = rotate(down[:, L:], pos, R, base, "interleaved")                 # [T, R], shared by the heads
    qr = rotate(q[..., D:], pos, R, base, "interleaved")
    kp = (c @ w[p + "uk"].T).view(T, H, D)
    v = (c @ w[p + "uv"].T).view(T, H, V)
    scores = (torch.einsum("ihd,jhd->hij", q[..., :D], kp) + torch.einsum("ihr,jr->hij", qr, kr)) * m["scale"]
    a = attention_weights(scores, visible(T, "window", m["mask"]["size"]), w[p + "sink"])
    o = torch.einsum("hij,jhv->ihv", a, v).reshape(T, H * V)
    return (o * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def mixer(kind, h, w, p, m, eps):
    if kind == "attention":
        return grouped_attention(h, w, p, m, eps, layout="interleaved", rule="chunk", sink_zero=True, softcap=None,
                                 gate_per_head=True)
    if kind == "attention_2":
        return grouped_attention(h, w, p, m, eps, layout="half", rule="causal", sink_zero=False,
                                 softcap=m["softcap"], gate_per_head=False)
    if kind == "latent_attention":
        return latent_attention(h, w, p, m, eps)
    raise ValueError(kind)


def silu_glu(h, gate, up, down):
    z = h @ gate.T
    return ((z * torch.sigmoid(z)) * (h @ up.T)) @ down.T


def route(h, router, bias, top):
    """(chosen experts [T, top], their weights, margin between the last chosen and the first unchosen logit)."""
    z = h @ router.T + bias
    order = torch.argsort(z, dim=-1, descending=True, stable=True)
    chosen = order[:, :top]
    picked = torch.gather(z, 1, chosen)
    weights = torch.softmax(picked, dim=-1)
    if z.shape[1] > top:
        margin = picked[:, -1] - torch.gather(z, 1, order[:, top:top + 1])[:, 0]
    else:
        margin = torch.full((h.shape[0],), math.inf, dtype=F64)
    return chosen, weights, margin


def feed_forward(h, w, p, f, forced=None, heard=None):
    """``f``: the layer's ``mlp`` config. ``forced`` [T, top]: expert choices to use instead of the router's own
    (weights are still the softmax over those experts' logits). ``heard``: a list that receives (the router's own
    choice, its margin) of a routed layer."""
    if f["kind"] == "dense":
        return silu_glu(h, w[p + "gate"], w[p + "up"], w[p + "down"])
    top = f["router"]["top"]
    z = h @ w[p + "router"].T + w[p + "router.b"]
    own, _, margin = route(h, w[p + "router"], w[p + "router.b"], top)
    if heard is not None:
        heard.append((own, margin))
    chosen = own if forced is None else torch.as_tensor(forced).long()
    weights = torch.softmax(torch.gather(z, 1, chosen), dim=-1)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for slot in range(top):
            e = int(chosen[t, slot])
            q = f"{p}e{e}."
            out[t] += weights[t, slot] * silu_glu(h[t:t + 1], w[q + "gate"], w[q + "up"], w[q + "down"])[0]
    return out


def layer_order(config):
    """[(layer index, pass number or None)] in the order of execution; a pass number marks the first layer of a
    pass of the repeated run."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, None) for i in range(start)]
    for t in range(times):
        order += [(i, t if i == start else None) for i in range(start, stop)]
    return order + [(i, None) for i in range(stop, n)]


def routed_runs(config):
    """The layer runs (indices into ``layer_order``) whose layer has routed experts, in order."""
    return [run for run, (i, _) in enumerate(layer_order(config))
            if (config["layers"][i].get("mlp") or {}).get("kind") == "moe"]


def forward(config, w, tokens, return_layers=False, forced=None, heard=None):
    """Logits [T, vocab] of one sequence. ``forced``: {layer-run index: [T, top] expert choices}; ``heard``: a list
    that receives (own choice, margin) of every routed layer run."""
    eps = config["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)].to(F64)
    x0 = x.clone()
    taps = []
    for run, (i, begins_pass) in enumerate(layer_order(config)):
        if begins_pass is not None:
            x = torch.cat([x, x0], dim=-1) @ w["loop.in"].T + w["loop.step"][begins_pass]
        layer = config["layers"][i]
        p = f"l{i}."
        x = x + rms_norm(mixer(layer["type"], rms_norm(x, w[p + "norm1"], eps), w, p + "mix.", layer["mixer"], eps),
                         w[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            fed = feed_forward(rms_norm(x, w[p + "norm2"], eps), w, p + "mlp.", layer["mlp"],
                               None if forced is None else forced.get(run), heard)
            x = x + rms_norm(fed, w[p + "norm2b"], eps)
        taps.append(x.clone())
    logits = (rms_norm(x, w["final.norm"], eps) @ w["embed"].T) * config.get("logit_scale", 1.0)
    return (logits, torch.stack(taps)) if return_layers else logits
