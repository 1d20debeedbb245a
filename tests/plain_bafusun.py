"""A plain, slow Bafusun: every mechanism as one function of float64 tensors, one sequence at a time.

This is the yardstick the engine's Bafusun parts are compared with. It shares no code with the
package: it takes a configuration as the plain dictionary that ``config.json`` holds and weights as
a name -> tensor dictionary, keeps no cache (every call sees the whole sequence) and runs on the CPU.

Notation: x is the [T, width] residual stream of one sequence, positions count from 0, a sublayer
reads x itself and its result is normalised, scaled entry by entry and added:
``x <- x + ls * norm(sublayer(x))``.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def layer_norm(x, weight, eps):
    """Mean taken off, divided by the root of the mean squared deviation (eps inside), times a weight."""
    centred = x - x.mean(dim=-1, keepdim=True)
    return centred / torch.sqrt((centred * centred).mean(dim=-1, keepdim=True) + eps) * weight


def rms_unit(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


# ---------------------------------------------------------------------------- rotary positions
def rotate(x, positions, rot):
    """x [T, heads, n]: entry i < dims/2 of every head is paired with entry i + dims/2 and the pair is turned
    by ``position * base^(-2i/dims)``; the entries from ``dims`` on pass unchanged."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    if half == 0:
        return x
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    angle = positions.to(F64)[:, None] * freq[None, :]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], dim=-1)


# ---------------------------------------------------------------------------- attention
def visible(i: int, j: int, mask: dict | None) -> bool:
    """Whether the query at position i sees the key at position j: never the future; with a mask, the last
    ``size`` positions (its own among them) and, wherever the query stands, the first ``keep_first`` ones."""
    if j > i:
        return False
    if mask is None:
        return True
    return i - j < int(mask["size"]) or j < int(mask.get("keep_first", 0))


def mask_matrix(positions, mask: dict | None):
    """``visible`` for every (query, key) pair at once: a boolean [T, T]."""
    i, j = positions[:, None], positions[None, :]
    seen = j <= i
    if mask is not None:
        seen = seen & ((i - j < int(mask["size"])) | (j < int(mask.get("keep_first", 0))))
    return seen


def attention_weights(q, k, m, eps, positions=None):
    """Softmax weights [heads, T, T] from projected q [T, heads, dim] and k [T, kv heads, dim]: rotation, then
    every head divided by its root mean square, scaled scores, the mask, an ordinary softmax."""
    T, H, G = q.shape[0], int(m["heads"]), int(m["kv_heads"])
    if positions is None:
        positions = torch.arange(T)
    rot = m.get("rot")
    if rot is not None:
        q, k = rotate(q, positions, rot), rotate(k, positions, rot)
    q, k = rms_unit(q, eps), rms_unit(k, eps)
    seen = mask_matrix(positions, m.get("mask"))
    weights = torch.zeros((H, T, T), dtype=F64)
    for h in range(H):
        g = h // (H // G)
        scores = (q[:, h] @ k[:, g].T) * float(m["scale"])
        weights[h] = torch.softmax(scores.masked_fill(~seen, -math.inf), dim=-1)
    return weights


def attention(x, w, p, m, eps):
    """The attention mixer on a whole sequence: [T, width] -> [T, width]."""
    T, H, G = x.shape[0], int(m["heads"]), int(m["kv_heads"])
    dim, vdim = int(m["dim"]), int(m.get("vdim", m["dim"]))
    q = (x @ w[p + "q"].T).view(T, H, dim)
    k = (x @ w[p + "k"].T).view(T, G, dim)
    v = (x @ w[p + "v"].T).view(T, G, vdim)
    weights = attention_weights(q, k, m, eps)
    heads = [weights[h] @ v[:, h // (H // G)] for h in range(H)]
    return torch.cat(heads, dim=-1) @ w[p + "o"].T


# ---------------------------------------------------------------------------- feed-forward
def clamped_expert(h, w, p, limit):
    """One gated feed-forward: the gate capped from above, the linear branch from both sides."""
    g = torch.clamp(h @ w[p + "gate"].T, max=float(limit))
    u = torch.clamp(h @ w[p + "up"].T, min=-float(limit), max=float(limit))
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def route(h, w, p, router):
    """(chosen [T, top], weights [T, top]): softmax over all router outputs; the choice adds the correction,
    the weights do not; the chosen scores are divided by their sum."""
    scores = torch.softmax(h @ w[p + "router"].T, dim=-1)
    choice = scores + w[p + "correction"]
    chosen = torch.topk(choice, int(router["top"]), dim=-1).indices
    picked = torch.gather(scores, 1, chosen)
    return chosen, picked / (picked.sum(dim=-1, keepdim=True) + 1e-20)


def choice_margin(h, w, p, router):
    """Per token, by how much a router logit would have to move for the last chosen expert and the best one not
    chosen to change places (infinite when all are chosen): the gap of their choice scores over the sum of their
    plain scores, since a logit's change of d moves a score s by about s d."""
    scores = torch.softmax(h @ w[p + "router"].T, dim=-1)
    top = int(router["top"])
    if top >= scores.shape[-1]:
        return torch.full((h.shape[0],), math.inf, dtype=F64)
    best, index = torch.sort(scores + w[p + "correction"], dim=-1, descending=True)
    both = scores.gather(1, index[:, top - 1:top + 1]).sum(dim=-1)
    return (best[:, top - 1] - best[:, top]) / both


def mixture(h, w, p, f, margins=None, forced=None, choices=None):
    """The routed feed-forward: the last ``identity`` router outputs stand for experts that return their input.
    ``margins``: a list that receives ``choice_margin`` of this call. ``forced`` [T, top]: experts to use in
    place of the router's own choice (their weights are still their plain scores over their sum); ``choices``
    receives the router's own choice all the same."""
    router = f["router"]
    real = int(router["experts"])
    chosen, weights = route(h, w, p, router)
    if choices is not None:
        choices.append(chosen)
    if forced is not None:
        chosen = torch.as_tensor(forced, dtype=torch.long)
        picked = torch.gather(torch.softmax(h @ w[p + "router"].T, dim=-1), 1, chosen)
        weights = picked / (picked.sum(dim=-1, keepdim=True) + 1e-20)
    if margins is not None:
        margins.append(choice_margin(h, w, p, router))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, weight in zip(chosen[t].tolist(), weights[t]):
            if e >= real:
                out[t] += weight * h[t]
            else:
                out[t] += weight * clamped_expert(h[t:t + 1], w, f"{p}e{e}.", f["expert"]["limit"])[0]
    if f.get("shared") is not None:
        out = out + clamped_expert(h, w, p + "shared.", f["shared"]["limit"])
    return out


# ---------------------------------------------------------------------------- per-layer token input
def token_input(x, tokens, w, layer: int, dim: int, eps):
    """What a layer adds from the token itself: the layer's slice of a second embedding, gated by the stream,
    projected to the width, divided by its root mean square and scaled."""
    p = f"l{layer}.side."
    e = w["side.embed"][tokens][:, layer * dim:(layer + 1) * dim]
    y = (gelu_tanh(x @ w[p + "gate"].T) * e) @ w[p + "proj"].T
    return rms_unit(y, eps) * w[p + "norm"]


# ---------------------------------------------------------------------------- the model
def to_f64(weights: dict) -> dict:
    return {name: (t.to(F64) if t.is_floating_point() else t) for name, t in weights.items()}


def forward(config: dict, weights: dict, tokens, return_layers: bool = False, margins: list | None = None,
            forced: list | None = None, choices: list | None = None):
    """Logits [T, vocab] of one whole sequence (and, when asked, the stream after every layer). ``margins``
    receives every routed layer's ``choice_margin`` and ``choices`` its router's own choice; ``forced`` gives
    every routed layer's experts, layer by layer (``mixture``)."""
    w = to_f64(weights)
    eps = float(config["norm"]["eps"])
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    x = w["embed"][tokens] * float(config.get("embedding", {}).get("scale", 1.0))
    side = config.get("token_side")
    taps, routed = [], 0
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        if layer["type"] != "attention":
            raise ValueError(f"unknown layer type {layer['type']!r}")
        mixed = attention(x, w, p + "mix.", layer["mixer"], eps)
        x = x + layer_norm(mixed, w[p + "norm1"], eps) * w[p + "ls1"]
        if layer.get("mlp") is not None:
            fed = mixture(x, w, p + "mlp.", layer["mlp"], margins, forced[routed] if forced is not None else None,
                          choices)
            routed += 1
            x = x + layer_norm(fed, w[p + "norm2"], eps) * w[p + "ls2"]
        if side is not None:
            x = x + token_input(x, tokens, w, i, int(side["dim"]), eps)
        taps.append(x)
    logits = layer_norm(x, w["final.norm"], eps) @ w["embed"].T * float(config.get("logit_scale", 1.0))
    return (logits, torch.stack(taps)) if return_layers else logits
