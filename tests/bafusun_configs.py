"""Small Bafusun configurations of the tests (sizes, orders and constants of their own) and helpers that draw
their weights. Queries and keys of this design have unit root mean square, so the sharpness of the softmax is set
by the configuration's ``scale`` alone: the tests choose it so that single keys carry most of the weight and a
key wrongly seen or missed moves the logits."""

from __future__ import annotations

import copy

import torch

from matricxon_b200.config.registry import config_from_dict
from matricxon_b200.weights.random_init import RandomInit, random_tensors


def moe(ff, limit, experts, identity, top, shared=None):
    """``shared`` = (ff, limit) or None."""
    out = {"kind": "moe", "expert": {"ff": ff, "limit": limit},
           "router": {"experts": experts, "identity": identity, "top": top}}
    if shared is not None:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


def attention(heads, kv_heads, dim, vdim, scale, rot=None, mask=None, mlp=None):
    """``rot`` = (dims, base) or None; ``mask`` = (size, keep_first) or None."""
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot is not None:
        mixer["rot"] = {"dims": rot[0], "base": rot[1]}
    if mask is not None:
        mixer["mask"] = {"size": mask[0], "keep_first": mask[1]}
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def model(width, vocab, embedding_scale, logit_scale, side_dim, layers, eps=1e-5):
    raw = {"architecture": "Bafusun", "width": width, "vocab": vocab, "embedding": {"scale": embedding_scale},
           "logit_scale": logit_scale, "norm": {"eps": eps}, "layers": layers}
    if side_dim:
        raw["token_side"] = {"dim": side_dim}
    return raw


# odd head sizes (keys wider and narrower than values), a window shorter than a page with a few kept tokens, a
# layer that sees everything and has no feed-forward, a window without kept tokens, more kept tokens than the
# window is long, a router with and without identity experts, with and without a shared expert, top 1 and a top
# that must take identity experts
MODEL_A = model(96, 211, 1.7, 0.6, 10, [
    attention(6, 3, 24, 40, 0.55, rot=(12, 1000.0), mask=(9, 3),
              mlp=moe(40, 0.8, 5, 2, 2, shared=(56, 1.2))),
    attention(4, 1, 40, 8, 0.4, rot=(40, 50000.0), mask=None, mlp=None),
    attention(3, 3, 16, 16, 0.7, rot=None, mask=(33, 0), mlp=moe(24, 2.0, 3, 0, 1)),
    attention(2, 2, 48, 48, 0.35, rot=(16, 300.0), mask=(5, 21), mlp=moe(32, 0.5, 2, 3, 4, shared=(16, 3.0))),
])

# head sizes that the tensor-core attention kernels take (64 and 128), groups of four, two and one query heads,
# kept tokens that end inside a page, at a page's border and beyond the window, one layer that sees everything;
# no token input, embedding and logit scales of one
MODEL_B = model(128, 257, 1.0, 1.0, 0, [
    attention(8, 2, 64, 64, 0.3, rot=(64, 10000.0), mask=(37, 18), mlp=moe(96, 1.0, 4, 1, 2, shared=(64, 1.0))),
    attention(4, 2, 128, 128, 0.2, rot=(32, 700.0), mask=(70, 5), mlp=None),
    attention(2, 2, 64, 128, 0.3, rot=(16, 10000.0), mask=(16, 32), mlp=moe(64, 4.0, 9, 0, 3)),
    attention(4, 1, 128, 64, 0.2, rot=None, mask=None, mlp=moe(72, 1.0, 2, 2, 1, shared=(128, 0.7))),
    attention(4, 4, 128, 128, 0.2, rot=(128, 100000.0), mask=(48, 0), mlp=None),
])

# sizes that are multiples of nothing useful: width 100, odd vocabulary, heads of 12 and 20, six rotated entries
MODEL_C = model(100, 131, 3.0, 2.0, 7, [
    attention(5, 5, 12, 20, 0.8, rot=(6, 90.0), mask=(21, 2), mlp=moe(52, 1.5, 10, 3, 3, shared=(44, 1.0))),
    attention(5, 1, 20, 12, 0.6, rot=(20, 10000.0), mask=(1, 1), mlp=moe(36, 1.0, 1, 1, 2)),
])

# a middle size for long prompts: products of more than a thousand rows, windows of many chunks with kept tokens
# of more than one chunk, heads of 64 in a group of four and of 128 in a group of two
MODEL_L = model(256, 512, 2.0, 0.5, 16, [
    attention(8, 2, 64, 64, 0.3, rot=(64, 10000.0), mask=(130, 40), mlp=moe(128, 1.0, 8, 2, 2, shared=(256, 2.0))),
    attention(4, 2, 128, 128, 0.2, rot=(64, 10000.0), mask=(300, 70), mlp=moe(64, 1.0, 6, 0, 3)),
    attention(4, 2, 128, 128, 0.2, rot=(128, 500000.0), mask=(200, 0), mlp=None),
])

MODELS = {"A": MODEL_A, "B": MODEL_B, "C": MODEL_C, "L": MODEL_L}
INIT = RandomInit(weight_std=0.08, bias_std=0.05, norm_weight_std=0.2, norm_bias_std=0.1)


def single_layer(layer: dict, width=64, vocab=120, embedding_scale=2.5, logit_scale=1.5, side_dim=0) -> dict:
    return model(width, vocab, embedding_scale, logit_scale, side_dim, [copy.deepcopy(layer)])


def draw(raw: dict, seed: int, store_dtype=torch.float32, router_gain: float = 1.0) -> dict[str, torch.Tensor]:
    """Random weights with the tensors away from the values that hide them: router scores apart from one
    another, a correction large enough to change the choice, branch scales of both signs, logits of a few units.
    ``router_gain`` sharpens the routers further: with a large one, few tokens have two experts so close that
    16-bit rounding decides between them."""
    tensors = random_tensors(config_from_dict(copy.deepcopy(raw)), seed, INIT, store_dtype)
    generator = torch.Generator().manual_seed(seed + 1)
    for name in tensors:
        shape = tensors[name].shape
        if name.endswith(".mlp.router"):
            tensors[name] = (tensors[name].float() * 4.0 * router_gain).to(store_dtype)
        elif name.endswith(".mlp.correction"):
            tensors[name] = (torch.randn(shape, generator=generator) * 0.15).to(store_dtype)
        elif name.endswith(".ls1") or name.endswith(".ls2"):
            tensors[name] = (torch.randn(shape, generator=generator) * 0.6).to(store_dtype)
        elif name == "embed":
            tensors[name] = (tensors[name].float() * 6.0).to(store_dtype)
        elif name == "side.embed":
            tensors[name] = (tensors[name].float() * 8.0).to(store_dtype)
        elif name.endswith(".gate") or name.endswith(".up"):
            tensors[name] = (tensors[name].float() * 2.0).to(store_dtype)      # some entries reach the clamps
    return tensors


def ids(count: int, vocab: int, seed: int) -> list[int]:
    generator = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (count,), generator=generator).tolist()
