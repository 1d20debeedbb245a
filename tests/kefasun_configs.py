"""Small Kefasun configurations of the tests (sizes, orders and constants of their own) and helpers that draw their
weights. Queries and keys are RMS-normalised with weights near one, so the sharpness of the softmax is set by the
configuration's ``scale``: the tests choose it so that single keys carry much of the weight and a key wrongly seen
or missed moves the logits."""

from __future__ import annotations

import copy

import torch

from matricxon_b200.config.registry import config_from_dict
from matricxon_b200.weights.random_init import RandomInit, random_tensors


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def blocks(heads, kv_heads, dim, vdim, scale, rot, size, mlp=None):
    """The block-masked kind; ``rot`` = (dims, base) or None."""
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": size}}
    if rot is not None:
        mixer["rot"] = {"dims": rot[0], "base": rot[1]}
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def capped(heads, kv_heads, dim, vdim, scale, rot, softcap, mlp=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "softcap": softcap}
    if rot is not None:
        mixer["rot"] = {"dims": rot[0], "base": rot[1]}
    return {"type": "attention_2", "mixer": mixer, "mlp": mlp}


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base, window, mlp=None):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
             "scale": scale, "rot": {"dims": rot_dim, "base": base}, "mask": {"size": window}}
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


def model(width, vocab, logit_scale, layers, loop=None, eps=1e-5):
    raw = {"architecture": "Kefasun", "width": width, "vocab": vocab, "logit_scale": logit_scale, "norm": {"eps": eps},
           "layers": layers}
    if loop is not None:
        raw["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return raw


# odd head sizes (keys wider and narrower than values), blocks shorter than a page and not a multiple of one, a
# window shorter than a page, a layer without a feed-forward, top 1 and top 3, a run of two layers repeated three
# times that starts at the first layer
MODEL_A = model(96, 211, 0.6, [
    blocks(6, 3, 24, 40, 0.5, (12, 1000.0), 11, mlp=moe(40, 5, 2)),
    latent(3, 24, 8, 20, 40, 32, 0.35, 300.0, 9, mlp=None),
    capped(4, 1, 40, 8, 0.5, (40, 50000.0), 3.0, mlp=dense(72)),
    latent(5, 16, 4, 16, 24, 48, 0.4, 10000.0, 37, mlp=moe(24, 3, 1)),
], loop=(0, 2, 3))

# head sizes that the tensor-core attention kernels take (64 and 128) and a latent whose rank they take, groups of
# four, two and one query heads, a block of one page, a run of one layer repeated twice in the middle, a logit
# scale of one, the capped kind first and the block-masked kind last
MODEL_B = model(128, 257, 1.0, [
    capped(8, 2, 64, 64, 0.15, (64, 10000.0), 30.0, mlp=moe(96, 4, 2)),
    blocks(4, 2, 128, 128, 0.1, (32, 700.0), 16, mlp=None),
    latent(4, 32, 16, 32, 64, 64, 0.2, 5000.0, 40, mlp=dense(160)),
    blocks(2, 2, 64, 128, 0.15, (16, 10000.0), 50, mlp=moe(64, 9, 3)),
], loop=(1, 2, 2))

# sizes that are multiples of nothing useful: width 100, odd vocabulary, heads of 12 and 20, six rotated entries,
# a latent of 20 with a rotated part of 6, a window of one, blocks of one position; no repeated run at all; a run
# that covers every layer once
MODEL_C = model(100, 131, 2.0, [
    blocks(5, 5, 12, 20, 0.7, (6, 90.0), 1, mlp=moe(52, 10, 3)),
    latent(2, 12, 6, 20, 28, 20, 0.5, 77.0, 1, mlp=moe(36, 2, 2)),
    capped(5, 1, 20, 12, 0.6, None, 1.5, mlp=None),
])
MODEL_D = model(64, 97, 1.5, [
    latent(9, 16, 8, 8, 16, 24, 0.4, 1000.0, 300, mlp=dense(48)),
    blocks(2, 1, 32, 32, 0.4, (32, 10000.0), 1000, mlp=dense(40)),
], loop=(0, 2, 1))

# a middle size for long prompts: products of more than a thousand rows, blocks and windows of many key chunks, heads
# of 64 in a group of four and of 128 in a group of two
MODEL_L = model(256, 512, 0.5, [
    blocks(8, 2, 64, 64, 0.15, (64, 10000.0), 300, mlp=moe(128, 8, 2)),
    latent(4, 64, 32, 64, 96, 128, 0.12, 10000.0, 200, mlp=moe(64, 6, 3)),
    capped(4, 2, 128, 128, 0.1, (128, 500000.0), 20.0, mlp=dense(384)),
    blocks(4, 2, 128, 128, 0.1, (64, 10000.0), 130, mlp=None),
], loop=(1, 3, 2))

MODELS = {"A": MODEL_A, "B": MODEL_B, "C": MODEL_C, "D": MODEL_D, "L": MODEL_L}
INIT = RandomInit(weight_std=0.08, bias_std=0.05, norm_weight_std=0.2, norm_bias_std=0.1)


def single_layer(layer: dict, width=64, vocab=120, logit_scale=1.5, loop=None) -> dict:
    return model(width, vocab, logit_scale, [copy.deepcopy(layer)], loop=loop)


def draw(raw: dict, seed: int, store_dtype=torch.float32, router_gain: float = 1.0) -> dict[str, torch.Tensor]:
    """Random weights with the tensors away from the values that hide them: router logits apart from one another
    with biases large enough to change the choice, sinks of both signs, pass vectors of a size that shows, an
    embedding of a few units. ``router_gain`` sharpens the routers further: with a large one, few tokens have two
    experts so close that 16-bit rounding decides between them."""
    tensors = random_tensors(config_from_dict(copy.deepcopy(raw)), seed, INIT, store_dtype)
    generator = torch.Generator().manual_seed(seed + 1)
    for name in tensors:
        shape = tensors[name].shape
        if name.endswith(".mlp.router"):
            tensors[name] = (tensors[name].float() * 4.0 * router_gain).to(store_dtype)
        elif name.endswith(".mlp.router.b"):
            tensors[name] = (torch.randn(shape, generator=generator) * 0.5 * router_gain).to(store_dtype)
        elif name.endswith(".mix.sink"):
            tensors[name] = (torch.randn(shape, generator=generator) * 1.5).to(store_dtype)
        elif name == "loop.step":
            tensors[name] = (torch.randn(shape, generator=generator) * 0.7).to(store_dtype)
        elif name == "embed":
            tensors[name] = (tensors[name].float() * 6.0).to(store_dtype)
        elif name.endswith(".gate") or name.endswith(".up") or name.endswith(".mix.g"):
            tensors[name] = (tensors[name].float() * 2.0).to(store_dtype)
    return tensors


def ids(count: int, vocab: int, seed: int) -> list[int]:
    generator = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (count,), generator=generator).tolist()
