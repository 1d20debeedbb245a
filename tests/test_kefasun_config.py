"""Kefasun on the CPU: configuration, names, cache plan and schedule of the engine's description, and properties of
the plain implementation that the GPU tests measure against."""

import copy
import math

import pytest
import torch

import plain_kefasun as plain
from kefasun_configs import MODELS, blocks, capped, dense, draw, ids, latent, model, moe, single_layer
from matricxon_b200.config import ConfigError, config_from_dict, resolve_architecture
from matricxon_b200.config.kefasun import KefasunConfig
from matricxon_b200.models.decoder import model_weight_specs, plan_cache
from matricxon_b200.parts.rotary import paired_frequencies
from matricxon_b200.parts.spec import PairedRotarySpec

F64 = torch.float64


def doubles(tensors):
    return {name: value.double() for name, value in tensors.items()}


@pytest.mark.parametrize("name", list(MODELS))
def test_registry_and_round_trip(name):
    raw = MODELS[name]
    assert resolve_architecture(raw).config_class is KefasunConfig
    config = config_from_dict(copy.deepcopy(raw))
    assert config.to_dict() == raw
    assert config_from_dict(config.to_dict()) == config


def test_tensor_names_and_shapes():
    spec = config_from_dict(copy.deepcopy(MODELS["A"])).model_spec()
    shapes = {w.name: tuple(w.shape) for w in model_weight_specs(spec)}
    assert shapes["embed"] == (211, 96) and shapes["final.norm"] == (96,)
    assert shapes["loop.in"] == (96, 192) and shapes["loop.step"] == (3, 96)
    for fragment in ("norm1", "norm1b", "norm2", "norm2b"):
        assert shapes[f"l0.{fragment}"] == (96,)
    assert shapes["l0.mix.q"] == (144, 96) and shapes["l0.mix.k"] == (72, 96) and shapes["l0.mix.v"] == (120, 96)
    assert shapes["l0.mix.q.norm"] == (24,) and shapes["l0.mix.k.norm"] == (24,)
    assert shapes["l0.mix.g"] == (6, 96) and shapes["l0.mix.o"] == (96, 240)
    assert shapes["l0.mlp.router"] == (5, 96) and shapes["l0.mlp.router.b"] == (5,)
    assert shapes["l0.mlp.e4.gate"] == (40, 96) and shapes["l0.mlp.e4.down"] == (96, 40)
    assert shapes["l1.mix.dq"] == (40, 96) and shapes["l1.mix.dq.norm"] == (40,) and shapes["l1.mix.uq"] == (96, 40)
    assert shapes["l1.mix.dkv"] == (40, 96) and shapes["l1.mix.dkv.norm"] == (32,)
    assert shapes["l1.mix.uk"] == (72, 32) and shapes["l1.mix.uv"] == (60, 32) and shapes["l1.mix.sink"] == (3,)
    assert shapes["l1.mix.g"] == (60, 96) and shapes["l1.mix.o"] == (96, 60)
    assert "l1.norm2" not in shapes and "l1.mlp.gate" not in shapes           # a layer without a feed-forward
    assert shapes["l2.mix.g"] == (32, 96) and shapes["l2.mlp.gate"] == (72, 96) and shapes["l2.mlp.down"] == (96, 72)
    assert not any(name.endswith(".weight") for name in shapes)


def test_schedule_and_cache_plan():
    spec = config_from_dict(copy.deepcopy(MODELS["A"])).model_spec()
    assert [(e.layer, e.pass_index) for e in spec.schedule] == [(0, 0), (1, None), (0, 1), (1, None), (0, 2), (1, None),
                                                                 (2, None), (3, None)]
    plan = plan_cache(spec)
    by_request = {(g.request.num_kv_heads, g.request.head_dim, g.request.window, g.request.planes): g.entries
                  for g in plan.groups}
    assert by_request[(3, 48, None, 2)] == (0, 2, 4)              # every pass keeps a cache of its own
    assert [g.request.block for g in plan.groups if g.entries == (0, 2, 4)] == [11]      # pages live by blocks
    assert [g.request.block for g in plan.groups if g.entries == (6,)] == [None]
    assert by_request[(1, 40, 9, 1)] == (1, 3, 5)                 # latent + rotated part, one plane, windowed
    assert by_request[(1, 48, None, 2)] == (6,)
    assert by_request[(1, 52, 37, 1)] == (7,)
    middle = config_from_dict(copy.deepcopy(MODELS["B"])).model_spec()
    assert [(e.layer, e.pass_index) for e in middle.schedule] == [(0, None), (1, 0), (1, 1), (2, None), (3, None)]
    none = config_from_dict(copy.deepcopy(MODELS["C"])).model_spec()
    assert none.pass_input is None and [e.layer for e in none.schedule] == [0, 1, 2]
    assert [order for order in plain.layer_order(MODELS["A"])] == [(e.layer, e.pass_index) for e in spec.schedule]


def test_pages_of_blocks_the_sequence_has_left_come_back():
    from matricxon_b200.cache.manager import CacheManager, GroupRule

    cache = CacheManager([GroupRule(window=None, block=10), GroupRule(window=None)], [12, 12], 4, 2)
    cache.add_request("a")
    for tokens, held in ((9, [0, 1, 2]), (1, [2]), (7, [2, 3, 4]), (3, []), (19, [7, 8, 9])):
        cache.reserve("a", tokens)
        cache.commit("a", tokens)
        table = cache.record("a").tables[0]
        # after `length` tokens the next query sits in the block of position `length`: earlier pages are gone
        assert [lp for lp, page in enumerate(table) if page >= 0] == held, (cache.record("a").length, table)
        assert all(page >= 0 for page in cache.record("a").tables[1])
        cache.check_invariants()
    with pytest.raises(ValueError):
        GroupRule(window=5, block=5)


def test_tensors_fill_in_ranks_and_note_what_lies_unused():
    raw = copy.deepcopy(MODELS["C"])
    del raw["layers"][1]["mixer"]["q_rank"], raw["layers"][1]["mixer"]["kv_rank"]
    shapes = {"l1.mix.dq": (28, 100), "l1.mix.dkv": (26, 100), "l2.norm2": (100,), "l2.norm2b": (100,),
              "loop.in": (100, 200), "loop.step": (2, 100)}
    config = config_from_dict(raw).with_tensor_shapes(lambda name: shapes.get(name))
    assert (config.layers[1].q_rank, config.layers[1].kv_rank) == (28, 20)
    assert dict(config.unused_tensors) == {"l2.norm2": (100,), "l2.norm2b": (100,), "loop.in": (100, 200),
                                           "loop.step": (2, 100)}
    names = {w.name for w in model_weight_specs(config.model_spec())}
    assert {"l2.norm2", "loop.in"} <= names
    with pytest.raises(ConfigError, match="q_rank"):
        config_from_dict(raw).model_spec()


@pytest.mark.parametrize("change, key", [
    (lambda r: r["layers"][0].update(type="mamba"), "mamba"),
    (lambda r: r["layers"][0]["mixer"].pop("heads"), "heads"),
    (lambda r: r["layers"][0]["mixer"].update(kv_heads=4), "kv_heads"),
    (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=7), "dims"),
    (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=26), "dims"),
    (lambda r: r["layers"][1]["mixer"].pop("rot_dim"), "rot_dim"),
    (lambda r: r["layers"][2]["mixer"].pop("softcap"), "softcap"),
    (lambda r: r["layers"][0]["mlp"]["router"].update(top=6), "top"),
    (lambda r: r["layers"][2]["mlp"].update(kind="sparse"), "sparse"),
    (lambda r: r["loop"].update(stop=5), "loop"),
    (lambda r: r["loop"].update(times=0), "times"),
    (lambda r: r.pop("norm"), "norm"),
    (lambda r: r.pop("vocab"), "vocab"),
])
def test_errors_name_the_key(change, key):
    raw = copy.deepcopy(MODELS["A"])
    change(raw)
    with pytest.raises(ConfigError, match=key):
        config_from_dict(raw)


def test_absent_keys_mean_absent_mechanisms():
    raw = model(64, 50, 1.0, [blocks(2, 1, 16, 16, 0.3, None, 8)])
    del raw["layers"][0]["mixer"]["mask"]
    spec = config_from_dict(raw).model_spec()
    mixer = spec.layers[0].mixer
    assert mixer.position is None and mixer.mask == "causal" and mixer.sink == "zero" and mixer.gate == "head"
    assert spec.pass_input is None and spec.layers[0].feed_forward is None and spec.layers[0].ffn_out_norm is None
    looped = model(64, 50, 1.0, [blocks(2, 1, 16, 16, 0.3, None, 8)], loop=(1, 1, 4))      # an empty run repeats nothing
    assert config_from_dict(looped).model_spec().pass_input is None


def test_frequency_table_is_the_plain_one():
    for dims, base in ((40, 300000.0), (12, 70000.0), (6, 90.0), (2, 10.0)):
        table = paired_frequencies(PairedRotarySpec(rotary_dim=dims, theta=base))
        want = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)
        assert torch.equal(table, want)
    with pytest.raises(ValueError):
        PairedRotarySpec(rotary_dim=5, theta=10.0)
    with pytest.raises(ValueError):
        PairedRotarySpec(rotary_dim=4, theta=10.0, pairing="quarter")


# ---------------------------------------------------------------------- the plain model's own properties
def test_both_pairings_rotate_by_the_positions_distance():
    gen = torch.Generator().manual_seed(1)
    q, k = torch.randn(1, 12, generator=gen, dtype=F64), torch.randn(1, 12, generator=gen, dtype=F64)
    for layout in ("interleaved", "half"):
        def score(pq, pk):
            return float(plain.rotate(q, torch.tensor([pq]), 8, 100.0, layout)[0] @ plain.rotate(k, torch.tensor([pk]), 8, 100.0, layout)[0])
        assert abs(score(40, 33) - score(1007, 1000)) < 1e-9
        assert abs(score(40, 33) - score(40, 32)) > 1e-3
        turned = plain.rotate(q, torch.tensor([5]), 8, 100.0, layout)
        assert torch.equal(turned[0, 8:], q[0, 8:]) and not torch.allclose(turned[0, :8], q[0, :8])
    a = plain.rotate(q, torch.tensor([3]), 8, 100.0, "interleaved")[0]
    b = plain.rotate(q[:, [0, 2, 4, 6, 1, 3, 5, 7, 8, 9, 10, 11]], torch.tensor([3]), 8, 100.0, "half")[0]
    assert torch.allclose(a[[0, 2, 4, 6, 1, 3, 5, 7]], b[:8])


def test_visibility_rules():
    seen = plain.visible(12, "chunk", 5)
    assert seen[7].tolist() == [False] * 5 + [True] * 3 + [False] * 4
    assert seen[5].tolist() == [False] * 5 + [True] + [False] * 6
    assert seen[4].tolist() == [True] * 5 + [False] * 7
    window = plain.visible(12, "window", 3)
    assert window[7].tolist() == [False] * 5 + [True] * 3 + [False] * 4
    assert window[1].tolist() == [True, True] + [False] * 10
    assert plain.visible(4, "causal", 0)[2].tolist() == [True, True, True, False]


def test_sink_takes_weight_and_brings_nothing():
    scores = torch.tensor([[[1.0, 2.0, 0.5]]], dtype=F64)
    seen = torch.tensor([[True, True, True]])
    plain_weights = plain.attention_weights(scores, seen)
    assert abs(float(plain_weights.sum()) - 1.0) < 1e-12
    zero = plain.attention_weights(scores, seen, torch.zeros(1, dtype=F64))
    assert abs(float(zero.sum()) - (1 - 1 / (1 + float(torch.exp(scores).sum())))) < 1e-12
    big = plain.attention_weights(scores, seen, torch.tensor([50.0], dtype=F64))
    assert float(big.sum()) < 1e-18
    gone = plain.attention_weights(scores, seen, torch.tensor([-50.0], dtype=F64))
    assert torch.allclose(gone, plain_weights)


def test_router_takes_the_largest_logits_with_their_bias():
    h = torch.tensor([[1.0, 0.0], [0.0, 1.0]], dtype=F64)
    router = torch.tensor([[1.0, 0.0], [0.5, 0.2], [0.0, 1.0]], dtype=F64)
    bias = torch.tensor([0.0, 0.7, 0.0], dtype=F64)
    chosen, weights, margin = plain.route(h, router, bias, 2)
    assert chosen.tolist() == [[1, 0], [2, 1]]
    assert torch.allclose(weights[0], torch.softmax(torch.tensor([1.2, 1.0], dtype=F64), 0))
    assert abs(float(margin[0]) - 1.0) < 1e-12
    assert plain.route(h, router, torch.zeros(3, dtype=F64), 2)[0].tolist() == [[0, 1], [2, 1]]


def test_every_tensor_is_used_and_a_prefix_does_not_depend_on_what_follows():
    for name in ("A", "C"):
        raw = MODELS[name]
        weights = doubles(draw(raw, seed=5))
        tokens = ids(45, raw["vocab"], seed=2)
        full = plain.forward(raw, weights, tokens)
        assert torch.allclose(plain.forward(raw, weights, tokens[:30]), full[:30], atol=1e-9)
        for tensor in weights:
            changed = dict(weights)
            changed[tensor] = weights[tensor] * 1.5 + 0.01
            assert not torch.allclose(plain.forward(raw, changed, tokens), full, atol=1e-7), tensor


def test_the_pass_vector_and_the_embedding_enter_before_every_pass():
    raw = single_layer(blocks(2, 2, 16, 16, 0.4, (8, 100.0), 13, mlp=dense(40)), loop=(0, 1, 3))
    weights = doubles(draw(raw, seed=3))
    tokens = ids(20, raw["vocab"], seed=1)
    logits, taps = plain.forward(raw, weights, tokens, return_layers=True)
    assert taps.shape[0] == 3
    x0 = weights["embed"][tokens]
    first_in = torch.cat([x0, x0], -1) @ weights["loop.in"].T + weights["loop.step"][0]
    eps = raw["norm"]["eps"]
    mixed = plain.mixer("attention", plain.rms_norm(first_in, weights["l0.norm1"], eps), weights, "l0.mix.",
                        raw["layers"][0]["mixer"], eps)
    after_mixer = first_in + plain.rms_norm(mixed, weights["l0.norm1b"], eps)
    fed = plain.feed_forward(plain.rms_norm(after_mixer, weights["l0.norm2"], eps), weights, "l0.mlp.", raw["layers"][0]["mlp"])
    assert torch.allclose(taps[0], after_mixer + plain.rms_norm(fed, weights["l0.norm2b"], eps), atol=1e-10)
    for t in (1, 2):
        changed = dict(weights)
        step = weights["loop.step"].clone()
        step[t] += 1.0
        changed["loop.step"] = step
        other = plain.forward(raw, changed, tokens, return_layers=True)[1]
        assert torch.allclose(other[:t], taps[:t]) and not torch.allclose(other[t], taps[t])


def test_softcap_and_block_edges_in_the_plain_mixers():
    raw = single_layer(capped(2, 1, 16, 16, 1e6, None, 1.5))
    weights = doubles(draw(raw, seed=4))
    tokens = ids(30, raw["vocab"], seed=3)
    # a huge scale saturates every score at the cap: the weights become those of scores +-cap
    saturated = plain.forward(raw, weights, tokens)
    raw2 = copy.deepcopy(raw)
    raw2["layers"][0]["mixer"]["scale"] = 1e9
    assert torch.allclose(plain.forward(raw2, weights, tokens), saturated, atol=1e-6)
    edge = single_layer(blocks(2, 1, 16, 16, 0.5, None, 10))
    weights = doubles(draw(edge, seed=6))
    tokens = ids(30, edge["vocab"], seed=4)
    base = plain.forward(edge, weights, tokens)
    moved = list(tokens)
    moved[9] = (tokens[9] + 1) % edge["vocab"]
    other = plain.forward(edge, weights, moved)
    assert not torch.allclose(other[9], base[9]) and torch.allclose(other[10:], base[10:], atol=1e-12)
    assert math.isfinite(float(base.abs().max()))
