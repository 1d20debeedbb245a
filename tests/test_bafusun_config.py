"""Bafusun on the CPU: configuration and registry, tensor names and shapes, the cache plan and its page rules,
errors that name the key, and properties of the plain model itself (tests/plain_bafusun.py), which is the
yardstick of the GPU tests."""

import copy
import math

import pytest
import torch

import plain_bafusun as plain
from bafusun_configs import MODELS, attention, draw, ids, model, moe, single_layer
from matricxon_b200.cache.manager import CacheManager, GroupRule
from matricxon_b200.config.bafusun import BafusunConfig
from matricxon_b200.config.base import ConfigError
from matricxon_b200.config.registry import config_from_dict, resolve_architecture
from matricxon_b200.models.decoder import model_weight_specs, plan_cache
from matricxon_b200.weights.loader import DictSource, WeightLoadError, check_weights

F64 = torch.float64


def test_registry_and_round_trip():
    for raw in MODELS.values():
        assert resolve_architecture(raw).config_class is BafusunConfig
        config = config_from_dict(copy.deepcopy(raw))
        assert config_from_dict(config.to_dict()) == config
    assert resolve_architecture({"model_type": "bafusun"}).name == "Bafusun"


def test_tensor_names_shapes_and_cache_plan():
    raw = MODELS["A"]
    config = config_from_dict(copy.deepcopy(raw))
    spec = config.model_spec()
    specs = model_weight_specs(spec)
    names = [s.name for s in specs]
    assert len(names) == len(set(names)), "the token table is one tensor however many layers read it"
    shapes = {s.name: tuple(s.shape) for s in specs}
    assert shapes["embed"] == (211, 96) and "head" not in shapes          # the logits come from the table itself
    assert shapes["side.embed"] == (211, 4 * 10) and shapes["final.norm"] == (96,)
    # layer 0: 6 heads over 3, keys 24 wide and values 40; 5 experts with matrices beside 2 without; a shared one
    assert shapes["l0.mix.q"] == (144, 96) and shapes["l0.mix.k"] == (72, 96) and shapes["l0.mix.v"] == (120, 96)
    assert shapes["l0.mix.o"] == (96, 240) and not any(n.endswith(".b") for n in shapes)
    assert shapes["l0.mlp.router"] == (7, 96) and shapes["l0.mlp.correction"] == (7,)
    assert shapes["l0.mlp.e4.gate"] == (40, 96) and shapes["l0.mlp.e4.down"] == (96, 40) and "l0.mlp.e5.gate" not in shapes
    assert shapes["l0.mlp.shared.up"] == (56, 96) and shapes["l0.mlp.shared.down"] == (96, 56)
    assert shapes["l0.norm1"] == (96,) and shapes["l0.ls1"] == (96,) and shapes["l0.ls2"] == (96,)
    assert shapes["l0.side.gate"] == (10, 96) and shapes["l0.side.proj"] == (96, 10) and shapes["l0.side.norm"] == (96,)
    # layer 1 has no feed-forward: no second norm, no second scale; it still takes its token input
    assert "l1.norm2" not in shapes and "l1.ls2" not in shapes and not any(n.startswith("l1.mlp") for n in shapes)
    assert shapes["l1.side.proj"] == (96, 10)
    # layer 2 has no shared expert and no identity experts
    assert shapes["l2.mlp.router"] == (3, 96) and "l2.mlp.shared.gate" not in shapes
    # layer 3: two experts with matrices, three without, four chosen
    assert shapes["l3.mlp.router"] == (5, 96) and "l3.mlp.e2.gate" not in shapes
    plan = plan_cache(spec)
    groups = sorted((g.request.num_kv_heads, g.request.head_dim, g.request.window, g.request.keep_first)
                    for g in plan.groups)
    # heads padded to the wider of key and value, rounded up to 16; kept tokens only under a window
    assert groups == [(1, 48, None, 0), (2, 48, 5, 21), (3, 16, 33, 0), (3, 48, 9, 3)]
    assert all(s is None for s in plan.state_of_entry)
    # a model without token input names no table
    config_b = config_from_dict(copy.deepcopy(MODELS["B"]))
    assert not any("side" in s.name for s in model_weight_specs(config_b.model_spec()))


def test_weight_errors_name_every_tensor():
    raw = MODELS["C"]
    tensors = draw(raw, 1)
    specs = model_weight_specs(config_from_dict(copy.deepcopy(raw)).model_spec())
    check_weights(specs, DictSource(tensors))
    broken = dict(tensors)
    del broken["l0.mlp.correction"]
    broken["l1.side.gate"] = torch.zeros(7, 99)
    broken["l0.mlp.e12.gate"] = torch.zeros(52, 100)             # an identity expert has no tensors
    with pytest.raises(WeightLoadError) as error:
        check_weights(specs, DictSource(broken))
    assert error.value.missing == ["l0.mlp.correction"] and error.value.unexpected == ["l0.mlp.e12.gate"]
    assert error.value.wrong_shape[0][0] == "l1.side.gate"


def test_second_norm_of_a_layer_without_feed_forward_may_lie_in_a_folder():
    raw = MODELS["A"]
    tensors = draw(raw, 1)
    config = config_from_dict(copy.deepcopy(raw))
    extra = dict(tensors)
    extra["l1.norm2"] = torch.ones(96)
    extra["l1.ls2"] = torch.ones(96)
    with pytest.raises(WeightLoadError):
        check_weights(model_weight_specs(config.model_spec()), DictSource(extra))
    shaped = config.with_tensor_shapes(lambda name: tuple(extra[name].shape) if name in extra else None)
    assert {name for name, _ in shaped.unused_tensors} == {"l1.norm2", "l1.ls2"}
    check_weights(model_weight_specs(shaped.model_spec()), DictSource(extra))
    bare = config.with_tensor_shapes(lambda name: tuple(tensors[name].shape) if name in tensors else None)
    assert bare.unused_tensors == ()


@pytest.mark.parametrize("change, needle", [
    (lambda r: r.pop("vocab"), "'vocab'"),
    (lambda r: r.pop("norm"), "'norm'"),
    (lambda r: r["layers"][0]["mixer"].pop("heads"), "'heads'"),
    (lambda r: r["layers"][0]["mixer"].update(kv_heads=4), "multiple of kv_heads"),
    (lambda r: r["layers"][0]["mixer"].pop("scale"), "'scale'"),
    (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=13), "'dims'"),
    (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=26), "'dims'"),
    (lambda r: r["layers"][0]["mixer"]["mask"].update(size=0), "'size'"),
    (lambda r: r["layers"][0]["mixer"].update(dim=300), "no attention kernel"),
    (lambda r: r["layers"][0]["mlp"]["router"].update(top=8), "'top'"),
    (lambda r: r["layers"][0]["mlp"]["expert"].pop("limit"), "'limit'"),
    (lambda r: r["layers"][0]["mlp"].update(kind="dense"), "unknown feed-forward kind"),
    (lambda r: r["layers"][1].update(type="recurrent"), "unknown layer type"),
    (lambda r: r.update(layers=[]), "'layers'"),
])
def test_configuration_errors_name_the_key(change, needle):
    raw = copy.deepcopy(MODELS["A"])
    change(raw)
    with pytest.raises(ConfigError) as error:
        config_from_dict(raw)
    assert needle in str(error.value)


def test_absent_keys_mean_absent_mechanisms():
    layer = attention(2, 2, 8, 8, 0.5)                   # no rotation, no mask, no feed-forward
    raw = model(32, 40, 1.0, 1.0, 0, [layer])
    del raw["embedding"], raw["logit_scale"]
    config = config_from_dict(raw)
    assert config.embedding_scale == 1.0 and config.logit_scale == 1.0 and config.side_dim == 0
    mixer = config.model_spec().layers[0].mixer
    assert mixer.position is None and mixer.window is None and mixer.keep_first == 0
    assert config.model_spec().layers[0].feed_forward is None and config.model_spec().layers[0].side_input is None
    assert config.model_spec().layers[0].ffn_norm is None


# ---------------------------------------------------------------------------- pages under a window that keeps
def test_pages_of_the_first_tokens_are_never_given_back():
    """Window 9 with 3 kept tokens and pages of 4: page 0 stays for good, the others leave as the window passes;
    with 0 kept tokens page 0 leaves too; with 6 kept tokens pages 0 and 1 stay."""
    for keep, held in ((3, {0}), (0, set()), (6, {0, 1}), (8, {0, 1})):
        cache = CacheManager([GroupRule(window=9, keep_first=keep)], [12], 4, 2)
        cache.add_request("a")
        length = 0
        for portion in (5, 1, 1, 7, 1, 1, 1, 13, 1):
            cache.reserve("a", portion)
            cache.commit("a", portion)
            length += portion
            table = cache.record("a").tables[0]
            # the next query stands at ``length`` and sees positions > length - 9: their pages are held
            first_needed = max(length - 9 + 1, 0) // 4
            for logical, page in enumerate(table):
                if logical in held or logical >= first_needed:
                    assert page >= 0, (keep, length, logical)
                else:
                    assert page < 0, (keep, length, logical)
            cache.check_invariants()
        cache.free_request("a")
        assert cache.free_pages() == [12]


# ---------------------------------------------------------------------------- the plain model's own properties
def test_plain_window_sees_its_last_keys_and_the_first_ones():
    mask = {"size": 4, "keep_first": 2}
    seen = [[plain.visible(i, j, mask) for j in range(9)] for i in range(9)]
    assert seen[8] == [True, True, False, False, False, True, True, True, True]
    assert seen[3] == [True, True, True, True] + [False] * 5           # the window still covers everything
    assert seen[5] == [True, True, True, True, True, True, False, False, False]
    assert torch.equal(plain.mask_matrix(torch.arange(9), mask), torch.tensor(seen))
    assert plain.visible(7, 0, {"size": 4, "keep_first": 0}) is False and plain.visible(7, 0, None) is True
    assert plain.visible(7, 4, {"size": 4}) and not plain.visible(7, 3, {"size": 4})


def test_plain_attention_rotates_the_first_entries_only_and_by_distance():
    gen = torch.Generator().manual_seed(3)
    x = torch.randn(6, 2, 10, generator=gen, dtype=F64)
    rot = {"dims": 6, "base": 50.0}
    turned = plain.rotate(x, torch.arange(6), rot)
    assert torch.equal(turned[..., 6:], x[..., 6:]) and torch.equal(turned[0], x[0])
    assert not torch.allclose(turned[1:, :, :6], x[1:, :, :6])
    # entry 1 pairs with entry 4 and turns by position * 50^(-2/6)
    a = 5 * 50.0 ** (-2.0 / 6)
    assert math.isclose(float(turned[5, 0, 1]), float(x[5, 0, 1] * math.cos(a) - x[5, 0, 4] * math.sin(a)), abs_tol=1e-12)
    assert math.isclose(float(turned[5, 0, 4]), float(x[5, 0, 4] * math.cos(a) + x[5, 0, 1] * math.sin(a)), abs_tol=1e-12)
    # scores depend on the distance alone: the same rows ten positions on give the same products
    later = plain.rotate(x, torch.arange(6) + 10, rot)
    assert torch.allclose(torch.einsum("thd,shd->hts", turned, turned), torch.einsum("thd,shd->hts", later, later))


def test_plain_scores_are_of_unit_norm_queries_and_keys():
    """Scaling a token's query or key rows changes nothing (beyond eps): the softmax's sharpness is the scale's."""
    gen = torch.Generator().manual_seed(4)
    q, k = torch.randn(7, 4, 12, generator=gen, dtype=F64), torch.randn(7, 2, 12, generator=gen, dtype=F64)
    m = {"heads": 4, "kv_heads": 2, "scale": 0.9, "rot": {"dims": 4, "base": 100.0}, "mask": {"size": 3, "keep_first": 1}}
    w = plain.attention_weights(q, k, m, 1e-12)
    assert torch.allclose(plain.attention_weights(q * 7.0, k * 0.1, m, 1e-12), w, atol=1e-9)
    assert torch.allclose(w.sum(-1), torch.ones(4, 7, dtype=F64))
    assert float(w[:, 6, 1:4].abs().max()) == 0.0 and float(w[:, 6, 0].min()) > 0.0
    # the largest possible score is scale * dim: two equal unit-norm rows
    same = plain.attention_weights(k[:, :1].repeat(1, 4, 1), k[:, :1], {**m, "kv_heads": 1, "rot": None, "mask": None}, 0.0)
    assert torch.allclose(same[0, 0, 0], torch.tensor(1.0, dtype=F64))


def test_plain_expert_clamps_gate_from_above_and_linear_branch_from_both_sides():
    w = {"e.gate": torch.eye(3, dtype=F64), "e.up": torch.eye(3, dtype=F64), "e.down": torch.eye(3, dtype=F64)}
    h = torch.tensor([[5.0, -5.0, 0.5]], dtype=F64)
    got = plain.clamped_expert(h, w, "e.", 2.0)
    sig = lambda g: 1.0 / (1.0 + math.exp(-1.702 * g))
    want = [2.0 * sig(2.0) * 3.0, -5.0 * sig(-5.0) * (-2.0 + 1.0), 0.5 * sig(0.5) * 1.5]
    assert torch.allclose(got, torch.tensor([want], dtype=F64))


def test_plain_routing_corrects_the_choice_and_not_the_weights():
    gen = torch.Generator().manual_seed(5)
    h = torch.randn(40, 16, generator=gen, dtype=F64)
    w = {"r.router": torch.randn(6, 16, generator=gen, dtype=F64), "r.correction": torch.zeros(6, dtype=F64)}
    router = {"experts": 4, "identity": 2, "top": 2}
    chosen, weights = plain.route(h, w, "r.", router)
    scores = torch.softmax(h @ w["r.router"].T, dim=-1)
    assert torch.equal(chosen, torch.topk(scores, 2).indices)
    assert torch.allclose(weights.sum(-1), torch.ones(40, dtype=F64))
    assert torch.allclose(weights[:, 0] / weights[:, 1], scores.gather(1, chosen)[:, 0] / scores.gather(1, chosen)[:, 1])
    w["r.correction"] = torch.tensor([0.0, 0.0, 0.0, 0.0, 0.0, 5.0], dtype=F64)
    chosen2, weights2 = plain.route(h, w, "r.", router)
    assert bool((chosen2[:, 0] == 5).all())                         # the correction decides the choice ...
    picked = scores.gather(1, chosen2)
    assert torch.allclose(weights2, picked / picked.sum(-1, keepdim=True))     # ... the weights never see it


def test_plain_identity_experts_return_their_input():
    """All experts without matrices and top = all of them: the routed sum is the input itself."""
    gen = torch.Generator().manual_seed(6)
    h = torch.randn(9, 8, generator=gen, dtype=F64)
    w = {"f.router": torch.randn(3, 8, generator=gen, dtype=F64), "f.correction": torch.randn(3, generator=gen, dtype=F64)}
    f = {"expert": {"ff": 4, "limit": 1.0}, "router": {"experts": 0, "identity": 3, "top": 3}}
    assert torch.allclose(plain.mixture(h, w, "f.", f), h)
    f["router"]["top"] = 1
    assert torch.allclose(plain.mixture(h, w, "f.", f), h)          # one weight, divided by itself


def test_plain_model_is_independent_of_what_follows_and_uses_every_tensor():
    raw = MODELS["A"]
    tensors = draw(raw, 3)
    tokens = ids(40, raw["vocab"], seed=1)
    whole, taps = plain.forward(raw, tensors, tokens, return_layers=True)
    assert taps.shape == (4, 40, 96)
    assert torch.allclose(plain.forward(raw, tensors, tokens[:23]), whole[:23], atol=1e-9)
    for name in ("l0.ls1", "l3.ls2", "l1.side.norm", "l0.mlp.correction", "l3.mlp.shared.down", "side.embed",
                 "l2.mlp.e1.up", "final.norm"):
        changed = dict(tensors)
        changed[name] = tensors[name] * 1.5 + 0.01
        assert not torch.allclose(plain.forward(raw, changed, tokens), whole, atol=1e-6), name
    # the logits come from the table without the embedding's scale, times the logit scale
    twice = copy.deepcopy(raw)
    twice["logit_scale"] = raw["logit_scale"] * 2
    assert torch.allclose(plain.forward(twice, tensors, tokens), whole * 2)


def test_plain_window_edge_decides_with_sharp_scores():
    """One layer, window 9 with 3 kept tokens: moving a token changes the last position's logits if and only
    if the last query sees it."""
    layer = attention(2, 1, 16, 16, 2.0, rot=(8, 100.0), mask=(9, 3))
    raw = single_layer(layer, width=32, vocab=50)
    tensors = draw(raw, 7)
    tokens = ids(30, 49, seed=2)
    base = plain.forward(raw, tensors, tokens)[-1]
    for j, seen in ((0, True), (2, True), (3, False), (20, False), (21, True), (28, True)):
        moved = list(tokens)
        moved[j] = 49
        delta = float((plain.forward(raw, tensors, moved)[-1] - base).abs().max())
        assert (delta > 1e-6) == seen, (j, delta)


def test_benchmark_configurations_describe_runnable_models():
    """The sizes ``bench.py --compare bafusun`` times: they parse, name every tensor once, plan one cache group
    under the window with its kept tokens, and keep no state."""
    import bench

    for size in bench.COMPARE_SIZES.values():
        config = config_from_dict(bench.bafusun_config(size))
        spec = config.model_spec()
        names = [s.name for s in model_weight_specs(spec)]
        assert len(names) == len(set(names))
        plan = plan_cache(spec)
        assert len(plan.groups) == 1 and plan.groups[0].request.head_dim == 128
        assert plan.groups[0].request.window == bench.COMPARE_WINDOW
        assert plan.groups[0].request.keep_first == bench.BAFUSUN_KEEP_FIRST
        assert all(s is None for s in plan.state_of_entry)


def test_plain_model_under_given_experts():
    """Handing the plain model its own choice changes nothing; another choice changes those positions; the
    margin says how far a router logit is from changing the choice."""
    raw = MODELS["C"]
    tensors = draw(raw, 4)
    tokens = ids(30, raw["vocab"], seed=9)
    margins, choices = [], []
    whole = plain.forward(raw, tensors, tokens, margins=margins, choices=choices)
    assert len(margins) == len(choices) == 2 and choices[0].shape == (30, 3) and margins[0].shape == (30,)
    assert float(margins[1].min()) == math.inf                      # two router outputs, both chosen
    assert float(margins[0].min()) > 0.0
    again = plain.forward(raw, tensors, tokens, forced=[c.tolist() for c in choices])
    assert torch.allclose(again, whole, atol=1e-12)
    other = [c.tolist() for c in choices]
    spare = [e for e in range(13) if e not in other[0][17]]
    other[0][17] = [spare[0]] + other[0][17][1:]
    moved = plain.forward(raw, tensors, tokens, forced=other)
    assert torch.allclose(moved[:17], whole[:17], atol=1e-12) and not torch.allclose(moved[17], whole[17], atol=1e-6)
