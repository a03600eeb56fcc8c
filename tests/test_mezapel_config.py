"""Host-side tests of the Mezapel configuration, its model plan, the tensors the plan asks for, what
the cache keeps, the rotation tables, and the plain implementation's own mechanisms (no GPU)."""

import copy
import math

import pytest
import torch

import mezapel_tiny as mz
import plain_mezapel as plain
from freetoken_b200.cache import CacheManager, StateNeed
from freetoken_b200.cache.manager import CompositeNeed, PagedKVNeed
from freetoken_b200.config.mezapel import MezapelConfig, build_plan
from freetoken_b200.config.model_plan import ConfigError
from freetoken_b200.models.model import Model
from freetoken_b200.parts.position import rotary_table, scaled_frequencies
from freetoken_b200.registry import architecture_of
from freetoken_b200.weights.loader import WeightError, plan_loading
from freetoken_b200.weights.spec import leaves


def test_registry_picks_the_design_by_its_singular_key():
    arch = architecture_of(mz.MZ_A)
    assert arch.name == "Mezapel"
    cfg = arch.read_config(mz.MZ_A)
    assert isinstance(cfg, MezapelConfig) and cfg.to_dict() == mz.MZ_A


@pytest.mark.parametrize("which", list(mz.MZ))
def test_plan_hands_every_constant_to_a_part(which):
    raw = mz.MZ[which]
    cfg = MezapelConfig.from_dict(raw)
    plan = build_plan(cfg)
    assert plan.residual_streams == (raw.get("streams") or 1)
    assert [s.layer for s in plan.schedule] == plain.run_order(raw)
    assert all(s.owns_cache for s in plan.schedule)
    assert plan.final_norm.kind == "hyper_norm" and plan.final_norm.params["connection"] is None
    e, big = plan.embedding.params, raw["embedding"].get("bigram")
    assert e["scale"] == raw["embedding"]["scale"]
    if big:
        assert (e["pair_tensor"], e["buckets"], e["mul_prev"], e["mul_cur"]) == \
            ("bigram", big["buckets"], big["mul_prev"], big["mul_cur"])
    else:
        assert "pair_tensor" not in e
    for i, (spec, layer) in enumerate(zip(plan.layers, raw["layers"])):
        assert spec.block.kind == "hyper" and spec.mixer.kind == "paged_attention"
        assert (spec.feed_forward is None) == (layer["mlp"] is None)
        for q, n in ((1, spec.all_norms()["mixer"]), (2, spec.all_norms().get("feed_forward"))):
            if n is None:
                continue
            assert (n.params["eps"], n.params["center"], n.params["tensor"]) == (raw["norm"]["eps"], True, f"norm{q}")
            assert n.params["connection"] == (f"hc{q}" if "streams" in raw else "identity")
        m, p = layer["mixer"], spec.mixer.params
        assert (p["num_heads"], p["num_kv_heads"], p["head_dim"], p["value_dim"], p["sm_scale"], p["qk_norm_eps"]) == \
            (m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["scale"], raw["norm"]["eps"])
        assert p["fill_heads"] is True
        pos = p["position"]
        assert (pos.kind, pos.params["rotary_dim"], pos.params["theta"]) == ("rotary_neox", m["rot"]["dims"], m["rot"]["base"])
        scaling = m["rot"].get("scaling") if m["rot"]["dims"] else None
        if layer["type"] == "attention":
            assert (p["qk_norm"], p["chunk"], p["sink_value"], p["gate"]) == ("per_layer", m["mask"]["size"], 0.0, "head")
            assert not p.get("sliding_window") and not p.get("softcap") and not p.get("conv_taps") and not p.get("sink")
            want = {"kind": "yarn", **scaling} if scaling else None
        else:
            assert (p["qk_norm"], p["sliding_window"], p["sink"], p["gate"], p["conv_taps"]) == \
                ("per_head", m["mask"]["size"], True, "element", m.get("conv", 0))
            assert (p["softcap"] or 0.0) == m.get("softcap", 0.0) and not p.get("chunk") and p.get("sink_value") is None
            want = {"kind": "llama3", **scaling} if scaling else None
        assert pos.params["scaling"] == want
        if layer["mlp"]:
            f = spec.feed_forward.params
            assert (spec.feed_forward.kind, f["intermediate_size"], f["activation"], f["gated"]) == \
                ("dense_mlp", layer["mlp"]["ff"], "silu", True)


@pytest.mark.parametrize("which", list(mz.MZ))
def test_the_plan_asks_for_exactly_the_tensors_of_a_checkpoint(which):
    raw = mz.MZ[which]
    model = Model(build_plan(MezapelConfig.from_dict(raw)))
    asked = {}
    for spec in model.tensor_specs():
        for leaf in leaves(spec.all_sources()[0]):
            asked[leaf.name] = tuple(leaf.shape)
    assert asked == plain.expected_tensors(raw)
    shapes = dict(asked)
    plan_loading(model.tensor_specs(), shapes)
    first = next(iter(sorted(shapes)))
    del shapes[first]
    shapes["l0.mix.stranger"] = (3,)
    with pytest.raises(WeightError) as err:
        plan_loading(model.tensor_specs(), shapes)
    assert first in err.value.missing and "l0.mix.stranger" in err.value.unexpected


def test_cache_needs_pages_conv_inputs_and_the_last_token():
    raw = mz.MZ_A
    model = Model(build_plan(MezapelConfig.from_dict(raw)))
    needs = model.cache_needs()
    order = plain.run_order(raw)
    assert len(needs) == len(order) + 1 and needs[-1] == StateNeed((1,), "int32")      # the hashed table's previous token
    for need, i in zip(needs, order):
        m = raw["layers"][i]["mixer"]
        d = max(m["dim"], m["vdim"])
        paged = PagedKVNeed(m["kv_heads"], d, m["mask"]["size"])
        if m.get("conv", 0) > 1:
            assert need == CompositeNeed((paged, StateNeed(((m["conv"] - 1) * (m["heads"] + 2 * m["kv_heads"]) * d,))))
        else:
            assert need == paged
    assert len(Model(build_plan(MezapelConfig.from_dict(mz.MZ_C))).cache_needs()) == len(plain.run_order(mz.MZ_C))
    cache = CacheManager(needs, 4, 20, 2, 64)
    cache.admit("a")
    cache.grow("a", 30)
    cache.advance("a", 30)
    assert cache.held_pages("a")[0] < 8        # chunks that are over gave their pages back
    cache.release("a")
    assert cache.free_pages() == cache.total_pages()


def _broken(path, value):
    raw = copy.deepcopy(mz.MZ_A)
    node = raw
    for key in path[:-1]:
        node = node[key]
    if value is None:
        node.pop(path[-1])
    else:
        node[path[-1]] = value
    return raw


@pytest.mark.parametrize("path,value", [
    (("vocab",), None), (("width",), 0), (("norm",), None), (("streams",), 0), (("streams",), 9),
    (("layers",), []), (("layers", 0, "type"), "attention_3"), (("layers", 0, "mixer", "heads"), None),
    (("layers", 0, "mixer", "kv_heads"), 3), (("layers", 0, "mixer", "scale"), None),
    (("layers", 0, "mixer", "rot", "dims"), 7), (("layers", 0, "mixer", "rot", "dims"), 14),
    (("layers", 0, "mixer", "rot", "scaling", "fast"), None), (("layers", 1, "mixer", "rot", "scaling", "high"), 0.0),
    (("layers", 1, "mixer", "rot", "scaling", "factor"), 0.0), (("layers", 0, "mlp", "kind"), "moe"),
    (("layers", 0, "mlp", "ff"), None), (("loop", "stop"), 9), (("loop", "times"), 0),
    (("embedding", "bigram", "buckets"), 0), (("embedding", "bigram", "mul_cur"), None),
])
def test_refusals_name_the_key(path, value):
    with pytest.raises(ConfigError) as err:
        MezapelConfig.from_dict(_broken(path, value))
    assert str(path[-1]) in str(err.value) or str(path[-2]) in str(err.value)


def test_rotation_tables_follow_both_scaling_rules():
    for dims, base, rule, s in ((24, 1000.0, "yarn", mz.yarn(4.0, 64)), (16, 50000.0, "yarn", mz.yarn(16.0, 8, 4.0, 0.5)),
                                (32, 1e4, "llama3", mz.llama3(8.0, 64)), (8, 10.0, "llama3", mz.llama3(3.0, 16, 0.25, 2.0))):
        want_f, want_m = plain.rotation({"base": base, "dims": dims, "scaling": s}, rule)
        got_f, got_m = scaled_frequencies(dims, base, {"kind": rule, **s})
        assert torch.allclose(got_f, torch.tensor(want_f, dtype=torch.float64), rtol=1e-14, atol=0) and got_m == want_m
        table = rotary_table(dims, base, "cpu", 300, True, {"kind": rule, **s})
        a = torch.arange(300, dtype=torch.float64)[:, None] * torch.tensor(want_f, dtype=torch.float64)[None]
        assert torch.equal(table, (torch.cat((a.cos(), a.sin()), -1) * want_m).float())
    # the three regimes of the second rule, and the ramp of the first, are all met in these cases
    f, _ = scaled_frequencies(32, 1e4, {"kind": "llama3", **mz.llama3(8.0, 64)})
    plainf = torch.tensor(plain.plain_frequencies(1e4, 32), dtype=torch.float64)
    ratio = f / plainf
    assert (ratio == 1).any() and torch.isclose(ratio, torch.tensor(0.125, dtype=torch.float64)).any() and \
        ((ratio > 0.126) & (ratio < 0.999)).any()
    assert not torch.equal(rotary_table(24, 1000.0, "cpu", 10, True, None), rotary_table(24, 1000.0, "cpu", 10, True, {"kind": "yarn", **mz.yarn(4.0, 64)}))


# ------------------------------------------------- the plain implementation's own mechanisms
def test_plain_hash_rows_and_first_token():
    big = {"buckets": 7, "mul_prev": 5, "mul_cur": 3}
    assert plain.bigram_rows([4, 6, 0, 6], big) == [7, (4 * 5 + 6 * 3) % 7, (6 * 5) % 7, (6 * 3) % 7]


def test_plain_masks_and_sinks():
    torch.manual_seed(0)
    s = torch.randn(9, 9, dtype=torch.float64)
    w = plain.masked_softmax_with_sink(s, lambda a, b: b <= a and a // 4 == b // 4, 0.0)
    assert (w[4, :4] == 0).all() and (w[3, :4] > 0).all() and (w[8, :8] == 0).all()
    assert math.isclose(float(w[8, 8]), math.exp(s[8, 8]) / (1 + math.exp(s[8, 8])))
    w = plain.masked_softmax_with_sink(s, lambda a, b: 0 <= a - b < 3, 2.0)
    assert (w[5, :3] == 0).all() and (w[5, 3:6] > 0).all() and (w[5, 6:] == 0).all()
    e = torch.exp(s[5, 3:6])
    assert torch.allclose(w[5, 3:6], e / (e.sum() + math.exp(2.0)))
    # a very large sink takes all the weight and overflows nothing
    assert float(plain.masked_softmax_with_sink(s, lambda a, b: b <= a, 800.0).sum()) < 1e-300


def test_plain_loop_repeats_the_range_as_a_whole():
    assert plain.run_order({"layers": [0] * 5, "loop": {"start": 2, "stop": 4, "times": 2}}) == [0, 1, 2, 3, 2, 3, 4]
    assert plain.run_order({"layers": [0] * 2}) == [0, 1]
    cfg = MezapelConfig.from_dict(mz.MZ_B)
    assert cfg.run_order() == plain.run_order(mz.MZ_B)


def test_plain_streams_of_one_with_unit_weights_are_the_plain_residual():
    """One stream whose connection weights are all one is ``x + sublayer(norm(x))``."""
    config = copy.deepcopy(mz.MZ_D)
    state = mz.random_state(config, 5)
    toks = mz.tokens(2, 17, config["vocab"])
    want = plain.forward(config, state, toks)
    config["streams"] = 1
    for i, layer in enumerate(config["layers"]):
        for q in (1, 2):
            state[f"l{i}.hc{q}.in"] = torch.ones(1, dtype=torch.float64)
            state[f"l{i}.hc{q}.out"] = torch.ones(1, dtype=torch.float64)
            state[f"l{i}.hc{q}.mix"] = torch.ones(1, 1, dtype=torch.float64)
    assert torch.allclose(plain.forward(config, state, toks), want, rtol=1e-12, atol=1e-12)
