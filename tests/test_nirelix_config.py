"""Host-side tests of the Nirelix configuration, its model plan, the tensors the plan asks for, the
size that only a checkpoint's tensor shapes state, and the plain implementation's own mechanisms
(no GPU)."""

import copy
import json
import os

import pytest
import torch

import nirelix_tiny as nx
import plain_nirelix as plain
from freetoken_b200.cache import CacheManager, PagedKeyNeed, StateNeed
from freetoken_b200.config.model_plan import ConfigError
from freetoken_b200.config.nirelix import NirelixConfig, build_plan, sizes_from_tensors
from freetoken_b200.models.model import Model
from freetoken_b200.registry import architecture_of, read_model_config
from freetoken_b200.weights.loader import WeightError, plan_loading
from freetoken_b200.weights.spec import leaves


def test_registry_picks_the_design_by_its_singular_key():
    arch = architecture_of(nx.NX_A)
    assert arch.name == "Nirelix"
    cfg = arch.read_config(nx.NX_A)
    assert isinstance(cfg, NirelixConfig) and cfg.to_dict() == nx.NX_A


@pytest.mark.parametrize("which", list(nx.NX))
def test_plan_hands_every_constant_to_a_part(which):
    raw = nx.NX[which]
    plan = build_plan(NirelixConfig.from_dict(raw))
    assert plan.residual_streams == raw["streams"]
    assert [s.layer for s in plan.schedule] == list(range(len(raw["layers"])))
    assert plan.final_norm.kind == "hyper_norm" and plan.final_norm.params["connection"] is None
    for spec, layer in zip(plan.layers, raw["layers"]):
        assert spec.block.kind == "hyper"
        assert (spec.feed_forward is None) == (layer["mlp"] is None)
        assert sorted(spec.all_norms()) == (["feed_forward", "mixer"] if layer["mlp"] else ["mixer"])
        for n in spec.all_norms().values():
            assert (n.params["eps"], n.params["streams"], n.params["center"]) == (raw["norm"]["eps"], raw["streams"], True)
            assert n.params["bias_tensor"] == n.params["tensor"] + ".b"
        m, p = layer["mixer"], spec.mixer.params
        assert spec.mixer.kind == layer["type"]
        if layer["type"] == "retention":
            assert (p["heads"], p["key_dim"], p["head_dim"], list(p["decay"])) == (m["heads"], m["dim"], m["vdim"], m["decay"])
            assert (p["position"].kind, p["position"].params["rotary_dim"], p["position"].params["theta"]) == \
                ("rotary_neox", m["rot"]["dims"], m["rot"]["base"])
        elif layer["type"] == "channel_delta":
            assert (p["heads"], p["key_heads"], p["key_dim"], p["head_dim"], p["conv_taps"], p["low_rank"],
                    p["gate_rank"]) == \
                (m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"], m["low_rank"],
                 m.get("gate_rank") or m["low_rank"])
        else:
            assert (p["num_heads"], p["qk_dim"], p["rot_dim"], p["v_dim"], p["q_rank"], p["rank"], p["sm_scale"],
                    p["sliding_window"], p["gate_per"]) == \
                (m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["q_rank"], m["kv_rank"], m["scale"], m["mask"]["size"],
                 "element")
            assert (p["position"].kind, p["position"].params["theta"]) == ("rotary_interleaved", m["rot"]["base"])
        mlp = layer["mlp"]
        if mlp and mlp["kind"] == "moe":
            f, r = spec.feed_forward.params, mlp["router"]
            assert (f["num_experts"], f["top_k"], f["scale"], f["groups"], f["keep_groups"], f["intermediate_size"]) == \
                (r["experts"], r["top"], r["scale"], r["groups"]["count"], r["groups"]["keep"], mlp["expert"]["ff"])
            assert f["scoring"] == "sigmoid" and f["renormalize"] and f["activation"] == "silu"
        elif mlp:
            f = spec.feed_forward.params
            assert (f["activation"], f["act_limit"], f["act_alpha"], f["gated"]) == ("swigluoai", mlp["limit"], 1.702, True)


@pytest.mark.parametrize("which", list(nx.NX))
def test_the_plan_asks_for_exactly_the_tensors_of_a_checkpoint(which):
    raw = nx.NX[which]
    model = Model(build_plan(NirelixConfig.from_dict(raw)))
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


def test_cache_needs_rows_of_latent_plus_rotated_part_and_states():
    raw = nx.NX_A
    model = Model(build_plan(NirelixConfig.from_dict(raw)))
    needs = model.cache_needs()
    for need, layer in zip(needs, raw["layers"]):
        m = layer["mixer"]
        if layer["type"] == "latent_attention":
            assert need == PagedKeyNeed(1, m["kv_rank"] + m["rot_dim"], m["mask"]["size"])
        elif layer["type"] == "retention":
            assert need == StateNeed((m["heads"] * m["dim"] * m["vdim"],), "float32")
        else:
            conv = (m["conv"] - 1) * (2 * m["kv_heads"] * m["dim"] + m["heads"] * m["vdim"])
            assert need == StateNeed((conv + m["heads"] * m["dim"] * m["vdim"],), "float32")
    cache = CacheManager(needs, 4, 20, 2, 64)
    cache.admit("a")
    cache.grow("a", 30)
    cache.advance("a", 30)
    cache.release("a")
    assert cache.free_pages() == cache.total_pages()


def test_a_size_only_the_checkpoint_states(tmp_path):
    """config.json does not give the widths of the middles of the delta rule's two-step projections:
    they are the row counts of the first steps' matrices in the checkpoint (the gate's may differ
    from the decay's)."""
    config = nx.NX_C
    folder = nx.write(str(tmp_path / "m"), config, nx.random_state(config, 3))
    on_disk = json.load(open(os.path.join(folder, "config.json")))
    assert all("low_rank" not in layer["mixer"] and "gate_rank" not in layer["mixer"] for layer in on_disk["layers"])
    arch, cfg = read_model_config(folder)
    assert [(l.mixer.low_rank, l.mixer.gate_rank) for l in cfg.layers if l.type == "channel_delta"] == [(3, 3), (24, 8)]
    with pytest.raises(ConfigError, match="low_rank"):
        NirelixConfig.from_dict(on_disk)
    sized = sizes_from_tensors(on_disk, {"l1.mix.a1": (3, 70), "l2.mix.a1": (24, 70), "l2.mix.g1": (8, 70)})
    assert (sized["layers"][2]["mixer"]["low_rank"], sized["layers"][2]["mixer"]["gate_rank"]) == (24, 8)
    assert "gate_rank" not in sized["layers"][1]["mixer"]


def _broken(path, value):
    raw = copy.deepcopy(nx.NX_A)
    node = raw
    for key in path[:-1]:
        node = node[key]
    if value is None:
        del node[path[-1]]
    else:
        node[path[-1]] = value
    return raw


@pytest.mark.parametrize("path,value,match", [
    (("layers", 0, "type"), "mystery", "type"),
    (("layers", 0, "mixer", "kv_heads"), 3, "kv_heads"),
    (("layers", 0, "mlp", "router", "groups"), {"count": 4, "keep": 2}, "groups"),
    (("layers", 0, "mlp", "router", "top"), 5, "do not fit"),
    (("layers", 0, "mlp", "router", "top"), 9, "top"),
    (("layers", 1, "mixer", "rot"), {"base": 100.0, "dims": 6}, "rot.dims"),
    (("layers", 1, "mixer", "mask"), None, "mask"),
    (("layers", 1, "mlp", "limit"), None, "limit"),
    (("layers", 2, "mixer", "decay"), [0.9, 0.8], "decay"),
    (("layers", 2, "mixer", "rot"), {"base": 10.0, "dims": 12}, "rot.dims"),
    (("streams",), 9, "streams"),
    (("norm",), None, "norm"),
])
def test_refusals(path, value, match):
    with pytest.raises(ConfigError, match=match):
        NirelixConfig.from_dict(_broken(path, value))


def test_plain_mechanisms_against_their_definitions():
    """The plain implementation's own pieces, each against a second way of writing it."""
    torch.manual_seed(0)
    # rotation in pairs is a rotation: lengths stay, position 0 turns nothing, angles add up
    v = torch.randn(5, 2, 8, dtype=torch.float64)
    r = plain.rotate_pairs(v, 100.0, 6)
    assert torch.allclose(r[0], v[0]) and torch.allclose(r[..., 6:], v[..., 6:])
    assert torch.allclose((r[..., :6] ** 2).sum(-1), (v[..., :6] ** 2).sum(-1))
    assert torch.allclose(plain.rotate_pairs(v, 100.0, 6, first=3)[0], plain.rotate_pairs(v[:1].repeat(4, 1, 1), 100.0, 6)[3])
    h = plain.rotate_halves(v, 100.0, 6)
    assert torch.allclose(h[1, 0, 0], v[1, 0, 0] * torch.cos(torch.tensor(1.0)) - v[1, 0, 3] * torch.sin(torch.tensor(1.0)))
    assert torch.allclose(r[1, 0, 0], v[1, 0, 0] * torch.cos(torch.tensor(1.0)) - v[1, 0, 1] * torch.sin(torch.tensor(1.0)))
    # retention's recurrence is a decayed sum over the past
    cfg = nx.one_layer(nx.retention(1, 4, 3, (0.5,), 0), vocab=10, width=8)
    w = nx.random_state(cfg, 1)
    x = torch.randn(6, 8, dtype=torch.float64)
    q, k, val = x @ w["l0.mix.q"].T, x @ w["l0.mix.k"].T * 4 ** -0.5, x @ w["l0.mix.v"].T
    o = torch.stack([sum(0.5 ** (t - j) * (q[t] @ k[j]) * val[j] for j in range(t + 1)) for t in range(6)])
    want = (plain.rms(o, 1e-6) * plain.silu(x @ w["l0.mix.g"].T)) @ w["l0.mix.o"].T
    assert torch.allclose(plain.retention(x, w, "l0.mix.", cfg["layers"][0]["mixer"], 1e-6), want)
    # a dropped group stays dropped although its scores are the only positive ones left
    router = {"experts": 4, "top": 2, "scale": 1.0, "groups": {"count": 2, "keep": 1}}
    ww = {"r.router": torch.eye(4, dtype=torch.float64), "r.correction": torch.tensor([-3.0, -3.0, 0.0, -9.0], dtype=torch.float64)}
    ids, weights = plain.choose_experts(torch.zeros(1, 4, dtype=torch.float64), ww, "r.", router)
    assert sorted(ids[0].tolist()) == [0, 1] and torch.allclose(weights.sum(), torch.tensor(1.0, dtype=torch.float64))
    # streams: with in = out = 1, mix = identity and one stream the sublayer is the plain pre-norm residual
    wts = {"l0.hc1.in": torch.ones(1, dtype=torch.float64), "l0.hc1.out": torch.ones(1, dtype=torch.float64),
           "l0.hc1.mix": torch.eye(1, dtype=torch.float64), "l0.norm1": torch.ones(8, dtype=torch.float64),
           "l0.norm1.b": torch.zeros(8, dtype=torch.float64)}
    s = torch.randn(1, 6, 8, dtype=torch.float64)
    out = plain.sublayer(s, wts, "l0.", 1, lambda z: 2 * z, 1e-6)
    assert torch.allclose(out[0], s[0] + 2 * plain.layer_norm(s[0], wts["l0.norm1"], wts["l0.norm1.b"], 1e-6))
