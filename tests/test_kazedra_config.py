"""Kazedra on the host: config.json keys and refusals, the plan it becomes, the tensors it expects, and the
caches its layers ask for (a paged one and a state per layer).  Needs no GPU."""
import copy
import json

import pytest

from imp_b200.cache.manager import CacheManager, PagedKVSpec, StateSpec
from imp_b200.config.model_config import ConfigError, KazedraConfig
from imp_b200.config.registry import config_from_dict, known_architectures, load_config, plan_for
from plain import kazedra_plain as K

CFG = {
    "architecture": "Kazedra", "vocab": 97, "width": 64, "norm": {"eps": 3e-5}, "logit_scale": 1.7,
    "layers": [
        {"type": "parallel",
         "mixer": {"left": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 16, "bias_max": 20, "scale": 0.3, "q_temp": {"coef": 0.35, "every": 7}},
                   "right": {"heads": 2, "kv_heads": 1, "dim": 24, "vdim": 40, "conv": 3}, "left_scale": 0.6, "right_scale": 1.1},
         "mlp": {"kind": "dense", "ff": 72}},
        {"type": "parallel",
         "mixer": {"left": {"heads": 3, "kv_heads": 3, "dim": 32, "vdim": 32, "bias_max": 11, "scale": 0.2, "q_temp": {"coef": 0.1, "every": 5}},
                   "right": {"heads": 4, "kv_heads": 4, "dim": 16, "vdim": 16, "conv": 2}, "left_scale": 1.2, "right_scale": 0.7},
         "mlp": None},
    ],
}


def test_architecture_is_known_and_named_by_a_single_string():
    assert "Kazedra" in known_architectures()
    c = config_from_dict(CFG)
    assert isinstance(c, KazedraConfig)
    assert (c.architecture, c.vocab_size, c.hidden_size, c.num_hidden_layers) == ("Kazedra", 97, 64, 2)


def test_round_trip_through_folder(tmp_path):
    c = config_from_dict(CFG)
    c.save(str(tmp_path))
    assert load_config(str(tmp_path)) == c
    assert json.load(open(tmp_path / "config.json"))["layers"][1]["mlp"] is None


def test_plan_takes_every_size_and_constant_from_the_layer_entries():
    plan = plan_for(config_from_dict(CFG))
    assert [l.block for l in plan.layers] == ["parallel_prenorm"] * 2
    assert list(plan.layers[0].parts) == ["mixer_norm", "left", "right", "ffn_norm", "feed_forward"]
    assert list(plan.layers[1].parts) == ["mixer_norm", "left", "right"]            # no feed-forward, no second norm
    l0, l1 = plan.layers
    assert l0.block_params == {"left_scale": 0.6, "right_scale": 1.1, "has_ffn": True}
    assert l1.block_params == {"left_scale": 1.2, "right_scale": 0.7, "has_ffn": False}
    a = l1.left
    assert a.kind == "sink_bias_attention"
    assert (a.params["num_heads"], a.params["num_kv_heads"], a.params["head_dim"], a.params["scale"], a.params["q_temp_coef"],
            a.params["q_temp_every"], a.params["bias_max_distance"], a.params["norm_eps"]) == (3, 3, 32, 0.2, 0.1, 5, 11, 3e-5)
    b = l0.right
    assert b.kind == "gated_delta_rule"
    assert (b.params["num_heads"], b.params["num_kv_heads"], b.params["key_dim"], b.params["value_dim"], b.params["conv_taps"]) == (2, 1, 24, 40, 3)
    assert l0.mixer_norm.params["weight_offset"] == 1.0 and plan.final_norm.params["weight_offset"] == 1.0
    assert plan.head.params["scale"] == 1.7
    assert l0.feed_forward.params["intermediate_size"] == 72


def test_expected_tensors_and_the_table_whose_rows_the_checkpoint_gives():
    plan = plan_for(config_from_dict(CFG))
    exp = plan.expected_tensors()
    assert list(exp["l0.mix.left.q"].shape) == [64, 64] and list(exp["l0.mix.left.k.b"].shape) == [32]
    assert list(exp["l1.mix.left.q.norm"].shape) == [96] and list(exp["l1.mix.left.sink"].shape) == [3]
    assert list(exp["l0.mix.right.v.conv"].shape) == [80, 3] and list(exp["l0.mix.right.q.conv"].shape) == [24, 3]
    assert list(exp["l1.mix.right.b"].shape) == [4, 64] and list(exp["l1.mix.right.norm"].shape) == [16]
    assert list(exp["l0.mix.left.rel"].shape) == [-1, 4]            # any number of rows
    assert "l1.norm2" not in exp and "l1.mlp.gate" not in exp and "l0.norm2" in exp
    assert list(exp["embed"].shape) == [97, 64] and list(exp["head"].shape) == [97, 64] and list(exp["final.norm"].shape) == [64]
    fixed = plan_for(config_from_dict(dict(CFG, bias_buckets=12))).expected_tensors()
    assert list(fixed["l0.mix.left.rel"].shape) == [12, 4]


@pytest.mark.parametrize("edit,match", [
    (lambda d: d["layers"][0].update(type="serial"), "unknown layer type"),
    (lambda d: d["layers"][0]["mixer"]["left"].update(vdim=8), "vdim"),
    (lambda d: d["layers"][1]["mixer"]["left"].update(heads=4), "multiple of kv_heads"),
    (lambda d: d["layers"][1]["mixer"]["right"].pop("conv"), "conv"),
    (lambda d: d.pop("norm"), "norm"),
    (lambda d: d["layers"][0]["mlp"].update(kind="routed"), "unknown kind"),
    (lambda d: d.pop("width"), "width"),
    (lambda d: d.update(layers=[]), "layers"),
])
def test_refusals_name_the_key(edit, match):
    d = copy.deepcopy(CFG)
    edit(d)
    with pytest.raises(ConfigError, match=match):
        config_from_dict(d)


def test_each_layer_holds_pages_and_a_state_slot_and_gives_both_back():
    """The caches of a two-layer model as the engine lays them out: per layer a paged entry and a state entry; layers of
    different sizes do not share a group; pages and slots return when a request ends."""
    specs = [PagedKVSpec(2, 16), StateSpec(tensors=(("S", (2, 24, 40), "float32"), ("conv", (2, 128), "float32"))),
             PagedKVSpec(3, 32), StateSpec(tensors=(("S", (4, 16, 16), "float32"), ("conv", (1, 192), "float32")))]
    m = CacheManager(specs, page_size=4, num_pages=10, num_state_slots=2)
    info = m.info()
    assert [p["kind"] for p in info["positions"]] == ["paged", "state", "paged", "state"]
    assert len(info["paged"]) == 2 and len(info["state"]) == 2
    s0 = m.add_request(1)
    m.reserve(1, 17)
    m.commit(1, 17)
    s1 = m.add_request(2)
    assert s0 != s1
    with pytest.raises(Exception):
        m.add_request(3)                       # both slots are held
    m.reserve(2, 9)
    m.commit(2, 9)
    assert m.free_pages() == 10 - 5 - 3
    m.release(1)
    assert m.add_request(3) == s0              # the slot that came back is used again
    m.reserve(3, 20)
    m.check_invariants()
    m.release(2)
    m.release(3)
    assert m.free_pages() == 10 and m.info()["free_slots"] == 2


def test_distance_buckets_of_the_plain_implementation():
    B, D = 12, 40
    b = [K.distance_bucket(n, B, D) for n in range(200)]
    assert b[:6] == list(range(6))                                  # exact below half the table
    assert all(x <= y for x, y in zip(b, b[1:])) and set(b) == set(range(B))
    assert b[D - 1] <= B - 1 and all(x == B - 1 for x in b[D:])     # from the largest distance on: the last row
    assert K.query_temperature(0, 0.5, 4) == 1.0 and K.query_temperature(2, 0.5, 4) == 1.0
    assert K.query_temperature(3, 0.5, 4) == pytest.approx(1 + 0.5 * 0.6931471805599453)
