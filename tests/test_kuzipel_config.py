"""Kuzipel on the host: config.json keys and refusals, the plan it becomes (a repeated run of layers with a cache per
pass, blocks with tensors of their own), the tensors it expects and the caches its layers ask for.  Needs no GPU."""
import copy
import json

import pytest

from imp_b200.cache.manager import CacheManager
from imp_b200.config.model_config import ConfigError, KuzipelConfig
from imp_b200.config.registry import config_from_dict, known_architectures, load_config, plan_for
from imp_b200.parts.registry import mixer_cache_spec
from plain import kuzipel_plain as Z


def latent(heads, dim, rot, vdim, kv_rank, q_rank, base=5000.0):
    return {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": 0.21,
            "rot": {"base": base, "dims": rot}}


def moe(experts, top, ff, shared):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}, "shared": {"ff": shared} if shared else None}


CFG = {
    "architecture": "Kuzipel", "vocab": 101, "width": 64, "norm": {"eps": 2e-5}, "residual_mult": 1.3,
    "layers": [
        {"type": "wkv", "mixer": {"heads": 2, "dim": 24}, "mlp": moe(5, 2, 24, 16)},
        {"type": "latent_attention", "mixer": latent(3, 16, 8, 20, 40, 28), "mlp": None},
        {"type": "latent_attention", "mixer": latent(2, 32, 16, 32, 48, 24, base=100.0), "mlp": moe(3, 3, 8, 0)},
    ],
    "loop": {"start": 1, "stop": 3, "times": 2},
}


def test_architecture_is_known_and_round_trips(tmp_path):
    assert "Kuzipel" in known_architectures()
    c = config_from_dict(CFG)
    assert isinstance(c, KuzipelConfig)
    assert (c.architecture, c.vocab_size, c.hidden_size, c.num_hidden_layers) == ("Kuzipel", 101, 64, 3)
    assert c.run_order() == [0, 1, 2, 1, 2] == Z.run_order(CFG)[0]
    c.save(str(tmp_path))
    assert load_config(str(tmp_path)) == c
    assert json.load(open(tmp_path / "config.json"))["layers"][1]["mlp"] is None


def test_plan_takes_every_size_and_constant_from_config():
    plan = plan_for(config_from_dict(CFG))
    assert [l.block for l in plan.layers] == ["scaled_prenorm"] * 3 + ["stream_reinject"]
    # the map over the stream and the embedding runs before every pass of the repeated layers, which come twice
    assert plan.order == [0, 3, 1, 2, 3, 1, 2]
    l0, l1, l2, inj = plan.layers
    assert list(l0.parts) == ["mixer_norm", "mixer", "ffn_norm", "feed_forward"] and list(l1.parts) == ["mixer_norm", "mixer"]
    assert l0.block_params == {"hidden_size": 64, "residual_mult": 1.3, "has_ffn": True} and l1.block_params["has_ffn"] is False
    assert l0.block_tensors == {"mixer_scale": "l0.ls1", "ffn_scale": "l0.ls2"} and l1.block_tensors == {"mixer_scale": "l1.ls1"}
    assert inj.block_tensors == {"weight": "loop.in"} and not inj.parts
    assert l0.mixer.kind == "wkv" and (l0.mixer.params["num_heads"], l0.mixer.params["head_dim"], l0.mixer.params["norm_eps"]) == (2, 24, 2e-5)
    a = l2.mixer
    assert a.kind == "latent_attention"
    assert (a.params["num_heads"], a.params["head_dim"], a.params["rot_dim"], a.params["value_dim"], a.params["kv_rank"], a.params["q_rank"],
            a.params["scale"], a.params["rot_base"], a.params["rot_dims"]) == (2, 32, 16, 32, 48, 24, 0.21, 100.0, 16)
    f = l0.feed_forward
    assert f.kind == "routed_experts"
    assert (f.params["num_experts"], f.params["top_k"], f.params["expert_size"], f.params["shared_size"]) == (5, 2, 24, 16)
    assert l2.feed_forward.params["shared_size"] == 0 and "shared_gate" not in l2.feed_forward.tensors
    assert l0.mixer_norm.kind == plan.final_norm.kind == "layernorm" and plan.final_norm.params["eps"] == 2e-5


def test_expected_tensors_are_the_checkpoint_names():
    exp = plan_for(config_from_dict(CFG)).expected_tensors()
    assert tuple(exp["loop.in"].shape) == (64, 128)
    assert tuple(exp["l0.mix.u"].shape) == (2, 24) and tuple(exp["l0.mix.r"].shape) == (48, 64) and tuple(exp["l0.mix.o"].shape) == (64, 48)
    assert tuple(exp["l0.mix.w1"].shape) == (-1, 64) and tuple(exp["l0.mix.w2"].shape) == (48, -1)       # the checkpoint gives the inner size
    assert tuple(exp["l0.mlp.e4.down"].shape) == (64, 24) and tuple(exp["l0.mlp.router.b"].shape) == (5,)
    assert tuple(exp["l0.mlp.shared.sg"].shape) == (1, 64) and tuple(exp["l0.mlp.shared.gate"].shape) == (16, 64)
    assert tuple(exp["l1.mix.dkv"].shape) == (48, 64) and tuple(exp["l1.mix.dkv.norm"].shape) == (40,)
    assert tuple(exp["l1.mix.uq"].shape) == (3 * 24, 28) and tuple(exp["l1.mix.uk"].shape) == (48, 40) and tuple(exp["l1.mix.uv"].shape) == (60, 40)
    assert "l1.norm2" not in exp and "l1.ls2" not in exp and "l2.mlp.shared.gate" not in exp
    assert tuple(exp["l2.ls2"].shape) == (64,) and tuple(exp["final.norm"].shape) == (64,)
    with_rank = copy.deepcopy(CFG)
    with_rank["layers"][0]["mixer"]["decay_rank"] = 12          # random weights need the size
    assert tuple(plan_for(config_from_dict(with_rank)).expected_tensors()["l0.mix.w1"].shape) == (12, 64)


def test_without_a_repeated_run_there_is_no_map_and_no_order():
    cfg = {k: v for k, v in CFG.items() if k != "loop"}
    plan = plan_for(config_from_dict(cfg))
    assert len(plan.layers) == 3 and plan.order is None and "loop.in" not in plan.expected_tensors()
    cfg["loop"] = None
    assert plan_for(config_from_dict(cfg)).order is None


def test_caches_one_per_run_and_keys_only_for_the_latent():
    spec = mixer_cache_spec("latent_attention", plan_for(config_from_dict(CFG)).layers[1].mixer.params)
    assert spec == {"kind": "paged", "num_kv_heads": 1, "head_dim": 48, "window": 0, "keys_only": True}
    state = mixer_cache_spec("wkv", plan_for(config_from_dict(CFG)).layers[0].mixer.params)
    assert [(t["name"], t["shape"], t["dtype"]) for t in state["tensors"]] == [("S", [2, 24, 48], "float32"), ("prev", [64], "float32")]   # S with room for 64-bit words
    # run positions: wkv, map, latent(48), latent(64), map, latent(48), latent(64): the repeated layers own a cache per pass
    spec2 = mixer_cache_spec("latent_attention", plan_for(config_from_dict(CFG)).layers[2].mixer.params)
    mgr = CacheManager([state, None, spec, spec2, None, spec, spec2], page_size=4, num_pages=32, num_state_slots=2)
    info = mgr.info()
    assert sorted(len(g["layers"]) for g in info["paged"]) == [2, 2] and len(info["state"]) == 1
    mgr.add_request(1)
    mgr.reserve(1, 9)
    mgr.commit(1, 9)
    mgr.check_invariants()
    assert mgr.free_pages() == 32 - 3
    mgr.release(1)
    assert mgr.free_pages() == 32


@pytest.mark.parametrize("edit, text", [
    (lambda c: c["layers"][0].update(type="conv"), "unknown layer type 'conv'"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "unknown kind 'dense'"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=6), "top 6 exceeds the 5 experts"),
    (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "dims 7 must be even"),
    (lambda c: c["loop"].update(stop=4), "start < stop <= 3"),
    (lambda c: c["loop"].update(times=0), "'times' must be positive"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_refusals_name_the_key(edit, text):
    cfg = copy.deepcopy(CFG)
    edit(cfg)
    with pytest.raises(ConfigError) as e:
        config_from_dict(cfg)
    assert text in str(e.value)
