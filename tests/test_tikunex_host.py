"""Tikunex without a GPU: its configuration, the order in which its layers run, what its mixers ask of
the cache, the tensors it declares, and the cache's book-keeping for kept first tokens and for requests
made of several parts."""
import copy

import pytest

from friday_inference_engine_b200 import ConfigError, WeightsError, check_weights, describe_model, read_config
from friday_inference_engine_b200.cache import PAGE, CacheBook, kv_request, several, state_request

import plain_tikunex as plain
import tiny_configs

MOE = {"kind": "moe", "expert": {"ff": 24}, "router": {"experts": 5, "top": 2}}
GLA = {"heads": 3, "dim": 8, "vdim": 16, "tau": 4.0, "decay_rank": 4}
PAR = {"left": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 24, "scale": 0.3, "mask": {"size": 100, "keep_first": 70}},
       "right": {"heads": 2, "dim": 8, "decay_rank": 4}, "left_scale": 0.7, "right_scale": 1.3}
CFG = {"architecture": "Tikunex", "vocab": 50, "width": 32, "norm": {"eps": 1e-5},
       "layers": [{"type": "gla", "mixer": GLA, "mlp": MOE}, {"type": "parallel", "mixer": PAR, "mlp": None},
                  {"type": "parallel", "mixer": PAR, "mlp": MOE}, {"type": "gla", "mixer": GLA, "mlp": None}],
       "loop": {"start": 1, "stop": 3, "times": 3}, "token_side": {"dim": 4}}


def test_the_name_selects_the_design():
    assert read_config(CFG)["architecture"] == "Tikunex"
    assert describe_model(CFG)["architecture"] == "Tikunex"


def test_run_order_and_injections():
    d = describe_model(CFG)
    prog = d["program"]
    assert [c["layer"] for c in prog] == [0, 1, 2, 1, 2, 1, 2, 3]
    assert [c["cache"] for c in prog] == list(range(8))                 # every run has memory of its own
    assert [c["inject"] for c in prog] == [-1, 0, -1, 0, -1, 0, -1, -1]  # right before the first layer of every pass
    assert [(i, first) for i, first in plain.run_order(CFG)] == [(c["layer"], c["inject"] >= 0) for c in prog]
    no_loop = {k: v for k, v in CFG.items() if k != "loop"}
    d = describe_model(no_loop)
    assert [c["layer"] for c in d["program"]] == [0, 1, 2, 3] and all(c["inject"] < 0 for c in d["program"])
    assert "loop.in" not in [p["name"] for p in d["params"]]


def test_cache_requests():
    reqs = describe_model(CFG)["cache_requests"]
    assert reqs["0"] == {"kind": "state", "shape": [3 * 8 * 16], "dtype": "float32"}
    p = reqs["1"]
    assert p["kind"] == "several" and len(p["parts"]) == 2
    assert p["parts"][0] == {"kind": "kv", "n_kv_heads": 2, "head_dim": 8, "window": 100, "v_head_dim": 24, "keep_first": 70}
    assert p["parts"][1] == {"kind": "state", "shape": [32 + 2 * 8 * 8], "dtype": "float32"}


def test_declared_tensors():
    d = describe_model(CFG)
    shapes = {p["name"]: p["shape"] for p in d["params"]}
    assert shapes["embed"] == [50, 32] and shapes["head"] == [50, 32] and shapes["loop.in"] == [32, 64]
    assert shapes["side.embed"] == [50, 4 * 4] and shapes["l2.side.gate"] == [4, 32] and shapes["l2.side.proj"] == [32, 4]
    assert shapes["l0.mix.a1"] == [4, 32] and shapes["l0.mix.a2"] == [24, 4] and shapes["l0.mix.norm"] == [16]
    assert shapes["l1.mix.left.q"] == [32, 32] and shapes["l1.mix.left.v"] == [48, 32] and shapes["l1.mix.left.o"] == [32, 96]
    assert shapes["l1.mix.right.u"] == [2, 8] and shapes["l1.mix.right.w2"] == [16, 4] and shapes["l1.mix.right.mu.w"] == [32]
    assert shapes["l2.mlp.e4.down"] == [32, 24] and shapes["l2.mlp.router.b"] == [5]
    assert "l1.norm2" not in shapes and "l1.norm2" in d["ignorable"]     # no feed-forward: no second norm
    assert "l1.mlp.router" not in shapes
    # without "decay_rank" the size is the checkpoint's
    cfg = copy.deepcopy(CFG)
    del cfg["layers"][0]["mixer"]["decay_rank"]
    shapes = {p["name"]: p["shape"] for p in describe_model(cfg)["params"]}
    assert shapes["l0.mix.a1"] == [-1, 32] and shapes["l0.mix.a2"] == [24, -1]


@pytest.mark.parametrize("change,word", [
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c["layers"][0].update(type="mamba"), "mamba"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "dense"),
    (lambda c: c["layers"][1]["mixer"]["left"].update(kv_heads=3), "share"),
    (lambda c: c["layers"][1]["mixer"]["left"]["mask"].pop("size"), "size"),
    (lambda c: c["layers"][2]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c["token_side"].update(dim=0), "dim"),
    (lambda c: c["layers"][0]["mixer"].update(tau=0.0), "tau"),
])
def test_bad_config_names_the_key(change, word):
    cfg = copy.deepcopy(CFG)
    change(cfg)
    with pytest.raises(ConfigError) as e:
        read_config(cfg)
    assert word in str(e.value)


def test_folder_round_trip_and_sizes_left_to_the_checkpoint(tmp_path):
    d = tiny_configs.make_model_dir(str(tmp_path / "m"), CFG, 5)
    check_weights(d)
    cfg, t = plain.load(d)
    assert t["l0.mix.a1"].shape == (4, 32) and t["side.embed"].shape == (50, 16)
    # the same folder read by a configuration that does not name the decay's inner size
    import json
    import os
    for L in cfg["layers"]:
        m = L["mixer"]
        m.pop("decay_rank", None)
        if "right" in m:
            m["right"].pop("decay_rank", None)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    check_weights(d)
    # ... but random weights cannot be drawn for it
    with pytest.raises(WeightsError):
        tiny_configs.make_model_dir(str(tmp_path / "n"), cfg, 5)


def test_kept_first_pages_are_never_given_back():
    # window 100, 70 kept tokens: logical pages 0 and 1 hold kept tokens
    c = CacheBook({0: kv_request(2, 8, 100, v_head_dim=24, keep_first=70)}, 16 * PAGE, 16 * PAGE, max_slots=2)
    g = c.info()["groups"][0]
    assert g["pool_shape"][-1] == 8 and g["value_pool_shape"][-1] == 24 and g["keep_first"] == 70
    s = c.alloc_slot()
    c.reserve([s], [10 * PAGE])
    c.commit([s], [10 * PAGE])
    table = c.info()["groups"][0]["table"][s]
    held = [lp for lp, p in enumerate(table) if p >= 0]
    # the window's pages: positions 541..639 -> logical pages 8, 9; the kept ones: 0, 1
    assert held == [0, 1, 8, 9]
    for _ in range(3 * PAGE):                       # decoding on: the window moves, the kept pages stay
        c.reserve([s], [1])
        c.commit([s], [1])
    held = [lp for lp, p in enumerate(c.info()["groups"][0]["table"][s]) if p >= 0]
    assert held[:2] == [0, 1] and held[2] >= 11 and len(held) <= 5
    c.free_slot(s)
    assert c.info()["groups"][0]["pages_held"] == 0
    # a window without kept tokens gives everything behind it back
    c = CacheBook({0: kv_request(2, 8, 100)}, 16 * PAGE, 16 * PAGE, max_slots=2)
    s = c.alloc_slot()
    c.reserve([s], [10 * PAGE])
    c.commit([s], [10 * PAGE])
    assert [lp for lp, p in enumerate(c.info()["groups"][0]["table"][s]) if p >= 0] == [8, 9]


def test_requests_made_of_several_parts():
    reqs = {0: state_request((5,)),
            1: several(kv_request(2, 8, 100, 24, 70), state_request((7,))),
            2: several(kv_request(2, 8, 100, 24, 70), state_request((7,))),
            3: several(kv_request(1, 8), state_request((9,)))}
    c = CacheBook(reqs, 8 * PAGE, 8 * PAGE, max_slots=3)
    info = c.info()
    assert len(info["groups"]) == 2                           # the two windowed parts share a group, the third has its own
    assert len(info["groups"][0]["entries"]) == 2 and len(info["groups"][1]["entries"]) == 1
    assert sorted(v[1] for v in info["states"].values()) == [5, 7, 7, 9]
    s = c.alloc_slot()
    c.reserve([s], [PAGE + 1])
    c.commit([s], [PAGE + 1])
    assert all(g["pages_held"] == 2 for g in c.info()["groups"])
    c.free_slot(s)
    assert all(g["pages_held"] == 0 for g in c.info()["groups"])
