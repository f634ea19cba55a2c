"""Beletar without a GPU: its configuration, the order in which its layers run, what its mixers ask of
the cache, the tensors it declares, and the plain implementation's own mechanisms against hand-made cases."""
import copy

import numpy as np
import pytest

from friday_inference_engine_b200 import ConfigError, check_weights, describe_model, read_config

import plain_beletar as plain

LAT = {"heads": 3, "dim": 16, "rot_dim": 8, "vdim": 24, "kv_rank": 40, "scale": 0.2,
       "rot": {"base": 10000.0, "dims": 8, "scaling": {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 2.0}}}
DEL = {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "conv": 4}
CHA = {"heads": 6, "kv_heads": 3, "dim": 16, "vdim": 8, "conv": 2}
MLP = {"kind": "dense", "ff": 40}
CFG = {"architecture": "Beletar", "vocab": 50, "width": 32, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0},
       "layers": [{"type": "delta", "mixer": DEL, "mlp": MLP}, {"type": "latent_attention", "mixer": LAT, "mlp": None},
                  {"type": "channel_delta", "mixer": CHA, "mlp": MLP}, {"type": "delta", "mixer": DEL, "mlp": None}],
       "loop": {"start": 1, "stop": 3, "times": 3}}


def test_the_name_selects_the_design():
    assert read_config(CFG)["architecture"] == "Beletar"
    assert describe_model(CFG)["architecture"] == "Beletar"


def test_run_order_and_where_the_input_comes_back():
    prog = describe_model(CFG)["program"]
    assert [c["layer"] for c in prog] == [0, 1, 2, 1, 2, 1, 2, 3]
    assert [c["cache"] for c in prog] == list(range(8))                  # every run has memory of its own
    assert [c["add_input"] for c in prog] == [False, False, False, True, False, True, False, False]
    assert plain.run_order(CFG) == [(c["layer"], c["add_input"]) for c in prog]
    no_loop = {k: v for k, v in CFG.items() if k != "loop"}
    prog = describe_model(no_loop)["program"]
    assert [c["layer"] for c in prog] == [0, 1, 2, 3] and not any(c["add_input"] for c in prog)
    once = dict(CFG, loop={"start": 0, "stop": 4, "times": 1})
    assert not any(c["add_input"] for c in describe_model(once)["program"])


def test_cache_requests():
    reqs = describe_model(CFG)["cache_requests"]
    # delta: three rows of inputs before the heads' matrices
    assert reqs["0"] == {"kind": "state", "shape": [3 * (2 * 2 * 16 + 4 * 24) + 4 * 16 * 24], "dtype": "float32"}
    # the latent and the rotated key part, one row per position whatever the number of heads
    assert reqs["1"] == {"kind": "kv", "n_kv_heads": 1, "head_dim": 40, "window": 0, "v_head_dim": 8, "keep_first": 0}
    assert reqs["2"] == {"kind": "state", "shape": [1 * (2 * 3 * 16 + 6 * 8) + 6 * 16 * 8], "dtype": "float32"}
    assert reqs["3"] == reqs["1"] and reqs["4"] == reqs["2"]


def test_declared_tensors():
    d = describe_model(CFG)
    shapes = {p["name"]: p["shape"] for p in d["params"]}
    assert shapes["embed"] == [50, 32] and "head" not in shapes
    assert shapes["final.norm"] == [32] and shapes["final.norm.b"] == [32] and shapes["l0.norm1.b"] == [32]
    assert shapes["l0.mix.q"] == [32, 32] and shapes["l0.mix.v"] == [96, 32] and shapes["l0.mix.k.conv"] == [32, 4]
    assert shapes["l0.mix.a"] == [4, 32] and shapes["l0.mix.dt_bias"] == [4] and shapes["l0.mix.g"] == [96, 32]
    assert shapes["l1.mix.q"] == [3 * 24, 32] and shapes["l1.mix.dkv"] == [48, 32] and shapes["l1.mix.dkv.norm"] == [40]
    assert shapes["l1.mix.uk"] == [48, 40] and shapes["l1.mix.uv"] == [72, 40] and shapes["l1.mix.sink"] == [3]
    assert shapes["l1.mix.g"] == [3, 32] and shapes["l1.mix.o"] == [32, 72]
    assert shapes["l2.mix.a1"] == [-1, 32] and shapes["l2.mix.a2"] == [96, -1] and shapes["l2.mix.dt_bias"] == [96]
    assert shapes["l2.mix.g2"] == [48, -1] and shapes["l2.mix.A_log"] == [6] and shapes["l2.mix.norm"] == [8]
    assert shapes["l2.mlp.gate"] == [40, 32] and shapes["l2.mlp.down"] == [32, 40]
    assert "l1.norm2" not in shapes and "l1.norm2" in d["ignorable"] and "l1.mlp.gate" not in shapes


@pytest.mark.parametrize("change,word", [
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c["layers"][0].update(type="mamba"), "mamba"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "moe"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "share"),
    (lambda c: c["layers"][0]["mixer"].update(conv=9), "conv"),
    (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=10), "dims"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=3), "dims"),
    (lambda c: c["layers"][1]["mixer"]["rot"]["scaling"].update(factor=0), "factor"),
    (lambda c: c["loop"].update(stop=9), "loop"),
])
def test_bad_config_names_the_key(change, word):
    cfg = copy.deepcopy(CFG)
    change(cfg)
    with pytest.raises(ConfigError) as e:
        read_config(cfg)
    assert word in str(e.value)


# ---- the plain implementation's mechanisms against cases worked by hand
def test_plain_convolution_and_norms():
    x = np.arange(8, dtype=np.float64).reshape(4, 2)
    w = np.array([[1.0, 10.0, 100.0], [0.0, 0.0, 2.0]])
    y = plain.short_convolution(x, w)
    assert y[0].tolist() == [0.0, 2.0] and y[1].tolist() == [200.0, 6.0] and y[3].tolist() == [1 * 2 + 10 * 4 + 100 * 6, 14.0]
    v = np.array([[3.0, 4.0]])
    assert np.allclose(plain.unit(v), v / np.sqrt(25.0 + 1e-6))
    ln = plain.layer_norm(np.array([[1.0, 3.0]]), np.array([2.0, 2.0]), np.array([0.5, 0.5]), 0.0)
    assert np.allclose(ln, [[-1.5, 2.5]])


def test_plain_delta_rule_writes_then_reads():
    # one head, no decay, beta 1: after writing (k, v) the state returns v for the query k
    k = np.array([[[1.0, 0.0]], [[0.0, 1.0]], [[1.0, 0.0]]])
    v = np.array([[[5.0]], [[7.0]], [[9.0]]])
    one = np.ones((3, 1))
    o = plain.delta_rule(k, k, v, one, np.ones((3, 1, 1)))
    assert o[:, 0, 0].tolist() == [5.0, 7.0, 9.0]                      # the third token overwrites what the first wrote
    half = plain.delta_rule(k, k, v, 0.5 * one, np.ones((3, 1, 1)))
    assert half[:, 0, 0].tolist() == [2.5, 3.5, 2.5 + 0.5 * (9.0 - 2.5)]
    # a decay of zero forgets everything before the present token
    o = plain.delta_rule(k, k, v, one, np.zeros((3, 1, 1)))
    assert o[:, 0, 0].tolist() == [5.0, 7.0, 9.0]


def test_plain_rotation_tables():
    f, mult = plain.rotary_frequencies({"base": 100.0, "dims": 4})
    assert np.allclose(f, [1.0, 0.1]) and mult == 1.0
    f, mult = plain.rotary_frequencies({"base": 100.0, "dims": 4, "scaling": {"factor": 4.0, "original": 64, "fast": 32.0, "slow": 1.0}})
    assert np.isclose(mult, 0.1 * np.log(4.0) + 1.0)
    assert np.isclose(f[0], 1.0) and f[1] < 0.1 and f[1] >= 0.1 / 4.0            # the short wavelength stays, the long one is stretched
    x = np.array([[1.0, 0.0, 1.0, 0.0]])
    r = plain.rotate_pairs(x, [2], {"base": 100.0, "dims": 4})
    assert np.allclose(r, [[np.cos(2.0), np.sin(2.0), np.cos(0.2), np.sin(0.2)]])
