"""Beletar through the engine against the plain implementation (tests/plain_beletar.py), on small
configurations of the tests' own with weights drawn here: each mechanism alone, whole prompts, decoding
token by token, prompts cut into portions, batches of unequal requests, slots and pages used again,
keys far away and at page borders, the first tokens of a sequence, long decoding, and greedy generation
through Engine.generate.

Weights N(0, 0.02) everywhere would hide faults (a flat softmax, states that forget at once, a sink that
weighs nothing), so the folders are written with: queries, latents and key expansions scaled up (peaked
attention that often picks a key hundreds of tokens back), sinks of the size of the scores, decay rates
and biases for which the states remember a hundred tokens and still depend on the token, convolution
taps and betas of ordinary size, norm biases that matter.

float32 must agree with the plain implementation to summation order; bfloat16 within bounds relative to
the logits' spread.
"""
import json
import os

import numpy as np
import pytest

import harness
import plain_beletar as plain
import tiny_configs
from friday_inference_engine_b200 import Engine
from friday_inference_engine_b200.weights import write_safetensors

pytestmark = pytest.mark.gpu
DTYPES = [pytest.param("float32", id="f32"), pytest.param("bfloat16", id="bf16")]


def latent(heads, dim, rot, vdim, rank, base=10000.0, scaling=None, scale=None, turning=None):
    rot_spec = {"base": base, "dims": turning or rot}
    if scaling:
        rot_spec["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": rank,
                      "scale": scale if scale is not None else (dim + rot) ** -0.5, "rot": rot_spec}}


def delta(heads, kv, dim, vdim, conv, channel=False):
    return {"type": "channel_delta" if channel else "delta",
            "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}}


def config(width, vocab, layers, ffs, loop=None, eps=1e-5, scale=1.0):
    c = {"architecture": "Beletar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": scale}, "layers": []}
    for L, ff in zip(layers, ffs):
        c["layers"].append(dict(L, mlp={"kind": "dense", "ff": ff} if ff else None))
    if loop:
        c["loop"] = dict(zip(("start", "stop", "times"), loop))
    return c


CONFIGS = {
    # all three mixers; a loop over the middle layers run three times; a layer without feed-forward; stretched wavelengths
    "P": (config(96, 300, [delta(4, 2, 16, 24, 4), latent(3, 16, 8, 24, 40, 10000.0, (8.0, 64, 16.0, 2.0)),
                           delta(6, 3, 16, 8, 2, channel=True), delta(2, 2, 32, 16, 3)],
                 [40, 56, None, 24], loop=(1, 3, 3), eps=3e-6, scale=3.0), {"l2": (5, 7)}),
    # no loop; one head everywhere; no stretching; a convolution of one tap (none); embedding multiplier 1
    "Q": (config(64, 200, [latent(1, 32, 16, 8, 24, 500.0), delta(1, 1, 8, 40, 1), delta(1, 1, 24, 8, 5, channel=True)],
                 [16, None, 32]), {"l2": (3, 2)}),
    # sizes that the tensor-core products like; prompts of several pages; a loop of the first layers run twice
    "R": (config(128, 512, [latent(4, 32, 32, 64, 64, 20000.0, (4.0, 256, 32.0, 1.0), 0.11), delta(4, 2, 32, 32, 4),
                            delta(4, 4, 64, 32, 3, channel=True), latent(2, 64, 16, 32, 96, 1000.0, turning=8)],
                 [128, 64, 128, None], loop=(0, 2, 2), scale=11.3), {"l2": (16, 8)}),
    # sizes that fit no tile: a width that is no multiple of 8 (no tensor-core product at all), odd head sizes, a latent
    # that no warp divides, a loop that is run once
    "S": (config(100, 333, [delta(6, 2, 24, 40, 3, channel=True), latent(5, 24, 6, 40, 50, 777.0, (2.0, 100, 8.0, 0.5)),
                            delta(3, 1, 40, 24, 6)],
                 [56, 6, 30], loop=(0, 3, 1), scale=0.5), {"l0": (6, 10)}),
    # sizes that nothing divides (and a rotated part of which only the first four numbers turn): key channels of 10 and 6, value channels of 12 and 5, an odd latent, eight taps, five heads
    # on five and on one query/key head, a width that is a multiple of 4 only
    "T": (config(52, 97, [delta(5, 5, 10, 12, 8), latent(3, 10, 6, 7, 17, 300.0, (3.0, 50, 4.0, 0.25), 0.4, turning=4),
                          delta(5, 1, 6, 5, 2, channel=True)],
                 [10, 22, None], loop=(1, 2, 2), scale=1.7), {"l2": (3, 5)}),
    # heads as large as real models have them: key channels of 128 and 256, a latent of 512 with a rotated part of 64
    "U": (config(256, 200, [delta(2, 1, 128, 128, 4), latent(2, 128, 64, 128, 512, 10000.0, (4.0, 128, 32.0, 1.0)),
                            delta(2, 2, 256, 64, 4, channel=True)],
                 [64, None, 64], loop=(0, 3, 2), scale=4.0), {"l2": (16, 16)}),
    # single mechanisms
    "delta_only": (config(64, 100, [delta(4, 2, 16, 24, 4)], [None]), {}),
    "channel_only": (config(64, 100, [delta(2, 1, 16, 24, 3, channel=True)], [None]), {"l0": (4, 6)}),
    "latent_only": (config(64, 100, [latent(4, 16, 8, 12, 20, 10000.0, (4.0, 32, 8.0, 1.0))], [None]), {}),
    "mlp_loop": (config(64, 100, [delta(1, 1, 16, 16, 2)], [48], loop=(0, 1, 3), scale=2.0), {}),
}
SEEDS = {name: 70 + i for i, name in enumerate(CONFIGS)}


def tensors_of(cfg, ranks, rng):
    """Every tensor of the design by name, float32, already shaped so that faults show."""
    w = cfg["width"]
    out = {}

    def normal(shape, std=0.02, mean=0.0):
        return (rng.standard_normal(shape) * std + mean).astype(np.float32)

    out["embed"] = normal((cfg["vocab"], w), 0.3)
    out["final.norm"] = normal((w,), 0.1, 1.0)
    out["final.norm.b"] = normal((w,), 0.1)
    for i, L in enumerate(cfg["layers"]):
        p = "l%d." % i
        m = L["mixer"]
        out[p + "norm1"] = normal((w,), 0.1, 1.0)
        out[p + "norm1.b"] = normal((w,), 0.2)
        if L["type"] == "latent_attention":
            H, dim, rd, vd, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            # scores of a few units whatever the sizes: peaked, but not so that two keys within rounding of each other swap
            out[p + "mix.q"] = normal((H * (dim + rd), w), 0.5 * min(1.0, (32.0 / (dim + rd)) ** 0.5) * min(1.0, (96.0 / w) ** 0.5))
            out[p + "mix.dkv"] = normal((rank + rd, w), 0.3 * min(1.0, (96.0 / w) ** 0.5))
            out[p + "mix.dkv.norm"] = normal((rank,), 0.1, 1.0)
            out[p + "mix.uk"] = normal((H * dim, rank), 0.3 * min(1.0, (64.0 / rank) ** 0.5))
            out[p + "mix.uv"] = normal((H * vd, rank), 0.1)
            out[p + "mix.sink"] = normal((H,), 2.0, 1.0)
            out[p + "mix.g"] = normal((H, w), 0.2)
            out[p + "mix.o"] = normal((w, H * vd), 0.05)
        else:
            H, G, dk, dv, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            for n, rows in (("q", G * dk), ("k", G * dk), ("v", H * dv)):
                out[p + "mix." + n] = normal((rows, w), 0.2)
                out[p + "mix." + n + ".conv"] = normal((rows, taps), 0.5, 0.3)
            out[p + "mix.b"] = normal((H, w), 0.2)
            out[p + "mix.A_log"] = normal((H,), 0.5, -2.5)
            out[p + "mix.norm"] = normal((dv,), 0.1, 1.0)
            out[p + "mix.o"] = normal((w, H * dv), 0.05)
            if L["type"] == "channel_delta":
                ra, rg = ranks["l%d" % i]
                out[p + "mix.a1"] = normal((ra, w), 0.2)
                out[p + "mix.a2"] = normal((H * dk, ra), 0.3)
                out[p + "mix.dt_bias"] = normal((H * dk,), 0.8, -2.0)
                out[p + "mix.g1"] = normal((rg, w), 0.2)
                out[p + "mix.g2"] = normal((H * dv, rg), 0.3)
            else:
                out[p + "mix.a"] = normal((H, w), 0.2)
                out[p + "mix.dt_bias"] = normal((H,), 0.8, -2.0)
                out[p + "mix.g"] = normal((H * dv, w), 0.2)
        if L.get("mlp"):
            ff = L["mlp"]["ff"]
            out[p + "norm2"] = normal((w,), 0.1, 1.0)
            out[p + "norm2.b"] = normal((w,), 0.2)
            out[p + "mlp.gate"] = normal((ff, w), 0.15)
            out[p + "mlp.up"] = normal((ff, w), 0.15)
            out[p + "mlp.down"] = normal((w, ff), 0.1)
    return out


def write_folder(path, cfg, ranks, seed):
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    t = tensors_of(cfg, ranks, np.random.default_rng(seed))
    write_safetensors(os.path.join(path, "model.safetensors"),
                      [(n, "BF16", list(x.shape), harness.f32_to_bf16_bytes(x)) for n, x in t.items()])
    return path


_made = {}


def model(root, name):
    key = (str(root), name)
    if key not in _made:
        cfg, ranks = CONFIGS[name]
        d = write_folder(os.path.join(str(root), "beletar_" + name), cfg, ranks, SEEDS[name])
        _made[key] = (d,) + plain.load(d)
    return _made[key]


@pytest.fixture(scope="module")
def root(tmp_path_factory):
    return tmp_path_factory.mktemp("beletar")


def engine(root, name, dtype, **kw):
    d, cfg, t = model(root, name)
    kw.setdefault("max_ctx", 1024)
    kw.setdefault("max_batch", 6)
    return Engine(model_path=d, dtype=dtype, **kw), cfg, t


_plain = {}


def plain_logits(root, name, prompt):
    key = (str(root), name, tuple(prompt))
    if key not in _plain:
        _, cfg, t = model(root, name)
        _plain[key] = plain.forward(cfg, t, prompt)
    return _plain[key]


def agree(got, root, name, prompt, places, dtype, what):
    ref = plain_logits(root, name, prompt)
    got = np.asarray(got, dtype=np.float64)
    assert got.shape == (len(places), ref.shape[1]), what
    assert np.isfinite(got).all(), what
    if dtype == "float32":
        spread = np.sqrt((ref ** 2).mean())
        err = np.abs(got - ref[places]).max()
        assert err <= 1e-4 * max(spread, 1.0), "%s: |engine - plain| = %.3g (spread %.3g)" % (what, err, spread)
        return
    for i in range(len(places)):
        ok, text = harness.bf16_ok(got[i], ref[places[i]], what, harness.BF16_WIDE)
        assert ok, "%s, place %d: %s" % (what, places[i], text)


def prompts(lengths, vocab, seed):
    return tiny_configs.random_prompts(lengths, vocab, seed)


def nothing_held(eng):
    st = eng.stats()
    return st["slots_held"] == 0 and all(g["pages_held"] == 0 for g in st["groups"])


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["delta_only", "channel_only", "latent_only", "mlp_loop"])
def test_each_mechanism_alone(root, name, dtype):
    eng, cfg, _ = engine(root, name, dtype)
    for n, p in zip([1, 2, 40, 90], prompts([1, 2, 40, 90], cfg["vocab"], 3)):
        s = eng.alloc_slot()
        got = eng.step([s], [p], [list(range(n))], to="host")
        eng.free_slot(s)
        agree(got, root, name, p, list(range(n)), dtype, "%s alone, %d tokens" % (name, n))
    eng.check()
    assert nothing_held(eng)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,n", [("P", 150), ("Q", 70), ("R", 300), ("S", 200), ("T", 130), ("U", 100)])
def test_whole_prompt(root, name, n, dtype):
    eng, cfg, _ = engine(root, name, dtype)
    (p,) = prompts([n], cfg["vocab"], 5)
    s = eng.alloc_slot()
    got = eng.step([s], [p], [list(range(n))], to="host")
    eng.free_slot(s)
    agree(got, root, name, p, list(range(n)), dtype, "%s whole %d" % (name, n))
    assert nothing_held(eng)


def test_faults_would_show(root):
    """What the comparisons above would see: the plain implementation with one mechanism changed a little differs from
    itself by far more than the float32 bound: a far key dropped, the sink left out, a state that forgets, the
    a late start (keys, state and the convolution's history lost), a pass of the loop left out."""
    _, cfg, t = model(root, "P")
    (p,) = prompts([150], cfg["vocab"], 5)
    ref = plain.forward(cfg, t, p)
    bound = 100 * 1e-4 * max(np.sqrt((ref ** 2).mean()), 1.0)
    no_sink = dict(t)
    no_sink["l1.mix.sink"] = t["l1.mix.sink"] - 30.0
    assert np.abs(plain.forward(cfg, no_sink, p) - ref).max() > bound
    forgetful = dict(t)
    forgetful["l0.mix.A_log"] = t["l0.mix.A_log"] + 1.0
    assert np.abs(plain.forward(cfg, forgetful, p) - ref).max() > bound
    # a sequence that starts 100 tokens late misses keys and state: the last logits must differ
    late = plain.forward(cfg, t, p[100:])
    assert np.abs(late[-1] - ref[-1]).max() > bound
    # ... and the attention alone, too: a key 100 back carries weight
    _, lcfg, lt = model(root, "latent_only")
    (lp,) = prompts([140], lcfg["vocab"], 5)
    a, b = plain.forward(lcfg, lt, lp), plain.forward(lcfg, lt, lp[100:])
    assert np.abs(a[-1] - b[-1]).max() > 100 * 1e-4 * max(np.sqrt((a ** 2).mean()), 1.0)
    once = dict(cfg, loop=dict(cfg["loop"], times=cfg["loop"]["times"] - 1))
    assert np.abs(plain.forward(once, t, p) - ref).max() > bound


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "R", "S", "T", "U"])
def test_prompt_then_token_by_token(root, name, dtype):
    """The last tokens one by one, across page borders of 64: states, the convolution's history and the cached latents
    go from step to step."""
    eng, cfg, _ = engine(root, name, dtype)
    n, tail = (330, 150) if name == "R" else (120, 60)
    (p,) = prompts([n], cfg["vocab"], 6)
    s = eng.alloc_slot()
    got = [eng.step([s], [p[:n - tail]], [[n - tail - 1]], to="host")]
    for i in range(n - tail, n):
        got.append(eng.step([s], [[p[i]]], [[0]], to="host"))
    eng.free_slot(s)
    agree(np.concatenate(got), root, name, p, list(range(n - tail - 1, n)), dtype, "%s decode" % name)
    assert nothing_held(eng)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "Q"])
def test_all_tokens_one_by_one(root, name, dtype):
    """From the very first token: states start at zero, the inputs before the first are zero."""
    eng, cfg, _ = engine(root, name, dtype)
    (p,) = prompts([70], cfg["vocab"], 7)
    s = eng.alloc_slot()
    got = [eng.step([s], [[tok]], [[0]], to="host") for tok in p]
    eng.free_slot(s)
    agree(np.concatenate(got), root, name, p, list(range(70)), dtype, "%s one by one" % name)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,cuts", [("P", [2, 3, 7, 64, 65, 9, 1, 1, 2]), ("R", [64, 2, 128, 100, 6]), ("Q", [1, 2, 30, 37, 3]),
                                       ("S", [5, 64, 3, 70, 2, 2]), ("T", [3, 2, 40, 1, 5, 66, 2])])
def test_portions(root, name, cuts, dtype):
    """A prompt cut into steps of several sizes, down to two tokens (and one): portions shorter than the convolution
    keep part of the history that was there."""
    eng, cfg, _ = engine(root, name, dtype)
    n = sum(cuts)
    (p,) = prompts([n], cfg["vocab"], 8)
    s = eng.alloc_slot()
    got, at = [], 0
    for c in cuts:
        got.append(eng.step([s], [p[at:at + c]], [list(range(c))], to="host"))
        at += c
    eng.free_slot(s)
    agree(np.concatenate(got), root, name, p, list(range(n)), dtype, "%s portions %s" % (name, cuts))


@pytest.mark.parametrize("dtype", DTYPES)
def test_passes_of_the_step_function(root, dtype):
    """A prompt longer than the step function's pass: state, history and cache go from pass to pass."""
    eng, cfg, _ = engine(root, "R", dtype, prefill_chunk=64)
    (p,) = prompts([300], cfg["vocab"], 9)
    s = eng.alloc_slot()
    got = eng.step([s], [p], [list(range(300))], to="host")
    eng.free_slot(s)
    agree(got, root, "R", p, list(range(300)), dtype, "R in passes of 64")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "R"])
def test_batch_of_unequal_requests(root, name, dtype):
    """Requests of different lengths in one batch (one of a single token), then decoded together; the shorter ones
    end earlier.  Every request must come out as it does alone."""
    eng, cfg, _ = engine(root, name, dtype)
    lengths = [1, 70, 131, 40] if name == "P" else [1, 200, 90]
    tail = 20
    ps = prompts([n + tail for n in lengths], cfg["vocab"], 10)
    slots = [eng.alloc_slot() for _ in ps]
    got = {i: [] for i in range(len(ps))}
    first = eng.step(slots, [p[:n] for p, n in zip(ps, lengths)], [[n - 1] for n in lengths], to="host")
    for i in range(len(ps)):
        got[i].append(first[i:i + 1])
    live = list(range(len(ps)))
    for k in range(tail):
        if k == 7:
            eng.free_slot(slots[live.pop(0)])               # the first request ends early
        out = eng.step([slots[i] for i in live], [[ps[i][lengths[i] + k]] for i in live], [[0]] * len(live), to="host")
        for j, i in enumerate(live):
            got[i].append(out[j:j + 1])
    for i in live:
        eng.free_slot(slots[i])
    for i, p in enumerate(ps):
        n = lengths[i]
        places = list(range(n - 1, n - 1 + len(got[i])))
        agree(np.concatenate(got[i]), root, name, p, places, dtype, "%s request %d of a batch" % (name, i))
    assert nothing_held(eng)


@pytest.mark.parametrize("dtype", DTYPES)
def test_slots_and_pages_used_again(root, dtype):
    """A slot that held a long request is given to a short one: the states and the history start at zero again, stale
    pages are not read."""
    eng, cfg, _ = engine(root, "P", dtype, max_batch=2, max_ctx=256, max_tokens=512)
    a, b, c = prompts([200, 30, 90], cfg["vocab"], 11)
    for p in (a, b, c, b):
        s = eng.alloc_slot()
        got = eng.step([s], [p], [list(range(len(p)))], to="host")
        eng.free_slot(s)
        agree(got, root, "P", p, list(range(len(p))), dtype, "P in a slot used before (%d tokens)" % len(p))
    s1, s2 = eng.alloc_slot(), eng.alloc_slot()
    g1 = eng.step([s1, s2], [c[:50], b], [[49], [len(b) - 1]], to="host")
    g2 = eng.step([s1], [c[50:]], [list(range(40))], to="host")
    eng.free_slot(s1)
    eng.free_slot(s2)
    agree(np.concatenate([g1[:1], g2]), root, "P", c, [49] + list(range(50, 90)), dtype, "P cut in two, in a used slot")
    agree(g1[1:], root, "P", b, [len(b) - 1], dtype, "P beside it")
    assert nothing_held(eng)


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(root, dtype):
    """Hundreds of single-token steps: the states run on, keys hundreds of tokens back stay in sight."""
    eng, cfg, _ = engine(root, "R", dtype)
    (p,) = prompts([10 + 400], cfg["vocab"], 12)
    s = eng.alloc_slot()
    eng.step([s], [p[:10]], [[]], to="host")
    got = [eng.step([s], [[tok]], [[0]], to="host") for tok in p[10:]]
    eng.free_slot(s)
    agree(np.concatenate(got), root, "R", p, list(range(10, 410)), dtype, "R long decoding")


@pytest.mark.parametrize("name", ["P", "R"])
def test_greedy_generation(root, name):
    """Engine.generate (the library's scheduler, its decoder with captured steps, its sampler) chooses the tokens
    that the plain implementation chooses."""
    eng, cfg, t = engine(root, name, "float32", max_batch=3)
    ps = prompts([5, 23, 64, 9], cfg["vocab"], 13)
    out = eng.generate(ps, max_new_tokens=12, temperature=0.0, ignore_eos=True)
    for p, g in zip(ps, out):
        want = plain.greedy(cfg, t, p, 12)
        for i, (a, b) in enumerate(zip(g.tokens, want)):
            if a != b:
                lg = plain.forward(cfg, t, p + want[:i])[-1]
                top2 = np.sort(lg)[-2:]
                assert top2[1] - top2[0] < 1e-4, "%s: token %d is %d, plain chooses %d" % (name, i, a, b)
                break
    assert nothing_held(eng)


def test_bf16_generation_runs_and_repeats(root):
    eng, cfg, _ = engine(root, "R", "bfloat16", max_batch=4)
    ps = prompts([5, 23, 64, 9], cfg["vocab"], 14)
    a = eng.generate(ps, max_new_tokens=20, temperature=0.0, ignore_eos=True)
    b = eng.generate(ps, max_new_tokens=20, temperature=0.0, ignore_eos=True)
    assert [g.tokens for g in a] == [g.tokens for g in b]
    assert all(len(g.tokens) == 20 for g in a)
    assert nothing_held(eng)
