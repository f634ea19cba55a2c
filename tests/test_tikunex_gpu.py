"""Tikunex through the engine against the plain implementation (tests/plain_tikunex.py), on small
configurations of the tests' own with random weights: each mechanism alone, whole prompts, decoding
token by token, prompts cut into portions, batches of unequal requests, slots and pages used again,
keys at the edges of the window and of the kept first tokens, long decoding, and greedy generation
through Engine.generate.

Random N(0, 0.02) weights would hide faults (flat softmax, decays that forget at once, routers that
barely prefer anybody), so the folders are rewritten: queries, keys and the token table are scaled up
(peaked attention), the decays' biases are set so that the states remember hundreds of tokens, and the
routers are scaled so that their choices are clear.

float32 must agree with the plain implementation to summation order.  In bfloat16 a router's close
call can go the other way, and a different expert is a different function, not a rounding; with random
inputs some token's choice is always close.  The bfloat16 runs therefore use folders whose routers are
dominated by well-separated biases (the choice is clear at every token; which expert a token gets is
then the same for all tokens), and are compared with a bound relative to the logits' spread.
"""
import os

import numpy as np
import pytest

import harness
import plain_tikunex as plain
import tiny_configs
from friday_inference_engine_b200 import Engine

pytestmark = pytest.mark.gpu
DTYPES = [pytest.param("float32", id="f32"), pytest.param("bfloat16", id="bf16")]


def moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def gla(heads, dim, vdim, tau, rank):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "decay_rank": rank}


def par(heads, kv, dim, vdim, size, keep, scale, rheads, rdim, rank, ls, rs):
    return {"left": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale,
                     "mask": {"size": size, "keep_first": keep}},
            "right": {"heads": rheads, "dim": rdim, "decay_rank": rank}, "left_scale": ls, "right_scale": rs}


def config(width, vocab, layers, loop=None, side=None, eps=1e-5):
    c = {"architecture": "Tikunex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if loop:
        c["loop"] = dict(zip(("start", "stop", "times"), loop))
    if side:
        c["token_side"] = {"dim": side}
    return c


CONFIGS = {
    # every mechanism; a loop from the first layer run three times; a layer without feed-forward; one expert chosen
    "X": config(96, 300, [
        {"type": "parallel", "mixer": par(4, 1, 16, 48, 20, 3, 0.3, 3, 16, 8, 0.7, 1.3), "mlp": moe(5, 1, 40)},
        {"type": "gla", "mixer": gla(3, 16, 32, 4.0, 8), "mlp": moe(4, 3, 24)},
        {"type": "parallel", "mixer": par(2, 2, 32, 16, 33, 0, 0.2, 1, 32, 4, 1.0, 0.5), "mlp": None},
    ], loop=(0, 2, 3), side=8, eps=3e-6),
    # no loop, no token input; one head everywhere; every expert chosen; a window that no prompt outgrows
    "Y": config(64, 200, [
        {"type": "gla", "mixer": gla(1, 32, 8, 1.0, 4), "mlp": moe(3, 3, 16)},
        {"type": "parallel", "mixer": par(1, 1, 8, 8, 1000, 2, 0.5, 1, 8, 4, 1.0, 1.0), "mlp": moe(6, 2, 32)},
    ]),
    # sizes that the tensor-core products like; kept first tokens that cross a page of 64; a loop of the last layers
    "Z": config(128, 512, [
        {"type": "gla", "mixer": gla(2, 64, 64, 8.0, 16), "mlp": moe(8, 2, 64)},
        {"type": "parallel", "mixer": par(4, 2, 32, 64, 130, 70, 0.18, 2, 32, 16, 1.1, 0.9), "mlp": moe(8, 2, 64)},
        {"type": "gla", "mixer": gla(4, 32, 16, 12.0, 8), "mlp": None},
    ], loop=(1, 3, 2), side=16),
    # sizes that fit no tile: a width that is no multiple of 8 (no tensor-core product at all), head sizes of 24 and 40,
    # inner sizes of 6 and 56, more kept tokens than the window is long, three passes of the loop
    "W": config(100, 333, [
        {"type": "parallel", "mixer": par(6, 3, 24, 40, 50, 70, 0.2, 2, 24, 6, 0.9, 1.1), "mlp": moe(3, 2, 56)},
        {"type": "gla", "mixer": gla(2, 24, 40, 3.0, 6), "mlp": moe(3, 1, 56)},
    ], loop=(0, 2, 3), side=6),
    # the same head sizes on a width that the tensor cores take; so many experts that prompts, too, run them per (row, choice)
    "V": config(192, 333, [
        {"type": "gla", "mixer": gla(2, 24, 40, 3.0, 6), "mlp": moe(40, 2, 24)},
        {"type": "parallel", "mixer": par(6, 3, 24, 40, 50, 70, 0.2, 2, 24, 6, 0.9, 1.1), "mlp": moe(40, 2, 24)},
    ], side=6),
    # single mechanisms
    "gla_only": config(64, 100, [{"type": "gla", "mixer": gla(2, 16, 24, 2.0, 4), "mlp": None}]),
    "parallel_only": config(64, 100, [{"type": "parallel", "mixer": par(4, 2, 16, 8, 12, 2, 0.4, 2, 16, 4, 1.2, 0.8), "mlp": None}]),
    "experts": config(64, 100, [{"type": "gla", "mixer": gla(1, 16, 16, 2.0, 4), "mlp": moe(7, 2, 24)}]),
    "token_input": config(64, 100, [{"type": "gla", "mixer": gla(1, 16, 16, 2.0, 4), "mlp": None}], side=4),
    "loop_only": config(64, 100, [{"type": "gla", "mixer": gla(1, 16, 16, 2.0, 4), "mlp": None}], loop=(0, 1, 2)),
}
SEEDS = {name: 40 + i for i, name in enumerate(CONFIGS)}


def sharpen(model_dir, calm_routers):
    def change(n, x):
        if calm_routers and n.endswith(".router"):
            return x * np.float32(4.0)
        if calm_routers and n.endswith(".router.b"):
            return np.random.default_rng(len(x)).permutation(len(x)).astype(np.float32) * np.float32(8.0)
        if n.endswith(".left.q") or n.endswith(".left.k"):
            return x * np.float32(40.0)
        if n == "embed" or n == "side.embed":
            return x * np.float32(20.0)
        if n.endswith(".mix.q") or n.endswith(".mix.k") or n.endswith(".right.r") or n.endswith(".right.k"):
            return x * np.float32(8.0)
        if n.endswith(".a2.b"):
            return x * np.float32(40.0) + np.float32(4.0)         # sigmoid(4)^(1/tau): a long memory
        if n.endswith(".a2") or n.endswith(".w2"):
            return x * np.float32(30.0)                           # ... that still depends on the token
        if n.endswith(".w0"):
            return x * np.float32(40.0) - np.float32(4.0)         # exp(-exp(-4)) = 0.98
        if n.endswith(".right.u"):
            return x * np.float32(30.0)
        if n.endswith(".router") or n.endswith(".router.b"):
            return x * np.float32(60.0)
        if n.endswith(".side.gate") or n.endswith(".mu.r") or n.endswith(".mu.k") or n.endswith(".mu.v") or n.endswith(".mu.w") or n.endswith(".mu.g"):
            return x * np.float32(15.0)
        if n == "loop.in":
            return x * np.float32(6.0)
        return None
    harness.rewrite(model_dir, change)


_made = {}


def model(root, name, dtype="float32"):
    calm = dtype != "float32"
    key = (str(root), name, calm)
    if key not in _made:
        d = tiny_configs.make_model_dir(os.path.join(str(root), "tikunex_%s_%d" % (name, calm)), CONFIGS[name], SEEDS[name])
        sharpen(d, calm)
        _made[key] = (d,) + plain.load(d)
    return _made[key]


@pytest.fixture(scope="module")
def root(tmp_path_factory):
    return tmp_path_factory.mktemp("tikunex")


def engine(root, name, dtype, **kw):
    d, cfg, t = model(root, name, dtype)
    kw.setdefault("max_ctx", 1024)
    kw.setdefault("max_batch", 6)
    return Engine(model_path=d, dtype=dtype, **kw), cfg, t


_plain = {}


def plain_logits(root, name, prompt, dtype):
    """(logits [T, vocab], first position whose routing was a close call or T)."""
    key = (str(root), name, tuple(prompt), dtype != "float32")
    if key not in _plain:
        _, cfg, t = model(root, name, dtype)
        gaps = np.full((len(prompt),), np.inf)
        lg = plain.forward(cfg, t, prompt, gaps=gaps)
        close = np.nonzero(gaps < 0.25)[0]
        _plain[key] = (lg, int(close[0]) if len(close) else len(prompt))
    return _plain[key]


def agree(got, root, name, prompt, places, dtype, what):
    """Engine logits at `places` of `prompt` against the plain implementation."""
    ref, clear = plain_logits(root, name, prompt, dtype)
    got = np.asarray(got, dtype=np.float64)
    assert got.shape == (len(places), ref.shape[1]), what
    assert np.isfinite(got).all(), what
    if dtype == "float32":
        spread = np.sqrt((ref ** 2).mean())
        err = np.abs(got - ref[places]).max()
        assert err <= 1e-4 * max(spread, 1.0), "%s: |engine - plain| = %.3g (spread %.3g)" % (what, err, spread)
        return
    assert clear == len(prompt), "%s: the routing at token %d is a close call; this folder was made so that none is" % (what, clear)
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
@pytest.mark.parametrize("name", ["gla_only", "parallel_only", "experts", "token_input", "loop_only"])
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
@pytest.mark.parametrize("name,n", [("X", 150), ("Y", 70), ("Z", 300), ("W", 200), ("V", 200)])
def test_whole_prompt(root, name, n, dtype):
    eng, cfg, _ = engine(root, name, dtype)
    (p,) = prompts([n], cfg["vocab"], 5)
    s = eng.alloc_slot()
    got = eng.step([s], [p], [list(range(n))], to="host")
    eng.free_slot(s)
    agree(got, root, name, p, list(range(n)), dtype, "%s whole %d" % (name, n))
    assert nothing_held(eng)


@pytest.mark.parametrize("form", ["grouped", "dense", "pairs"])
@pytest.mark.parametrize("name", ["Z", "V"])
def test_every_form_of_the_experts(root, name, form, monkeypatch):
    """The three ways in which routed experts run for many rows in bfloat16 (rows gathered by expert, all experts
    with zero weights for the unchosen, one block per row and choice) agree with the plain implementation."""
    monkeypatch.setenv("FRIDAY_EXPERTS", form)
    eng, cfg, _ = engine(root, name, "bfloat16")
    lengths = [150, 3, 70]
    ps = prompts(lengths, cfg["vocab"], 21)
    slots = [eng.alloc_slot() for _ in ps]
    got = eng.step(slots, ps, [list(range(n)) for n in lengths], to="host")
    at = 0
    for s, p, n in zip(slots, ps, lengths):
        eng.free_slot(s)
        agree(got[at:at + n], root, name, p, list(range(n)), "bfloat16", "%s experts %s, %d tokens" % (name, form, n))
        at += n


def test_the_window_and_the_kept_tokens_show(root):
    """The comparison above would see a window or a count of kept tokens that is off by one: the plain implementation
    with either changed by one differs from itself by far more than the bound."""
    _, cfg, t = model(root, "X")
    (p,) = prompts([150], cfg["vocab"], 5)
    ref = plain.forward(cfg, t, p)
    spread = np.sqrt((ref ** 2).mean())
    import copy
    for key, delta in (("size", 1), ("size", -1), ("keep_first", 1), ("keep_first", -1)):
        other = copy.deepcopy(cfg)
        other["layers"][0]["mixer"]["left"]["mask"][key] += delta
        assert np.abs(plain.forward(other, t, p) - ref).max() > 100 * 1e-4 * spread, (key, delta)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["X", "Z", "W", "V"])
def test_prompt_then_token_by_token(root, name, dtype):
    """The last tokens one by one: the window passes over decoded tokens, pages fill and are given back, the kept
    first tokens stay."""
    eng, cfg, _ = engine(root, name, dtype)
    n, tail = (330, 150) if name == "Z" else (120, 60)
    (p,) = prompts([n], cfg["vocab"], 6)
    s = eng.alloc_slot()
    got = [eng.step([s], [p[:n - tail]], [[n - tail - 1]], to="host")]
    for i in range(n - tail, n):
        got.append(eng.step([s], [[p[i]]], [[0]], to="host"))
    eng.free_slot(s)
    agree(np.concatenate(got), root, name, p, list(range(n - tail - 1, n)), dtype, "%s decode" % name)
    assert nothing_held(eng)


@pytest.mark.parametrize("dtype", DTYPES)
def test_all_tokens_one_by_one(root, dtype):
    """From the very first token: states start at zero, the row before the first is zero."""
    eng, cfg, _ = engine(root, "X", dtype)
    (p,) = prompts([45], cfg["vocab"], 7)
    s = eng.alloc_slot()
    got = [eng.step([s], [[tok]], [[0]], to="host") for tok in p]
    eng.free_slot(s)
    agree(np.concatenate(got), root, "X", p, list(range(45)), dtype, "X one by one")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,cuts", [("X", [2, 3, 7, 64, 65, 9]), ("Z", [64, 2, 128, 100, 6]), ("Y", [1, 2, 30, 37]), ("W", [5, 64, 3, 70])])
def test_portions(root, name, cuts, dtype):
    """A prompt cut into steps of several sizes, down to two tokens (and one)."""
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
    """A prompt longer than the step function's pass: the states, the row before and the window go from pass to pass."""
    eng, cfg, _ = engine(root, "Z", dtype, prefill_chunk=64)
    (p,) = prompts([300], cfg["vocab"], 9)
    s = eng.alloc_slot()
    got = eng.step([s], [p], [list(range(300))], to="host")
    eng.free_slot(s)
    agree(got, root, "Z", p, list(range(300)), dtype, "Z in passes of 64")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["X", "Z"])
def test_batch_of_unequal_requests(root, name, dtype):
    """Requests of different lengths in one batch (one of a single token), then decoded together; the shorter ones
    end earlier.  Every request must come out as it does alone."""
    eng, cfg, _ = engine(root, name, dtype)
    lengths = [1, 70, 131, 40] if name == "X" else [1, 200, 90]
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
    """A slot that held a long request is given to a short one: the states start at zero again, stale pages are not read."""
    eng, cfg, _ = engine(root, "X", dtype, max_batch=2, max_ctx=256, max_tokens=512)
    a, b, c = prompts([200, 30, 90], cfg["vocab"], 11)
    for p in (a, b, c, b):
        s = eng.alloc_slot()
        got = eng.step([s], [p], [list(range(len(p)))], to="host")
        eng.free_slot(s)
        agree(got, root, "X", p, list(range(len(p))), dtype, "X in a slot used before (%d tokens)" % len(p))
    # two at once, in slots that others held, after one of them was cut in two
    s1, s2 = eng.alloc_slot(), eng.alloc_slot()
    g1 = eng.step([s1, s2], [c[:50], b], [[49], [len(b) - 1]], to="host")
    g2 = eng.step([s1], [c[50:]], [list(range(40))], to="host")
    eng.free_slot(s1)
    eng.free_slot(s2)
    agree(np.concatenate([g1[:1], g2]), root, "X", c, [49] + list(range(50, 90)), dtype, "X cut in two, in a used slot")
    agree(g1[1:], root, "X", b, [len(b) - 1], dtype, "X beside it")
    assert nothing_held(eng)


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(root, dtype):
    """Hundreds of single-token steps: pages of the window are given back on the way, the kept tokens' pages never."""
    eng, cfg, _ = engine(root, "Z", dtype)
    (p,) = prompts([10 + 400], cfg["vocab"], 12)
    s = eng.alloc_slot()
    eng.step([s], [p[:10]], [[]], to="host")
    got = [eng.step([s], [[tok]], [[0]], to="host") for tok in p[10:]]
    held = eng.stats()["groups"][0]["pages_held"]
    eng.free_slot(s)
    places = list(range(10, 410))
    agree(np.concatenate(got), root, "Z", p, places, dtype, "Z long decoding")
    # window 130 and 70 kept tokens: 2 kept pages + at most 4 of the window, of the 7 that 410 tokens fill
    assert held <= 6, held


@pytest.mark.parametrize("name", ["X", "Z"])
def test_greedy_generation(root, name):
    """Engine.generate (the library's scheduler, its decoder with captured steps, its sampler) chooses the tokens
    that the plain implementation chooses."""
    eng, cfg, t = engine(root, name, "float32", max_batch=3)
    ps = prompts([5, 23, 64, 9], cfg["vocab"], 13)
    out = eng.generate(ps, max_new_tokens=12, temperature=0.0, ignore_eos=True)
    for p, g in zip(ps, out):
        want = plain.greedy(cfg, t, p, 12)
        # a tie within rounding may go either way: accept a run that leaves the plain one only where the two best
        # logits of the plain implementation are closer than 1e-4
        for i, (a, b) in enumerate(zip(g.tokens, want)):
            if a != b:
                lg = plain.forward(cfg, t, p + want[:i])[-1]
                top2 = np.sort(lg)[-2:]
                assert top2[1] - top2[0] < 1e-4, "%s: token %d is %d, plain chooses %d" % (name, i, a, b)
                break
    assert nothing_held(eng)


def test_bf16_generation_runs_and_repeats(root):
    eng, cfg, _ = engine(root, "Z", "bfloat16", max_batch=4)
    ps = prompts([5, 23, 64, 9], cfg["vocab"], 14)
    a = eng.generate(ps, max_new_tokens=20, temperature=0.0, ignore_eos=True)
    b = eng.generate(ps, max_new_tokens=20, temperature=0.0, ignore_eos=True)
    assert [g.tokens for g in a] == [g.tokens for g in b]
    assert all(len(g.tokens) == 20 for g in a)
    assert nothing_held(eng)
