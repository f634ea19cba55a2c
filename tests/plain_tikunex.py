"""Plain, slow statement of the Tikunex decoder: whole sequences, float64, no cache, no
batching, no kernels; one function per mechanism.  It shares no code with the package
under test (own reader of config.json and of the safetensors file).

Notation: X is [T, width] (the residual stream of one sequence), h a mixer's or a
feed-forward's input.  Weights are [out, in] and act as h @ W.T.

The design, in this file's words:
  x0 = unit_offset_norm(embed[tokens], embed.norm)
  layers run in config order; the layers loop.start .. loop.stop-1 run loop.times times
  in a row with the same weights (own memory each time); before the first layer of each
  such pass X = [X, x0] @ loop.in.T
  a layer:  X += mixer(norm1(X));  X += moe(norm2(X)) (if it has one);  X += token_side(X, tokens)
  logits = norm(X, final.norm) @ head.T
"""
import json
import math
import os
import struct

import numpy as np

F64 = np.float64


def read_safetensors(path):
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n).decode("utf-8"))
        blob = f.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        raw = blob[lo:hi]
        shape = tuple(info["shape"])
        if info["dtype"] == "BF16":
            arr = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32).astype(F64)
        elif info["dtype"] == "F32":
            arr = np.frombuffer(raw, dtype="<f4").astype(F64)
        elif info["dtype"] == "I32":
            arr = np.frombuffer(raw, dtype="<i4")
        else:
            raise ValueError("dtype %s" % info["dtype"])
        out[name] = arr.reshape(shape)
    return out


def load(model_dir):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(model_dir, "model.safetensors"))


# ---------------------------------------------------------------------------
# small functions
# ---------------------------------------------------------------------------
def rms_scale(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)


def unit_offset_norm(x, w, eps):
    return rms_scale(x, eps) * (1.0 + w)


def plain_norm(x, w, eps):
    return rms_scale(x, eps) * w


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


# ---------------------------------------------------------------------------
# mixers
# ---------------------------------------------------------------------------
def window_sink_attention(h, t, p, m):
    """Softmax attention without position encoding.  Query i sees key j if j <= i and
    (i - j < mask.size or j < mask.keep_first)."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    size, keep = m["mask"]["size"], m["mask"]["keep_first"]
    q = (h @ t[p + "q"].T).reshape(T, H, dk)
    k = (h @ t[p + "k"].T).reshape(T, G, dk)
    v = (h @ t[p + "v"].T).reshape(T, G, dv)
    out = np.zeros((T, H, dv), dtype=F64)
    i = np.arange(T)[:, None]
    j = np.arange(T)[None, :]
    seen = (j <= i) & ((i - j < size) | (j < keep))
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * m["scale"]
        s = np.where(seen, s, -np.inf)
        s = s - s.max(axis=1, keepdims=True)
        w = np.exp(s)
        w = w / w.sum(axis=1, keepdims=True)
        out[:, hd] = w @ v[:, g]
    return out.reshape(T, H * dv) @ t[p + "o"].T


def shifted_decay_mix(h, t, p, m, eps):
    """Token-shift time mixing with a per-channel decay that depends on the token and a
    bonus for the present token."""
    T, W = h.shape
    H, d = m["heads"], m["dim"]
    prev = np.vstack([np.zeros((1, W), dtype=F64), h[:-1]])
    mix = {s: h + (prev - h) * t[p + "mu." + s] for s in "rkvgw"}
    r = (mix["r"] @ t[p + "r"].T).reshape(T, H, d)
    k = (mix["k"] @ t[p + "k"].T).reshape(T, H, d)
    v = (mix["v"] @ t[p + "v"].T).reshape(T, H, d)
    gate = silu(mix["g"] @ t[p + "g"].T)
    w = np.exp(-np.exp(np.tanh(mix["w"] @ t[p + "w1"].T) @ t[p + "w2"].T + t[p + "w0"])).reshape(T, H, d)
    u = t[p + "u"].reshape(H, d)
    o = np.zeros((T, H, d), dtype=F64)
    for hd in range(H):
        S = np.zeros((d, d), dtype=F64)            # [key channel, value channel]
        for i in range(T):
            kv = np.outer(k[i, hd], v[i, hd])
            o[i, hd] = (S + u[hd][:, None] * kv).T @ r[i, hd]
            S = w[i, hd][:, None] * S + kv
    o = rms_scale(o, eps).reshape(T, H * d) * t[p + "norm"] * gate
    return o @ t[p + "o"].T


def parallel_mixer(h, t, p, m, eps):
    left = window_sink_attention(h, t, p + "left.", m["left"])
    right = shifted_decay_mix(h, t, p + "right.", m["right"], eps)
    return m["left_scale"] * left + m["right_scale"] * right


def gated_linear_attention(h, t, p, m, eps):
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ t[p + "q"].T).reshape(T, H, dk) * dk ** -0.5
    k = (h @ t[p + "k"].T).reshape(T, H, dk)
    v = (h @ t[p + "v"].T).reshape(T, H, dv)
    z = (h @ t[p + "a1"].T) @ t[p + "a2"].T + t[p + "a2.b"]
    alpha = (sigmoid(z) ** (1.0 / m["tau"])).reshape(T, H, dk)
    o = np.zeros((T, H, dv), dtype=F64)
    for hd in range(H):
        S = np.zeros((dk, dv), dtype=F64)
        for i in range(T):
            S = alpha[i, hd][:, None] * S + np.outer(k[i, hd], v[i, hd])
            o[i, hd] = S.T @ q[i, hd]
    o = plain_norm(o, t[p + "norm"], eps).reshape(T, H * dv)
    return (o * silu(h @ t[p + "g"].T)) @ t[p + "o"].T


# ---------------------------------------------------------------------------
# feed-forward and the per-layer token input
# ---------------------------------------------------------------------------
def routed_experts(h, t, p, m, gaps=None):
    """gaps, if given, is an array [T] that keeps, per token, the smallest distance seen so far between the last
    chosen logit and the first one that was not chosen (how close the choice was)."""
    E, top = m["router"]["experts"], m["router"]["top"]
    z = h @ t[p + "router"].T + t[p + "router.b"]
    out = np.zeros((h.shape[0], t[p + "e0.down"].shape[0]), dtype=F64)
    for i in range(h.shape[0]):
        chosen = np.argsort(-z[i], kind="stable")[:top]
        if gaps is not None and top < E:
            ordered = np.sort(z[i])[::-1]
            gaps[i] = min(gaps[i], ordered[top - 1] - ordered[top])
        w = np.exp(z[i, chosen] - z[i, chosen].max())
        w = w / w.sum()
        for e, we in zip(chosen, w):
            pe = "%se%d." % (p, e)
            a = silu(h[i] @ t[pe + "gate"].T) * (h[i] @ t[pe + "up"].T)
            out[i] += we * (a @ t[pe + "down"].T)
    return out


def token_side(x, tokens, layer, t, p, dim, eps):
    e = t["side.embed"][np.asarray(tokens)][:, layer * dim:(layer + 1) * dim]
    g = gelu_tanh(x @ t[p + "gate"].T) * e
    y = g @ t[p + "proj"].T
    return rms_scale(y, eps) * t[p + "norm"]


# ---------------------------------------------------------------------------
# the model
# ---------------------------------------------------------------------------
def run_order(cfg):
    """[(layer, first of a pass)] in the order the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, False) for i in range(a)]
    for _ in range(times):
        order += [(i, i == a) for i in range(a, b)]
    order += [(i, False) for i in range(b, n)]
    return order


def layer_forward(cfg, t, i, X, tokens, gaps=None):
    L = cfg["layers"][i]
    eps = cfg["norm"]["eps"]
    p = "l%d." % i
    h = unit_offset_norm(X, t[p + "norm1"], eps)
    if L["type"] == "gla":
        X = X + gated_linear_attention(h, t, p + "mix.", L["mixer"], eps)
    elif L["type"] == "parallel":
        X = X + parallel_mixer(h, t, p + "mix.", L["mixer"], eps)
    else:
        raise ValueError("mixer type %r" % L["type"])
    if L.get("mlp"):
        X = X + routed_experts(unit_offset_norm(X, t[p + "norm2"], eps), t, p + "mlp.", L["mlp"], gaps)
    side = cfg.get("token_side")
    if side:
        X = X + token_side(X, tokens, i, t, p + "side.", side["dim"], eps)
    return X


def forward(cfg, t, tokens, keep_layers=False, gaps=None):
    """logits [T, vocab]; with keep_layers also the residual stream after every layer run."""
    eps = cfg["norm"]["eps"]
    x0 = unit_offset_norm(t["embed"][np.asarray(tokens)], t["embed.norm"], eps)
    X = x0
    after = []
    for i, first in run_order(cfg):
        if first:
            X = np.concatenate([X, x0], axis=1) @ t["loop.in"].T
        X = layer_forward(cfg, t, i, X, tokens, gaps)
        after.append(X)
    logits = unit_offset_norm(X, t["final.norm"], eps) @ t["head"].T
    return (logits, np.stack(after)) if keep_layers else logits


def greedy(cfg, t, prompt, n_new):
    """The tokens that greedy decoding appends to `prompt` (the first maximum wins)."""
    tokens = list(prompt)
    for _ in range(n_new):
        tokens.append(int(np.argmax(forward(cfg, t, tokens)[-1])))
    return tokens[len(prompt):]
