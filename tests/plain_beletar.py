"""Plain, slow statement of the Beletar decoder: whole sequences, float64, no cache, no
batching, no kernels; one function per mechanism.  It shares no code with the package
under test (own reader of config.json and of the safetensors file).

Notation: X is [T, width] (the residual stream of one sequence), h a mixer's or a
feed-forward's input.  Weights are [out, in] and act as h @ W.T.

The design, in this file's words:
  x0 = embed[tokens] * embedding.scale
  layers run in config order; the layers loop.start .. loop.stop-1 run loop.times times
  in a row with the same weights (own memory each time); before the first layer of every
  pass after the first, X += x0
  a layer:  X += mixer(layer_norm(X, norm1));  X += gated_mlp(layer_norm(X, norm2)) (if it has one)
  mixers: "delta" and "channel_delta" (delta rule with a decay per head, or per head and key
  channel), "latent_attention" (keys and values expanded from one small latent per token,
  a rotated key part shared by the heads, a sink in the softmax, a gate per head)
  logits = layer_norm(X, final.norm) @ embed.T
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
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def layer_norm(x, w, b, eps):
    mu = x.mean(axis=-1, keepdims=True)
    d = x - mu
    var = (d * d).mean(axis=-1, keepdims=True)
    return d / np.sqrt(var + eps) * w + b


def rms_scale(x, eps):
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)


def unit(x):
    """x / sqrt(sum(x^2) + 1e-6) over the last axis."""
    return x / np.sqrt((x * x).sum(axis=-1, keepdims=True) + 1e-6)


# ---------------------------------------------------------------------------
# rotation with stretched frequencies
# ---------------------------------------------------------------------------
def rotary_frequencies(rot):
    """The dims/2 angular frequencies and the multiplier of cos and sin."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    f = np.array([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def turn_dim(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_dim(float(sc["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(sc["slow"]))), dims - 1)
    ramp = np.clip((np.arange(half, dtype=F64) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    stretched = f / factor * ramp + f * (1.0 - ramp)
    return stretched, 0.1 * math.log(factor) + 1.0


def rotate_pairs(x, positions, rot):
    """x [T, ..., dims]: (x[2i], x[2i+1]) turns by positions[t] * f_i."""
    f, mult = rotary_frequencies(rot)
    dims = int(rot["dims"])
    ang = np.asarray(positions, dtype=F64)[:, None] * f[None, :]           # [T, dims/2]
    shape = (x.shape[0],) + (1,) * (x.ndim - 2) + (dims // 2,)
    c, s = (np.cos(ang) * mult).reshape(shape), (np.sin(ang) * mult).reshape(shape)
    out = x.copy()
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


# ---------------------------------------------------------------------------
# mixers
# ---------------------------------------------------------------------------
def latent_attention(h, m, W, p, eps, positions=None):
    """Causal softmax attention whose keys and values come from a latent of kv_rank numbers per token."""
    T = h.shape[0]
    H, dim, rd, vd, rank = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    pos = np.arange(T) if positions is None else np.asarray(positions)
    q = (h @ W[p + "q"].T).reshape(T, H, dim + rd)
    q_plain, q_rot = q[..., :dim], rotate_pairs(q[..., dim:], pos, m["rot"])
    dkv = h @ W[p + "dkv"].T
    c = rms_scale(dkv[:, :rank], eps) * W[p + "dkv.norm"]
    k_rot = rotate_pairs(dkv[:, rank:], pos, m["rot"])                      # [T, rd], one for all heads
    k_plain = (c @ W[p + "uk"].T).reshape(T, H, dim)
    v = (c @ W[p + "uv"].T).reshape(T, H, vd)
    gate = sigmoid(h @ W[p + "g"].T)                                        # [T, H]
    out = np.zeros((T, H, vd), dtype=F64)
    causal = np.tril(np.ones((T, T), dtype=bool))
    for a in range(H):
        s = (q_plain[:, a] @ k_plain[:, a].T + q_rot[:, a] @ k_rot.T) * float(m["scale"])
        s = np.where(causal, s, -np.inf)
        sink = W[p + "sink"][a]
        top = np.maximum(s.max(axis=1), sink)
        e = np.exp(s - top[:, None])
        w = e / (e.sum(axis=1) + np.exp(sink - top))[:, None]
        out[:, a] = (w @ v[:, a]) * gate[:, a:a + 1]
    return out.reshape(T, H * vd) @ W[p + "o"].T


def short_convolution(x, taps_w):
    """x [T, C], taps_w [C, taps]: y[t] = sum_j w[:, j] x[t - (taps-1) + j], zeros before the start."""
    T, C = x.shape
    taps = taps_w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, C), dtype=F64), x], axis=0)
    y = np.zeros_like(x)
    for j in range(taps):
        y += padded[j:j + T] * taps_w[:, j][None, :]
    return y


def delta_rule(q, k, v, beta, decay):
    """Per head: S = decay * S; u = beta (v - S^T k); S += k u^T; o = S^T q.
    q, k [T, H, dk], v [T, H, dv], beta [T, H], decay [T, H, dk] (or [T, H, 1])."""
    T, H, dk = q.shape
    dv = v.shape[2]
    S = np.zeros((H, dk, dv), dtype=F64)
    o = np.zeros((T, H, dv), dtype=F64)
    for t in range(T):
        S = S * decay[t][:, :, None]
        u = beta[t][:, None] * (v[t] - np.einsum("hkv,hk->hv", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        o[t] = np.einsum("hkv,hk->hv", S, q[t])
    return o


def delta_mixer(h, m, W, p, eps, per_channel):
    T = h.shape[0]
    H, G, dk, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = silu(short_convolution(h @ W[p + "q"].T, W[p + "q.conv"])).reshape(T, G, dk)
    k = silu(short_convolution(h @ W[p + "k"].T, W[p + "k.conv"])).reshape(T, G, dk)
    v = silu(short_convolution(h @ W[p + "v"].T, W[p + "v.conv"])).reshape(T, H, dv)
    q = unit(q) * dk ** -0.5
    k = unit(k)
    share = H // G
    q = np.repeat(q, share, axis=1)                 # head a reads group a // share
    k = np.repeat(k, share, axis=1)
    beta = sigmoid(h @ W[p + "b"].T)
    rate = np.exp(W[p + "A_log"])                   # [H]
    if per_channel:
        raw = (h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "dt_bias"]
        decay = np.exp(-rate[None, :, None] * softplus(raw).reshape(T, H, dk))
        gate = sigmoid((h @ W[p + "g1"].T) @ W[p + "g2"].T)
    else:
        raw = h @ W[p + "a"].T + W[p + "dt_bias"]
        decay = np.exp(-rate[None, :] * softplus(raw))[:, :, None]
        gate = silu(h @ W[p + "g"].T)
    o = delta_rule(q, k, v, beta, decay)
    o = rms_scale(o, eps) * W[p + "norm"]
    return (o.reshape(T, H * dv) * gate) @ W[p + "o"].T


def gated_mlp(h, W, p):
    return (silu(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


# ---------------------------------------------------------------------------
# the model
# ---------------------------------------------------------------------------
def run_order(cfg):
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(i, False) for i in range(a)]
    for t in range(times):
        order += [(i, t > 0 and i == a) for i in range(a, b)]
    return order + [(i, False) for i in range(b, n)]


def layer(X, i, cfg, W):
    L = cfg["layers"][i]
    eps = float(cfg["norm"]["eps"])
    p = "l%d." % i
    h = layer_norm(X, W[p + "norm1"], W[p + "norm1.b"], eps)
    kind = L["type"]
    if kind == "latent_attention":
        X = X + latent_attention(h, L["mixer"], W, p + "mix.", eps)
    elif kind in ("delta", "channel_delta"):
        X = X + delta_mixer(h, L["mixer"], W, p + "mix.", eps, kind == "channel_delta")
    else:
        raise ValueError("mixer type %r" % kind)
    if L.get("mlp"):
        X = X + gated_mlp(layer_norm(X, W[p + "norm2"], W[p + "norm2.b"], eps), W, p + "mlp.")
    return X


def forward(cfg, W, tokens, streams=None):
    """logits [T, vocab] of one sequence; `streams`, if a list, receives X after every layer run."""
    x0 = W["embed"][np.asarray(tokens)] * float(cfg["embedding"]["scale"])
    X = x0.copy()
    for i, add_input in run_order(cfg):
        if add_input:
            X = X + x0
        X = layer(X, i, cfg, W)
        if streams is not None:
            streams.append(X.copy())
    h = layer_norm(X, W["final.norm"], W["final.norm.b"], float(cfg["norm"]["eps"]))
    return h @ W["embed"].T


def greedy(cfg, W, prompt, n_new):
    """The tokens that greedy decoding appends to `prompt` (the first maximum wins)."""
    tokens = list(prompt)
    for _ in range(n_new):
        tokens.append(int(np.argmax(forward(cfg, W, tokens)[-1])))
    return tokens[len(prompt):]
