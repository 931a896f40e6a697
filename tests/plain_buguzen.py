"""A plain, slow implementation of the Buguzen decoder in NumPy float64: whole sequences, no cache, no
batches, one function per mechanism.  It shares no code with the package; the tests hold the package to it.

A model is (config dict, {tensor name: array}).  Layer i's tensors are `l<i>.norm1`, `l<i>.norm2`,
`l<i>.mix.*`, `l<i>.mlp.*`, `l<i>.side.*`; linear weights are [out, in].

    layer:   x <- x + mixer(norm1(x));  x <- x + ff(norm2(x)) if it has one;  x <- x + side(x, token)
    norm:    x / sqrt(mean(x^2) + eps) * w
    loop:    layers start .. stop-1 are run `times` times; before pass t, x <- x + loop.step[t]
"""
from __future__ import annotations

import math

import numpy as np


def rms_unit(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def norm(x, w, eps):
    return rms_unit(x, eps) * w


def silu(z):
    return z / (1.0 + np.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


# -- positions ---------------------------------------------------------------------------------------------

def frequencies(rot):
    """The rotation's angular frequencies, one per pair, after the scaling that `rot` names: a `scaling`
    with `factor` alone divides all of them; one with low/high/original leaves short wavelengths, divides
    long ones and blends in between."""
    dims, base = rot["dims"], rot["base"]
    f = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)])
    sc = rot.get("scaling")
    if not sc:
        return f
    if "original" not in sc:
        return f / sc["factor"]
    out = np.empty_like(f)
    for i, fi in enumerate(f):
        wavelength = 2.0 * math.pi / fi
        if wavelength < sc["original"] / sc["high"]:
            out[i] = fi
        elif wavelength > sc["original"] / sc["low"]:
            out[i] = fi / sc["factor"]
        else:
            s = (sc["original"] / wavelength - sc["low"]) / (sc["high"] - sc["low"])
            out[i] = (1.0 - s) * fi / sc["factor"] + s * fi
    return out


def rotate(x, positions, rot, layout):
    """x [T, ..., D]: the first rot.dims dimensions are turned pair by pair.  layout "neighbours" pairs
    (2i, 2i+1), "halves" pairs (i, i + dims/2)."""
    dims = rot["dims"]
    half = dims // 2
    out = np.array(x, dtype=np.float64, copy=True)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * frequencies(rot)[None, :]
    shape = (len(positions),) + (1,) * (x.ndim - 2) + (half,)
    c, s = np.cos(ang).reshape(shape), np.sin(ang).reshape(shape)
    if layout == "neighbours":
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * c - v * s
        out[..., 1:dims:2] = v * c + u * s
    else:
        u, v = x[..., :half], x[..., half:dims]
        out[..., :half] = u * c - v * s
        out[..., half:dims] = v * c + u * s
    return out


def visible(T, window, positions=None):
    """mask[i, j]: token i sees token j (0 <= i - j < window)."""
    p = np.arange(T) if positions is None else np.asarray(positions)
    d = p[:, None] - p[None, :]
    return (d >= 0) & (d < window)


def softmax(scores, sink=None):
    """Over the last axis; entries of -inf count nothing.  `sink`: one more term exp(sink) in the denominator."""
    m = scores.max(axis=-1, keepdims=True)
    if sink is not None:
        m = np.maximum(m, sink)
    e = np.exp(scores - m)
    den = e.sum(axis=-1, keepdims=True)
    if sink is not None:
        den = den + np.exp(sink - m)
    return e / den


# -- mixers ------------------------------------------------------------------------------------------------

def lightning(h, w, mx, eps, state=None):
    """Linear attention with a fixed decay per head.  Returns (output [T, E], state [H, dim, vdim])."""
    T = h.shape[0]
    H, D, V = mx["heads"], mx["dim"], mx["vdim"]
    q = silu(h @ w["q"].T).reshape(T, H, D)
    k = silu(h @ w["k"].T).reshape(T, H, D)
    v = silu(h @ w["v"].T).reshape(T, H, V)
    S = np.zeros((H, D, V)) if state is None else np.array(state, dtype=np.float64)
    o = np.zeros((T, H, V))
    for t in range(T):
        for a in range(H):
            S[a] = mx["decay"][a] * S[a] + np.outer(k[t, a], v[t, a])
            o[t, a] = S[a].T @ q[t, a]
    y = norm(o.reshape(T, H * V), w["norm"], eps) * sigmoid(h @ w["g"].T)
    return y @ w["o"].T, S


def diff_attention(h, w, mx, eps, positions=None):
    """Two softmax maps per head over the same values, subtracted."""
    T = h.shape[0]
    H, G, D, V = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    pos = np.arange(T) if positions is None else np.asarray(positions)
    q = (h @ w["q"].T + w["q.b"]).reshape(T, H, 2, D)
    k = (h @ w["k"].T + w["k.b"]).reshape(T, G, 2, D)
    v = (h @ w["v"].T + w["v.b"]).reshape(T, G, V)
    q = rotate(q, pos, mx["rot"], "neighbours")
    k = rotate(k, pos, mx["rot"], "neighbours")
    lam = math.exp(float(np.sum(w["lq1"] * w["lk1"]))) - math.exp(float(np.sum(w["lq2"] * w["lk2"]))) + mx["diff"]
    mask = visible(T, mx["mask"]["size"], pos)
    out = np.zeros((T, H, V))
    for a in range(H):
        g = a // (H // G)
        maps = []
        for m in range(2):
            s = (q[:, a, m] @ k[:, g, m].T) * mx["scale"]
            maps.append(softmax(np.where(mask, s, -np.inf)) @ v[:, g])
        o = maps[0] - lam * maps[1]
        out[:, a] = rms_unit(o, eps) * (1.0 - mx["diff"])
    return out.reshape(T, H * V) @ w["o"].T


def keyvalue_attention(h, w, mx, eps, positions=None):
    """Attention whose values are its keys as projected; query and key norm; a sink in the softmax."""
    T = h.shape[0]
    H, G, D = mx["heads"], mx["kv_heads"], mx["dim"]
    pos = np.arange(T) if positions is None else np.asarray(positions)
    q = (h @ w["q"].T + w["q.b"]).reshape(T, H, D)
    k = (h @ w["k"].T + w["k.b"]).reshape(T, G, D)
    v = k.copy()
    q = rotate(norm(q, w["q.norm"], eps), pos, mx["rot"], "halves")
    k = rotate(norm(k, w["k.norm"], eps), pos, mx["rot"], "halves")
    mask = visible(T, mx["mask"]["size"], pos)
    out = np.zeros((T, H, D))
    for a in range(H):
        g = a // (H // G)
        s = (q[:, a] @ k[:, g].T) * mx["scale"]
        out[:, a] = softmax(np.where(mask, s, -np.inf), float(w["sink"][a])) @ v[:, g]
    return out.reshape(T, H * D) @ w["o"].T


# -- the rest of a layer -------------------------------------------------------------------------------------

def dense_relu(h, w):
    return (np.maximum(h @ w["gate"].T, 0.0) * (h @ w["up"].T)) @ w["down"].T


def token_side(x, e, w, eps):
    """x [T, E], e [T, dim]: the layer's part of the side table's rows of the tokens."""
    y = (gelu_tanh(x @ w["gate"].T) * e) @ w["proj"].T
    return rms_unit(y, eps) * w["norm"]


def _sub(weights, prefix):
    n = len(prefix) + 1
    return {k[n:]: np.asarray(v, dtype=np.float64) for k, v in weights.items() if k.startswith(prefix + ".")}


def run_order(config):
    """[(layer, pass or None)]: the order in which the layers run."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    out = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        out += [(i, t) for i in range(loop["start"], loop["stop"])]
    return out + [(i, None) for i in range(loop["stop"], n)]


def forward(config, weights, tokens, trace=None):
    """Logits [T, vocab] of one whole sequence.  `trace`: a list that gets the stream after every layer run."""
    W = {k: np.asarray(v, dtype=np.float64) for k, v in weights.items()}
    eps = config["norm"]["eps"]
    tokens = np.asarray(tokens)
    x = W["embed"][tokens]
    side_dim = config["token_side"]["dim"] if config.get("token_side") else 0
    loop = config.get("loop")
    for i, t in run_order(config):
        layer, p = config["layers"][i], f"l{i}"
        if t is not None and i == loop["start"]:
            x = x + W["loop.step"][t]
        h = norm(x, W[f"{p}.norm1"], eps)
        mw = _sub(W, f"{p}.mix")
        if layer["type"] == "lightning":
            y, _ = lightning(h, mw, layer["mixer"], eps)
        elif layer["type"] == "attention":
            y = diff_attention(h, mw, layer["mixer"], eps)
        elif layer["type"] == "attention_2":
            y = keyvalue_attention(h, mw, layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + y
        if layer.get("mlp") is not None:
            x = x + dense_relu(norm(x, W[f"{p}.norm2"], eps), _sub(W, f"{p}.mlp"))
        if side_dim:
            e = W["side.embed"][tokens][:, i * side_dim:(i + 1) * side_dim]
            x = x + token_side(x, e, _sub(W, f"{p}.side"), eps)
        if trace is not None:
            trace.append(x.copy())
    return norm(x, W["final.norm"], eps) @ W["head"].T
