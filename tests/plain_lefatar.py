"""A plain, slow implementation of the Lefatar decoder in NumPy float64: whole sequences, no cache, no
batches, one function per mechanism.  It shares no code with the package; the tests hold the package to it.

A model is (config dict, {tensor name: array}).  Layer i's tensors are `l<i>.norm1`, `l<i>.mix.*`,
`l<i>.mlp.*`; linear weights are [out, in].

    layer:   h = norm1(x);  x <- x + (mixer(h) + ff(h))
    norm1:   x / sqrt(mean(x^2) + eps) * (1 + w)
"""
from __future__ import annotations

import math

import numpy as np


def rms_unit(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def norm_offset(x, w, eps):
    """The layer norm and the final norm multiply by 1 + w."""
    return rms_unit(x, eps) * (1.0 + w)


def norm_plain(x, w, eps):
    return rms_unit(x, eps) * w


def rotate_pairs(x, positions, dims, base):
    """x [T, ..., D]: the first `dims` dimensions, pairs (2i, 2i+1), turned by positions * base^(-2i/dims)."""
    out = np.array(x, dtype=np.float64, copy=True)
    half = dims // 2
    freq = np.array([base ** (-2.0 * i / dims) for i in range(half)])
    ang = np.asarray(positions, dtype=np.float64)[:, None] * freq[None, :]          # [T, half]
    shape = (len(positions),) + (1,) * (x.ndim - 2) + (half,)
    c, s = np.cos(ang).reshape(shape), np.sin(ang).reshape(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def softmax_with_sink(scores, sink):
    """scores [..., n]; the denominator also holds exp(sink), which has no value."""
    m = np.maximum(scores.max(axis=-1, keepdims=True), sink)
    e = np.exp(scores - m)
    return e / (e.sum(axis=-1, keepdims=True) + np.exp(sink - m))


def latent_attention(h, w, mx, eps, positions=None):
    """h [T, E]; `w` maps the mixer's short tensor names ('dq', 'dq.norm', ...) to arrays."""
    T = h.shape[0]
    H, D, R, V, C = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
    pos = np.arange(T) if positions is None else np.asarray(positions)
    cq = norm_plain(h @ w["dq"].T, w["dq.norm"], eps)
    q = (cq @ w["uq"].T).reshape(T, H, D + R)
    dkv = h @ w["dkv"].T
    c = norm_plain(dkv[:, :C], w["dkv.norm"], eps)
    k_rot = rotate_pairs(dkv[:, C:], pos, mx["rot"]["dims"], mx["rot"]["base"])         # [T, R], all heads
    q_rot = rotate_pairs(q[:, :, D:], pos, mx["rot"]["dims"], mx["rot"]["base"])        # [T, H, R]
    k_un = (c @ w["uk"].T).reshape(T, H, D)
    v = (c @ w["uv"].T).reshape(T, H, V)
    out = np.zeros((T, H, V))
    causal = np.tril(np.ones((T, T), dtype=bool))
    for a in range(H):
        s = (q[:, a, :D] @ k_un[:, a].T + q_rot[:, a] @ k_rot.T) * mx["scale"]
        s = np.where(causal, s, -np.inf)
        out[:, a] = softmax_with_sink(s, float(w["sink"][a])) @ v[:, a]
    return out.reshape(T, H * V) @ w["o"].T


def mlstm(h, w, mx, eps, state=None):
    """Matrix-memory recurrence, token by token.  Returns (output [T, E], state) where state is
    (S [H, dim, vdim], n [H, dim], m [H]); a sequence starts with zeros, m included."""
    T = h.shape[0]
    H, D, V, cap = mx["heads"], mx["dim"], mx["vdim"], mx["gate_cap"]
    q = (h @ w["q"].T).reshape(T, H, D) * D ** -0.5
    k = (h @ w["k"].T).reshape(T, H, D)
    v = (h @ w["v"].T).reshape(T, H, V)
    gi = cap * np.tanh((h @ w["i"].T + w["i.b"]) / cap)                                 # log input gate
    zf = cap * np.tanh((h @ w["f"].T + w["f.b"]) / cap)
    gf = -np.logaddexp(0.0, -zf)                                                        # logsigmoid
    if state is None:
        S, n, m = np.zeros((H, D, V)), np.zeros((H, D)), np.zeros(H)
    else:
        S, n, m = (np.array(a, dtype=np.float64) for a in state)
    o = np.zeros((T, H, V))
    for t in range(T):
        for a in range(H):
            m_new = max(gf[t, a] + m[a], gi[t, a])
            keep, add = math.exp(gf[t, a] + m[a] - m_new), math.exp(gi[t, a] - m_new)
            S[a] = keep * S[a] + add * np.outer(k[t, a], v[t, a])
            n[a] = keep * n[a] + add * k[t, a]
            m[a] = m_new
            o[t, a] = S[a].T @ q[t, a] / (max(abs(n[a] @ q[t, a]), math.exp(-m_new)) + 1e-6)
    o = rms_unit(o, eps).reshape(T, H * V) * w["norm"]
    gate = 1.0 / (1.0 + np.exp(-(h @ w["g"].T)))
    return (o * gate) @ w["o"].T, (S, n, m)


def dense_ff(h, w):
    g = h @ w["gate"].T
    return ((g / (1.0 + np.exp(-g))) * (h @ w["up"].T)) @ w["down"].T


def route(h, router_w, rt, with_margin=False):
    """(chosen experts [T, top], their weights [T, top]); with_margin: also, per token, how far the choice is
    from another one, in units of the router's logits: the smaller of (last chosen - best not chosen among
    the allowed experts) and (last kept group - best dropped group)."""
    z = h @ router_w.T
    z = z - z.max(axis=-1, keepdims=True)
    s = np.exp(z)
    s = s / s.sum(axis=-1, keepdims=True)
    T, E = s.shape
    G, keep, top = rt["groups"]["count"], rt["groups"]["keep"], rt["top"]
    per = E // G
    best = np.argsort(-s.reshape(T, G, per).max(axis=-1), axis=-1, kind="stable")[:, :keep]
    allowed = np.zeros((T, G), dtype=bool)
    np.put_along_axis(allowed, best, True, axis=-1)
    masked = np.where(np.repeat(allowed, per, axis=-1), s, -1.0)
    idx = np.argsort(-masked, axis=-1, kind="stable")[:, :top]
    wts = np.take_along_axis(s, idx, axis=-1)
    wts_out = wts / (wts.sum(axis=-1, keepdims=True) + 1e-20) * rt["scale"]
    if not with_margin:
        return idx, wts_out
    margin = np.full(T, np.inf)
    ranked = -np.sort(-masked, axis=-1)
    if top < E and keep * per > top:
        margin = np.log(ranked[:, top - 1]) - np.log(np.maximum(ranked[:, top], 1e-300))
    if keep < G:
        gs = -np.sort(-s.reshape(T, G, per).max(axis=-1), axis=-1)
        margin = np.minimum(margin, np.log(gs[:, keep - 1]) - np.log(gs[:, keep]))
    return idx, wts_out, margin


def gelu_erf(z):
    return 0.5 * z * (1.0 + np.vectorize(math.erf)(z / math.sqrt(2.0)))


def moe_ff(h, w, mlp, margins=None):
    idx, wts, margin = route(h, w["router"], mlp["router"], with_margin=True)
    if margins is not None:
        margins.append(margin)
    out = np.zeros((h.shape[0], w["e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for e, g in zip(idx[t], wts[t]):
            out[t] += g * (w[f"e{e}.down"] @ gelu_erf(w[f"e{e}.up"] @ h[t]))
    return out


def sub(weights, prefix):
    return {k[len(prefix):]: np.asarray(v, dtype=np.float64) for k, v in weights.items() if k.startswith(prefix)}


def forward(config, weights, tokens, return_layers=False, margins=None):
    """Logits [T, vocab] of one whole sequence (and the residual stream after every layer).  `margins`: a list
    that gets, for every layer with routed experts, each token's distance from another choice (see `route`)."""
    eps = config["norm"]["eps"]
    x = np.asarray(weights["embed"], dtype=np.float64)[np.asarray(tokens)]
    after = []
    for i, layer in enumerate(config["layers"]):
        h = norm_offset(x, np.asarray(weights[f"l{i}.norm1"], dtype=np.float64), eps)
        mw = sub(weights, f"l{i}.mix.")
        if layer["type"] == "latent_attention":
            y = latent_attention(h, mw, layer["mixer"], eps)
        elif layer["type"] == "mlstm":
            y, _ = mlstm(h, mw, layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        mlp = layer.get("mlp")
        if mlp is not None:
            fw = sub(weights, f"l{i}.mlp.")
            y = y + (dense_ff(h, fw) if mlp["kind"] == "dense" else moe_ff(h, fw, mlp, margins))
        x = x + y
        after.append(x.copy())
    logits = norm_offset(x, np.asarray(weights["final.norm"], dtype=np.float64), eps) @ \
        np.asarray(weights["head"], dtype=np.float64).T
    return (logits, np.stack(after)) if return_layers else logits
