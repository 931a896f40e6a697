"""Small Buguzen configurations and weights for the tests.

The configurations differ from each other in every size and constant, and within one configuration no two
sizes that a layer kind shares with another are equal by accident (key and value sizes, head counts, widths and
feed-forward widths differ; one model has equal key and value sizes and as many key/value heads as heads, which
the others keep apart).  Windows of 9, 33, 64, 70 and 130 tokens: shorter than a page, a page exactly, and across
one and two page borders.  Rotations over part of a vector and over all of it; frequency scalings whose blended
range is hit; decays of exactly 1 and well below; loops at the start, in the middle (one pass only) and none;
with and without the per-layer token input; a feed-forward width that is no multiple of 8; head sizes that
take the tensor-core kernels in bfloat16 (32, 48) and ones that do not (20, 24).

`make_weights` draws values that a bfloat16 holds exactly, so that the plain implementation, the 32-bit
engine and the bfloat16 engine read the same numbers.  Scales are chosen so that faults show: matrices with
scores of order 1 and more (sharp attention), sinks around +1 (a sink that is left out changes every row),
key and query norm weights away from 1, pass offsets and token tables of order 1.
"""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np


def _lightning(heads, dim, vdim, decay):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}


def _diff(heads, kv_heads, dim, vdim, window, scale, diff, base, dims, factor=None):
    rot = {"base": base, "dims": dims}
    if factor is not None:
        rot["scaling"] = {"factor": factor}
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff,
            "mask": {"size": window}, "rot": rot}


def _keyval(heads, kv_heads, dim, window, scale, base, dims, scaling=None):
    rot = {"base": base, "dims": dims}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "scale": scale, "mask": {"size": window}, "rot": rot}


TINY_U = {
    "architecture": "Buguzen", "vocab": 101, "width": 40, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "attention", "mixer": _diff(4, 2, 16, 24, 9, 0.3, 0.25, 10000.0, 8, 2.0), "mlp": {"kind": "dense", "ff": 56}},
        {"type": "lightning", "mixer": _lightning(3, 8, 12, (0.5, 0.9, 1.0)), "mlp": None},
        {"type": "attention_2", "mixer": _keyval(4, 1, 20, 70, 0.25, 5000.0, 12, (4.0, 1.0, 3.0, 48)),
         "mlp": {"kind": "dense", "ff": 28}},
    ],
    "loop": {"start": 0, "stop": 2, "times": 3},
    "token_side": {"dim": 5},
}

TINY_W = {
    "architecture": "Buguzen", "vocab": 67, "width": 64, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "lightning", "mixer": _lightning(1, 40, 36, (0.97,)), "mlp": {"kind": "dense", "ff": 48}},
        {"type": "attention_2", "mixer": _keyval(2, 2, 32, 33, 0.2, 300.0, 32, (6.0, 1.0, 4.0, 64)), "mlp": None},
        {"type": "attention", "mixer": _diff(2, 1, 32, 16, 130, 0.18, 0.4, 50000.0, 32), "mlp": {"kind": "dense", "ff": 80}},
        {"type": "lightning", "mixer": _lightning(2, 16, 72, (0.8, 0.999)), "mlp": None},
    ],
}

TINY_X = {
    "architecture": "Buguzen", "vocab": 131, "width": 48, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "attention_2", "mixer": _keyval(3, 3, 48, 64, 0.15, 20000.0, 16), "mlp": {"kind": "dense", "ff": 64}},
        {"type": "attention", "mixer": _diff(2, 2, 24, 24, 1000, 0.22, 0.1, 1000.0, 24, 1.5), "mlp": None},
        {"type": "lightning", "mixer": _lightning(2, 24, 20, (0.6, 0.95)), "mlp": {"kind": "dense", "ff": 40}},
        {"type": "attention_2", "mixer": _keyval(6, 2, 24, 7, 0.3, 100.0, 8, (2.0, 1.0, 2.0, 16)), "mlp": None},
    ],
    "loop": {"start": 1, "stop": 3, "times": 1},
    "token_side": {"dim": 8},
}

CONFIGS = {"u": TINY_U, "w": TINY_W, "x": TINY_X}


def bf16_exact(x):
    """Rounds float32 values to the nearest bfloat16 (ties to even), returned as float32."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    bits = x.view(np.uint32).astype(np.uint64)
    bits = (bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000
    return bits.astype(np.uint32).view(np.float32).reshape(x.shape)


def tensor_shapes(config) -> dict:
    E, V = config["width"], config["vocab"]
    out = {"embed": (V, E), "head": (V, E), "final.norm": (E,)}
    side = config["token_side"]["dim"] if config.get("token_side") else 0
    if side:
        out["side.embed"] = (V, side * len(config["layers"]))
    if config.get("loop"):
        out["loop.step"] = (config["loop"]["times"], E)
    for i, layer in enumerate(config["layers"]):
        p, mx = f"l{i}", layer["mixer"]
        out[f"{p}.norm1"] = (E,)
        H, D = mx["heads"], mx["dim"]
        if layer["type"] == "lightning":
            Vd = mx["vdim"]
            out.update({f"{p}.mix.q": (H * D, E), f"{p}.mix.k": (H * D, E), f"{p}.mix.v": (H * Vd, E),
                        f"{p}.mix.g": (H * Vd, E), f"{p}.mix.o": (E, H * Vd), f"{p}.mix.norm": (H * Vd,)})
        elif layer["type"] == "attention":
            G, Vd = mx["kv_heads"], mx["vdim"]
            out.update({f"{p}.mix.q": (H * 2 * D, E), f"{p}.mix.q.b": (H * 2 * D,), f"{p}.mix.k": (G * 2 * D, E),
                        f"{p}.mix.k.b": (G * 2 * D,), f"{p}.mix.v": (G * Vd, E), f"{p}.mix.v.b": (G * Vd,),
                        f"{p}.mix.lq1": (D,), f"{p}.mix.lk1": (D,), f"{p}.mix.lq2": (D,), f"{p}.mix.lk2": (D,),
                        f"{p}.mix.o": (E, H * Vd)})
        else:
            G = mx["kv_heads"]
            out.update({f"{p}.mix.q": (H * D, E), f"{p}.mix.q.b": (H * D,), f"{p}.mix.k": (G * D, E),
                        f"{p}.mix.k.b": (G * D,), f"{p}.mix.q.norm": (D,), f"{p}.mix.k.norm": (D,),
                        f"{p}.mix.sink": (H,), f"{p}.mix.o": (E, H * D)})
        if layer["mlp"] is not None:
            F = layer["mlp"]["ff"]
            out.update({f"{p}.norm2": (E,), f"{p}.mlp.gate": (F, E), f"{p}.mlp.up": (F, E), f"{p}.mlp.down": (E, F)})
        if side:
            out.update({f"{p}.side.gate": (side, E), f"{p}.side.proj": (E, side), f"{p}.side.norm": (E,)})
    return out


def make_weights(config, seed: int, std: float = 0.1) -> dict:
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        last = name.rsplit(".", 1)[-1]
        if last in ("norm", "norm1", "norm2"):
            x = 1.0 + rng.normal(0.0, 0.3, shape) if ".side." not in name else rng.normal(0.0, 0.6, shape)
        elif last == "sink":
            x = rng.normal(1.0, 0.7, shape)
        elif last == "b":
            x = rng.normal(0.0, 0.3, shape)
        elif last in ("lq1", "lk1", "lq2", "lk2"):
            x = rng.normal(0.0, 0.25, shape)
        elif name in ("embed", "side.embed", "loop.step"):
            x = rng.normal(0.0, 1.0, shape)
        else:
            x = rng.normal(0.0, std * (48.0 / shape[-1]) ** 0.5 * 1.5, shape)
        out[name] = bf16_exact(x.astype(np.float32))
    return out


def write_model_dir(path, config, weights) -> Path:
    """config.json + model.safetensors (bfloat16), through the package's writer."""
    import torch
    from alpacca_b200.weights import write_safetensors
    path = Path(path)
    path.mkdir(parents=True, exist_ok=True)
    (path / "config.json").write_text(json.dumps(config))
    entries = [(n, "BF16", tuple(w.shape), (lambda w=w: torch.from_numpy(np.array(w)).to(torch.bfloat16)))
               for n, w in weights.items()]
    write_safetensors(path / "model.safetensors", entries)
    return path
