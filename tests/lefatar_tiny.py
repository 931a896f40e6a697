"""Small Lefatar configurations and weights for the tests.

The configurations differ from each other in every size and constant; none of the sizes that a layer kind
shares with another is equal by accident (value sizes, rotated and unrotated dims, widths and feed-forward
widths differ), the rotation covers part of the rotated dims in one layer and all of them in another, groups
of experts are 1, 2 and 3 with 1 or 2 kept, 1 to 3 experts chosen, one layer has no feed-forward, and one
dense feed-forward has an inner width that is no multiple of 8.

`make_weights` draws values that a bfloat16 holds exactly, so that the plain implementation, the 32-bit
engine and the bfloat16 engine read the same numbers.  Scales are chosen so that faults show: matrices
N(0, std) with std near 0.1 (scores of order 1 and more: sharp attention), sinks around +1.5 (a sink that is
left out changes every row), forget-gate biases around +3 and input-gate biases around -1 (a long memory).
"""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np


def _latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base, dims):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
            "scale": scale, "rot": {"base": base, "dims": dims}}


def _mlstm(heads, dim, vdim, cap):
    return {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}


def _moe(ff, experts, top, count, keep, scale):
    return {"kind": "moe", "expert": {"ff": ff},
            "router": {"experts": experts, "top": top, "scale": scale, "groups": {"count": count, "keep": keep}}}


TINY_P = {
    "architecture": "Lefatar", "vocab": 97, "width": 48, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "latent_attention", "mixer": _latent(3, 24, 12, 20, 40, 36, 0.17, 10000.0, 8),
         "mlp": {"kind": "dense", "ff": 72}},
        {"type": "mlstm", "mixer": _mlstm(3, 16, 24, 8.0), "mlp": _moe(40, 6, 2, 3, 2, 1.0)},
        {"type": "mlstm", "mixer": _mlstm(1, 24, 40, 30.0), "mlp": None},
        {"type": "latent_attention", "mixer": _latent(2, 16, 8, 28, 24, 56, 0.2, 300.0, 8),
         "mlp": _moe(24, 4, 1, 1, 1, 2.5)},
    ],
}

TINY_Q = {
    "architecture": "Lefatar", "vocab": 211, "width": 64, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "mlstm", "mixer": _mlstm(2, 32, 40, 11.0), "mlp": _moe(32, 8, 2, 4, 2, 1.5)},
        {"type": "latent_attention", "mixer": _latent(4, 32, 16, 24, 48, 64, 0.15, 40000.0, 16),
         "mlp": {"kind": "dense", "ff": 96}},
        {"type": "mlstm", "mixer": _mlstm(4, 64, 20, 12.0), "mlp": {"kind": "dense", "ff": 60}},
    ],
}

# TINY_P's mixers with dense feed-forwards only: no router whose choice rounding could tip, so that bfloat16
# runs are held to the plain implementation at every position
TINY_R = {
    "architecture": "Lefatar", "vocab": 113, "width": 48, "norm": {"eps": 1e-5},
    "layers": [dict(TINY_P["layers"][0]), dict(TINY_P["layers"][1], mlp={"kind": "dense", "ff": 40}),
               dict(TINY_P["layers"][2]), dict(TINY_P["layers"][3], mlp={"kind": "dense", "ff": 52})],
}

CONFIGS = {"p": TINY_P, "q": TINY_Q, "r": TINY_R}


def bf16_exact(x):
    """Rounds float32 values to the nearest bfloat16 (ties to even), returned as float32."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    bits = x.view(np.uint32).astype(np.uint64)
    bits = (bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000
    return bits.astype(np.uint32).view(np.float32).reshape(x.shape)


def tensor_shapes(config) -> dict:
    E, V = config["width"], config["vocab"]
    out = {"embed": (V, E), "head": (V, E), "final.norm": (E,)}
    for i, layer in enumerate(config["layers"]):
        p, mx = f"l{i}", layer["mixer"]
        out[f"{p}.norm1"] = (E,)
        if layer["type"] == "mlstm":
            H, D, Vd = mx["heads"], mx["dim"], mx["vdim"]
            out.update({f"{p}.mix.q": (H * D, E), f"{p}.mix.k": (H * D, E), f"{p}.mix.v": (H * Vd, E),
                        f"{p}.mix.g": (H * Vd, E), f"{p}.mix.o": (E, H * Vd), f"{p}.mix.norm": (H * Vd,),
                        f"{p}.mix.i": (H, E), f"{p}.mix.i.b": (H,), f"{p}.mix.f": (H, E), f"{p}.mix.f.b": (H,)})
        else:
            H, D, R, Vd, Q, C = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["q_rank"], mx["kv_rank"]
            out.update({f"{p}.mix.dq": (Q, E), f"{p}.mix.dq.norm": (Q,), f"{p}.mix.uq": (H * (D + R), Q),
                        f"{p}.mix.dkv": (C + R, E), f"{p}.mix.dkv.norm": (C,), f"{p}.mix.uk": (H * D, C),
                        f"{p}.mix.uv": (H * Vd, C), f"{p}.mix.sink": (H,), f"{p}.mix.o": (E, H * Vd)})
        mlp = layer["mlp"]
        if mlp is None:
            continue
        if mlp["kind"] == "dense":
            out.update({f"{p}.mlp.gate": (mlp["ff"], E), f"{p}.mlp.up": (mlp["ff"], E), f"{p}.mlp.down": (E, mlp["ff"])})
        else:
            F = mlp["expert"]["ff"]
            out[f"{p}.mlp.router"] = (mlp["router"]["experts"], E)
            for e in range(mlp["router"]["experts"]):
                out[f"{p}.mlp.e{e}.up"] = (F, E)
                out[f"{p}.mlp.e{e}.down"] = (E, F)
    return out


def make_weights(config, seed: int, std: float = 0.1) -> dict:
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        last = name.rsplit(".", 1)[-1]
        if name.endswith("norm1") or name == "final.norm":
            x = rng.normal(0.0, 0.2, shape)                      # multiplies as 1 + w
        elif last == "norm":
            x = 1.0 + rng.normal(0.0, 0.2, shape)
        elif last == "sink":
            x = rng.normal(1.5, 0.7, shape)
        elif name.endswith("f.b"):
            x = rng.normal(3.0, 1.0, shape)
        elif name.endswith("i.b"):
            x = rng.normal(-1.0, 0.7, shape)
        elif last == "router":
            x = rng.normal(0.0, 0.5, shape)                      # clear choices
        elif last in ("i", "f"):
            x = rng.normal(0.0, 0.3, shape)
        elif name == "embed":
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
