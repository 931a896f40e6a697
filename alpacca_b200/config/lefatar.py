"""The configuration of the Lefatar decoder, by its config.json keys.

    {"architecture": "Lefatar", "vocab": V, "width": E, "norm": {"eps": e},
     "layers": [{"type": "mlstm" | "latent_attention", "mixer": {...}, "mlp": {...} | null}, ...]}

A layer's mixer sizes:
    mlstm             heads, dim, vdim, gate_cap
    latent_attention  heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, rot: {base, dims}
and its feed-forward: {"kind": "dense", "ff": F} or
    {"kind": "moe", "expert": {"ff": F}, "router": {"experts", "top", "scale", "groups": {"count", "keep"}}}.
Every size and constant is read from here; the configuration sets no limit on positions.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from .base import ModelConfig

MIXERS = {
    "mlstm": {"heads": int, "dim": int, "vdim": int, "gate_cap": float},
    "latent_attention": {"heads": int, "dim": int, "rot_dim": int, "vdim": int, "q_rank": int, "kv_rank": int,
                         "scale": float, "rot": dict},
}


def _is_int(v) -> bool:
    return isinstance(v, int) and not isinstance(v, bool)


def _is_num(v) -> bool:
    return isinstance(v, (int, float)) and not isinstance(v, bool)


def _check_keys(where: str, d, wanted: dict, bad: list) -> bool:
    if not isinstance(d, dict):
        bad.append(f"{where} must be an object")
        return False
    ok = True
    for key, kind in wanted.items():
        v = d.get(key)
        if key not in d:
            bad.append(f"{where}: missing key '{key}'")
            ok = False
        elif kind is int and not (_is_int(v) and v > 0):
            bad.append(f"{where}.{key} must be a positive integer, got {v!r}")
            ok = False
        elif kind is float and not _is_num(v):
            bad.append(f"{where}.{key} must be a number, got {v!r}")
            ok = False
        elif kind is dict and not isinstance(v, dict):
            bad.append(f"{where}.{key} must be an object")
            ok = False
    return ok


@dataclass(frozen=True)
class LefatarConfig(ModelConfig):
    vocab: int = None
    width: int = None
    norm: dict = field(default_factory=dict)
    layers: list = field(default_factory=list)
    bos_token_id: int | None = None
    eos_token_id: int | list | None = None

    @property
    def eps(self) -> float:
        return float(self.norm["eps"])

    @property
    def stop_tokens(self) -> tuple[int, ...]:
        e = self.eos_token_id
        if e is None:
            return ()
        return tuple(e) if isinstance(e, (list, tuple)) else (int(e),)

    @property
    def bos_token(self) -> int | None:
        return self.bos_token_id

    def to_dict(self) -> dict:
        out = super().to_dict()
        out.pop("architectures", None)
        out = {"architecture": self.architecture, **out}
        for key in ("bos_token_id", "eos_token_id"):
            if out.get(key) is None:
                out.pop(key, None)
        return out

    def validate(self) -> list[str]:
        bad: list[str] = []
        for name in ("vocab", "width"):
            v = getattr(self, name)
            if not (_is_int(v) and v > 0):
                bad.append(f"key '{name}' must be a positive integer, got {v!r}")
        if not (isinstance(self.norm, dict) and _is_num(self.norm.get("eps")) and self.norm["eps"] >= 0):
            bad.append("norm.eps must be a number that is not negative")
        if not isinstance(self.layers, list) or not self.layers:
            bad.append("'layers' must be a list with at least one layer")
            return bad
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict):
                bad.append(f"{where} must be an object")
                continue
            kind = layer.get("type")
            if kind not in MIXERS:
                bad.append(f"{where}.type {kind!r} is not supported (supported: {', '.join(sorted(MIXERS))})")
                continue
            mx = layer.get("mixer")
            if _check_keys(f"{where}.mixer", mx, MIXERS[kind], bad):
                if kind == "mlstm" and not mx["gate_cap"] > 0:
                    bad.append(f"{where}.mixer.gate_cap must be positive")
                if kind == "latent_attention":
                    rot = mx["rot"]
                    if _check_keys(f"{where}.mixer.rot", rot, {"base": float, "dims": int}, bad):
                        if rot["dims"] % 2 or rot["dims"] > mx["rot_dim"]:
                            bad.append(f"{where}.mixer.rot.dims {rot['dims']} must be even and at most rot_dim "
                                       f"{mx['rot_dim']}")
                        if not rot["base"] > 0:
                            bad.append(f"{where}.mixer.rot.base must be positive")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
                bad.append(f"{where}.mlp must be null or an object of kind 'dense' or 'moe'")
                continue
            if mlp["kind"] == "dense":
                _check_keys(f"{where}.mlp", mlp, {"ff": int}, bad)
                continue
            ok = _check_keys(f"{where}.mlp", mlp, {"expert": dict, "router": dict}, bad)
            if ok and _check_keys(f"{where}.mlp.expert", mlp["expert"], {"ff": int}, bad) and \
                    _check_keys(f"{where}.mlp.router", mlp["router"],
                                {"experts": int, "top": int, "scale": float, "groups": dict}, bad):
                rt = mlp["router"]
                if _check_keys(f"{where}.mlp.router.groups", rt["groups"], {"count": int, "keep": int}, bad):
                    E, G, keep = rt["experts"], rt["groups"]["count"], rt["groups"]["keep"]
                    if E % G:
                        bad.append(f"{where}.mlp.router: {E} experts do not form {G} equal groups")
                    elif keep > G or rt["top"] > keep * (E // G):
                        bad.append(f"{where}.mlp.router: {rt['top']} experts cannot be chosen from {keep} of {G} "
                                   f"groups of {E // G}")
        for t in self.stop_tokens if not bad else ():
            if not 0 <= t < self.vocab:
                bad.append(f"eos_token_id {t} lies outside the vocabulary of {self.vocab}")
        return bad
