"""The configuration of the Buguzen decoder, by its config.json keys.

    {"architecture": "Buguzen", "vocab": V, "width": E, "norm": {"eps": e},
     "layers": [{"type": "lightning" | "attention" | "attention_2", "mixer": {...}, "mlp": {...} | null}, ...],
     "loop": {"start": a, "stop": b, "times": n},          (optional: layers a .. b-1 run n times in a row)
     "token_side": {"dim": d}}                             (optional: a per-layer token input of d columns)

A layer's mixer sizes:
    lightning     heads, dim, vdim, decay (one number per head, in (0, 1])
    attention     heads, kv_heads, dim, vdim, scale, diff, mask: {size}, rot: {base, dims, scaling: {factor}}
    attention_2   heads, kv_heads, dim, scale, mask: {size},
                  rot: {base, dims, scaling: {factor, low, high, original}}
and its feed-forward: {"kind": "dense", "ff": F}.  `rot.scaling` may be left out (no scaling).
Every size and constant is read from here; the configuration sets no limit on positions.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from .base import ModelConfig
from .lefatar import _check_keys, _is_int, _is_num

MIXERS = {
    "lightning": {"heads": int, "dim": int, "vdim": int, "decay": list},
    "attention": {"heads": int, "kv_heads": int, "dim": int, "vdim": int, "scale": float, "diff": float,
                  "mask": dict, "rot": dict},
    "attention_2": {"heads": int, "kv_heads": int, "dim": int, "scale": float, "mask": dict, "rot": dict},
}


def _check_rot(where: str, rot: dict, dim: int, blended: bool, bad: list) -> None:
    if not _check_keys(where, rot, {"base": float}, bad):
        return
    dims = rot.get("dims")
    if not (_is_int(dims) and dims >= 0 and dims % 2 == 0 and dims <= dim):
        bad.append(f"{where}.dims {dims!r} must be even and at most dim {dim} (0: no rotation)")
    if not rot["base"] > 0:
        bad.append(f"{where}.base must be positive")
    sc = rot.get("scaling")
    if sc is None:
        return
    keys = {"factor": float, "low": float, "high": float, "original": float} if blended else {"factor": float}
    if _check_keys(f"{where}.scaling", sc, keys, bad):
        if not sc["factor"] > 0:
            bad.append(f"{where}.scaling.factor must be positive")
        if blended and not (sc["high"] > sc["low"] >= 0 and sc["original"] > 0):
            bad.append(f"{where}.scaling needs 0 <= low < high and a positive original length")


@dataclass(frozen=True)
class BuguzenConfig(ModelConfig):
    vocab: int = None
    width: int = None
    norm: dict = field(default_factory=dict)
    layers: list = field(default_factory=list)
    loop: dict | None = None
    token_side: dict | None = None
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

    def run_order(self) -> list[tuple[int, int | None]]:
        """(layer, pass) in the order in which the layers run; pass None outside the loop."""
        n = len(self.layers)
        if not self.loop:
            return [(i, None) for i in range(n)]
        a, b, times = self.loop["start"], self.loop["stop"], self.loop["times"]
        out = [(i, None) for i in range(a)]
        for t in range(times):
            out += [(i, t) for i in range(a, b)]
        return out + [(i, None) for i in range(b, n)]

    def to_dict(self) -> dict:
        out = super().to_dict()
        out.pop("architectures", None)
        out = {"architecture": self.architecture, **out}
        for key in ("bos_token_id", "eos_token_id", "loop", "token_side"):
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
            if _check_keys(f"{where}.mixer", mx, {k: t for k, t in MIXERS[kind].items() if t is not list}, bad):
                if kind == "lightning":
                    decay = mx.get("decay")
                    if not (isinstance(decay, list) and len(decay) == mx["heads"]
                            and all(_is_num(a) and 0 < a <= 1 for a in decay)):
                        bad.append(f"{where}.mixer.decay must list one number in (0, 1] per head")
                else:
                    if mx["heads"] % mx["kv_heads"]:
                        bad.append(f"{where}.mixer: {mx['heads']} heads cannot share {mx['kv_heads']} key/value heads")
                    _check_keys(f"{where}.mixer.mask", mx["mask"], {"size": int}, bad)
                    _check_rot(f"{where}.mixer.rot", mx["rot"], mx["dim"], kind == "attention_2", bad)
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                bad.append(f"{where}.mlp must be null or an object of kind 'dense'")
                continue
            _check_keys(f"{where}.mlp", mlp, {"ff": int}, bad)
        if self.loop is not None:
            if _check_keys("loop", self.loop, {"stop": int, "times": int}, bad):
                a, b = self.loop.get("start"), self.loop["stop"]
                if not (_is_int(a) and 0 <= a < b <= len(self.layers)):
                    bad.append(f"loop: start {a!r} and stop {b} must satisfy 0 <= start < stop <= {len(self.layers)}")
        if self.token_side is not None:
            _check_keys("token_side", self.token_side, {"dim": int}, bad)
        for t in self.stop_tokens if not bad else ():
            if not 0 <= t < self.vocab:
                bad.append(f"eos_token_id {t} lies outside the vocabulary of {self.vocab}")
        return bad
