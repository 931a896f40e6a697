"""Buguzen configurations drawn at random from fixed seeds: 2 to 5 layers in any order, 1 to 6 heads in groups of 1 to
3, key and value sizes from 8 to 80 of which some are multiples of 16 (the tensor-core kernels in bfloat16) and some
are not (the last six seeds: widths that are no multiples of 8 or 4 or 2, odd head sizes, head sizes 64 and 128,
rotations over no dims at all),
sizes that happen to be equal or 1 (one head, one key/value head, a window of 1, a loop of one pass, a
rotation over the whole vector), windows shorter and longer than the prompts and at page borders, loops anywhere,
with and without token inputs.  Each whole, in portions, and with its last tokens one by one, in both precisions."""
import functools

import numpy as np
import pytest

import buguzen_tiny as bt
import plain_buguzen as plain

pytestmark = pytest.mark.gpu

SEEDS = list(range(16))


def draw_config(seed: int) -> dict:
    rng = np.random.default_rng(1000 + seed)
    pick = lambda xs: xs[int(rng.integers(len(xs)))]        # noqa: E731
    n_layers = int(rng.integers(2, 6))
    layers = []
    for _ in range(n_layers):
        kind = pick(["lightning", "attention", "attention_2"])
        mlp = pick([None, {"kind": "dense", "ff": pick([9, 24, 40, 64])}])
        if kind == "lightning":
            heads = pick([1, 2, 3])
            mixer = {"heads": heads, "dim": pick([8, 12, 16, 36, 64] if seed < 10 else [5, 30, 128]),
                     "vdim": pick([8, 20, 33, 64]),
                     "decay": [float(pick([0.3, 0.8, 0.95, 0.999, 1.0])) for _ in range(heads)]}
        else:
            group = pick([1, 2, 3])
            kv = pick([1, 2])
            dim = pick([8, 16, 24, 32, 48, 80] if seed < 10 else [10, 25, 18, 64, 128])
            even = dim - dim % 2
            dims = pick([d for d in ((2, 4, 8, 16, even) if seed < 14 else (0, 0, 6, even)) if d <= dim])
            rot = {"base": float(pick([100.0, 10000.0, 1e6])), "dims": dims}
            mixer = {"heads": kv * group, "kv_heads": kv, "dim": dim, "scale": float(pick([0.1, 0.2, dim ** -0.5])),
                     "mask": {"size": pick([1, 5, 63, 64, 65, 100, 4096])}, "rot": rot}
            if kind == "attention":
                mixer.update(vdim=pick([8, 16, 2 * dim, 40]), diff=float(pick([0.1, 0.3, 0.6])))
                if rng.random() < 0.6:
                    rot["scaling"] = {"factor": float(pick([1.0, 2.0, 8.0]))}
            elif rng.random() < 0.7:
                rot["scaling"] = {"factor": float(pick([2.0, 8.0])), "low": 1.0, "high": float(pick([2.0, 4.0])),
                                  "original": pick([16, 64, 256])}
        layers.append({"type": kind, "mixer": mixer, "mlp": mlp})
    cfg = {"architecture": "Buguzen", "vocab": pick([37, 97, 260]),
           "width": pick([24, 40, 64, 72] if seed < 10 else [36, 50, 27]),
           "norm": {"eps": float(pick([1e-5, 1e-6]))}, "layers": layers}
    if rng.random() < 0.7:
        a = int(rng.integers(0, n_layers))
        b = int(rng.integers(a + 1, n_layers + 1))
        cfg["loop"] = {"start": a, "stop": b, "times": pick([1, 2, 3])}
    if rng.random() < 0.7:
        cfg["token_side"] = {"dim": pick([1, 6, 16])}
    return cfg


@functools.lru_cache(maxsize=None)
def model_of(seed, dtype):
    """A token input of ONE column is kept for the 32-bit runs only: its output y = W_proj a is a fixed direction
    times a number, so y / rms(y) is that direction times the number's SIGN, and where the number is within
    rounding of zero a bfloat16 run may get the other sign (no fault, and not small)."""
    cfg = draw_config(seed)
    if dtype == "bfloat16" and cfg.get("token_side", {}).get("dim") == 1:
        cfg["token_side"] = {"dim": 6}
    return cfg, bt.make_weights(cfg, 500 + seed)


@pytest.fixture(scope="module")
def root(tmp_path_factory):
    return tmp_path_factory.mktemp("buguzen_random")


def check(got, want, dtype, what, one_column=False):
    """`one_column`: the model has a token input of one column, whose output is a fixed direction times
    g / sqrt(g^2 c + eps) for a number g: where g is near sqrt(eps) the float32 rounding of g is passed on
    enlarged, so single logits get more room there (the mean does not)."""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert got.shape == want.shape and np.isfinite(got).all(), what
    d = np.abs(got - want)
    if dtype == "float32":
        most = 1e-3 if one_column else 3e-4
        assert d.max() <= most and d.mean() <= 2e-5, f"{what}: max |diff| {d.max():.3e}, mean {d.mean():.3e}"
        return
    spread = max(float(want.std()), 1e-30)
    assert d.max() <= 0.6 * spread and d.mean() <= 0.03 * spread, \
        f"{what}: max |diff| {d.max() / spread:.3f}, mean {d.mean() / spread:.4f} of the spread"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", SEEDS)
def test_random_configuration(root, seed, dtype):
    from alpacca_b200.engine.engine import Engine
    from alpacca_b200.engine.loading import load_model_dir
    from alpacca_b200.engine.step import StepEntry
    cfg, weights = model_of(seed, dtype)
    folder = bt.write_model_dir(root / f"m{seed}_{dtype}", cfg, weights)
    eng = Engine(load_model_dir(folder, dtype, "cuda", max_positions=512), max_tokens=1024, max_slots=3)
    rng = np.random.default_rng(seed)
    toks = rng.integers(0, cfg["vocab"], 140 if seed < 10 else 200).tolist()
    other = rng.integers(0, cfg["vocab"], 30).tolist()
    want, want_other = plain.forward(cfg, weights, toks), plain.forward(cfg, weights, other)

    def run(entries):
        out = eng.step([StepEntry(s, t, list(range(len(t)))) for s, t in entries]).cpu().numpy()
        eng.wait()
        return out
    a, b = eng.alloc_slot(), eng.alloc_slot()
    both = run([(b, other), (a, toks)])                                      # whole, beside another request
    one = (cfg.get("token_side") or {}).get("dim") == 1
    check(both[30:], want, dtype, f"seed {seed} whole", one)
    check(both[:30], want_other, dtype, f"seed {seed} the request beside it", one)
    eng.free_slot(a)
    eng.free_slot(b)
    a = eng.alloc_slot()
    got, at = [], 0
    for n in ((2, 61, 1, 2, 40) if seed < 10 else (30, 136)) + (1,) * 34:    # portions, then token by token
        got.append(run([(a, toks[at:at + n])]))
        at += n
    check(np.concatenate(got), want, dtype, f"seed {seed} in portions and decoded", one)
    eng.free_slot(a)
    eng.cache.check()
