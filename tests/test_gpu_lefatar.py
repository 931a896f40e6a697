"""The Lefatar decoder in the engine against the plain implementation (tests/plain_lefatar.py): whole prompts,
decoding through cache and state, prompts in portions, unequal batches, slots and pages used again, long
decoding, the first tokens, greedy generation through the package's entry point, and trace replay."""
import functools
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

import lefatar_tiny as lt
import plain_lefatar as plain
from helpers import check_logits

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
DTYPES = ("float32", "bfloat16")
WEIGHTS = {name: lt.make_weights(cfg, seed) for (name, cfg), seed in zip(lt.CONFIGS.items(), (5, 6, 7))}


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    root = tmp_path_factory.mktemp("lefatar")
    return {name: lt.write_model_dir(root / name, cfg, WEIGHTS[name]) for name, cfg in lt.CONFIGS.items()}


@functools.lru_cache(maxsize=None)
def _plain(name, tokens):
    margins = []
    logits = plain.forward(lt.CONFIGS[name], WEIGHTS[name], list(tokens), margins=margins)
    return logits, (np.min(np.stack(margins), axis=0) if margins else np.full(len(tokens), np.inf))


def plain_logits(name, tokens):
    return _plain(name, tuple(int(t) for t in tokens))[0]


CLOSE_CALL = 0.08     # in units of the router's logits


def check(got, name, tokens, dtype, what, rows=None):
    """Holds the engine's logits to the plain ones.  In bfloat16 a router's choice between two experts whose
    logits are closer than the rounding of the activations may fall the other way, which is no fault but changes
    that position and, through the memory and the cached latent, the positions after it: a bfloat16 run is
    compared up to its first such position (configuration "r" has no router and is compared in full).  In
    32-bit every position is compared."""
    want, margin = _plain(name, tuple(int(t) for t in tokens))
    got = np.asarray(got)
    assert got.shape == want.shape and np.isfinite(got).all(), what
    if dtype == "bfloat16":
        close_calls = np.nonzero(margin <= CLOSE_CALL)[0]
        upto = int(close_calls[0]) if len(close_calls) else len(margin)
        if upto:
            check_logits(got[:upto], want[:upto], dtype, what)
        return
    # 32-bit: sums of float32 roundings through gates, denominators and head norms that divide by small numbers
    # in places; logits of order 1
    diff = np.abs(np.asarray(got, np.float64) - want)
    assert diff.max() <= 2e-4 and diff.mean() <= 1e-5, f"{what}: max |diff| {diff.max():.3e}, mean {diff.mean():.3e}"


def some_tokens(name, n, seed):
    return np.random.default_rng(seed).integers(0, lt.CONFIGS[name]["vocab"], n).tolist()


_ENGINES: dict = {}


def engine_of(dirs, name, dtype, max_tokens=2048, max_slots=6):
    from alpacca_b200.engine.engine import Engine
    from alpacca_b200.engine.loading import load_model_dir
    key = (name, dtype, max_tokens, max_slots)
    if key not in _ENGINES:
        model = load_model_dir(dirs[name], dtype, "cuda", max_positions=1024)
        _ENGINES[key] = Engine(model, max_tokens=max_tokens, max_slots=max_slots)
    return _ENGINES[key]


def run(eng, slot, tokens, want=None):
    from alpacca_b200.engine.step import StepEntry
    want = list(range(len(tokens))) if want is None else want
    out = eng.step([StepEntry(slot, tokens, want)]).cpu().numpy()
    eng.wait()
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(lt.CONFIGS))
def test_whole_prompt(dirs, name, dtype):
    eng = engine_of(dirs, name, dtype)
    toks = some_tokens(name, 150, 1)
    s = eng.alloc_slot()
    try:
        check(run(eng, s, toks), name, toks, dtype, f"lefatar {name} whole")
    finally:
        eng.free_slot(s)
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(lt.CONFIGS))
def test_prompt_then_long_decoding(dirs, name, dtype):
    """60 tokens at once, then 90 one by one: the page borders at 64 and 128 are passed while decoding, the
    matrix memory is carried through 90 steps, and from the third step on the steps are graph replays."""
    eng = engine_of(dirs, name, dtype)
    toks = some_tokens(name, 150, 2)
    want = plain_logits(name, toks)
    s = eng.alloc_slot()
    try:
        got = [run(eng, s, toks[:60])]
        for p in range(60, 150):
            got.append(run(eng, s, [toks[p]]))
        check(np.concatenate(got), name, toks, dtype, f"lefatar {name} decode")
    finally:
        eng.free_slot(s)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(lt.CONFIGS))
@pytest.mark.parametrize("cuts", [(2, 3, 59, 1, 64, 2, 19), (63, 2, 63, 22), (1, 1, 2, 126, 20), (65, 85)])
def test_prompt_in_portions(dirs, name, dtype, cuts):
    eng = engine_of(dirs, name, dtype)
    toks = some_tokens(name, sum(cuts), 3)
    want = plain_logits(name, toks)
    s = eng.alloc_slot()
    try:
        got, at = [], 0
        for n in cuts:
            got.append(run(eng, s, toks[at:at + n]))
            at += n
        check(np.concatenate(got), name, toks, dtype, f"lefatar {name} portions")
    finally:
        eng.free_slot(s)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(lt.CONFIGS))
def test_unequal_batch_against_each_alone(dirs, name, dtype):
    """Three prompts of 1, 70 and 33 tokens in one step, then decoded together; the shortest request ends
    first.  Every request's logits are those of the request alone."""
    from alpacca_b200.engine.step import StepEntry
    eng = engine_of(dirs, name, dtype)
    full = [some_tokens(name, n, 10 + i) for i, n in enumerate((4, 78, 39))]
    first = (1, 70, 33)
    slots = [eng.alloc_slot() for _ in full]
    try:
        got = [[] for _ in full]
        out = eng.step([StepEntry(s, t[:n], list(range(n))) for s, t, n in zip(slots, full, first)]).cpu().numpy()
        at = 0
        for i, n in enumerate(first):
            got[i].append(out[at:at + n])
            at += n
        pos = list(first)
        while any(p < len(t) for p, t in zip(pos, full)):
            live = [i for i in range(len(full)) if pos[i] < len(full[i])]
            out = eng.step([StepEntry(slots[i], [full[i][pos[i]]], [0]) for i in live]).cpu().numpy()
            for j, i in enumerate(live):
                got[i].append(out[j:j + 1])
                pos[i] += 1
        eng.wait()
        for i, t in enumerate(full):
            check(np.concatenate(got[i]), name, t, dtype, f"lefatar {name} batch row {i}")
    finally:
        for s in slots:
            eng.free_slot(s)
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_slots_and_pages_used_again(dirs, dtype):
    """A cache of four pages and two slots: every new sequence gets a slot and pages that another one has just
    given back, with its keys still in the pages and its matrix memory still in the state's row."""
    name = "r" if dtype == "bfloat16" else "p"
    eng = engine_of(dirs, name, dtype, max_tokens=256, max_slots=2)
    for k, n in enumerate((130, 100, 3, 128, 65)):
        toks = some_tokens(name, n, 20 + k)
        s = eng.alloc_slot()
        other = eng.alloc_slot() if n <= 100 else None
        try:
            cut = max(1, n - 3)
            got = [run(eng, s, toks[:cut])]
            if other is not None:
                run(eng, other, some_tokens(name, 40, 99))       # a neighbour that writes pages and state too
            for p in range(cut, n):
                got.append(run(eng, s, [toks[p]]))
            check(np.concatenate(got), name, toks, dtype, f"lefatar reuse {k}")
        finally:
            eng.free_slot(s)
            if other is not None:
                eng.free_slot(other)
        eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(lt.CONFIGS))
def test_first_tokens(dirs, name, dtype):
    eng = engine_of(dirs, name, dtype)
    toks = some_tokens(name, 3, 30)
    want = plain_logits(name, toks)
    for cuts in ((3,), (1, 1, 1), (1, 2), (2, 1)):
        s = eng.alloc_slot()
        try:
            got, at = [], 0
            for n in cuts:
                got.append(run(eng, s, toks[at:at + n]))
                at += n
            check(np.concatenate(got), name, toks, dtype, f"lefatar {name} first tokens")
        finally:
            eng.free_slot(s)


def test_wanted_places_only(dirs):
    eng = engine_of(dirs, "q", "float32")
    toks = some_tokens("q", 90, 31)
    want = [0, 17, 63, 64, 89]
    s = eng.alloc_slot()
    try:
        check_logits(run(eng, s, toks, want), plain_logits("q", toks)[want], "float32", "lefatar wanted places")
    finally:
        eng.free_slot(s)


def plain_greedy(name, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(np.argmax(plain_logits(name, toks)[-1])))
    return toks[len(prompt):]


@pytest.mark.parametrize("graphs", [True, False])
def test_greedy_generation_through_the_entry_point(dirs, graphs):
    """`Model.load` + `generate` (the scheduler, the graph decoder with its padded rows, the device sampler)
    give the plain implementation's greedy tokens, for prompts of unequal lengths that end at different steps."""
    from alpacca_b200.api import Model, generate
    from alpacca_b200.sampling import SamplerParams
    name = "p"
    model = Model.load(dirs[name], n_ctx=256, dtype="float32", max_batch=4, progress=False)
    if not graphs:
        model.use_graphs = False
    prompts = [some_tokens(name, n, 40 + i) for i, n in enumerate((5, 70, 1))]
    budgets = 9
    res = generate(model, prompts, SamplerParams.greedy(), n_predict=budgets)
    for p, r in zip(prompts, res):
        assert r.token_ids == plain_greedy(name, p, budgets)
    # a second batch in the same slots
    again = generate(model, prompts[::-1], SamplerParams.greedy(), n_predict=4)
    for p, r in zip(prompts[::-1], again):
        assert r.token_ids == plain_greedy(name, p, 4)


def test_generation_in_bfloat16_runs(dirs):
    from alpacca_b200.api import Model, generate
    from alpacca_b200.sampling import SamplerParams
    model = Model.load(dirs["q"], n_ctx=256, dtype="bfloat16", max_batch=4, progress=False)
    res = generate(model, [some_tokens("q", 30, 50), some_tokens("q", 2, 51)], SamplerParams(temperature=0.8, seed=3),
                   n_predict=20)
    assert all(len(r.token_ids) == 20 and all(0 <= t < lt.CONFIGS["q"]["vocab"] for t in r.token_ids) for r in res)


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_replay(dirs, dtype, tmp_path):
    name = "q"
    a, b = some_tokens(name, 70, 60), some_tokens(name, 9, 61)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:66], "want": [0, 65]},
                                     {"id": "b", "tokens": b[:7], "want": [6]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[66:67], "want": [0]},
                                     {"id": "b", "tokens": b[7:8], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[67:68], "want": [0]},
                                     {"id": "b", "tokens": b[8:9], "want": [0]}], "end": ["b"]},
             {"step": 3, "entries": [{"id": "a", "tokens": a[68:70], "want": [1]}], "end": ["a"]}]
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(dirs[name]), "--dtype", dtype,
                           "--out", str(out), "--max-tokens", "256"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [ln for ln in proc.stdout.splitlines() if ln.startswith("done")] == [f"done {i}" for i in range(4)]
    V = lt.CONFIGS[name]["vocab"]
    pa, pb = plain_logits(name, a), plain_logits(name, b)
    want = {0: np.stack([pa[0], pa[65], pb[6]]), 1: pa[66:67], 2: np.stack([pa[67], pb[8]]), 3: pa[69:70]}
    for i, w in want.items():
        got = np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, V)
        check_logits(got, w, dtype, "lefatar trace replay")


def test_run_command(dirs):
    """`python -m alpacca_b200 run` with a Lefatar folder: two prompts as one batch, greedy, in 32-bit."""
    name = "p"
    prompts = [some_tokens(name, 6, 70), some_tokens(name, 2, 71)]
    text = " / ".join(" ".join(map(str, p)) for p in prompts)
    proc = subprocess.run([sys.executable, "-m", "alpacca_b200", "run", str(dirs[name]), text, "--temp", "0",
                           "--repeat-penalty", "1.0", "--n-predict", "5", "--dtype", "float32", "--ctx", "64"],
                          capture_output=True, text=True, timeout=600, cwd=str(ROOT))
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [ln for ln in proc.stdout.splitlines() if ln.strip()]
    assert [[int(t) for t in ln.split()] for ln in lines] == [plain_greedy(name, p, 5) for p in prompts]


def test_trace_replay_of_many_short_requests(dirs, tmp_path):
    """Thirty requests of three tokens live at once, with --max-tokens exactly what they hold: every request has a
    slot and a page of its own although the tokens alone would fill two pages."""
    name = "q"
    reqs = [some_tokens(name, 3, 200 + i) for i in range(30)]
    steps = [{"step": 0, "entries": [{"id": f"r{i}", "tokens": r[:2], "want": [1]} for i, r in enumerate(reqs)], "end": []},
             {"step": 1, "entries": [{"id": f"r{i}", "tokens": r[2:], "want": [0]} for i, r in enumerate(reqs)],
              "end": [f"r{i}" for i in range(30)]}]
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(dirs[name]), "--dtype", "float32",
                           "--out", str(out), "--max-tokens", "90"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    V = lt.CONFIGS[name]["vocab"]
    for step, pos in ((0, 1), (1, 2)):
        got = np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(-1, V)
        want = np.stack([plain_logits(name, r)[pos] for r in reqs])
        assert np.abs(got - want).max() < 2e-4


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["q", "r"])
def test_prompt_steps_replayed_from_their_graph(dirs, name, dtype):
    """Five prompt steps of one shape (two prompts of 70 and 9 tokens on empty slots): the second is captured, the
    later ones are replays with other tokens, slots and pages, and every one gives the plain logits."""
    from alpacca_b200.engine.step import StepEntry
    eng = engine_of(dirs, name, dtype)
    held = eng.alloc_slot()          # shifts the slots of the later rounds
    for k in range(5):
        a, b = some_tokens(name, 70, 300 + k), some_tokens(name, 9, 320 + k)
        if k == 3:
            eng.free_slot(held)
            held = None
        sa, sb = eng.alloc_slot(), eng.alloc_slot()
        out = eng.step([StepEntry(sa, a, list(range(70))), StepEntry(sb, b, list(range(9)))]).cpu().numpy()
        eng.wait()
        check(out[:70], name, a, dtype, f"lefatar {name} replayed prompt step {k}")
        check(out[70:], name, b, dtype, f"lefatar {name} replayed prompt step {k}, second prompt")
        eng.free_slot(sa)
        eng.free_slot(sb)
    assert len(eng._graphs) >= 1
