"""Each mechanism of the Buguzen decoder alone, against its function in tests/plain_buguzen.py: linear attention
with a fixed decay, attention with two score maps whose difference is taken, attention whose values are its keys
with query and key norm and a sink, the gated feed-forward with ReLU, the per-layer token input, the pass offset.
Sizes differ from test to test; inputs are made so that faults show."""
import numpy as np
import pytest
import torch

import plain_buguzen as plain
from helpers import PartHarness, load_part

pytestmark = pytest.mark.gpu

TOL = {"float32": (2e-4, 2e-5), "bfloat16": (0.12, 0.02)}      # (largest, mean) |difference| as shares of the spread
# the difference of two maps, divided by its own root mean square, passes the rounding of the maps on at full size
# (largest seen: 0.13 of the spread for one value, 0.009 for the mean, on the tensor-core kernels, whose softmax
# weights are bfloat16 in the product with the values)
TOL_DIFF_BF16 = (0.25, 0.02)


def close(got, want, dtype, what, tol=None):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert got.shape == want.shape and np.isfinite(got).all(), what
    spread = max(float(want.std()), 1e-30)
    d = np.abs(got - want) / spread
    big, mean = tol or TOL[dtype]
    assert d.max() <= big and d.mean() <= mean, f"{what}: max {d.max():.3e} mean {d.mean():.3e} of the spread"


def opts_of(dtype, max_positions=1024):
    from alpacca_b200.parts import BuildOptions
    return BuildOptions(dtype={"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype], device="cuda",
                        max_positions=max_positions)


def hidden(rng, n, width, dtype):
    """Activations [n, width] that both precisions hold exactly."""
    x = torch.from_numpy(rng.normal(0.0, 1.0, (n, width)).astype(np.float32)).to(torch.bfloat16)
    dt = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    return x.to(dt).cuda().contiguous(), x.double().numpy()


def short(weights, prefix):
    return {k[len(prefix) + 1:]: v for k, v in weights.items() if k.startswith(prefix + ".")}


def feed(part, hs, slot, x, cuts):
    """Runs `x` through a mixer in portions; returns the outputs as one array."""
    out, at = [], 0
    for n in cuts:
        ctx = hs.step([(slot, n)])
        view = hs.cache.entry_view(0, ctx.block_tables)
        out.append(part.forward(x[at:at + n].contiguous(), ctx, view).float().cpu().numpy())
        hs.done()
        at += n
    assert at == x.shape[0]
    return np.concatenate(out)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,D,V,decay", [(2, 16, 24, (0.7, 1.0)), (1, 24, 40, (0.99,)), (3, 64, 20, (0.3, 0.9, 0.999)),
                                         (2, 128, 36, (0.95, 0.5)), (1, 40, 70, (0.9,)), (1, 7, 33, (0.8,)),
                                         (1, 200, 130, (0.97,))])
def test_linear_attention(dtype, H, D, V, decay):
    """Two sequences side by side, fed in portions of unequal sizes down to one token; the state is carried from
    step to step.  Head sizes from 7 to 200 take every register form of the kernel; value sizes that are no
    multiple of the 32 columns of a block."""
    from alpacca_b200.parts import DecayLinearAttention
    width, eps = 56, 1e-5
    part = DecayLinearAttention(opts_of(dtype), width, H, D, V, decay, eps, "m")
    w = short(load_part(part, seed=H * 100 + D, dtype=dtype, std=0.25), "m")
    mx = {"heads": H, "dim": D, "vdim": V, "decay": list(decay)}
    rng = np.random.default_rng(D)
    lens = (75, 31)
    xs = [hidden(rng, n, width, dtype) for n in lens]
    want = [plain.lightning(x64, w, mx, eps)[0] for _, x64 in xs]
    hs = PartHarness([part.cache_spec()], dtype, max_slots=3)
    s0, s1 = hs.cache.alloc_slot(), hs.cache.alloc_slot()
    # both in one step, then each alone in portions
    ctx = hs.step([(s0, 20), (s1, 9)])
    view = hs.cache.entry_view(0, ctx.block_tables)
    first = part.forward(torch.cat([xs[0][0][:20], xs[1][0][:9]]).contiguous(), ctx, view).float().cpu().numpy()
    hs.done()
    got0 = np.concatenate([first[:20], feed(part, hs, s0, xs[0][0][20:], (1, 2, 17, 1, 34))])
    got1 = np.concatenate([first[20:], feed(part, hs, s1, xs[1][0][9:], (2, 2, 1, 17))])
    close(got0, want[0], dtype, "linear attention, first sequence")
    close(got1, want[1], dtype, "linear attention, second sequence")
    # the state of a slot that is given back and taken again starts at zero
    hs.cache.free_slot(s0)
    s2 = hs.cache.alloc_slot()
    assert s2 == s0
    close(feed(part, hs, s2, xs[1][0], (31,)), want[1], dtype, "linear attention, a slot used again")
    # a long prompt in one step is cut into pieces that are walked side by side; the state they leave is the one
    # that the next portion starts from
    long_x, long64 = hidden(rng, 330, width, dtype)
    s3 = hs.cache.alloc_slot()
    close(feed(part, hs, s3, long_x, (300, 30)), plain.lightning(long64, w, mx, eps)[0], dtype,
          "linear attention, a long prompt in pieces")
    state = hs.cache.entry_view(0, None).state[s2].double().cpu().numpy()
    close(state, plain.lightning(xs[1][1], w, mx, eps)[1], dtype, "linear attention, the state", tol=(0.05, 0.01) if dtype == "bfloat16" else None)


def attention_part(dtype, kind, width, H, G, D, V, window, rot, scale, eps, diff=0.35):
    from alpacca_b200.parts import MapsAttention, RotaryEncoding
    sc = rot.get("scaling")
    scaling = None
    if sc:
        scaling = ({"rope_type": "linear", "factor": sc["factor"]} if "original" not in sc else
                   {"rope_type": "llama3", "factor": sc["factor"], "low_freq_factor": sc["low"],
                    "high_freq_factor": sc["high"], "original_max_position_embeddings": sc["original"]})
    opts = opts_of(dtype)
    if kind == "diff":
        pos = RotaryEncoding(opts, D, rot["dims"], rot["base"], "llama", scaling)
        part = MapsAttention(opts, width, H, G, D, V, pos, "a", scale, eps, window=window, n_maps=2, bias=True,
                             difference=diff)
        mx = {"heads": H, "kv_heads": G, "dim": D, "vdim": V, "scale": scale, "diff": diff, "mask": {"size": window},
              "rot": rot}
        return part, mx, plain.diff_attention
    pos = RotaryEncoding(opts, D, rot["dims"], rot["base"], "neox", scaling)
    part = MapsAttention(opts, width, H, G, D, None, pos, "a", scale, eps, window=window, bias=True, qk_norm=True,
                         values_are_keys=True, sink=True)
    mx = {"heads": H, "kv_heads": G, "dim": D, "scale": scale, "mask": {"size": window}, "rot": rot}
    return part, mx, plain.keyvalue_attention


SHAPES = [
    ("diff", 4, 2, 16, 24, 9, {"base": 10000.0, "dims": 8, "scaling": {"factor": 2.0}}),
    ("diff", 2, 1, 32, 16, 130, {"base": 500.0, "dims": 32}),
    ("diff", 3, 3, 20, 20, 64, {"base": 100.0, "dims": 10, "scaling": {"factor": 3.0}}),
    ("diff", 1, 1, 72, 136, 65, {"base": 1000.0, "dims": 72}),
    ("keys", 4, 1, 20, None, 70, {"base": 5000.0, "dims": 12, "scaling": {"factor": 4.0, "low": 1.0, "high": 3.0, "original": 48}}),
    ("keys", 2, 2, 32, None, 33, {"base": 300.0, "dims": 32, "scaling": {"factor": 5.0, "low": 1.0, "high": 4.0, "original": 64}}),
    ("keys", 6, 2, 48, None, 64, {"base": 20000.0, "dims": 16}),
    ("keys", 2, 1, 144, None, 63, {"base": 20000.0, "dims": 100}),
    # head sizes 64 and 128: prompts of 128 tokens and more take the tcgen05 kernel in bfloat16
    ("keys", 4, 2, 64, None, 100, {"base": 20000.0, "dims": 32}),
    ("keys", 2, 1, 128, None, 70, {"base": 1000.0, "dims": 64, "scaling": {"factor": 6.0, "low": 1.0, "high": 3.0, "original": 64}}),
    ("diff", 4, 2, 64, 128, 100, {"base": 200000.0, "dims": 32, "scaling": {"factor": 3.0}}),
]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind,H,G,D,V,window,rot", SHAPES)
def test_attention_whole_portions_and_single_tokens(dtype, kind, H, G, D, V, window, rot):
    """A sequence of 150 tokens: whole; in portions down to two tokens; its last 90 tokens one by one (the window
    passes over decoded tokens and page borders); beside another sequence in the same step."""
    width, eps = 40, 1e-5
    part, mx, fn = attention_part(dtype, kind, width, H, G, D, V, window, rot, 0.25, eps)
    w = short(load_part(part, seed=H * 10 + D, dtype=dtype, std=0.3), "a")
    if kind == "keys":
        w["sink"] = w["sink"] + 1.0
        part.sink += 1.0
    rng = np.random.default_rng(D + window)
    x, x64 = hidden(rng, 150, width, dtype)
    y, y64 = hidden(rng, 40, width, dtype)
    want, want_y = fn(x64, w, mx, eps), fn(y64, w, mx, eps)
    tol = TOL_DIFF_BF16 if (kind, dtype) == ("diff", "bfloat16") else None
    hs = PartHarness([part.cache_spec()], dtype, max_slots=4)
    for cuts in ((150,), (2, 3, 59, 1, 64, 2, 19), (20, 130), (60,) + (1,) * 90):
        s = hs.cache.alloc_slot()
        close(feed(part, hs, s, x, cuts), want, dtype, f"attention {kind} in portions {cuts[:4]}", tol=tol)
        hs.cache.free_slot(s)
    s, s2 = hs.cache.alloc_slot(), hs.cache.alloc_slot()
    ctx = hs.step([(s2, 40), (s, 100)])
    view = hs.cache.entry_view(0, ctx.block_tables)
    both = part.forward(torch.cat([y, x[:100]]).contiguous(), ctx, view).float().cpu().numpy()
    hs.done()
    close(both[:40], want_y, dtype, f"attention {kind}, the short sequence of a batch", tol=tol)
    close(both[40:], want[:100], dtype, f"attention {kind}, the long sequence of a batch", tol=tol)
    # both go on by one token each in one step
    ctx = hs.step([(s2, 1), (s, 1)])
    view = hs.cache.entry_view(0, ctx.block_tables)
    y2, y2_64 = hidden(rng, 1, width, dtype)
    nxt = part.forward(torch.cat([y2, x[100:101]]).contiguous(), ctx, view).float().cpu().numpy()
    hs.done()
    close(nxt[1:], want[100:101], dtype, f"attention {kind}, a decode step of two sequences", tol=tol)
    close(nxt[:1], fn(np.concatenate([y64, y2_64]), w, mx, eps)[40:], dtype, f"attention {kind}, the other row", tol=tol)
    hs.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind,window,D,V", [("diff", 33, 16, 24), ("diff", 64, 32, 16), ("diff", 100, 24, 40),
                                             ("keys", 33, 32, None), ("keys", 64, 20, None), ("keys", 129, 48, None),
                                             # a key among six hundred, nine pages back
                                             ("diff", 600, 32, 48), ("keys", 600, 64, None)])
@pytest.mark.parametrize("decode", [False, True])
def test_a_key_just_inside_and_just_outside_the_window(dtype, kind, window, D, V, decode):
    """One early token carries a value that no other has, and queries that look for it.  With scores made so
    that this key outweighs all others by far, the token at distance window - 1 still sees it and the token at
    distance window does not: the outputs at those two places differ by the planted value, in prompts and in
    decoding, for distances at and around a page border."""
    width, eps, H, G = 40, 1e-5, 2, 1
    rot = {"base": 10000.0, "dims": 8}
    part, mx, fn = attention_part(dtype, kind, width, H, G, D, V, window, rot, 1.0, eps, diff=0.2)
    w = short(load_part(part, seed=D, dtype=dtype, std=0.05), "a")
    # input column 0 drives an unrotated dim (the last) of every query vector, column 2 the same dim of every key
    # vector, and, in the attention with values of their own, column 1 one value column per group
    dt = part.qkv.weight.dtype
    W = part.qkv.weight.float()
    n_q, n_k = part.H * part.M * part.Dk, part.G * part.M * part.Dk
    W[:, :3] = 0.0
    for name in ("q", "k", "v"):
        if name in w:
            w[name][:, :3] = 0.0
    for v in range(part.H * part.M):
        W[v * D + D - 1, 0] = 4.0
        w["q"][v * D + D - 1, 0] = 4.0
    for v in range(part.G * part.M):
        W[n_q + v * D + D - 1, 2] = 4.0
        w["k"][v * D + D - 1, 2] = 4.0
    if kind == "diff":
        for g in range(part.G):
            W[n_q + n_k + g * V + 1, 1] = 2.0
            w["v"][g * V + 1, 1] = 2.0
    else:                               # the norm would flatten the planted component: a weight of 1, and a
        part.q_weight.fill_(1.0)        # vector that is little else than that component
        part.k_weight.fill_(1.0)
        w["q.norm"][:] = 1.0
        w["k.norm"][:] = 1.0
    part.qkv.weight = W.to(dt).contiguous()
    rng = np.random.default_rng(window)
    n = window + 70
    planted = 5
    inside, outside = planted + window - 1, planted + window
    x, x64 = hidden(rng, n, width, dtype)
    x[:, :3] = 0.0
    x64[:, :3] = 0.0
    for p, col in ((planted, 2), (planted, 1), (inside, 0), (outside, 0)):
        x[p, col] = 3.0
        x64[p, col] = 3.0
    want = fn(x64, w, mx, eps)
    hs = PartHarness([part.cache_spec()], dtype, max_slots=2)
    s = hs.cache.alloc_slot()
    cuts = (planted + 3,) + (1,) * (n - planted - 3) if decode else (n,)
    got = feed(part, hs, s, x, cuts)
    close(got, want, dtype, f"attention {kind} with a planted key, window {window}",
          tol=(0.2, 0.02) if dtype == "bfloat16" else None)
    # the plain outputs at the two places differ (the planted key matters), and so do the kernel's, alike
    gap = np.abs(want[inside] - want[outside]).max()
    assert gap > 0.05 * np.abs(want).max(), "the planted key does not show in the plain implementation"
    close(got[inside] - got[outside], want[inside] - want[outside], dtype, "the window's edge",
          tol=(0.25, 0.08) if dtype == "bfloat16" else (1e-3, 1e-4))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("level", [-30.0, 0.0, 8.0, 40.0])
def test_sink_far_below_and_far_above_the_scores(dtype, level):
    width, eps, H, G, D = 40, 1e-5, 4, 2, 32
    part, mx, fn = attention_part(dtype, "keys", width, H, G, D, None, 50, {"base": 100.0, "dims": 16}, 0.3, eps)
    w = short(load_part(part, seed=3, dtype=dtype, std=0.3), "a")
    part.sink.fill_(level)
    w["sink"][:] = level
    x, x64 = hidden(np.random.default_rng(4), 70, width, dtype)
    hs = PartHarness([part.cache_spec()], dtype, max_slots=2)
    s = hs.cache.alloc_slot()
    got = feed(part, hs, s, x, (66, 1, 1, 1, 1))
    want = fn(x64, w, mx, eps)
    if level >= 40.0:
        assert np.abs(got).max() <= 1e-6 * max(1.0, np.abs(x64).max()) + np.abs(want).max() * 1.5 + 1e-12
    close(got, want, dtype, f"attention with sinks at {level}", tol=(0.15, 0.03) if dtype == "bfloat16" else None)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width,ff", [(40, 56), (64, 28), (48, 9)])
def test_gated_feed_forward_with_relu(dtype, width, ff):
    from alpacca_b200.parts import SwiGLU
    from alpacca_b200.engine.step import StepContext
    part = SwiGLU(opts_of(dtype), width, ff, "f", names=("gate", "up", "down"), weight_suffix="", activation="relu")
    w = short(load_part(part, seed=ff, dtype=dtype, std=0.3), "f")
    for n in (1, 5, 40):
        x, x64 = hidden(np.random.default_rng(n), n, width, dtype)
        hs = PartHarness([], dtype)
        s = hs.cache.alloc_slot()
        ctx = hs.step([(s, n)])
        got = part.forward(x, ctx).float().cpu().numpy()
        hs.done()
        close(got, plain.dense_relu(x64, w), dtype, f"gated feed-forward with relu, {n} rows")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width,dim,layer,n_layers", [(40, 5, 1, 3), (64, 24, 0, 1), (48, 8, 3, 4)])
def test_token_side_and_pass_offset(dtype, width, dim, layer, n_layers):
    from alpacca_b200.engine.step import StepEntry
    from alpacca_b200.parts import HiddenStream, PassOffset, TokenSide, TokenTable
    opts, eps, vocab = opts_of(dtype), 1e-5, 31
    table = TokenTable(opts, vocab, n_layers * dim, "side.embed")
    tw = load_part(table, seed=1, dtype=dtype, std=1.0)["side.embed"]
    side = TokenSide(opts, width, dim, table, layer * dim, eps, "s")
    w = short(load_part(side, seed=2, dtype=dtype, std=0.3), "s")
    offs = PassOffset(opts, 3, width, "loop.step")
    ow = load_part(offs, seed=3, dtype=dtype, std=1.0)["loop.step"]
    rng = np.random.default_rng(dim)
    n = 23
    tokens = rng.integers(0, vocab, n).tolist()
    x, x64 = hidden(rng, n, width, dtype)
    d, d64 = hidden(rng, n, width, dtype)
    hs = PartHarness([], dtype)
    s = hs.cache.alloc_slot()
    hs.cache.reserve([(s, n)])
    ctx = hs.builder.build([StepEntry(s, tokens, [])], [0], hs.cache)
    stream = HiddenStream(x.float().contiguous(), delta=d)
    side.forward(stream, ctx)
    assert stream.delta is None
    xs = x64 + d64
    want = xs + plain.token_side(xs, tw[np.asarray(tokens)][:, layer * dim:(layer + 1) * dim], w, eps)
    close(stream.residual.cpu().numpy(), want, dtype, "token side", tol=(0.05, 0.01) if dtype == "bfloat16" else None)
    before = stream.residual.double().cpu().numpy()
    offs.forward(stream, ctx, 2)
    close(stream.residual.cpu().numpy(), before + ow[2], "float32", "pass offset")
