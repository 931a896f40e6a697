"""Each mechanism of the Lefatar decoder alone, against its function in tests/plain_lefatar.py: the matrix memory,
attention over a cached latent with a sink, the grouped router, the routed experts, the norm that multiplies by
1 + w and the parallel block.  Sizes differ from test to test; inputs are drawn so that faults show."""
import numpy as np
import pytest
import torch

import plain_lefatar as plain
from helpers import PartHarness, load_part

pytestmark = pytest.mark.gpu

TOL = {"float32": (2e-4, 2e-5), "bfloat16": (0.12, 0.02)}      # (largest, mean) |difference| as shares of the spread


def close(got, want, dtype, what):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert got.shape == want.shape and np.isfinite(got).all(), what
    spread = max(float(want.std()), 1e-30)
    d = np.abs(got - want) / spread
    big, mean = TOL[dtype]
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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,D,V,cap", [(2, 16, 24, 8.0), (1, 24, 40, 30.0), (3, 64, 20, 14.0), (2, 128, 36, 12.0),
                                       (2, 40, 70, 5.0), (1, 32, 33, 20.0), (1, 272, 264, 10.0)])
def test_matrix_memory(dtype, H, D, V, cap):
    """Two sequences side by side, fed in portions of unequal sizes down to one token; the state is carried from
    step to step.  D 16, 32, 64, 128 take the register form of the kernel, 24, 40 and 272 the shared-memory form
    (272 x 64 columns: more shared memory than a kernel gets without asking)."""
    from alpacca_b200.parts import MatrixMemory
    width, eps = 56, 1e-5
    part = MatrixMemory(opts_of(dtype), width, H, D, V, cap, eps, "m")
    w = short(load_part(part, seed=H * 100 + D, dtype=dtype, std=0.25), "m")
    w["f.b"] = w["f.b"] + 2.0           # a memory that lasts
    part.bias_f += 2.0
    mx = {"heads": H, "dim": D, "vdim": V, "gate_cap": cap}
    rng = np.random.default_rng(D)
    lens = (75, 31)
    xs = [hidden(rng, n, width, dtype) for n in lens]
    want = [plain.mlstm(x64, w, mx, eps)[0] for _, x64 in xs]
    hs = PartHarness([part.cache_spec()], dtype, max_slots=3)
    spare = hs.cache.alloc_slot()        # slot 0 stays unused: the sequences live in slots 1 and 2
    slots = [hs.cache.alloc_slot(), hs.cache.alloc_slot()]
    got = [[], []]
    at = [0, 0]
    for portion in ((40, 2), (1, 1), (2, 20), (31, 1), (1, 7)):
        seqs = [(s, n) for s, n, a, L in zip(slots, portion, at, lens) if a + n <= L]
        ctx = hs.step(seqs)
        h = torch.cat([xs[slots.index(s)][0][at[slots.index(s)]:at[slots.index(s)] + n] for s, n in seqs])
        out = part.forward(h.contiguous(), ctx, hs.cache.entry_view(0, ctx.block_tables)).float().cpu().numpy()
        hs.done()
        o = 0
        for s, n in seqs:
            i = slots.index(s)
            got[i].append(out[o:o + n])
            o += n
            at[i] += n
    for i in range(2):
        g = np.concatenate(got[i])
        close(g, want[i][:len(g)], dtype, f"matrix memory, sequence {i}")
    assert at[0] == 75 and float(hs.cache.state_groups[0].state[0, spare].abs().max()) == 0.0


def test_matrix_memory_state_is_zeroed_when_a_slot_is_taken_again():
    from alpacca_b200.parts import MatrixMemory
    part = MatrixMemory(opts_of("float32"), 32, 2, 16, 24, 10.0, 1e-6, "m")
    w = short(load_part(part, seed=3, dtype="float32", std=0.25), "m")
    mx = {"heads": 2, "dim": 16, "vdim": 24, "gate_cap": 10.0}
    rng = np.random.default_rng(0)
    hs = PartHarness([part.cache_spec()], "float32", max_slots=1)
    for n in (20, 9):
        x, x64 = hidden(rng, n, 32, "float32")
        s = hs.cache.alloc_slot()
        ctx = hs.step([(s, n)])
        out = part.forward(x, ctx, hs.cache.entry_view(0, ctx.block_tables)).cpu().numpy()
        hs.done()
        close(out, plain.mlstm(x64, w, mx, 1e-6)[0], "float32", "matrix memory in a slot used again")
        hs.cache.free_slot(s)


LATENT_SIZES = [  # H, D, R, V, Q, C, rotated dims, base, scale
    (3, 24, 12, 20, 40, 36, 8, 10000.0, 0.17),
    (2, 16, 8, 28, 24, 56, 8, 300.0, 0.2),
    (5, 32, 16, 24, 48, 112, 16, 70000.0, 0.12),
    (1, 8, 4, 8, 8, 8, 2, 50.0, 0.3),
    (2, 40, 24, 36, 72, 272, 24, 1000.0, 0.05),
]


def latent_part(dtype, sizes, width):
    from alpacca_b200.parts import LatentAttention, RotaryEncoding
    H, D, R, V, Q, C, dims, base, scale = sizes
    opts = opts_of(dtype)
    rope = RotaryEncoding(opts, R, dims, base, "llama")
    part = LatentAttention(opts, width, H, D, R, V, Q, C, scale, 1e-5, rope, "a")
    mx = {"heads": H, "dim": D, "rot_dim": R, "vdim": V, "q_rank": Q, "kv_rank": C, "scale": scale,
          "rot": {"base": base, "dims": dims}}
    return part, mx


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes", LATENT_SIZES)
def test_latent_attention(dtype, sizes):
    """A sequence of 200 tokens in portions (130, 2, 1, 1, 60, 1, 5) beside a short one: keys far away, at the
    page borders 64, 128 and 192, in prompts and in single-token steps."""
    width = 48
    part, mx = latent_part(dtype, sizes, width)
    w = short(load_part(part, seed=sizes[0] + sizes[5], dtype=dtype, std=0.3), "a")
    w["sink"] = w["sink"] + 1.0
    part.sink += 1.0
    rng = np.random.default_rng(sizes[5])
    lens = (200, 12)
    xs = [hidden(rng, n, width, dtype) for n in lens]
    want = [plain.latent_attention(x64, w, mx, 1e-5) for _, x64 in xs]
    hs = PartHarness([part.cache_spec()], dtype, max_tokens=64 * 6, max_slots=2)
    slots = [hs.cache.alloc_slot(), hs.cache.alloc_slot()]
    got, at = [[], []], [0, 0]
    for portion in ((130, 3), (2, 1), (1, 1), (1, 5), (60, 1), (1, 1), (5, 0)):
        seqs = [(i, n) for i, n in enumerate(portion) if n]
        ctx = hs.step([(slots[i], n) for i, n in seqs])
        h = torch.cat([xs[i][0][at[i]:at[i] + n] for i, n in seqs]).contiguous()
        out = part.forward(h, ctx, hs.cache.entry_view(0, ctx.block_tables)).float().cpu().numpy()
        hs.done()
        o = 0
        for i, n in seqs:
            got[i].append(out[o:o + n])
            o += n
            at[i] += n
    for i in range(2):
        close(np.concatenate(got[i]), want[i], dtype, f"latent attention, sequence {i}")


@pytest.mark.parametrize("where", [0, 1, 63, 64, 127, 128, 300])
@pytest.mark.parametrize("dtype,last", [("float32", 1), ("float32", 3), ("bfloat16", 1), ("bfloat16", 20)])
def test_latent_attention_finds_one_far_key(where, dtype, last):
    """One key among 400 is made to stand out for the last query (its cached row is the query's folded form,
    scaled): the output is that key's row, wherever it lies - the first tokens, a page's last or first row -
    when the query comes alone (a decode step) and when it is the last token of a portion of a prompt; in
    32-bit (the one-warp kernel) and in bfloat16 (the tensor-core kernels)."""
    from alpacca_b200 import ops
    sizes = (2, 16, 8, 12, 24, 40, 8, 10000.0, 0.25)
    part, mx = latent_part(dtype, sizes, 32)
    w = short(load_part(part, seed=9, dtype=dtype, std=0.3), "a")
    rng = np.random.default_rng(where)
    n = 400
    x, x64 = hidden(rng, n, 32, dtype)
    hs = PartHarness([part.cache_spec()], dtype, max_tokens=64 * 8, max_slots=1)
    s = hs.cache.alloc_slot()
    ctx = hs.step([(s, n - last)])
    view = hs.cache.entry_view(0, ctx.block_tables)
    part.forward(x[:n - last].contiguous(), ctx, view)
    hs.done()
    # plant the key: head 0's folded query of the last token, as the plain implementation forms it
    C, R, D = mx["kv_rank"], mx["rot_dim"], mx["dim"]
    cq = plain.norm_plain(x64[n - 1:] @ w["dq"].T, w["dq.norm"], 1e-5)
    q = (cq @ w["uq"].T).reshape(1, mx["heads"], D + R)
    q_lat = q[0, 0, :D] @ w["uk"].reshape(mx["heads"], D, C)[0]
    row = np.concatenate([q_lat, np.zeros(R)])
    row = 40.0 * row / np.linalg.norm(row)
    page = int(ctx.block_tables[0][0, where // 64])
    view.k[page, 0, where % 64] = torch.from_numpy(row).to(view.k.dtype).cuda()
    ctx = hs.step([(s, last)])
    seen = {}
    names = ("latent_attention", "latent_attention_mma")
    real = {k: getattr(ops, k) for k in names}

    def spy(name):
        def call(q_, out, *a, **k):
            r = real[name](q_, out, *a, **k)
            seen["o"] = out.float().clone()
            return r
        return call
    for k in names:
        setattr(ops, k, spy(k))
    try:
        part.forward(x[n - last:].contiguous(), ctx, hs.cache.entry_view(0, ctx.block_tables))
    finally:
        for k in names:
            setattr(ops, k, real[k])
    hs.done()
    head0 = seen["o"][last - 1, :C].cpu().numpy()        # the last token's first head: its weighted sum of c
    tol = 1e-3 if dtype == "float32" else 2e-2
    assert np.abs(head0 - row[:C]).max() < tol * np.abs(row).max(), "the planted key's row is not what head 0 returns"


def test_latent_attention_sink_takes_its_share():
    """With a sink far above every score the output vanishes; with one far below, it is plain softmax attention."""
    sizes = (2, 16, 8, 12, 24, 40, 8, 10000.0, 0.1)
    part, mx = latent_part("float32", sizes, 32)
    w = short(load_part(part, seed=4, dtype="float32", std=0.3), "a")
    x, x64 = hidden(np.random.default_rng(1), 70, 32, "float32")
    for sink in (30.0, -30.0, 0.5):
        part.sink.fill_(sink)
        w["sink"] = np.full(2, sink)
        hs = PartHarness([part.cache_spec()], "float32", max_slots=1)
        s = hs.cache.alloc_slot()
        ctx = hs.step([(s, 70)])
        out = part.forward(x, ctx, hs.cache.entry_view(0, ctx.block_tables)).cpu().numpy()
        hs.done()
        want = plain.latent_attention(x64, w, mx, 1e-5)
        assert np.abs(out - want).max() < 1e-4 * max(np.abs(want).max(), 1e-3) + 1e-7
        if sink == 30.0:
            assert np.abs(out).max() < 1e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E,groups,keep,top,scale", [(9, 3, 1, 3, 2.0), (6, 3, 2, 2, 1.0), (4, 1, 1, 1, 2.5), (40, 5, 3, 7, 1.5),
                                                      (12, 12, 4, 4, 1.0), (1, 1, 1, 1, 3.0), (64, 8, 8, 6, 1.0)])
def test_router(dtype, E, groups, keep, top, scale):
    from alpacca_b200 import ops
    rng = np.random.default_rng(E)
    width = 40
    x, x64 = hidden(rng, 67, width, dtype)
    router = torch.from_numpy(rng.normal(0, 0.6, (E, width)).astype(np.float32)).to(torch.bfloat16).float()
    idx, wts = ops.moe_route(x, router.cuda().contiguous(), 67, groups, keep, top, scale)
    rt = {"experts": E, "top": top, "scale": scale, "groups": {"count": groups, "keep": keep}}
    want_idx, want_w = plain.route(x64, router.double().numpy(), rt)
    assert (idx.cpu().numpy() == want_idx).all()
    assert np.abs(wts.cpu().numpy() - want_w).max() < 2e-5 * scale


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E,groups,keep,top,ff", [(6, 3, 2, 2, 40), (4, 1, 1, 1, 24), (9, 3, 1, 3, 33)])
@pytest.mark.parametrize("T", [5, 50])
def test_routed_experts(dtype, E, groups, keep, top, ff, T):
    """5 tokens: an expert's rows are read once for the pairs that chose it (or, for widths that are no multiple
    of 8 and in 32-bit, once per pair); 50 tokens in bfloat16: all experts in two products."""
    from types import SimpleNamespace
    from alpacca_b200.parts import RoutedExperts
    width = 48
    part = RoutedExperts(opts_of(dtype), width, ff, E, top, groups, keep, 1.7, "f")
    w = short(load_part(part, seed=E, dtype=dtype, std=0.3), "f")
    x, x64 = hidden(np.random.default_rng(ff), T, width, dtype)
    out = part.forward(x, SimpleNamespace(n_tokens=T)).float().cpu().numpy()
    mlp = {"router": {"experts": E, "top": top, "scale": 1.7, "groups": {"count": groups, "keep": keep}}}
    close(out, plain.moe_ff(x64, w, mlp), dtype, "routed experts")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_parallel_block_and_offset_norm(dtype):
    """h = norm(x) with 1 + w; x += mixer(h) + ff(h), the sum kept in 32-bit; a block without a feed-forward."""
    from alpacca_b200.parts import MatrixMemory, ParallelBlock, RMSNorm, SwiGLU
    from alpacca_b200.parts.block import HiddenStream
    width, eps = 40, 1e-5
    opts = opts_of(dtype)
    mx = {"heads": 2, "dim": 16, "vdim": 12, "gate_cap": 9.0}
    for with_ff in (True, False):
        block = ParallelBlock(RMSNorm(opts, width, eps, "n", weight_suffix="", unit_offset=True),
                              MatrixMemory(opts, width, 2, 16, 12, 9.0, eps, "m"),
                              SwiGLU(opts, width, 56, "f", names=("gate", "up", "down"), weight_suffix="") if with_ff else None)
        w = load_part(block, seed=7, dtype=dtype, std=0.2)
        x, x64 = hidden(np.random.default_rng(2), 33, width, dtype)
        hs = PartHarness(block.cache_specs(), dtype, max_slots=1)
        s = hs.cache.alloc_slot()
        ctx = hs.step([(s, 33)])
        stream = HiddenStream(x.float().clone())
        block.forward(stream, ctx, hs.cache.entry_view(0, ctx.block_tables))
        hs.done()
        got = (stream.residual + stream.delta.float()).cpu().numpy()
        h = plain.norm_offset(x64, w["n"], eps)
        want = x64 + plain.mlstm(h, short(w, "m"), mx, eps)[0]
        if with_ff:
            want = want + plain.dense_ff(h, short(w, "f"))
        close(got - x64, want - x64, dtype, "parallel block")
