"""The matrix memory of xLSTM (mLSTM) as a mixer with a state of fixed size per sequence.

Per head, q = W_q h / sqrt(D), k = W_k h (D dims each), v = W_v h (V dims), a log input gate
gi = cap tanh((W_i h + b_i) / cap) and a log forget gate gf = logsigmoid(cap tanh((W_f h + b_f) / cap)).
With a running maximum m (m = 0 before the first token), S = 0 and n = 0:

    m' = max(gf + m, gi);  S' = exp(gf + m - m') S + exp(gi - m') k v^T;  n' likewise with k alone
    o  = S'^T q / (max(|n' . q|, exp(-m')) + 1e-6)

Each head's o is divided by its root mean square, the heads are concatenated, multiplied by a weight
and by sigmoid(W_g h), and projected by W_o.  (Beck et al., "xLSTM: Extended Long Short-Term Memory".)

All six projections are one product with a float32 result; gates, decays, the state and the
normalisation are 32-bit arithmetic in both precisions (csrc/mlstm.cu).  The state (S, n, m) lives in
the cache's state group, one row per (slot, head), and is carried from step to step: a prompt may be
cut anywhere, and a decode step is a step of one token.
"""
from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import ParamSpec
from .base import BuildOptions, Mixer, StateSpec
from .linear import Linear


class MatrixMemory(Mixer):
    def __init__(self, opts: BuildOptions, width: int, n_heads: int, dim: int, vdim: int, gate_cap: float, eps: float,
                 prefix: str, names=("q", "k", "v", "g", "i", "f", "o", "norm"), weight_suffix: str = "",
                 out_dtype=None):
        self.opts = opts
        self.width, self.H, self.D, self.V = int(width), int(n_heads), int(dim), int(vdim)
        self.cap, self.eps, self.prefix = float(gate_cap), float(eps), prefix
        if not self.cap > 0:
            raise ValueError(f"gate cap {gate_cap} must be positive")
        q, k, v, g, i, f, o, norm = names
        H, D, V = self.H, self.D, self.V
        self.names = names
        rows = [(q, H * D), (k, H * D), (v, H * V), (g, H * V), (i, H), (f, H)]
        self.offsets, at = [], 0
        for _, r in rows:
            self.offsets.append(at)
            at += r
        # gates, decays and the recurrence are 32-bit: the projections leave the product in float32
        self.proj = Linear(opts, width, [(f"{prefix}.{n}", r) for n, r in rows], out_dtype=torch.float32,
                           weight_suffix=weight_suffix)
        self.out = Linear(opts, H * V, [(f"{prefix}.{o}", width)], weight_suffix=weight_suffix, out_dtype=out_dtype)
        self.bias_i = self.bias_f = self.norm_weight = None

    def own_param_specs(self):
        _, _, _, _, i, f, _, norm = self.names
        return [ParamSpec(f"{self.prefix}.{i}.b", (self.H,), "vector", "normal"),
                ParamSpec(f"{self.prefix}.{f}.b", (self.H,), "vector", "normal"),
                ParamSpec(f"{self.prefix}.{norm}", (self.H * self.V,), "vector", "one_plus_normal")]

    def load_own(self, fetch):
        self.bias_i, self.bias_f, self.norm_weight = (fetch(s) for s in self.own_param_specs())

    def cache_spec(self):
        return StateSpec((self.H, ops.mlstm_state_row(self.D, self.V)), torch.float32)

    def forward(self, h, ctx, cache, write_cache: bool = True):
        T = ctx.n_tokens
        proj = self.proj.forward(h, n_rows=T)
        mixed = torch.empty((proj.shape[0], self.H * self.V), dtype=self.opts.dtype, device=proj.device)
        ops.mlstm_step(proj, self.offsets, self.bias_i, self.bias_f, cache.state, ctx, self.H, self.D, self.V, self.cap,
                       self.D ** -0.5, self.norm_weight, self.eps, mixed, write_state=write_cache)
        return self.out.forward(mixed, n_rows=T)
