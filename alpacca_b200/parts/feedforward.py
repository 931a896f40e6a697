"""The gated feed-forward: a = silu(h Wg^T) * (h Wu^T); out = a Wd^T
(alpacca/model.py:510-514; SiLU on the gate, g/(1+exp(-g)), alpacca/tensor.py:150-160).

gate and up are held as one matrix, interleaved in groups of 8 rows, so that
one product feeds the activation kernel.  An inner width that is no multiple of
8 is padded with zero rows (and zero columns of the down matrix) when the
weights are loaded: silu(0) * 0 adds nothing.

The activation on the gate is SiLU unless another is named ("relu", "gelu_tanh": act(0) * 0 adds nothing
either); every form of the product applies the one that is named.
"""
from __future__ import annotations

from .. import ops
from .base import BuildOptions, FeedForward
from .linear import Linear


class SwiGLU(FeedForward):
    def __init__(self, opts: BuildOptions, width: int, inner: int, prefix: str, bias: bool = False,
                 names=("gate_proj", "up_proj", "down_proj"), weight_suffix: str = ".weight",
                 out_dtype=None, activation: str = "silu"):
        if activation not in ops.GATE_ACTIVATIONS:
            raise ValueError(f"activation {activation!r} is not one of {tuple(ops.GATE_ACTIVATIONS)}")
        self.opts, self.width, self.inner, self.activation = opts, int(width), int(inner), activation
        g, u, d = names
        self.gate_up = Linear(opts, width, [(f"{prefix}.{g}", inner), (f"{prefix}.{u}", inner)], bias=bias,
                              interleave8=True, weight_suffix=weight_suffix, pad_rows_to=8)
        self.down = Linear(opts, inner, [(f"{prefix}.{d}", width)], bias=bias, weight_suffix=weight_suffix,
                           out_dtype=out_dtype, pad_in_to=8)

    adds_to_residual = True

    def accepts_owed_norm(self, n_rows: int) -> bool:
        return self.gate_up.accepts_owed_norm(n_rows)

    def forward(self, h, ctx, then=None):
        T = ctx.n_tokens
        act = self.gate_up.forward_swiglu(h, n_rows=T, activation=self.activation)
        return self.down.forward(act, n_rows=T, then=then)
