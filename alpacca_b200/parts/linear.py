"""The matrix product y = x @ W^T (+ b), W stored [out, in] as in the checkpoint.

Several checkpoint matrices that read the same input can be held as one fused
matrix (q|k|v, gate|up).  In the 32-bit path the product is the package's own
FMA kernel; in the bfloat16 path it is the skinny-matrix kernel for the few rows
of a decode step and the library matrix product otherwise (the reference uses
BLAS for every product: alpacca/tensor.py:82-97).
"""
from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import ParamSpec
from .base import BuildOptions, OwedNorm, Part


class Linear(Part):
    def __init__(self, opts: BuildOptions, in_features: int, sources, bias: bool = False,
                 interleave8: bool = False, out_dtype: torch.dtype | None = None, weight_suffix: str = ".weight",
                 pad_rows_to: int = 0, pad_in_to: int = 0, bias_suffix: str = ".bias"):
        """`sources`: list of (checkpoint prefix, rows); tensors `<prefix>.weight`
        [rows, in] (and `<prefix>.bias` [rows]) are stacked in that order
        (`weight_suffix` "" for checkpoints that name a matrix by its prefix alone; `bias_suffix` likewise
        for the biases).
        `interleave8`: two sources of equal size are interleaved in groups of 8
        rows (8 of the first, 8 of the second, ...), the layout `ops.swiglu` reads.
        `out_dtype` float32 gives float32 results from bfloat16 inputs (logits).
        `pad_rows_to` / `pad_in_to`: every source's rows / the inputs are padded with zeros up to a
        multiple of that many when the matrix is loaded (the checkpoint keeps its own shapes):
        `out_features` and `in_features` are then the padded sizes."""
        self.opts = opts
        self.stored_in = int(in_features)
        self.stored_sources = [(p, int(r)) for p, r in sources]
        up = lambda n, m: -(-n // m) * m if m else n        # noqa: E731
        self.in_features = up(self.stored_in, int(pad_in_to))
        self.sources = [(p, up(r, int(pad_rows_to))) for p, r in self.stored_sources]
        self.out_features = sum(r for _, r in self.sources)
        self.has_bias = bool(bias)
        self.interleave8 = bool(interleave8)
        self.out_dtype = out_dtype or opts.dtype
        self.weight_suffix, self.bias_suffix = weight_suffix, bias_suffix
        if interleave8:
            if len(self.sources) != 2 or self.sources[0][1] != self.sources[1][1] or self.sources[0][1] % 8:
                raise ValueError("interleave8 needs two sources of equal size, a multiple of 8 rows "
                                 f"(got {[r for _, r in self.sources]})")
        self.weight = None
        self.bias = None

    def own_param_specs(self):
        specs = [ParamSpec(f"{p}{self.weight_suffix}", (r, self.stored_in), "matrix", "normal")
                 for p, r in self.stored_sources]
        if self.has_bias:
            specs += [ParamSpec(f"{p}{self.bias_suffix}", (r,), "vector", "normal") for p, r in self.stored_sources]
        return specs

    def _padded(self, t, rows):
        """`t` with zero rows up to `rows` and, for a matrix, zero columns up to `in_features`."""
        more_rows = rows - t.shape[0]
        more_cols = self.in_features - t.shape[1] if t.dim() == 2 else 0
        if more_rows == 0 and more_cols == 0:
            return t
        pad = (0, more_cols, 0, more_rows) if t.dim() == 2 else (0, more_rows)
        return torch.nn.functional.pad(t, pad).contiguous()

    def _stack(self, tensors):
        if len(tensors) == 1:
            return tensors[0]
        if self.interleave8:
            a, b = tensors
            tail = a.shape[1:]
            return torch.cat([a.reshape(-1, 8, *tail), b.reshape(-1, 8, *tail)], dim=1).reshape(-1, *tail).contiguous()
        return torch.cat(tensors, dim=0).contiguous()

    def load_own(self, fetch):
        self.weight = self._stack([self._padded(fetch(ParamSpec(f"{p}{self.weight_suffix}", (r, self.stored_in), "matrix")), rp)
                                   for (p, r), (_, rp) in zip(self.stored_sources, self.sources)])
        if self.has_bias:
            self.bias = self._stack([self._padded(fetch(ParamSpec(f"{p}{self.bias_suffix}", (r,), "vector")), rp)
                                     for (p, r), (_, rp) in zip(self.stored_sources, self.sources)])

    def share_weight(self, tensor: torch.Tensor):
        """Uses an existing tensor as the matrix (a tied head)."""
        self.weight = tensor

    def accepts_owed_norm(self, n_rows: int) -> bool:
        """Whether `forward` should be given an `OwedNorm` in a step of `n_rows` rows (it can take one
        whenever the skinny product runs; it pays only for some shapes, see `ops.owed_norm_pays`)."""
        return (self.opts.dtype == torch.bfloat16 and self.weight is not None
                and ops.owed_norm_pays(n_rows, self.out_features, self.in_features, self.weight.device))

    def forward(self, x, n_rows: int | None = None, start_early: bool = True, then=None, with_bias: bool = True):
        """`start_early` off: the product's kernel may not start before the kernel before it has ended
        (see `ops.gemv_bf16`).  `x` may be an `OwedNorm` (the division by the rms is applied to the
        sums).  `then` = (residual, norm): where the step has few enough rows, the result is added to
        the residual here and an `OwedNorm` for `norm` is returned instead of the result.  `with_bias` off: the
        caller adds `self.bias` itself (in a kernel that touches the result anyway)."""
        n = x.shape[0] if n_rows is None else n_rows
        owed = None
        if isinstance(x, OwedNorm):
            owed, x = (x.ss, x.width, x.eps), x.x
        if then is not None and x.dtype == torch.bfloat16 and self.out_dtype == torch.bfloat16:
            residual, norm = then
            d = norm.deferred()
            if (d is not None and d[1] == self.out_features and ops.defers_norm(n, self.out_features)
                    and self.in_features % 8 == 0):
                out = torch.empty((x.shape[0], self.out_features), dtype=torch.bfloat16, device=x.device)
                _, ss = ops.gemv_bf16(x, self.weight, out, bias=self.bias, n_rows=n, start_early=start_early,
                                      owed=owed, residual=residual, norm_weight=d[0])
                return OwedNorm(out, ss, d[1], d[2], norm)
        out = torch.empty((x.shape[0], self.out_features), dtype=self.out_dtype, device=x.device)
        bias = self.bias if with_bias else None
        if x.dtype == torch.float32:
            ops.gemm_f32(x, self.weight, out, bias=bias, n_rows=n)
            return out
        return ops.linear_bf16(x, self.weight, out, n_rows=n, bias=bias, start_early=start_early, owed=owed)

    def forward_swiglu(self, x, n_rows: int | None = None, activation: str = "silu") -> torch.Tensor:
        """act(gate) * up of the interleaved gate|up product, [M, out_features / 2] (`activation`: "silu",
        "relu" or "gelu_tanh" on the gate)."""
        n = x.shape[0] if n_rows is None else n_rows
        if isinstance(x, OwedNorm):
            act = torch.empty((x.shape[0], self.out_features // 2), dtype=x.dtype, device=x.device)
            return ops.gemv_bf16(x.x, self.weight, act, bias=self.bias, n_rows=n, swiglu=True,
                                 owed=(x.ss, x.width, x.eps), activation=activation)
        act = torch.empty((x.shape[0], self.out_features // 2), dtype=x.dtype, device=x.device)
        if x.dtype == torch.bfloat16 and self.in_features % 8 == 0:
            if n <= ops.GEMV_MAX_ROWS:
                return ops.gemv_bf16(x, self.weight, act, bias=self.bias, n_rows=n, swiglu=True, activation=activation)
            if n >= ops.TC_PERSISTENT_MIN_ROWS:
                # long prompts: the persistent tcgen05 product with the activation in its tail
                return ops.gemm_tc(x, self.weight, act, bias=self.bias, n_rows=n, swiglu=True, swap=False,
                                   activation=activation)
        return ops.gated_act(self.forward(x, n_rows=n), act, activation, n_rows=n)
