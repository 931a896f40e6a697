"""Parts that act on the residual stream itself, between or after the sub-layers.

`PassOffset`   a learned vector per pass of a loop over layers: before pass t the row t of a table
               [passes, width] is added to every token's stream.
`TokenTable`   a second embedding table [vocab, n_layers * dim]; layer i owns the columns [i*dim, (i+1)*dim).
`TokenSide`    a layer's token input from that table, added after its sub-layers:
                   e = table[token][i*dim:(i+1)*dim];  a = gelu_tanh(W_gate x) * e;  y = W_proj a
                   x <- x + y / sqrt(mean(y^2) + eps) * w
               x is the stream as it stands (no norm before W_gate); the norm of y is 32-bit.
`StreamCast`   stands where a part reads the stream itself in the activation dtype.  To the block it is a norm whose
               weight is 1 and whose division nobody owes: in a step of a few rows the product before it adds its
               result to the stream and leaves bf16(stream) behind (the skinny product's residual tail), and the
               kernel that casts the stream is not launched.
"""
from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import ParamSpec
from .base import BuildOptions, Norm, Part
from .linear import Linear


class StreamCast(Norm):
    def __init__(self, opts: BuildOptions, width: int):
        self.opts, self.width = opts, int(width)
        self.ones = torch.ones(self.width, dtype=torch.float32, device=opts.device)

    def deferred(self):
        if self.opts.dtype != torch.bfloat16:
            return None
        return self.ones, self.width, 0.0

    def forward(self, residual, delta, out=None, rows=None, n_rows=None):
        """residual += delta; the stream in the activation dtype."""
        if rows is not None:
            raise ValueError("the cast stream is read in full")
        if out is None:
            out = torch.empty(residual.shape, dtype=self.opts.dtype, device=residual.device)
        return ops.stream_cast(residual, delta, out, n_rows=n_rows)


class PassOffset(Part):
    def __init__(self, opts: BuildOptions, passes: int, width: int, name: str):
        self.opts, self.passes, self.width, self.name = opts, int(passes), int(width), name
        self.rows = None

    def own_param_specs(self):
        return [ParamSpec(self.name, (self.passes, self.width), "vector", "normal")]

    def load_own(self, fetch):
        self.rows = fetch(self.own_param_specs()[0])

    def forward(self, stream, ctx, index: int) -> None:
        if not 0 <= index < self.passes:
            raise ValueError(f"{self.name} has {self.passes} rows, row {index} was asked for")
        if stream.owed is not None:
            raise RuntimeError("rows prepared for a norm cannot take an offset any more")
        ops.add_row(stream.residual, self.rows[index], ctx)


class TokenTable(Part):
    def __init__(self, opts: BuildOptions, vocab: int, columns: int, name: str):
        self.opts, self.vocab, self.columns, self.name = opts, int(vocab), int(columns), name
        self.weight = None

    def own_param_specs(self):
        return [ParamSpec(self.name, (self.vocab, self.columns), "matrix", "normal")]

    def load_own(self, fetch):
        self.weight = fetch(self.own_param_specs()[0])


class TokenSide(Part):
    def __init__(self, opts: BuildOptions, width: int, dim: int, table: TokenTable, offset: int, eps: float,
                 prefix: str, names=("gate", "proj", "norm"), weight_suffix: str = ""):
        self.opts, self.width, self.dim, self.offset, self.eps = opts, int(width), int(dim), int(offset), float(eps)
        if self.offset < 0 or self.offset + self.dim > table.columns:
            raise ValueError(f"{prefix}: columns {self.offset}..{self.offset + self.dim} lie outside the table's "
                             f"{table.columns}")
        self.cast = StreamCast(opts, width)  # what the block may ask the part before this one to prepare
        self._table = {"part": table}       # shared by the layers and loaded once, by the model: not a child
        self.prefix, self.names = prefix, names
        gate, proj, _ = names
        self.gate = Linear(opts, width, [(f"{prefix}.{gate}", dim)], weight_suffix=weight_suffix)
        self.proj = Linear(opts, dim, [(f"{prefix}.{proj}", width)], weight_suffix=weight_suffix,
                           out_dtype=torch.float32)
        self.norm_weight = None

    def own_param_specs(self):
        return [ParamSpec(f"{self.prefix}.{self.names[2]}", (self.width,), "vector", "one_plus_normal")]

    def load_own(self, fetch):
        self.norm_weight = fetch(self.own_param_specs()[0])

    def forward(self, stream, ctx) -> None:
        T = ctx.n_tokens
        if stream.owed is not None:
            if stream.owed.norm is not self.cast:
                raise RuntimeError("rows prepared for a norm cannot be read as the stream")
            x, stream.owed = stream.owed.x, None      # the product before has added its result and left the cast
        else:
            x = self.cast.forward(stream.residual, stream.delta, n_rows=T)
            stream.delta = None
        z = self.gate.forward(x, n_rows=T)
        a = torch.empty_like(z)
        ops.token_gate(z, self._table["part"].weight, self.offset, ctx, a)
        y = self.proj.forward(a, n_rows=T)
        ops.add_unit_norm(stream.residual, y, self.norm_weight, self.eps, ctx)
