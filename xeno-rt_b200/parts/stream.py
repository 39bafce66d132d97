"""Steps on the residual stream between layers (role ``stream``)."""
from __future__ import annotations

import torch

from ..core import ConfigError, torch_dtype
from ..csrc import ops
from .linear import linear
from .registry import register_part


class MixWithEmbedding:
    """x <- W [x; x0]: the stream and what the embedding gave, side by side, through one matrix.  A model that
    runs a stretch of layers several times begins each pass with it.
    params: ``width``.  weights: ``weight`` [width, 2 * width], the stream's columns first."""

    graph_safe = True

    @classmethod
    def weight_shapes(cls, params):
        return {"weight": ((params["width"], 2 * params["width"]), "matrix")}

    def __init__(self, params, weights, dtype, device):
        self.width = int(params["width"])
        self.weight = weights["weight"]
        self.act_dtype = torch_dtype(dtype)

    def forward(self, x, x0, ctx):
        both = torch.empty((x.shape[0], 2 * self.width), dtype=self.act_dtype, device=x.device)
        ops.concat_cast(both, x, x0)
        return linear(both, self.weight, out_dtype=torch.float32)


class NormedStream:
    """x <- RMSNorm(x) * w in 32-bit: a norm on the residual stream itself (right after the embedding, say).
    params: ``width``, ``eps``.  weights: ``weight`` [width]."""

    graph_safe = True

    @classmethod
    def weight_shapes(cls, params):
        return {"weight": ((params["width"],), "vector")}

    def __init__(self, params, weights, dtype, device):
        self.width = int(params["width"])
        self.eps = float(params["eps"])
        self.weight = weights["weight"]

    def forward(self, x, x0, ctx):
        out = torch.empty_like(x)
        ops.rmsnorm(out, x, self.weight, self.eps, None)
        return out


class AddRow:
    """x <- x + R[row] in 32-bit, in place: one row of a table is added to every token's stream (a model that runs a
    stretch of layers several times may begin each pass with a row of its own).
    params: ``width``, ``rows`` (of the table), ``row``.  weights: ``weight`` [rows, width]."""

    graph_safe = True

    @classmethod
    def weight_shapes(cls, params):
        return {"weight": ((params["rows"], params["width"]), "matrix")}

    def __init__(self, params, weights, dtype, device):
        row, rows = int(params["row"]), int(params["rows"])
        if not 0 <= row < rows:
            raise ConfigError(f"row {row} is outside the table's {rows} rows")
        self.row = weights["weight"][row].to(torch.float32).contiguous()

    def forward(self, x, x0, ctx):
        ops.add_row(x, self.row)
        return x


register_part("stream", "add_row", AddRow)
register_part("stream", "mix_with_embedding", MixWithEmbedding)
register_part("stream", "rmsnorm", NormedStream)
