"""RMSNorm: y = (x / sqrt(mean(x^2) + eps)) * w, statistics in 32-bit
(crates/xrt-kernels/src/cpu/rmsnorm.rs:26-43), and a layer norm with a weight and no bias."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..core import torch_dtype
from ..csrc import ops
from .registry import register_part


@dataclass
class PendingNorm:
    """A norm's result that exists only up to its last step: ``scaled`` is the residual times the
    norm's weight (bfloat16 [rows, width]) and ``squares`` (float32 [parts, rows]) holds partial sums
    of squares of the residual's rows, both written by the product that added into the residual.  The
    product that takes this as its input multiplies row m of its result by
    1 / sqrt(sum of the row's parts / width + eps), since W . ((x * inv) * w) = inv * (W . (x * w)):
    no norm kernel runs between the two products of a decode step.  ``norm`` is the part whose result
    this stands for."""
    scaled: torch.Tensor
    squares: torch.Tensor
    eps: float
    norm: object

    @property
    def shape(self):
        return self.scaled.shape

    @property
    def dtype(self):
        return self.scaled.dtype

    @property
    def device(self):
        return self.scaled.device


@dataclass
class WeightedParts:
    """A sublayer's result that is still in parts: ``parts`` float32 [n, T, width], their sum sum_p scales[p] *
    parts[p] + bias being the result (``scales`` float32 [n] on the device, ``bias`` float32 [width] or None).  The
    norm that follows the sublayer adds them up in its own pass over the row."""
    parts: torch.Tensor
    scales: torch.Tensor
    bias: torch.Tensor | None = None


class RMSNorm:
    """params: ``width``, ``eps``; optional ``gain`` (a number g: ``add_into`` adds g times the norm; ``forward`` does
    not use it).  weights: ``weight`` [width]."""

    graph_safe = True

    @classmethod
    def weight_shapes(cls, params):
        return {"weight": ((params["width"],), "vector")}

    def __init__(self, params, weights, dtype, device):
        self.width = int(params["width"])
        self.eps = float(params["eps"])
        self.weight = weights["weight"]
        self.gain = float(params.get("gain") or 1.0)
        self.out_dtype = torch_dtype(dtype)

    def forward(self, x, rows=None):
        n = x.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.width), dtype=self.out_dtype, device=x.device)
        ops.rmsnorm(out, x, self.weight, self.eps, rows)
        return out

    def forward_f32(self, x):
        """The norm of the float32 rows ``x`` as float32 (a norm on the residual stream itself)."""
        out = torch.empty((x.shape[0], self.width), dtype=torch.float32, device=x.device)
        ops.rmsnorm(out, x, self.weight, self.eps, None)
        return out

    def add_into(self, residual, y, copy: bool = False, then=None):
        """residual += gain * norm(y), 32-bit (a norm that follows a sublayer).  ``y`` float32 [T, width] or [parts, T,
        width], whose parts are added in index order first; or a ``WeightedParts`` (parts with a factor each and a
        row added to their sum).  ``copy``: the new residual is also returned in the compute dtype, written in the
        same pass (what the next sublayer's products read), else None.  ``then``: another RMSNorm of this width whose
        weight has this one's dtype; its result over the new residual is returned, computed in the same pass (else None)."""
        scales = bias = None
        if isinstance(y, WeightedParts):
            y, scales, bias = y.parts, y.scales, y.bias
        if y.dim() == 3 and y.shape[0] == 1 and scales is None:
            y = y[0]
        out = following = None
        if copy:
            out = torch.empty(residual.shape, dtype=self.out_dtype, device=residual.device)
        elif isinstance(then, RMSNorm) and then.width == self.width and then.weight.dtype == self.weight.dtype:
            out = torch.empty(residual.shape, dtype=then.out_dtype, device=residual.device)
            following = (then.weight, then.eps, out)
        ops.rmsnorm_add(residual, y, self.weight, self.eps, copy=out if copy else None, factor=self.gain,
                        part_scales=scales, bias=bias, then=following)
        return out


class LayerNorm:
    """y = (x - mean(x)) / sqrt(mean((x - mean(x))^2) + eps) * w (+ b with ``bias``), statistics in 32-bit.
    params: ``width``, ``eps``, optional ``bias`` (bool).  weights: ``weight`` [width], with a bias ``bias`` [width].
    ``add_into(residual, y)`` adds the norm of ``y`` to the 32-bit residual stream in one pass (a norm that follows a
    sublayer); ``y`` may be [parts, T, width], whose parts are added in index order first."""

    graph_safe = True

    @classmethod
    def weight_shapes(cls, params):
        shapes = {"weight": ((params["width"],), "vector")}
        if params.get("bias"):
            shapes["bias"] = ((params["width"],), "vector")
        return shapes

    def __init__(self, params, weights, dtype, device):
        self.width = int(params["width"])
        self.eps = float(params["eps"])
        self.weight = weights["weight"]
        self.bias = weights["bias"].to(torch.float32).contiguous() if params.get("bias") else None
        self.weight32 = None
        self.out_dtype = torch_dtype(dtype)

    def _weight32(self):
        if self.weight32 is None:
            self.weight32 = self.weight.to(torch.float32).contiguous()
        return self.weight32

    def forward(self, x, rows=None):
        n = x.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.width), dtype=self.out_dtype, device=x.device)
        if self.bias is not None:
            ops.layernorm_affine(x, self._weight32(), self.bias, self.eps, out=out, rows=rows)
        else:
            ops.layernorm(out, x, self.weight, self.eps, rows)
        return out

    def add_into(self, residual, y, then=None):
        """residual += norm(y).  ``then``: another LayerNorm of the same width and eps; its result over the new
        residual is returned (computed in the same pass), else None."""
        if y.dim() == 3 and y.shape[0] == 1:
            y = y[0]
        parts = y.shape[0] if y.dim() == 3 else 1
        if isinstance(then, LayerNorm) and then.width == self.width and then.eps == self.eps:
            out = torch.empty(residual.shape, dtype=then.out_dtype, device=residual.device)
            ops.layernorm_affine(y, self._weight32(), self.bias, self.eps, out=out, residual=residual, n_parts=parts,
                                 then=(then._weight32(), then.bias))
            return out
        ops.layernorm_affine(y, self._weight32(), self.bias, self.eps, residual=residual, n_parts=parts)
        return None


register_part("norm", "rmsnorm", RMSNorm)
register_part("norm", "layernorm", LayerNorm)
