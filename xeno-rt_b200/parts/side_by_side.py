"""A mixer made of several mixers that read the same input side by side: each one's result is RMS-normed
over the model width with a weight of its own, and the mean of those is the mixer's result.

params: ``width``, ``eps``, ``branches``: a list of ``{"name", "kind", "params"}`` naming registered mixers
(each must offer ``mix``).  weights: for branch ``name`` the branch's own tensors under ``<name>.<role>``
and its norm weight under ``<name>.out`` [width].  The cache need is the list of the branches' needs.

``combine`` = "weighted" instead: the result is sum_b scale_b * result_b with a number ``scale`` in every branch's
dict; no norms and no ``<name>.out`` weights.  Such a mixer hands its result back in parts (``mix`` returns a
``WeightedParts``: the norm that follows it adds them up), or adds them into the stream itself (``forward``).
"""
from __future__ import annotations

import torch

from ..core import ConfigError
from ..csrc import ops
from .registry import part_class, register_part


class SideBySideMixer:

    @classmethod
    def _branches(cls, params):
        for branch in params["branches"]:
            yield branch["name"], part_class("mixer", branch["kind"]), branch.get("params", {})

    @classmethod
    def fused_weights(cls, params):
        fused = {}
        for name, branch_cls, branch_params in cls._branches(params):
            inner = getattr(branch_cls, "fused_weights", None)
            for role, roles in (inner(branch_params).items() if inner else ()):
                fused[f"{name}.{role}"] = tuple(f"{name}.{r}" for r in roles)
        return fused

    @classmethod
    def weight_shapes(cls, params):
        shapes = {}
        for name, branch_cls, branch_params in cls._branches(params):
            for role, shape in branch_cls.weight_shapes(branch_params).items():
                shapes[f"{name}.{role}"] = shape
            if params.get("combine", "normed_mean") != "weighted":
                shapes[f"{name}.out"] = ((params["width"],), "vector")
        return shapes

    def __init__(self, params, weights, dtype, device):
        self.width, self.eps = int(params["width"]), float(params.get("eps") or 0.0)
        self.combine = params.get("combine", "normed_mean")
        if self.combine not in ("normed_mean", "weighted"):
            raise ConfigError(f"side-by-side mixers are combined as normed_mean or weighted, not {self.combine!r}")
        self.branches, self.out_weights = [], []
        for name, branch_cls, branch_params in self._branches(params):
            if not hasattr(branch_cls, "mix"):
                raise ConfigError(f"mixer {branch_cls.__name__} cannot stand side by side: it has no 'mix'")
            own = {role[len(name) + 1:]: t for role, t in weights.items()
                   if role.startswith(name + ".") and role != f"{name}.out"}
            self.branches.append(branch_cls(branch_params, own, dtype, device))
            if self.combine != "weighted":
                self.out_weights.append(weights[f"{name}.out"].to(torch.float32).contiguous())
        self.bias = None
        if self.combine == "weighted":
            factors = [float(b["scale"]) for b in params["branches"]]
            self.scales = torch.tensor(factors, dtype=torch.float32, device=device)
            # a bias of a branch's last product is left for whoever adds the parts up: one row, sum_b scale_b * bias_b
            for branch, factor in zip(self.branches, factors):
                if getattr(branch, "o_bias", None) is not None:
                    row = branch.o_bias.to(torch.float32) * factor
                    self.bias = row if self.bias is None else self.bias + row
        if not self.branches:
            raise ConfigError("a side-by-side mixer needs at least one branch")
        self.graph_safe = all(getattr(b, "graph_safe", False) for b in self.branches)

    def cache_need(self):
        return [b.cache_need() for b in self.branches]

    def mix(self, h, ctx, store, owns_cache=True):
        """The branches' results as parts with their factors (``combine`` "weighted" only)."""
        from .norm import WeightedParts
        if self.combine != "weighted":
            raise ConfigError("side-by-side mixers whose results are normed and averaged add into the stream themselves")
        ctx.then_norm = None
        parts = torch.empty((len(self.branches), h.shape[0], self.width), dtype=torch.float32, device=h.device)
        for i, (branch, branch_store) in enumerate(zip(self.branches, store)):
            if getattr(branch, "o_bias", None) is not None:
                branch.mix(h, ctx, branch_store, owns_cache, out=parts[i], leave_bias=True)
            else:
                branch.mix(h, ctx, branch_store, owns_cache, out=parts[i])
        return WeightedParts(parts, self.scales, self.bias)

    def forward(self, h, residual, ctx, store, owns_cache=True):
        ctx.then_norm = None
        if self.combine == "weighted":
            y = self.mix(h, ctx, store, owns_cache)
            ops.add_scaled_parts(residual, y.parts, y.scales)
            if y.bias is not None:
                ops.add_row(residual, y.bias)
            return
        share = 1.0 / len(self.branches)
        for branch, weight, branch_store in zip(self.branches, self.out_weights, store):
            y = branch.mix(h, ctx, branch_store, owns_cache)
            ops.rms_scale_add(residual, y, weight, self.eps, share)


register_part("mixer", "side_by_side", SideBySideMixer)
