"""Feed-forwards.  SwiGLU: down( silu(gate(h)) * up(h) ), added to the residual
(crates/xrt-models/src/llama.rs:584-601; crates/xrt-kernels/src/cpu/silu.rs:1-3, 22-24).  Beside it a feed-forward
without a gate, down( relu(up(h))^2 ), and a mixture of small gated experts of which every token uses a few."""
from __future__ import annotations

import torch

from ..core import ConfigError, DType, torch_dtype
from ..csrc import ops
from .linear import linear
from .registry import register_part


class SwiGLUFeedForward:
    """params: ``width``, ``inner`` (the feed-forward width); optional ``activation`` of the gate: "silu" (default) or
    "gelu_tanh" (the tanh form of gelu: down( gelu_tanh(gate(h)) * up(h) )).
    weights: ``gate``, ``up`` [inner, width], ``down`` [width, inner]."""

    graph_safe = True

    @classmethod
    def fused_weights(cls, params):
        """gate and up are one matrix [gate rows, up rows] for one product."""
        return {"gate_up": ("gate", "up")}

    @classmethod
    def weight_shapes(cls, params):
        d, f = params["width"], params["inner"]
        return {"gate": ((f, d), "matrix"), "up": ((f, d), "matrix"), "down": ((d, f), "matrix")}

    def __init__(self, params, weights, dtype: DType, device):
        self.width = int(params["width"])
        self.inner = int(params["inner"])
        # one fused weight [2 * inner, width]: gate rows, then up rows
        self.w_gate_up = weights.get("gate_up")
        if self.w_gate_up is None:  # tensors that came one by one
            self.w_gate_up = torch.cat([weights["gate"], weights["up"]], dim=0).contiguous()
        self.w_down = weights["down"]
        self.act_dtype = torch_dtype(dtype)
        self.activation = params.get("activation", "silu")
        if self.activation not in ops.GATE_ACTS:
            raise ConfigError(f"the gate's activation {self.activation!r} is not one of {sorted(ops.GATE_ACTS)}")

    def takes_pending_norm(self, rows: int, device) -> bool:
        """Whether the first product of ``forward`` can finish a norm that the part before prepared."""
        if self.act_dtype != torch.bfloat16 or self.activation != "silu":
            return False
        from . import linear_bf16
        return linear_bf16.takes_pending(rows, self.inner, self.width, "swiglu", device)

    def _act(self, h):
        act = torch.empty((h.shape[0], self.inner), dtype=self.act_dtype, device=h.device)
        fused = False
        if self.act_dtype == torch.bfloat16 and h.dtype == torch.bfloat16:
            from . import linear_bf16
            fused = linear_bf16.run_swiglu(act, h, self.w_gate_up, self.inner, self.activation)
        if not fused:
            gate_up = linear(h, self.w_gate_up, out_dtype=torch.float32)
            ops.swiglu(act, gate_up, self.activation)
        return act

    def apply(self, h, ctx, out=None):
        """The result handed back, float32 [T, width] (written into ``out`` where that is given)."""
        ctx.then_norm = None
        return linear(self._act(h), self.w_down, out_dtype=torch.float32, out=out)

    def forward(self, h, residual, ctx):
        act = self._act(h)
        # the last product may prepare the norm that follows this part (ctx.then_norm, see parts/context.py)
        if getattr(ctx, "then_norm", None) is not None:
            _, ctx.pending = linear(act, self.w_down, accumulate_into=residual, then_norm=ctx.then_norm)
        else:
            linear(act, self.w_down, accumulate_into=residual)


class SquaredReluFeedForward:
    """down( relu(up(h))^2 ).  params: ``width``, ``inner``.  weights: ``up`` [inner, width], ``down`` [width, inner]."""

    graph_safe = True

    @classmethod
    def weight_shapes(cls, params):
        d, f = params["width"], params["inner"]
        return {"up": ((f, d), "matrix"), "down": ((d, f), "matrix")}

    def __init__(self, params, weights, dtype: DType, device):
        self.inner = int(params["inner"])
        self.w_up, self.w_down = weights["up"], weights["down"]
        self.act_dtype = torch_dtype(dtype)

    def _act(self, h):
        act = torch.empty((h.shape[0], self.inner), dtype=self.act_dtype, device=h.device)
        ops.relu_squared(act, linear(h, self.w_up, out_dtype=torch.float32))
        return act

    def apply(self, h, ctx):
        """The result handed back, float32 [T, width]."""
        return linear(self._act(h), self.w_down, out_dtype=torch.float32)

    def forward(self, h, residual, ctx):
        ctx.then_norm = None
        linear(self._act(h), self.w_down, accumulate_into=residual)


class RoutedExperts:
    """``experts`` small gated feed-forwards of which a token uses the ``top`` with the largest router logits
    z = W_router h + b (32-bit), weighted by the softmax over those logits alone.  An expert:
    g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit), y = g * sigmoid(alpha g) * (u + 1), W_down y.
    params: ``width``, ``inner`` (an expert's), ``experts``, ``top``, ``limit``, ``alpha``.
    weights: ``router`` [experts, width], ``router_bias`` [experts], and for expert i ``gate<i>``, ``up<i>``
    [inner, width], ``down<i>`` [width, inner]; they are kept as two buffers, [experts * 2 * inner, width] (an expert's
    gate rows, then its up rows) and [experts * width, inner].

    Other kinds of expert and of routing, by parameter:
    ``activation`` = "gelu": an expert is W_down gelu(W_up h) with the exact (erf) gelu and has no gate (no ``gate<i>``,
    ``limit`` or ``alpha``; the first buffer is [experts * inner, width]).
    ``routing`` = "scores": the weights are the softmax of the logits over ALL experts, as they are (not renormalized
    over the chosen); with ``groups`` (a number of equal groups of neighbouring experts) and ``keep_groups``, only
    experts of the ``keep_groups`` groups whose best score is largest can be chosen.  ``router_bias`` = False: the
    router has no bias tensor.
    ``activation`` = "gated_silu": an expert is W_down (silu(W_gate h) * (W_up h)), no limits.
    More options of ``routing`` = "scores": ``scores`` = "sigmoid" (every score is the sigmoid of its logit, not the
    softmax over all); ``correction`` = True (a tensor ``correction`` [experts] is added to the scores for every choice,
    of groups and of experts, but not for the weights); ``group_best`` (a group counts by the sum of so many of its
    largest choice scores, default 1); ``normalize`` (the chosen weights are divided by their sum + ``sum_eps``);
    ``weight_scale`` (they are multiplied by it).
    ``shared`` (an inner width): one more gated silu feed-forward ``shared_gate``, ``shared_up`` [shared, width],
    ``shared_down`` [width, shared] that every token uses with weight 1; its result is one more part of ``apply``'s."""

    graph_safe = True

    @staticmethod
    def _gated(params) -> bool:
        return params.get("activation", "gated_sigmoid") != "gelu"

    @staticmethod
    def _shared_spec(params):
        """The parameters of the shared feed-forward (a ``SwiGLUFeedForward`` whose tensors are this part's
        ``shared_*`` roles), or None."""
        if not params.get("shared"):
            return None
        return {"width": params["width"], "inner": int(params["shared"]), "activation": "silu"}

    @classmethod
    def fused_weights(cls, params):
        n = int(params["experts"])
        first = (lambda i: (f"gate{i}", f"up{i}")) if cls._gated(params) else (lambda i: (f"up{i}",))
        fused = {"experts_in": tuple(r for i in range(n) for r in first(i)),
                 "experts_out": tuple(f"down{i}" for i in range(n))}
        if cls._shared_spec(params):
            fused["shared_gate_up"] = ("shared_gate", "shared_up")
        return fused

    @classmethod
    def weight_shapes(cls, params):
        d, f, n = params["width"], params["inner"], int(params["experts"])
        shapes = {"router": ((n, d), "matrix")}
        if params.get("router_bias", True):
            shapes["router_bias"] = ((n,), "vector")
        for i in range(n):
            shapes.update({f"up{i}": ((f, d), "matrix"), f"down{i}": ((d, f), "matrix")})
            if cls._gated(params):
                shapes[f"gate{i}"] = ((f, d), "matrix")
        if params.get("correction"):
            shapes["correction"] = ((n,), "vector")
        shared = cls._shared_spec(params)
        if shared:
            for role, shape in SwiGLUFeedForward.weight_shapes(shared).items():
                shapes["shared_" + role] = shape
        return shapes

    def __init__(self, params, weights, dtype: DType, device):
        self.width, self.inner = int(params["width"]), int(params["inner"])
        self.experts, self.top = int(params["experts"]), int(params["top"])
        self.act = params.get("activation", "gated_sigmoid")
        if self.act not in ops.MOE_ACTS:
            raise ConfigError(f"experts' activation {self.act!r} is not one of {sorted(ops.MOE_ACTS)}")
        self.scores = params.get("scores", "softmax")
        self.group_best = int(params.get("group_best") or 1)
        self.normalize, self.sum_eps = bool(params.get("normalize")), float(params.get("sum_eps") or 0.0)
        self.weight_scale = float(params.get("weight_scale") or 1.0)
        self.correction = weights["correction"].to(torch.float32).contiguous() if params.get("correction") else None
        self.shared = None
        shared = self._shared_spec(params)
        if shared:
            own = {role[len("shared_"):]: t for role, t in weights.items() if role.startswith("shared_")}
            self.shared = SwiGLUFeedForward(shared, own, dtype, device)
        self.limit, self.alpha = float(params.get("limit") or 0.0), float(params.get("alpha") or 0.0)
        self.routing = params.get("routing", "top_softmax")
        if self.routing not in ("top_softmax", "scores"):
            raise ConfigError(f"routing {self.routing!r} is not top_softmax or scores")
        self.groups, self.keep_groups = int(params.get("groups") or 1), int(params.get("keep_groups") or 1)
        if self.routing == "scores":
            if self.experts % self.groups or not 1 <= self.keep_groups <= self.groups:
                raise ConfigError(f"{self.experts} experts do not form {self.groups} equal groups of which "
                                  f"{self.keep_groups} are kept")
            if self.top > self.experts // self.groups * self.keep_groups:
                raise ConfigError(f"top {self.top} exceeds the experts of {self.keep_groups} kept groups")
        self.w_router = weights["router"]
        self.router_bias = None
        if params.get("router_bias", True):
            self.router_bias = weights["router_bias"].to(torch.float32).contiguous()
        fused = self.fused_weights(params)
        self.w_in = weights.get("experts_in")
        if self.w_in is None:
            self.w_in = torch.cat([weights[r] for r in fused["experts_in"]], dim=0).contiguous()
        self.w_out = weights.get("experts_out")
        if self.w_out is None:
            self.w_out = torch.cat([weights[r] for r in fused["experts_out"]], dim=0).contiguous()

    def route(self, h):
        """(expert numbers int32 [T, top], weights float32 [T, top])."""
        n = h.shape[0]
        logits = linear(h, self.w_router, out_dtype=torch.float32)
        ids = torch.empty((n, self.top), dtype=torch.int32, device=h.device)
        weights = torch.empty((n, self.top), dtype=torch.float32, device=h.device)
        if self.routing == "scores":
            if self.router_bias is not None:
                logits += self.router_bias
            ops.moe_route_scores(ids, weights, logits, self.top, self.groups, self.keep_groups, scores=self.scores,
                                 correction=self.correction, group_best=self.group_best, normalize=self.normalize,
                                 sum_eps=self.sum_eps, scale=self.weight_scale)
        else:
            ops.moe_route(ids, weights, logits, self.router_bias, self.top)
        return ids, weights

    GROUPED_FROM = 4  # (token, choice) pairs an expert from which a step's rows are sorted by expert

    def apply(self, h, ctx):
        """The chosen experts' weighted results, float32 [top, T, width]; their sum in index order is the result.
        A step of few tokens runs every (token, choice) pair by itself, streaming that expert's matrices.  A step of
        many tokens (prompts, and decode steps of many sequences) sorts its rows by expert; in bfloat16 two launches
        then serve all experts with the row counts staying on the device (csrc/moe_grouped.cu: fit for a captured
        step), in float32 every expert's rows go through the library's product, for which the row counts are read back
        once (prompts only)."""
        n = h.shape[0]
        ids, weights = self.route(h)
        whole = torch.empty((self.top + (1 if self.shared else 0), n, self.width), dtype=torch.float32, device=h.device)
        out = whole[:self.top]
        if self.shared:
            self.shared.apply(h, ctx, out=whole[self.top])
        pairs = n * self.top
        one_launch = h.dtype == torch.bfloat16 and self.width % 8 == 0 and self.inner % 8 == 0
        fixed_shapes = getattr(ctx, "captured", False) or ctx.all_single  # no read-back inside such a step
        if pairs < self.GROUPED_FROM * self.experts or (fixed_shapes and not one_launch):
            ops.moe_experts(out, h, self.w_in, self.w_out, ids, weights, self.inner, self.limit, self.alpha, act=self.act)
            return whole
        offsets = torch.empty((self.experts + 1,), dtype=torch.int32, device=h.device)
        pos = torch.empty((pairs,), dtype=torch.int32, device=h.device)
        row_token = torch.empty((pairs,), dtype=torch.int32, device=h.device)
        ops.moe_group(offsets, pos, row_token, ids, self.experts)
        rows = torch.empty((pairs, self.width), dtype=h.dtype, device=h.device)
        ops.moe_gather(rows, h, row_token)
        if one_launch:
            # all experts in one launch a product: the blocks find their expert from the offsets on the device
            act = torch.empty((pairs, self.inner), dtype=h.dtype, device=h.device)
            y = torch.empty((pairs, self.width), dtype=torch.float32, device=h.device)
            ops.moe_grouped_product(act, rows, self.w_in, offsets, self.experts, self.inner, self.limit, self.alpha,
                                    act=self.act)
            ops.moe_grouped_product(y, act, self.w_out, offsets, self.experts)
        else:
            bounds = offsets.tolist()  # here the host waits for the device: how many rows each expert has
            act = torch.empty((pairs, self.inner), dtype=h.dtype, device=h.device)
            y = torch.zeros((pairs, self.width), dtype=torch.float32, device=h.device)
            for e in range(self.experts):
                lo, hi = bounds[e], bounds[e + 1]
                if hi > lo:
                    first = (1 if self.act == "gelu" else 2) * self.inner  # rows of an expert in the first buffer
                    gate_up = linear(rows[lo:hi], self.w_in[e * first:(e + 1) * first], out_dtype=torch.float32)
                    ops.moe_activation(act[lo:hi], gate_up, self.limit, self.alpha, kind=self.act)
                    linear(act[lo:hi], self.w_out[e * self.width:(e + 1) * self.width], accumulate_into=y[lo:hi])
        ops.moe_combine(out, y, pos, weights)
        return whole

    def forward(self, h, residual, ctx):
        ctx.then_norm = None
        parts = self.apply(h, ctx)
        for c in range(parts.shape[0]):
            residual.add_(parts[c])


register_part("feed_forward", "swiglu", SwiGLUFeedForward)
register_part("feed_forward", "relu_squared", SquaredReluFeedForward)
register_part("feed_forward", "routed_experts", RoutedExperts)
