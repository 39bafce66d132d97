"""Mixers that keep a matrix state per head instead of keys and values: gated linear attention, the gated delta
rule, and a delta rule with a decay and a removal rate per key channel (``DecayRemovalRule``, whose recurrence is in
its own text).  All run the same scan kernel (csrc/state_mixers.cu) over the tokens of a step,

    S_t = diag(a_t) S_(t-1) + k_t u_t^T,        o_t = S_t^T q_t,

with S [key size, value size] per head, a_t a decay per key channel, and u_t = v_t (gated linear
attention) or u_t = b_t (v_t - (diag(a_t) S_(t-1))^T k_t) (delta rule: the state is corrected by what it
already answers for k_t; the read-out sees the write).  The state, the decays, the unit norms and the
head norms are 32-bit in both compute dtypes; products take their inputs in the compute dtype.

The state lives in the cache as a ``StateNeed``: zero when a slot opens, carried from step to step,
laid out [heads, value size, key size] (a column of S is contiguous, which is how the kernel holds it).
"""
from __future__ import annotations

import torch

from ..cache import StateNeed
from ..core import ConfigError, DType, torch_dtype
from ..csrc import ops
from .linear import linear
from .registry import register_part


def _vector(t):
    """Small tensors of the recurrence are kept in 32-bit whatever the compute dtype."""
    return t.to(torch.float32).contiguous()


class _StateMixer:
    graph_safe = True

    def forward(self, h, residual, ctx, store, owns_cache=True):
        ctx.then_norm = None
        linear(self.heads_out(h, ctx, store, owns_cache), self.w_o, accumulate_into=residual)

    def mix(self, h, ctx, store, owns_cache=True, out=None):
        ctx.then_norm = None
        return linear(self.heads_out(h, ctx, store, owns_cache), self.w_o, out_dtype=torch.float32, out=out)

    @staticmethod
    def _rows(ctx):
        """How to make a buffer that the per-sequence kernels fill: they skip rows of no sequence (the padding rows
        of a captured step), which must then hold zeros and not whatever the memory held."""
        padded = getattr(ctx, "captured", False) or sum(ctx.new_lens) < ctx.n_tokens  # a captured step is replayed with padding rows
        return torch.zeros if padded else torch.empty

    @staticmethod
    def _owning(owns_cache):
        if not owns_cache:
            raise ConfigError("a mixer with a state cannot read another place's: the state is what the tokens left there")


class GatedLinearAttention(_StateMixer):
    """q = W_q h / sqrt(key size), k = W_k h, v = W_v h; decay a = sigmoid(W_a2 (W_a1 h) + bias)^(1 / tau) per
    head and key channel; scan; every head's o RMS-normed over the value size with one shared weight, times
    silu(W_g h), then W_o.
    params: ``width``, ``n_heads``, ``key_dim``, ``value_dim``, ``decay_rank`` (rows of a1), ``tau``, ``eps``.
    weights: ``q``, ``k`` [heads * key_dim, width], ``v``, ``g`` [heads * value_dim, width], ``a1`` [rank, width],
    ``a2`` [heads * key_dim, rank], ``a2_bias`` [heads * key_dim], ``norm`` [value_dim], ``o`` [width, heads * value_dim]."""

    @classmethod
    def fused_weights(cls, params):
        return {"qkvg": ("q", "k", "v", "g")}

    @classmethod
    def weight_shapes(cls, params):
        d, nh, kd, vd, r = (params[k] for k in ("width", "n_heads", "key_dim", "value_dim", "decay_rank"))
        return {"q": ((nh * kd, d), "matrix"), "k": ((nh * kd, d), "matrix"), "v": ((nh * vd, d), "matrix"),
                "g": ((nh * vd, d), "matrix"), "a1": ((r, d), "matrix"), "a2": ((nh * kd, r), "matrix"),
                "a2_bias": ((nh * kd,), "vector"), "norm": ((vd,), "vector"), "o": ((d, nh * vd), "matrix")}

    def __init__(self, params, weights, dtype: DType, device):
        self.n_heads, self.key_dim, self.value_dim = (int(params[k]) for k in ("n_heads", "key_dim", "value_dim"))
        self.tau, self.eps = float(params["tau"]), float(params["eps"])
        if not self.tau > 0:
            raise ConfigError(f"tau {self.tau} must be positive")
        self.w_in = weights.get("qkvg")
        if self.w_in is None:
            self.w_in = torch.cat([weights[r] for r in ("q", "k", "v", "g")], dim=0).contiguous()
        self.w_a1, self.w_a2, self.w_o = weights["a1"], weights["a2"], weights["o"]
        self.a2_bias, self.norm = _vector(weights["a2_bias"]), _vector(weights["norm"])
        self.act_dtype = torch_dtype(dtype)

    def cache_need(self):
        return StateNeed((self.n_heads, self.value_dim, self.key_dim), "float32")

    def heads_out(self, h, ctx, store, owns_cache=True):
        self._owning(owns_cache)
        nh, kd, vd = self.n_heads, self.key_dim, self.value_dim
        n = h.shape[0]
        p = linear(h, self.w_in, out_dtype=torch.float32)
        decay = linear(linear(h, self.w_a1, out_dtype=self.act_dtype), self.w_a2, out_dtype=torch.float32)
        ops.decay_from_gate(decay, self.a2_bias, nh, kd, self.tau)
        o = self._rows(ctx)((n, nh * vd), dtype=torch.float32, device=h.device)
        ops.state_scan(o, p, p[:, nh * kd:], p[:, 2 * nh * kd:], decay, None, store.state, ctx.cu_seqlens, ctx.seq_slot,
                       nh, nh, kd, vd, q_scale=kd ** -0.5, max_new=ctx.max_new)
        y = torch.empty((n, nh * vd), dtype=self.act_dtype, device=h.device)
        ops.head_norm_gate(y, o, self.norm, p[:, 2 * nh * kd + nh * vd:], nh, vd, self.eps, "silu")
        return y


class GatedDeltaRule(_StateMixer):
    """q = W_q h, k = W_k h (``n_qk_heads`` heads of key_dim), v = W_v h (``n_heads`` heads of value_dim; head i
    uses q/k head i // (n_heads / n_qk_heads)); each passes a short causal convolution per channel and silu; q and
    k become unit vectors per head (x / sqrt(sum x^2 + 1e-6)), q times key_dim^(-1/2); b = sigmoid(W_b h) per
    head; decay a = exp(-exp(A_log[head]) * softplus(W_a2 (W_a1 h) + dt_bias)) per head and key channel; scan with
    the delta rule; every head's o divided by its root mean square (eps), times the shared weight ``norm``, times
    sigmoid(W_g2 (W_g1 h)); then W_o.  The last taps - 1 inputs of the convolutions are state as well.
    params: ``width``, ``n_heads``, ``n_qk_heads``, ``key_dim``, ``value_dim``, ``taps``, ``decay_rank``,
    ``gate_rank``, ``eps``.
    weights: ``q``, ``k`` [qk heads * key_dim, width], ``v`` [heads * value_dim, width], ``q_conv``, ``k_conv``,
    ``v_conv`` [channels, taps], ``b`` [heads, width], ``A_log`` [heads], ``a1`` [decay_rank, width], ``a2``
    [heads * key_dim, decay_rank], ``dt_bias`` [heads * key_dim], ``g1`` [gate_rank, width], ``g2``
    [heads * value_dim, gate_rank], ``norm`` [value_dim], ``o`` [width, heads * value_dim]."""

    UNIT_EPS = 1e-6  # inside the root of the unit norms of q and k; a constant of the mixer

    @classmethod
    def fused_weights(cls, params):
        return {"qkvb": ("q", "k", "v", "b"), "a1g1": ("a1", "g1")}

    @classmethod
    def weight_shapes(cls, params):
        d, nh, nq, kd, vd, taps, ra, rg = (params[k] for k in ("width", "n_heads", "n_qk_heads", "key_dim", "value_dim",
                                                               "taps", "decay_rank", "gate_rank"))
        return {"q": ((nq * kd, d), "matrix"), "k": ((nq * kd, d), "matrix"), "v": ((nh * vd, d), "matrix"),
                "b": ((nh, d), "matrix"), "q_conv": ((nq * kd, taps), "vector"), "k_conv": ((nq * kd, taps), "vector"),
                "v_conv": ((nh * vd, taps), "vector"), "A_log": ((nh,), "vector"), "a1": ((ra, d), "matrix"),
                "a2": ((nh * kd, ra), "matrix"), "dt_bias": ((nh * kd,), "vector"), "g1": ((rg, d), "matrix"),
                "g2": ((nh * vd, rg), "matrix"), "norm": ((vd,), "vector"), "o": ((d, nh * vd), "matrix")}

    def __init__(self, params, weights, dtype: DType, device):
        self.n_heads, self.n_qk_heads, self.key_dim, self.value_dim, self.taps, self.decay_rank = (
            int(params[k]) for k in ("n_heads", "n_qk_heads", "key_dim", "value_dim", "taps", "decay_rank"))
        self.eps = float(params["eps"])
        if self.n_heads % self.n_qk_heads:
            raise ConfigError(f"{self.n_heads} heads are not a multiple of {self.n_qk_heads} q/k heads")
        if not (1 <= self.taps <= 9):
            raise ConfigError(f"a short convolution of {self.taps} taps is outside 1 to 9")
        self.w_in = weights.get("qkvb")
        if self.w_in is None:
            self.w_in = torch.cat([weights[r] for r in ("q", "k", "v", "b")], dim=0).contiguous()
        self.w_low = weights.get("a1g1")
        if self.w_low is None:
            self.w_low = torch.cat([weights["a1"], weights["g1"]], dim=0).contiguous()
        self.w_a2, self.w_g2, self.w_o = weights["a2"], weights["g2"], weights["o"]
        self.conv = torch.cat([_vector(weights[r]) for r in ("q_conv", "k_conv", "v_conv")], dim=0).contiguous()
        self.a_log, self.dt_bias, self.norm = _vector(weights["A_log"]), _vector(weights["dt_bias"]), _vector(weights["norm"])
        self.channels = 2 * self.n_qk_heads * self.key_dim + self.n_heads * self.value_dim
        self.act_dtype = torch_dtype(dtype)

    def cache_need(self):
        needs = [StateNeed((self.n_heads, self.value_dim, self.key_dim), "float32")]
        if self.taps > 1:
            needs.append(StateNeed((self.taps - 1, self.channels), "float32"))
        return needs

    def heads_out(self, h, ctx, store, owns_cache=True):
        self._owning(owns_cache)
        nh, nq, kd, vd = self.n_heads, self.n_qk_heads, self.key_dim, self.value_dim
        n = h.shape[0]
        p = linear(h, self.w_in, out_dtype=torch.float32)          # q | k | v | b
        low = linear(h, self.w_low, out_dtype=self.act_dtype)      # a1 h | g1 h
        decay = linear(low[:, :self.decay_rank], self.w_a2, out_dtype=torch.float32)
        gate = linear(low[:, self.decay_rank:], self.w_g2, out_dtype=torch.float32)
        ops.decay_from_step(decay, self.dt_bias, self.a_log, nh, kd)
        qkv = self._rows(ctx)((n, self.channels), dtype=torch.float32, device=h.device)
        conv_state = store[1].state if self.taps > 1 else None
        ops.short_conv(qkv, p, self.conv, conv_state, ctx.cu_seqlens, ctx.seq_slot, ctx.max_new, "silu")
        ops.unit_heads(qkv, 2 * nq, kd, self.UNIT_EPS, scaled_heads=nq, scale=kd ** -0.5)
        o = self._rows(ctx)((n, nh * vd), dtype=torch.float32, device=h.device)
        ops.state_scan(o, qkv, qkv[:, nq * kd:], qkv[:, 2 * nq * kd:], decay, p[:, self.channels:], store[0].state,
                       ctx.cu_seqlens, ctx.seq_slot, nh, nq, kd, vd, delta=True, max_new=ctx.max_new)
        y = torch.empty((n, nh * vd), dtype=self.act_dtype, device=h.device)
        ops.head_norm_gate(y, o, self.norm, gate, nh, vd, self.eps, "sigmoid")
        return y


class DecayRemovalRule(_StateMixer):
    """r = W_r h, k = W_k h, v = W_v h, all heads of ``dim``.  Per head and key channel a decay
    w = exp(-decay_rate * sigmoid(W_w2 tanh(W_w1 h) + w0)) and a removal rate a = sigmoid(W_a h + a_bias).  With the
    unit key n = k / sqrt(sum(k^2) + unit_eps) of a head, its state S [key, value] becomes
    S <- diag(w) S - (a * n) (n^T S) + k v^T, the decay and the removal both reading the state as the token found it,
    and o = S^T r.  Every head's o is divided by its root mean square (``eps``), times the weight ``norm`` (one a column
    of all heads), times sigmoid(W_g h); then W_o.  State, decays, rates, unit keys and head norms are 32-bit.
    params: ``width``, ``n_heads``, ``dim``, ``decay_rank`` (rows of w1), ``eps``, ``decay_rate``, ``unit_eps``.
    weights: ``r``, ``k``, ``v``, ``g``, ``a`` [heads * dim, width], ``a_bias``, ``w0``, ``norm`` [heads * dim],
    ``w1`` [decay_rank, width], ``w2`` [heads * dim, decay_rank], ``o`` [width, heads * dim]."""

    @classmethod
    def fused_weights(cls, params):
        return {"rkvgaw": ("r", "k", "v", "g", "a", "w1")}

    @classmethod
    def weight_shapes(cls, params):
        d, nh, hd, rank = (params[k] for k in ("width", "n_heads", "dim", "decay_rank"))
        shapes = {r: ((nh * hd, d), "matrix") for r in ("r", "k", "v", "g", "a")}
        shapes.update({"w1": ((rank, d), "matrix"), "w2": ((nh * hd, rank), "matrix"), "o": ((d, nh * hd), "matrix"),
                       "a_bias": ((nh * hd,), "vector"), "w0": ((nh * hd,), "vector"), "norm": ((nh * hd,), "vector")})
        return shapes

    def __init__(self, params, weights, dtype: DType, device):
        self.n_heads, self.dim, self.decay_rank = (int(params[k]) for k in ("n_heads", "dim", "decay_rank"))
        self.eps, self.decay_rate, self.unit_eps = (float(params[k]) for k in ("eps", "decay_rate", "unit_eps"))
        if not self.decay_rate > 0:
            raise ConfigError(f"decay_rate {self.decay_rate} must be positive")
        self.w_in = weights.get("rkvgaw")
        if self.w_in is None:
            self.w_in = torch.cat([weights[r] for r in ("r", "k", "v", "g", "a", "w1")], dim=0).contiguous()
        self.w_w2, self.w_o = weights["w2"], weights["o"]
        self.a_bias, self.w0, self.norm = _vector(weights["a_bias"]), _vector(weights["w0"]), _vector(weights["norm"])
        self.act_dtype = torch_dtype(dtype)

    def cache_need(self):
        return StateNeed((self.n_heads, self.dim, self.dim), "float32")

    def heads_out(self, h, ctx, store, owns_cache=True):
        self._owning(owns_cache)
        nh, hd = self.n_heads, self.dim
        n, w = h.shape[0], self.n_heads * self.dim
        p = linear(h, self.w_in, out_dtype=torch.float32)                   # r | k | v | g | a | w1 h
        low = torch.empty((n, self.decay_rank), dtype=self.act_dtype, device=h.device)
        ops.act_cast(low, p[:, 5 * w:], "tanh")
        decay = linear(low, self.w_w2, out_dtype=torch.float32)
        unit = torch.empty((n, w), dtype=torch.float32, device=h.device)
        removal = p[:, 4 * w:5 * w]
        ops.removal_gates(decay, self.w0, removal, self.a_bias, unit, p[:, w:2 * w], nh, hd, self.decay_rate, self.unit_eps)
        o = self._rows(ctx)((n, w), dtype=torch.float32, device=h.device)
        ops.state_scan(o, p, p[:, w:], p[:, 2 * w:], decay, None, store.state, ctx.cu_seqlens, ctx.seq_slot, nh, nh, hd, hd,
                       max_new=ctx.max_new, unit=unit, removal=removal)
        y = torch.empty((n, w), dtype=self.act_dtype, device=h.device)
        ops.head_norm_gate(y, o, self.norm, p[:, 3 * w:], nh, hd, self.eps, "sigmoid")
        return y


register_part("mixer", "decay_removal_rule", DecayRemovalRule)
register_part("mixer", "gated_linear_attention", GatedLinearAttention)
register_part("mixer", "gated_delta_rule", GatedDeltaRule)
