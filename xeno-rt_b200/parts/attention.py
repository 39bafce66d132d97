"""Grouped-query causal attention with optional per-head q/k RMSNorm and a position encoding.

Order, as in crates/xrt-models/src/llama.rs:447-577: q, k, v products; per-head norm of q and k if
the layer has one (488-496, 1025-1040); rotation (498-500); k and v into the cache (502); attention of
every query head over the keys of its group's kv head up to its own position with scale
1/sqrt(head_dim) (504-574); output product added to the residual (576-577).
"""
from __future__ import annotations

import math

import torch

from ..cache import KVNeed, StateNeed
from ..core import ConfigError, DType, Unsupported, torch_dtype
from ..csrc import ops
from .linear import linear
from .registry import part_class, register_part


def kernel_head_size(head_dim: int, v_head_dim: int) -> int:
    """The one head size that the attention kernels and the cache run a layer at: the larger of the key
    and the value size, rounded up to a multiple of 16."""
    return -(-max(int(head_dim), int(v_head_dim)) // 16) * 16


def _pad_rows(w, heads: int, size: int, to: int):
    """[heads * size, in] -> [heads * to, in], every head's rows followed by zero rows."""
    out = torch.zeros((heads, to, w.shape[1]), dtype=w.dtype, device=w.device)
    out[:, :size] = w.reshape(heads, size, w.shape[1])
    return out.reshape(heads * to, w.shape[1])


def _pad_columns(w, heads: int, size: int, to: int):
    """[out, heads * size] -> [out, heads * to], every head's columns followed by zero columns."""
    out = torch.zeros((w.shape[0], heads, to), dtype=w.dtype, device=w.device)
    out[:, :, :size] = w.reshape(w.shape[0], heads, size)
    return out.reshape(w.shape[0], heads * to).contiguous()


class GroupedQueryAttention:
    """params: ``width`` (model width), ``n_heads``, ``n_kv_heads``, ``head_dim``, ``qk_norm``
    (bool), ``eps`` (of the head norms), ``window`` (None = all keys), ``position`` (a PartSpec-like
    dict ``{"kind", "params"}``); optional: ``v_head_dim`` (the value size of a head, default
    head_dim), ``scale`` (of the scores, default 1 / sqrt(head_dim)), ``gate`` ("sigmoid" or "silu":
    the concatenated heads are multiplied by that function of a product ``g`` of the mixer's input
    before the output product; "sigmoid_head": one sigmoid gate a head, ``g`` [n_heads, width]), ``bias`` (q, k and v
    have biases ``q_bias``, ``k_bias``, ``v_bias``), ``qk_norm`` = "unit" (q and k heads divided by their root mean
    square, no weight), ``softcap`` (scores <- cap * tanh(scores / cap)), ``distance_rate`` r (head h's scores lose
    2^(-r (h + 1) / n_heads) for every position between query and key), ``keep_first`` (so many first keys of a
    sequence stay visible behind the window), ``value_blend`` (a name: the first layer of a model that gives this name
    keeps its values of the step's tokens, every later one caches (1 - b) v + b v_first with its own scalar ``blend``),
    ``qk_norm`` = "whole" (q and k are RMS-normed over the whole projection, all heads of a token at once, weights
    ``q_norm`` [n_heads*head_dim] and ``k_norm`` [n_kv_heads*head_dim], before the rotation), ``sink`` (a number s: the
    softmax's denominator holds one more term exp(s) that has no value, so a head may give less than an average of
    its values), ``own_kv`` = False (the layer has no k and v products, norms or cache of its own: it is scheduled
    with ``cache_from`` and reads the keys and values another layer cached, with its own queries, window and scale),
    ``conv`` (a number of taps: q, k and v pass a short causal convolution over time a channel, weights ``q_conv``,
    ``k_conv``, ``v_conv`` [channels, taps], right after the product and its bias, before norms and rotation; the
    last taps - 1 rows of the product are state of the sequence, so the part then asks for a ``StateNeed`` beside
    its keys), ``v_norm`` = "unit" (every value head is divided by its root mean square, ``eps``, no weight, before it
    is cached), ``o_bias`` (the output product has a bias ``o_bias`` [width]).
    weights: ``q`` [n_heads*head_dim, width], ``k`` [n_kv_heads*head_dim, width], ``v``
    [n_kv_heads*v_head_dim, width], ``o`` [width, n_heads*v_head_dim], with qk_norm ``q_norm``,
    ``k_norm`` [head_dim], with a gate ``g`` [n_heads*v_head_dim, width].

    The kernels and the cache run a layer at ONE head size.  Where the key and value sizes differ, or
    are no multiple of 16, every head is laid out at ``kernel_head_size`` with zero rows in q, k, v and
    g and zero columns in o: zero key dims add nothing to a score, zero value dims come out as zeros
    and meet zero columns, so the result is that of the true sizes."""

    graph_safe = True

    @classmethod
    def _sizes(cls, params):
        hd = int(params["head_dim"])
        vd = int(params.get("v_head_dim") or hd)
        return hd, vd, kernel_head_size(hd, vd)

    @classmethod
    def fused_weights(cls, params):
        """q, k and v (and the gate's matrix) are one matrix [q rows, k rows, v rows, g rows] for one product."""
        hd, vd, size = cls._sizes(params)
        if hd != size or vd != size or not params.get("own_kv", True):
            return {}  # the part lays the heads out itself
        return {"qkvg": ("q", "k", "v", "g")} if params.get("gate") else {"qkv": ("q", "k", "v")}

    @staticmethod
    def _unit_norm(params) -> bool:
        return params.get("qk_norm") == "unit"

    @staticmethod
    def _whole_norm(params) -> bool:
        return params.get("qk_norm") == "whole"

    @classmethod
    def weight_shapes(cls, params):
        d, nh, nkv = params["width"], params["n_heads"], params["n_kv_heads"]
        hd, vd, _ = cls._sizes(params)
        shapes = {"q": ((nh * hd, d), "matrix"), "k": ((nkv * hd, d), "matrix"), "v": ((nkv * vd, d), "matrix"),
                  "o": ((d, nh * vd), "matrix")}
        if params.get("qk_norm") and not cls._unit_norm(params):
            whole = cls._whole_norm(params)
            shapes["q_norm"] = ((nh * hd if whole else hd,), "vector")
            shapes["k_norm"] = ((nkv * hd if whole else hd,), "vector")
        if not params.get("own_kv", True):
            for role in ("k", "v", "k_norm"):
                shapes.pop(role, None)
        if params.get("gate"):
            shapes["g"] = ((nh if params["gate"] == "sigmoid_head" else nh * vd, d), "matrix")
        if params.get("bias"):
            shapes.update({"q_bias": ((nh * hd,), "vector"), "k_bias": ((nkv * hd,), "vector"),
                           "v_bias": ((nkv * vd,), "vector")})
        if params.get("value_blend"):
            shapes["blend"] = ((), "vector")
        if params.get("conv"):
            taps = int(params["conv"])
            shapes.update({"q_conv": ((nh * hd, taps), "vector"), "k_conv": ((nkv * hd, taps), "vector"),
                           "v_conv": ((nkv * vd, taps), "vector")})
        if params.get("o_bias"):
            shapes["o_bias"] = ((d,), "vector")
        return shapes

    def __init__(self, params, weights, dtype: DType, device):
        self.width = int(params["width"])
        self.n_heads = int(params["n_heads"])
        self.n_kv_heads = int(params["n_kv_heads"])
        true_dim, true_vdim, self.head_dim = self._sizes(params)  # head_dim: the size the kernels and the cache see
        self.eps = float(params.get("eps", 1e-5))
        self.window = params.get("window")
        self.gate = params.get("gate")
        if self.gate not in (None, "sigmoid", "silu", "sigmoid_head"):
            raise ConfigError(f"attention gate {self.gate!r} is not sigmoid, silu or sigmoid_head")
        self.unit_norm = self._unit_norm(params)
        self.whole_norm = self._whole_norm(params)
        self.own_kv = bool(params.get("own_kv", True))
        self.sink = None if params.get("sink") is None else float(params["sink"])
        if not self.own_kv and (params.get("bias") or params.get("value_blend")):
            raise Unsupported("a layer without keys and values of its own cannot have their biases or blend them")
        self.keep_first = int(params.get("keep_first") or 0) if self.window else 0
        self.softcap = float(params.get("softcap") or 0.0)
        self.distance_rate = float(params.get("distance_rate") or 0.0)
        self.value_blend = params.get("value_blend")
        self.true_dim, self.true_vdim = true_dim, true_vdim
        if self.n_heads % self.n_kv_heads:
            raise ConfigError(f"{self.n_heads} heads are not a multiple of {self.n_kv_heads} kv heads")
        if not (16 <= self.head_dim <= 256):
            raise Unsupported(f"head size {max(true_dim, true_vdim)}: the attention kernels take head sizes up to 256")
        if params.get("qk_norm") and not self.unit_norm and not self.whole_norm and true_dim != self.head_dim:
            raise Unsupported(f"q/k head norms with a head size of {true_dim} (no multiple of 16, or smaller than "
                              f"the value size) are not supported")
        self.q_width = self.n_heads * self.head_dim
        self.kv_width = self.n_kv_heads * self.head_dim
        # one fused weight for the products that read the mixer's input; the reference fuses only their dispatch (447-486)
        self.w_qkv = weights.get("qkvg" if self.gate else "qkv")
        self.w_o = weights["o"]
        if self.w_qkv is None:  # tensors that came one by one, or heads that are laid out at another size
            pieces = [_pad_rows(weights["q"], self.n_heads, true_dim, self.head_dim)]
            if self.own_kv:
                pieces += [_pad_rows(weights["k"], self.n_kv_heads, true_dim, self.head_dim),
                           _pad_rows(weights["v"], self.n_kv_heads, true_vdim, self.head_dim)]
            if self.gate == "sigmoid_head":
                pieces.append(weights["g"])
            elif self.gate:
                pieces.append(_pad_rows(weights["g"], self.n_heads, true_vdim, self.head_dim))
            self.w_qkv = torch.cat(pieces, dim=0).contiguous()
            if true_vdim != self.head_dim:
                self.w_o = _pad_columns(weights["o"], self.n_heads, true_vdim, self.head_dim)
        self.w_q = self.w_qkv[: self.q_width]
        self.gate_offset = self.q_width + 2 * self.kv_width
        weighted = params.get("qk_norm") and not self.unit_norm
        self.q_norm = weights.get("q_norm") if weighted else None
        self.k_norm = weights.get("k_norm") if weighted else None
        if self.whole_norm and true_dim != self.head_dim:  # one weight a column of the projection as it is laid out
            self.q_norm = _pad_rows(self.q_norm.reshape(-1, 1), self.n_heads, true_dim, self.head_dim).reshape(-1)
            if self.k_norm is not None:
                self.k_norm = _pad_rows(self.k_norm.reshape(-1, 1), self.n_kv_heads, true_dim, self.head_dim).reshape(-1)
        # one 32-bit bias a column of the q/k/v product's row, laid out as the row is (nothing for the gate's columns)
        self.bias = None
        if params.get("bias"):
            def as_row(t, heads, size):
                return _pad_rows(t.to(torch.float32).reshape(-1, 1), heads, size, self.head_dim).reshape(-1)
            self.bias = torch.cat([as_row(weights["q_bias"], self.n_heads, true_dim),
                                   as_row(weights["k_bias"], self.n_kv_heads, true_dim),
                                   as_row(weights["v_bias"], self.n_kv_heads, true_vdim)]).contiguous()
        self.blend = float(weights["blend"].to(torch.float32).reshape(-1)[0]) if self.value_blend else 0.0
        # a short convolution over time on every column of the q/k/v row (taps laid out as the row is)
        self.taps = int(params.get("conv") or 0)
        self.conv = None
        if self.taps:
            if not self.own_kv or self.gate:
                raise Unsupported("a convolution on q, k and v needs keys and values of the layer's own and no gate")
            if not 1 <= self.taps <= 9:
                raise ConfigError(f"a short convolution of {self.taps} taps is outside 1 to 9")
            def taps_of(t, heads, size):
                return _pad_rows(t.to(torch.float32), heads, size, self.head_dim)
            self.conv = torch.cat([taps_of(weights["q_conv"], self.n_heads, true_dim),
                                   taps_of(weights["k_conv"], self.n_kv_heads, true_dim),
                                   taps_of(weights["v_conv"], self.n_kv_heads, true_vdim)]).contiguous()
        self.v_unit = params.get("v_norm") == "unit"
        if params.get("v_norm") not in (None, "unit"):
            raise ConfigError(f"v_norm {params.get('v_norm')!r} is not unit")
        self.o_bias = weights["o_bias"].to(torch.float32).contiguous() if params.get("o_bias") else None
        # what the rotation kernel and the kernels that fold it in do not do: these layers prepare their heads with
        # ops.qkv_heads_write and attend with the kernels that take the score options
        self.plain_heads = (self.bias is None and not self.unit_norm and not self.whole_norm and not self.value_blend
                            and true_dim == self.head_dim and not self.taps and not self.v_unit)
        self.plain_scores = not (self.keep_first or self.softcap or self.distance_rate) and self.sink is None
        position = params.get("position") or {"kind": "none", "params": {}}
        self.position = part_class("position", position["kind"])(position.get("params", {}), {}, dtype, device)
        rope_dim = getattr(self.position, "rope_dim", 0)
        if rope_dim > true_dim:
            raise ConfigError(f"rope_dim {rope_dim} exceeds the head size {true_dim}")
        self.scale = float(params["scale"]) if params.get("scale") is not None else 1.0 / math.sqrt(true_dim)
        self.dtype = dtype
        self.act_dtype = torch_dtype(dtype)

    def cache_need(self):
        keys = KVNeed(self.n_kv_heads, self.head_dim, self.window, self.keep_first)
        if self.taps > 1:  # the convolution's last taps - 1 inputs, one row of the q/k/v product each
            return [keys, StateNeed((self.taps - 1, self.q_width + 2 * self.kv_width), "float32")]
        return keys

    def takes_pending_norm(self, rows: int, device) -> bool:
        """Whether the first product of ``forward`` can finish a norm that the part before prepared."""
        if self.dtype is not DType.BF16:
            return False
        from . import linear_bf16
        return linear_bf16.takes_pending(rows, self.w_qkv.shape[0], self.width, "store", device)

    def forward(self, h, residual, ctx, store, owns_cache=True):
        then_norm = getattr(ctx, "then_norm", None)  # for this part's last product only
        if then_norm is not None:
            ctx.then_norm = None
        attended = self.attended(h, ctx, store, owns_cache)
        if self.o_bias is not None:
            ops.add_row(residual, self.o_bias)
        if then_norm is not None:
            _, ctx.pending = linear(attended, self.w_o, accumulate_into=residual, then_norm=then_norm)
        else:
            linear(attended, self.w_o, accumulate_into=residual)

    def mix(self, h, ctx, store, owns_cache=True, out=None, leave_bias=False):
        """The mixer's result, float32 [T, width], for a caller that does something else with it than adding it
        (written into ``out`` where that is given).  ``leave_bias``: the caller adds ``o_bias`` itself."""
        ctx.then_norm = None
        y = linear(self.attended(h, ctx, store, owns_cache), self.w_o, out_dtype=torch.float32, out=out)
        if self.o_bias is not None and not leave_bias:
            ops.add_row(y, self.o_bias)
        return y

    def attended(self, h, ctx, store, owns_cache=True):
        """The concatenated heads (gated if the layer has a gate) in the compute dtype, [T, heads * head size]."""
        n = h.shape[0]
        gated = self.gate is not None
        bias = self.bias
        if self.taps > 1:
            if not owns_cache:
                raise ConfigError("a layer with a convolution on q, k and v cannot read another place's state")
            store, conv_store = store
        qkv = projected = linear(h, self.w_qkv if owns_cache or gated else self.w_q, out_dtype=torch.float32)
        if self.taps:
            # the product's bias is added on the convolution's way in; rows of no sequence are left alone there
            fresh = torch.zeros if getattr(ctx, "captured", False) or sum(ctx.new_lens) < ctx.n_tokens else torch.empty
            qkv = fresh(projected.shape, dtype=torch.float32, device=h.device)
            ops.short_conv(qkv, projected, self.conv, conv_store.state if self.taps > 1 else None, ctx.cu_seqlens,
                           ctx.seq_slot, ctx.max_new, "none", in_bias=bias)
            bias = None
        window = int(self.window) if self.window else 0
        pairing = getattr(self.position, "pairing", "split_half")
        cos_sin = self.position.tables(ctx)
        # padding rows belong to no sequence: kernels that walk sequences leave them unwritten
        # a captured step is replayed with padding rows, which the kernel of the scored layers leaves unwritten
        padded = (getattr(ctx, "captured", False) and not self.plain_scores) or sum(ctx.new_lens) < ctx.n_tokens
        attended = (torch.zeros if padded else torch.empty)((n, self.q_width), dtype=self.act_dtype, device=h.device)
        if self.dtype is DType.BF16 and self.plain_heads and self.plain_scores:
            from . import attention_bf16
            if attention_bf16.decode_from_qkv(attended, qkv, self.q_width, self.q_width + self.kv_width, self.q_norm,
                                              self.k_norm, self.eps, cos_sin, pairing, ctx, store, self.n_heads,
                                              self.n_kv_heads, self.head_dim, self.scale, window, owns_cache):
                qkv = None
        if qkv is not None:
            q = torch.empty((n, self.q_width), dtype=self.act_dtype, device=h.device)
            if self.plain_heads:
                ops.qk_rope_kv_write(q, store.k, store.v, qkv, self.q_width, self.q_width + self.kv_width, self.q_norm,
                                     self.k_norm, self.eps, cos_sin, ctx.tok_slot, ctx.tok_pos, store.block_table,
                                     self.n_heads, self.n_kv_heads, self.head_dim, write_kv=owns_cache, pairing=pairing)
            else:
                v_keep = v_first = None
                if self.value_blend and owns_cache:
                    v_first = ctx.shared.get(("value_blend", self.value_blend))
                    if v_first is not None and v_first.shape[1] != self.n_kv_heads * self.true_vdim:
                        raise ConfigError("layers that blend their values must have the same kv heads and value size")
                    if v_first is None:  # the first layer of this name in the step: its values are the ones blended in
                        v_keep = torch.zeros((n, self.n_kv_heads * self.true_vdim), dtype=torch.float32, device=h.device)
                        ctx.shared[("value_blend", self.value_blend)] = v_keep
                ops.qkv_heads_write(q, store.k, store.v, qkv, self.q_width, self.q_width + self.kv_width, bias,
                                    self.unit_norm, self.true_dim, self.eps, ctx.tok_slot, ctx.tok_pos, store.block_table,
                                    self.n_heads, self.n_kv_heads, self.head_dim, v_keep=v_keep, v_first=v_first,
                                    v_blend=self.blend if v_first is not None else 0.0, v_dim=self.true_vdim,
                                    write_kv=owns_cache, q_norm_w=self.q_norm, k_norm_w=self.k_norm if owns_cache else None,
                                    whole_q=self.n_heads * self.true_dim if self.whole_norm else 0,
                                    whole_k=self.n_kv_heads * self.true_dim if self.whole_norm else 0,
                                    cos_sin=cos_sin, pairing=pairing, v_unit=self.v_unit)
            self.attend(attended, q, ctx, store)
        if self.gate == "sigmoid_head":
            ops.gate_mul(attended, projected[:, self.gate_offset:], "sigmoid", group=self.head_dim)
        elif gated:
            ops.gate_mul(attended, projected[:, self.gate_offset:], self.gate)
        return attended

    def attend(self, out, q, ctx, store):
        window = int(self.window) if self.window else 0
        options = {} if self.plain_scores else {"keep_first": self.keep_first, "softcap": self.softcap,
                                                "distance_rate": self.distance_rate, "sink": self.sink}
        if self.dtype is DType.BF16:
            from . import attention_bf16
            if attention_bf16.run(out, q, ctx, store, self.n_heads, self.n_kv_heads, self.head_dim, self.scale,
                                  window, **options):
                return
        ops.attention_reference(out, q, store.k, store.v, ctx.tok_slot, ctx.tok_pos, store.block_table,
                                self.n_heads, self.n_kv_heads, self.head_dim, self.scale, window, **options)


register_part("mixer", "attention", GroupedQueryAttention)
