"""Latent attention: the keys and values of all heads are read out of one small normed vector a token (the latent
c), and one rotated key part is shared by all heads.

    q = W_q h, a head's row being [dim plain | rot rotated];  [c_raw | k_rot] = W_down h  (rank + rot rows)
    c = RMSNorm(c_raw) * w_c;  head a: k_a = W_uk,a c, v_a = W_uv,a c
    score = (q_plain . k_a + q_rot . k_rot) * scale over the visible keys, softmax, out = W_o [heads' sum p v]

Only c and the rotated part are cached: one row [c | k_rot] a token (``KVNeed(values_in_keys=True)``: one kv head whose
values are a part of its key rows).  Attention runs in the latent space: a head's query becomes [W_uk,a^T q_plain |
q_rot], all heads attend to the same cached rows with the library's attention kernels (one kv head, head size rank +
rot rounded up to 16), and W_uv,a is applied to the attended latent afterwards, which gives the same numbers since
q_plain . (W_uk c) = (W_uk^T q_plain) . c and sum p (W_uv c) = W_uv (sum p c).
"""
from __future__ import annotations

import torch

from ..cache import KVNeed
from ..core import ConfigError, DType, Unsupported, torch_dtype
from ..csrc import ops
from .linear import linear
from .registry import part_class, register_part


class LatentAttention:
    """params: ``width``, ``n_heads``, ``head_dim`` (a head's plain query/key size), ``rot_dim`` (its rotated size),
    ``v_head_dim``, ``kv_rank`` (the latent's size), ``eps`` (of the latent's norm), ``scale``, ``window`` (None = all
    keys), ``position`` (``{"kind", "params"}`` of a position part over ``rot_dim`` dims).
    weights: ``q`` [n_heads*(head_dim+rot_dim), width], ``down`` [kv_rank+rot_dim, width], ``down_norm`` [kv_rank],
    ``up_k`` [n_heads*head_dim, kv_rank], ``up_v`` [n_heads*v_head_dim, kv_rank], ``o`` [width, n_heads*v_head_dim]."""

    graph_safe = True

    @classmethod
    def fused_weights(cls, params):
        """q and the down product read the same input: one matrix [q rows, down rows] for one product."""
        return {"q_down": ("q", "down")}

    @classmethod
    def weight_shapes(cls, params):
        d, nh = params["width"], params["n_heads"]
        hd, rd, vd, rank = params["head_dim"], params["rot_dim"], params["v_head_dim"], params["kv_rank"]
        return {"q": ((nh * (hd + rd), d), "matrix"), "down": ((rank + rd, d), "matrix"),
                "down_norm": ((rank,), "vector"), "up_k": ((nh * hd, rank), "matrix"),
                "up_v": ((nh * vd, rank), "matrix"), "o": ((d, nh * vd), "matrix")}

    def __init__(self, params, weights, dtype: DType, device):
        self.width = int(params["width"])
        self.n_heads = int(params["n_heads"])
        self.dim, self.rot = int(params["head_dim"]), int(params["rot_dim"])
        self.vdim, self.rank = int(params["v_head_dim"]), int(params["kv_rank"])
        self.eps = float(params.get("eps", 1e-6))
        self.window = params.get("window")
        self.scale = float(params["scale"])
        self.head_size = -(-(self.rank + self.rot) // 16) * 16  # what the attention kernels and the cache see
        if self.head_size > 1024:  # rows wider than 256 run on the kernel that takes any case, in both dtypes
            raise Unsupported(f"latent attention: kv_rank + rot_dim = {self.rank + self.rot} exceeds the attention "
                              f"kernels' widest row of 1024")
        if self.rot % 2:
            raise ConfigError(f"rot_dim {self.rot} must be even")
        self.w_q_down = weights.get("q_down")
        if self.w_q_down is None:
            self.w_q_down = torch.cat([weights["q"], weights["down"]], dim=0).contiguous()
        self.q_rows = self.n_heads * (self.dim + self.rot)
        self.w_q = self.w_q_down[: self.q_rows]
        self.down_norm = weights["down_norm"]
        # a head's W_uk transposed, [heads, rank, dim]: the product that carries the plain query into the latent space
        self.w_uk_t = weights["up_k"].reshape(self.n_heads, self.dim, self.rank).transpose(1, 2).contiguous()
        self.w_uv = weights["up_v"].reshape(self.n_heads, self.vdim, self.rank).contiguous()
        self.w_o = weights["o"]
        position = params.get("position") or {"kind": "none", "params": {}}
        self.position = part_class("position", position["kind"])(position.get("params", {}), {}, dtype, device)
        if self.rot and getattr(self.position, "rope_dim", 0) != self.rot:
            raise ConfigError(f"latent attention rotates rot_dim = {self.rot} dims; the position part gives "
                              f"{getattr(self.position, 'rope_dim', 0)}")
        self.dtype = dtype
        self.act_dtype = torch_dtype(dtype)

    def cache_need(self):
        return KVNeed(1, self.head_size, self.window, 0, values_in_keys=True)

    HEADS_A_PASS = 16  # the attention kernels serve up to 16 query heads a kv head: more heads go in several passes

    def attended(self, h, ctx, store, owns_cache=True):
        """The heads' values side by side in the compute dtype, [T, heads * v_head_dim]."""
        n = h.shape[0]
        qd = linear(h, self.w_q_down if owns_cache else self.w_q, out_dtype=torch.float32)
        out = torch.empty((n, self.n_heads * self.vdim), dtype=self.act_dtype, device=h.device)
        padded = sum(ctx.new_lens) < ctx.n_tokens
        window = int(self.window) if self.window else 0
        tables = self.position.tables(ctx)
        pairing = getattr(self.position, "pairing", "interleaved")
        for first in range(0, self.n_heads, self.HEADS_A_PASS):
            heads = min(self.HEADS_A_PASS, self.n_heads - first)
            q = torch.empty((n, heads * self.head_size), dtype=self.act_dtype, device=h.device)
            ops.latent_prepare(q, store.k, qd, self.q_rows, self.down_norm, self.eps, tables, ctx.tok_slot, ctx.tok_pos,
                               store.block_table, heads, self.dim, self.rot, self.rank, self.head_size,
                               write_cache=owns_cache and first == 0, pairing=pairing, first_head=first)
            # [W_uk^T q_plain] into the first `rank` columns of every head's query row
            ops.head_product(q, self.head_size, 0, qd, self.dim + self.rot, first * (self.dim + self.rot),
                             self.w_uk_t[first:first + heads], heads)
            latent = (torch.zeros if padded else torch.empty)(q.shape, dtype=self.act_dtype, device=h.device)
            done = False
            if self.dtype is DType.BF16:
                from . import attention_bf16
                done = attention_bf16.run(latent, q, ctx, store, heads, 1, self.head_size, self.scale, window)
            if not done:
                ops.attention_reference(latent, q, store.k, store.v, ctx.tok_slot, ctx.tok_pos, store.block_table, heads,
                                        1, self.head_size, self.scale, window)
            ops.head_product(out, self.vdim, first * self.vdim, latent, self.head_size, 0, self.w_uv[first:first + heads],
                             heads)
        return out

    def mix(self, h, ctx, store, owns_cache=True):
        """The mixer's result, float32 [T, width]."""
        ctx.then_norm = None
        return linear(self.attended(h, ctx, store, owns_cache), self.w_o, out_dtype=torch.float32)

    def forward(self, h, residual, ctx, store, owns_cache=True):
        ctx.then_norm = None
        linear(self.attended(h, ctx, store, owns_cache), self.w_o, accumulate_into=residual)


register_part("mixer", "latent_attention", LatentAttention)
