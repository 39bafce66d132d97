"""Token shift (role ``shift``): what a mixer reads is blended, channel by channel, with what it read for the token
before, h_t <- h_t + (h_(t-1) - h_t) * s with h the layer's first norm of the stream and zeros before a sequence's
first token.  The token before a step's first token is state of the sequence: one float32 row a slot and place
(``cache_need``), zero when the slot opens.  Norm and blend are one kernel (csrc/token_shift.cu), 32-bit up to the
rounding of the result to the compute dtype."""
from __future__ import annotations

import torch

from ..cache import StateNeed
from ..core import ConfigError, torch_dtype
from ..csrc import ops
from .registry import register_part


class TokenShift:
    """params: ``width``.  weights: ``weight`` [width], the share of the token before in every channel.
    ``forward(x, norm, ctx, store)``: ``norm`` is the RMSNorm part whose result is shifted."""

    graph_safe = True

    @classmethod
    def weight_shapes(cls, params):
        return {"weight": ((params["width"],), "vector")}

    def __init__(self, params, weights, dtype, device):
        self.width = int(params["width"])
        self.shift = weights["weight"].to(torch.float32).contiguous()
        self.out_dtype = torch_dtype(dtype)

    def cache_need(self):
        return StateNeed((self.width,), "float32")

    def forward(self, x, norm, ctx, store, owns_cache=True):
        if not owns_cache:
            raise ConfigError("a token shift cannot read another place's state: it is what the tokens left there")
        out = torch.empty((x.shape[0], self.width), dtype=self.out_dtype, device=x.device)
        ops.rmsnorm_shift(out, x, norm.weight, self.shift, store.state,
                          (ctx.tok_slot, ctx.tok_pos, ctx.cu_seqlens, ctx.seq_slot), norm.eps,
                          single_tokens=ctx.max_new == 1)
        return out


register_part("shift", "token_shift", TokenShift)
