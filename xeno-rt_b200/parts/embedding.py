"""Token embedding and the output matrix."""
from __future__ import annotations

import torch

from ..csrc import ops
from .linear import linear
from .registry import register_part


class TokenEmbedding:
    """x = E[token], no scaling (crates/xrt-models/src/llama.rs:1042-1055); with ``scale`` x = E[token] * scale (32-bit).
    params: ``vocab_size``, ``width``, optional ``scale``.  weights: ``weight`` [vocab, width]."""

    graph_safe = True

    @classmethod
    def weight_shapes(cls, params):
        return {"weight": ((params["vocab_size"], params["width"]), "matrix")}

    def __init__(self, params, weights, dtype, device):
        self.vocab_size = int(params["vocab_size"])
        self.width = int(params["width"])
        self.weight = weights["weight"]
        self.scale = float(params.get("scale") or 1.0)

    def forward(self, token_ids, error_flag):
        out = torch.empty((token_ids.numel(), self.width), dtype=torch.float32, device=token_ids.device)
        ops.embedding(out, self.weight, token_ids, error_flag, self.scale)
        return out


class TokenPairEmbedding:
    """x = E[token] + P[(previous token * mul_prev + token * mul_cur) mod buckets]; a sequence's first token takes P's
    last row (number ``buckets``).  The previous token is state of the sequence (``state_need``): one int32 a slot,
    read by a step's first tokens and left holding the step's last.
    params: ``vocab_size``, ``width``, ``buckets``, ``mul_prev``, ``mul_cur``.
    weights: ``weight`` [vocab, width], ``pairs`` [buckets + 1, width]."""

    graph_safe = True

    @classmethod
    def weight_shapes(cls, params):
        return {"weight": ((params["vocab_size"], params["width"]), "matrix"),
                "pairs": ((params["buckets"] + 1, params["width"]), "matrix")}

    def __init__(self, params, weights, dtype, device):
        self.vocab_size = int(params["vocab_size"])
        self.width = int(params["width"])
        self.mul_prev, self.mul_cur = int(params["mul_prev"]), int(params["mul_cur"])
        self.weight, self.pairs = weights["weight"], weights["pairs"]

    def state_need(self):
        """(shape, dtype) of what the part keeps for every sequence."""
        return (), torch.int32

    def forward(self, token_ids, error_flag, ctx=None, state=None):
        out = torch.empty((token_ids.numel(), self.width), dtype=torch.float32, device=token_ids.device)
        ops.embedding_pair(out, self.weight, self.pairs, token_ids, ctx.tok_slot, ctx.tok_pos, state, ctx.cu_seqlens,
                           ctx.seq_slot, self.mul_prev, self.mul_cur, error_flag)
        return out


class OutputHead:
    """logits = W . normed, no scaling or cap (crates/xrt-models/src/llama.rs:604-613); W is the
    embedding when the model ties them (llama.rs:301-305), which the spec expresses by giving both
    parts the same tensor name.  params: ``vocab_size``, ``width``; optional ``scale`` (the logits are
    multiplied by it) and ``softcap`` (then logits <- softcap * tanh(logits / softcap)), both 32-bit.
    weights: ``weight``."""

    graph_safe = True

    @classmethod
    def weight_shapes(cls, params):
        return {"weight": ((params["vocab_size"], params["width"]), "matrix")}

    def __init__(self, params, weights, dtype, device):
        self.weight = weights["weight"]
        self.scale = float(params.get("scale") or 1.0)
        self.softcap = float(params["softcap"]) if params.get("softcap") else None

    def forward(self, normed):
        logits = linear(normed, self.weight, out_dtype=torch.float32)
        if self.scale != 1.0 or self.softcap is not None:
            ops.scale_softcap(logits, self.scale, self.softcap)
        return logits


register_part("embedding", "token", TokenEmbedding)
register_part("embedding", "token_pair", TokenPairEmbedding)
register_part("lm_head", "linear", OutputHead)
