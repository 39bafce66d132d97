"""Rotary position encoding.

The divisor table f_i = base^(2i / rope_dim) is computed once in float32 as the reference does
(crates/xrt-kernels/src/cpu/rope.rs:10-16); each step computes (cos, sin) of
pos * scale / f_i in 32-bit for the step's tokens (rope.rs:59-68).  The rotation itself is applied
by the attention mixer's fused kernel from this table, so any encoding that is a rotation of pairs
of a head's dims by position-dependent angles fits this interface by returning another table.  A
position part says which dims pair up with ``pairing``: "split_half" (i with i + rope_dim / 2, the
reference's and the default, rope.rs:19-35) or "interleaved" (2i with 2i + 1); dims from rope_dim on
stay as they are (rope.rs:19-35 rotates ``rope_dim`` dims of each head only).
"""
from __future__ import annotations

import numpy as np
import torch

from ..core import ConfigError
from ..csrc import ops
from .registry import register_part


class RotaryEncoding:
    """params: ``rope_dim`` (even, at most the head size), ``base``, ``scale`` (multiplies the
    position), ``pairing`` ("split_half" or "interleaved").  No weights."""

    @classmethod
    def weight_shapes(cls, params):
        return {}

    def __init__(self, params, weights, dtype, device):
        self.rope_dim = int(params["rope_dim"])
        self.base = float(params["base"])
        self.scale = float(params.get("scale", 1.0))
        self.pairing = str(params.get("pairing", "split_half"))
        if self.rope_dim <= 0 or self.rope_dim % 2:
            raise ConfigError(f"rope_dim {self.rope_dim} must be a positive even number")
        if self.pairing not in ("split_half", "interleaved"):
            raise ConfigError(f"pairing {self.pairing!r} is not split_half or interleaved")
        self.half = self.rope_dim // 2
        i = np.arange(self.half, dtype=np.float32)
        freq = np.power(np.float32(self.base), (np.float32(2.0) * i) / np.float32(self.rope_dim)).astype(np.float32)
        self.freq = torch.from_numpy(freq).to(device)
        self._key = ("rotary", self.rope_dim, self.base, self.scale)

    def tables(self, ctx):
        """(cos, sin) float32 [T, half, 2] for the tokens of the step; computed once a step."""
        table = ctx.shared.get(self._key)
        if table is None:
            table = torch.empty((ctx.n_tokens, self.half, 2), dtype=torch.float32, device=self.freq.device)
            ops.rope_table(table, ctx.tok_pos, self.freq, self.scale)
            ctx.shared[self._key] = table
        return table


class BlendedRotaryEncoding:
    """Rotary encoding whose frequencies are blended between the plain ones and ones divided by a factor
    (the scaling known as YaRN): with f_i = base^(-2i / rope_dim) and
    d(t) = rope_dim * ln(original / (2 pi t)) / (2 ln base), the dims below d(fast) keep f_i, the dims
    above d(slow) turn at f_i / factor, and those in between move linearly from one to the other:
    ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), lo = max(floor(d(fast)), 0),
    hi = min(ceil(d(slow)), rope_dim - 1); cos and sin are multiplied by 0.1 ln(factor) + 1.
    params: ``rope_dim``, ``base``, ``pairing``, and ``scaling`` = None or a dict with ``factor``,
    ``original`` (positions the frequencies were made for), ``fast`` and ``slow`` (turns over those
    positions); ``divide`` (optional, a number: every frequency is divided by it, the scaling known as linear or
    position interpolation; with ``scaling`` it applies first).  No weights.  The frequencies are worked out once in float64 and kept as two 32-bit
    terms; a step's angles are 32-bit products of position and frequency whose rounding error is carried along, so
    that far positions turn as exactly as near ones."""

    @classmethod
    def weight_shapes(cls, params):
        return {}

    def __init__(self, params, weights, dtype, device):
        import math
        self.rope_dim = int(params["rope_dim"])
        self.base = float(params["base"])
        self.pairing = str(params.get("pairing", "interleaved"))
        if self.rope_dim <= 0 or self.rope_dim % 2:
            raise ConfigError(f"rope_dim {self.rope_dim} must be a positive even number")
        if self.pairing not in ("split_half", "interleaved"):
            raise ConfigError(f"pairing {self.pairing!r} is not split_half or interleaved")
        if not self.base > 1.0:
            raise ConfigError(f"rotary base {self.base} must be above 1")
        self.half = self.rope_dim // 2
        i = np.arange(self.half, dtype=np.float64)
        freq = np.power(self.base, -2.0 * i / self.rope_dim)
        divide = float(params.get("divide") or 1.0)
        if not divide > 0:
            raise ConfigError(f"rotary divide {divide} must be positive")
        freq = freq / divide
        self.magnitude = 1.0
        scaling = params.get("scaling")
        if scaling:
            factor, original = float(scaling["factor"]), float(scaling["original"])
            if not (factor > 0 and original > 0 and float(scaling["fast"]) > 0 and float(scaling["slow"]) > 0):
                raise ConfigError(f"rotary scaling {scaling!r}: factor, original, fast and slow must be positive")
            where = lambda turns: self.rope_dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.base))
            lo = max(math.floor(where(float(scaling["fast"]))), 0)
            hi = min(math.ceil(where(float(scaling["slow"]))), self.rope_dim - 1)
            ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
            freq = freq / factor * ramp + freq * (1.0 - ramp)
            self.magnitude = 0.1 * math.log(factor) + 1.0
        self.freq = torch.from_numpy(freq.astype(np.float32)).to(device)
        # what the 32-bit frequency lost: the table kernel carries it, and its product's rounding error, into the angle
        self.freq_lo = torch.from_numpy((freq - freq.astype(np.float32).astype(np.float64)).astype(np.float32)).to(device)
        self._key = ("blended_rotary", self.rope_dim, self.base, divide, repr(sorted((scaling or {}).items())))

    def tables(self, ctx):
        """magnitude * (cos, sin) float32 [T, half, 2] for the tokens of the step; computed once a step."""
        table = ctx.shared.get(self._key)
        if table is None:
            table = torch.empty((ctx.n_tokens, self.half, 2), dtype=torch.float32, device=self.freq.device)
            ops.rotation_table(table, ctx.tok_pos, self.freq, self.magnitude, freq_lo=self.freq_lo)
            ctx.shared[self._key] = table
        return table


class NoPositionEncoding:
    """Leaves q and k as they are."""

    pairing = "split_half"

    @classmethod
    def weight_shapes(cls, params):
        return {}

    def __init__(self, params, weights, dtype, device):
        pass

    def tables(self, ctx):
        return None


register_part("position", "rotary", RotaryEncoding)
register_part("position", "none", NoPositionEncoding)
register_part("position", "blended_rotary", BlendedRotaryEncoding)
