"""Arrangements: how the parts of one layer are put together around the residual stream."""
from __future__ import annotations

import torch

from ..csrc import ops
from .registry import register_part


class LayerParts:
    """The built parts of one layer by the names its ``LayerSpec`` gave them: ``parts.mixer`` or
    ``parts["mixer"]``; ``parts.names()`` in the spec's order; ``parts.role(name)``."""

    def __init__(self, parts: dict, roles: dict | None = None):
        self._parts = dict(parts)
        self._roles = dict(roles or {})

    def __getattr__(self, name):
        try:
            return self.__dict__["_parts"][name]
        except KeyError:
            raise AttributeError(f"the layer has no part named {name!r}; it has {list(self.__dict__['_parts'])}") from None

    def __getitem__(self, name):
        return self._parts[name]

    def __contains__(self, name) -> bool:
        return name in self._parts

    def names(self) -> list:
        return list(self._parts)

    def role(self, name: str) -> str:
        return self._roles.get(name, "")

    def values(self):
        return self._parts.values()


def prenorm_residual(parts: LayerParts, x, ctx, stores, owns_cache: bool) -> None:
    """x += mixer(norm(x)); x += feed_forward(norm(x))   (crates/xrt-models/src/llama.rs:433-602).
    ``x`` is the float32 residual stream and is updated in place; the sums are 32-bit.  ``stores``
    maps a part's name to the cache storage it asked for."""
    h = ctx.take_pending(parts.mixer_norm)  # the layer before may have prepared this layer's first norm
    if h is None:
        h = parts.mixer_norm.forward(x)
    ctx.then_norm = _norm_that_can_wait(parts.ffn_norm, parts.ffn, ctx, x)
    parts.mixer.forward(h, x, ctx, stores.get("mixer"), owns_cache)
    h = ctx.take_pending(parts.ffn_norm)
    if h is None:
        h = parts.ffn_norm.forward(x)
    after = ctx.shared.get("next_layer")  # (norm, the part that takes its result) of the layer that runs next
    ctx.then_norm = _norm_that_can_wait(after[0], after[1], ctx, x) if after else None
    parts.ffn.forward(h, x, ctx)


def _norm_that_can_wait(norm, consumer, ctx, x):
    """``norm`` if the part that adds into the residual before it may prepare it (so that no norm
    kernel runs in between): the part that takes the norm's result must say that it can finish it."""
    can = getattr(consumer, "takes_pending_norm", None)
    return norm if can is not None and can(ctx.n_tokens, x.device) else None


def parallel_residual(parts: LayerParts, x, ctx, stores, owns_cache: bool) -> None:
    """x += mixer(norm(x)) + feed_forward(norm(x)): ONE norm whose result both read.  The layer's parts are
    ``norm``, ``mixer`` and, if it has one, ``ffn``.  Each adds its result into the 32-bit stream."""
    ctx.then_norm = ctx.pending = None
    h = parts.norm.forward(x)
    parts.mixer.forward(h, x, ctx, stores.get("mixer"), owns_cache)
    ctx.then_norm = ctx.pending = None
    if "ffn" in parts:
        parts.ffn.forward(h, x, ctx)
        ctx.then_norm = ctx.pending = None


def sandwich_residual(parts: LayerParts, x, ctx, stores, owns_cache: bool) -> None:
    """x += post_norm(mixer(norm(x))); x += post_norm(feed_forward(norm(x))): a norm before and after each sublayer.
    The layer's parts are ``mixer_norm``, ``mixer``, ``mixer_post`` and, if it has a feed-forward, ``ffn_norm``,
    ``ffn``, ``ffn_post``.  The mixer hands its result back (``mix``), the feed-forward too (``apply``: [T, width] or
    [parts, T, width] float32), and the norm after it adds into the 32-bit stream (``add_into``).
    The norm after a sublayer also computes the norm that the next sublayer begins with, in the same pass over the
    row (its own feed-forward's, or the first norm of the layer that runs next, left in ``ctx.pending``).
    A layer may have a part ``mixer_shift`` (role ``shift``): the mixer then reads its norm blended with that of the
    token before; such a layer's first norm is never prepared by the layer before it."""
    ready = ctx.take_pending(parts.mixer_norm)
    after = ctx.shared.get("next_layer")  # (first norm, the part that takes it) of the layer that runs next, or None
    if after is not None and len(after) > 2 and "mixer_shift" in after[2]:
        after = None  # that layer's first norm is blended with the token before: it runs it itself
    if "mixer_shift" in parts:
        h = parts.mixer_shift.forward(x, parts.mixer_norm, ctx, stores.get("mixer_shift"), owns_cache)
    else:
        h = ready.value if ready is not None else parts.mixer_norm.forward(x)
    has_ffn = "ffn" in parts
    following = parts.ffn_norm if has_ffn else (after[0] if after else None)
    h = parts.mixer_post.add_into(x, parts.mixer.mix(h, ctx, stores.get("mixer"), owns_cache), then=following)
    ctx.then_norm = ctx.pending = None
    if has_ffn:
        if h is None:
            h = parts.ffn_norm.forward(x)
        following = after[0] if after else None
        h = parts.ffn_post.add_into(x, parts.ffn.apply(h, ctx), then=following)
    if h is not None:
        ctx.pending = ReadyNorm(following, h)


def postnorm_residual(parts: LayerParts, x, ctx, stores, owns_cache: bool) -> None:
    """x += norm(mixer(x)); x += norm(feed_forward(x)): the sublayers read the residual stream itself and only what
    they give is normed.  The layer's parts are ``mixer``, ``mixer_post`` and, if it has a feed-forward, ``ffn`` and
    ``ffn_post``.  The mixer hands its result back (``mix``), the feed-forward too (``apply``: [T, width] or [parts, T,
    width] float32), and the norm after adds into the 32-bit stream (``add_into``).  In a 16-bit compute dtype the
    sublayers' products read a rounded copy of the stream, which the adding norm writes in the same pass (left in
    ``ctx.pending`` for the layer that runs next); only a layer that finds none there rounds the stream itself."""
    ready, ctx.pending, ctx.then_norm = ctx.pending, None, None
    rounds = parts.mixer_post.out_dtype != torch.float32
    if not rounds:
        h = x
    elif isinstance(ready, StreamCopy) and ready.of is x:
        h = ready.value
    else:
        h = torch.empty(x.shape, dtype=parts.mixer_post.out_dtype, device=x.device)
        ops.cast_rows(h, x)
    has_ffn = "ffn" in parts
    follows = ctx.shared.get("next_layer_reads_stream", False)
    h = parts.mixer_post.add_into(x, parts.mixer.mix(h, ctx, stores.get("mixer"), owns_cache),
                                  copy=rounds and (has_ffn or follows))
    ctx.then_norm = ctx.pending = None
    if has_ffn:
        h = parts.ffn_post.add_into(x, parts.ffn.apply(x if not rounds else h, ctx), copy=rounds and follows)
    if rounds and h is not None:
        ctx.pending = StreamCopy(x, h)


class StreamCopy:
    """The residual stream ``of`` rounded to the compute dtype by the part that wrote it last."""

    def __init__(self, of, value):
        self.of, self.value = of, value
        self.norm = None  # it stands for no norm: arrangements that look for a prepared norm pass it by


postnorm_residual.reads_stream = True
register_part("arrangement", "postnorm_residual", postnorm_residual)


class ReadyNorm:
    """A norm's finished result that the part before it computed on its way: ``norm`` is the part it stands for."""

    def __init__(self, norm, value):
        self.norm, self.value = norm, value


sandwich_residual.first_norm = lambda parts: (parts.mixer_norm, parts.mixer, parts)
register_part("arrangement", "parallel_residual", parallel_residual)
register_part("arrangement", "sandwich_residual", sandwich_residual)


# what a layer of this arrangement begins with: the norm it applies to the residual stream first, and the
# part that takes that norm's result
prenorm_residual.first_norm = lambda parts: (parts.mixer_norm, parts.mixer)
register_part("arrangement", "prenorm_residual", prenorm_residual)
