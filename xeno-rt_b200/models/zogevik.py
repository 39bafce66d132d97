"""Zogevik: a decoder that norms what a sublayer gives, not what it reads: x <- x + RMSNorm(mixer(x)), then, where the
layer has a feed-forward, x <- x + RMSNorm(ff(x)); the embedding output is RMS-normed once before the first layer.
A layer's mixer is grouped-query attention ("attention": q and k RMS-normed over the whole projection, rotation of
split-half pairs over the first dims of a head, a score scale of its own, a window of the most recent keys, and a
softmax whose denominator holds one more term of score 0 that has no value; a layer may read the keys and values
that an earlier layer cached instead of making its own) or latent attention ("latent_attention": the keys and
values of all heads are read out of one small normed vector a token, one rotated key part of interleaved pairs is shared
by all heads; plain softmax over a window).  A feed-forward is a mixture of small two-matrix experts with the exact
gelu, routed by the softmax over all experts among the experts of the best groups.  The logits are the final RMSNorm
times the head matrix.

config.json keys: ``architecture`` "Zogevik", ``vocab``, ``width``, ``norm.eps``, ``layers`` (a list of ``{"type",
"mixer", "mlp"}``), ``max_positions`` (optional).  An attention mixer: ``heads``, ``kv_heads``, ``dim``, ``vdim``,
``scale``, ``rot`` (``dims``, ``base``), ``mask.size``, ``kv_from`` (optional: the layer whose keys and values it reads).
A latent mixer: ``heads``, ``dim``, ``rot_dim``, ``vdim``, ``kv_rank``, ``scale``, ``rot`` (``dims``, ``base``),
``mask.size``.  ``mlp``: null or ``{"kind": "moe", "expert": {"ff"}, "router": {"experts", "top", "groups": {"count",
"keep"}}}``.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass

from ..config import ModelConfig, register_architecture
from ..core import ConfigError
from ..parts import LayerSpec, ModelSpec, PartSpec, SchedulePlace
from .givopel import DEFAULT_MAX_POSITIONS, _positive, _positive_int

SINK_SCORE = 0.0  # the score of the denominator's extra term: exp(0) = 1 is added to the sum


def _check_window(problems, where, m):
    mask = m.get("mask")
    if mask is None:
        return
    if not isinstance(mask, dict):
        problems.append(f"{where}.mask must be an object with size")
    else:
        _positive_int(problems, where + ".mask", mask, "size")


def _check_rotation(problems, where, m, most: int, exactly: bool = False):
    rot = m.get("rot")
    if rot is None and not exactly:
        return
    dims = _positive_int(problems, where + ".rot", rot, "dims")
    _positive(problems, where + ".rot", rot, "base")
    if dims % 2 or dims > most or (exactly and dims != most):
        problems.append(f"{where}.rot.dims {dims} must be even and {'equal to' if exactly else 'at most'} {most}")


def _check_attention(problems, where, m, index: int, layers: list):
    heads, kv = _positive_int(problems, where, m, "heads"), _positive_int(problems, where, m, "kv_heads")
    dim = _positive_int(problems, where, m, "dim")
    _positive_int(problems, where, m, "vdim")
    _positive(problems, where, m, "scale")
    if heads % kv:
        problems.append(f"{where}: {heads} heads are not a multiple of {kv} kv_heads")
    _check_rotation(problems, where, m, dim)
    _check_window(problems, where, m)
    source = m.get("kv_from")
    if source is None:
        return
    if isinstance(source, bool) or not isinstance(source, int) or not 0 <= source < index:
        problems.append(f"{where}.kv_from {source!r} must name an earlier layer")
        return
    other = layers[source] if isinstance(layers[source], dict) else {}
    theirs = other.get("mixer")
    if other.get("type") != "attention" or not isinstance(theirs, dict) or theirs.get("kv_from") is not None:
        problems.append(f"{where}.kv_from: layer {source} is not an attention layer with keys and values of its own")
    elif any(theirs.get(key) != m.get(key) for key in ("kv_heads", "dim", "vdim")) or theirs.get("rot") != m.get("rot"):
        problems.append(f"{where}.kv_from: layer {source} differs in kv_heads, dim, vdim or rot")


def _check_latent(problems, where, m):
    for key in ("heads", "dim", "vdim", "kv_rank"):
        _positive_int(problems, where, m, key)
    rot_dim = _positive_int(problems, where, m, "rot_dim")
    _positive(problems, where, m, "scale")
    _check_rotation(problems, where, m, rot_dim, exactly=True)
    _check_window(problems, where, m)


def _check_mlp(problems, where, mlp):
    if not isinstance(mlp, dict) or mlp.get("kind") != "moe":
        problems.append(f"{where}.kind {mlp.get('kind') if isinstance(mlp, dict) else mlp!r} is not moe")
        return
    _positive_int(problems, where + ".expert", mlp.get("expert"), "ff")
    router = mlp.get("router")
    experts = _positive_int(problems, where + ".router", router, "experts")
    top = _positive_int(problems, where + ".router", router, "top")
    count, keep = 1, 1
    groups = router.get("groups") if isinstance(router, dict) else None
    if groups is not None:
        count = _positive_int(problems, where + ".router.groups", groups, "count")
        keep = _positive_int(problems, where + ".router.groups", groups, "keep")
    if experts % count or keep > count:
        problems.append(f"{where}.router: {experts} experts do not form {count} equal groups of which {keep} are kept")
    elif top > experts // count * keep:
        problems.append(f"{where}.router: top {top} exceeds the experts of the {keep} kept groups")


@dataclass(frozen=True)
class ZogevikConfig(ModelConfig):
    architecture: str
    vocab: int
    width: int
    layers: tuple          # of dicts as config.json writes them (checked)
    norm_eps: float
    max_positions: int
    eos_token_ids: tuple = ()

    @classmethod
    def from_dict(cls, raw: dict) -> "ZogevikConfig":
        problems: list[str] = []
        vocab = _positive_int(problems, "config", raw, "vocab")
        width = _positive_int(problems, "config", raw, "width")
        eps = _positive(problems, "norm", raw.get("norm"), "eps")
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            problems.append("'layers' must be a non-empty list")
            layers = []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict) or not isinstance(layer.get("mixer"), dict):
                problems.append(f"{where} must be an object with a 'mixer'")
                continue
            kind, m = layer.get("type"), layer["mixer"]
            if kind == "attention":
                _check_attention(problems, where + ".mixer", m, i, layers)
            elif kind == "latent_attention":
                _check_latent(problems, where + ".mixer", m)
            else:
                problems.append(f"{where}.type {kind!r} is not one of attention, latent_attention")
            if layer.get("mlp") is not None:
                _check_mlp(problems, where + ".mlp", layer["mlp"])
        max_positions = raw.get("max_positions", DEFAULT_MAX_POSITIONS)
        if isinstance(max_positions, bool) or not isinstance(max_positions, int) or max_positions <= 0:
            problems.append(f"max_positions must be a positive integer, got {max_positions!r}")
        if problems:
            raise ConfigError("config.json: " + "; ".join(problems))
        eos = raw.get("eos_token_id")
        eos = () if eos is None else ((eos,) if isinstance(eos, int) else tuple(eos))
        return cls(architecture="Zogevik", vocab=vocab, width=width, layers=tuple(copy.deepcopy(layers)), norm_eps=eps,
                   max_positions=max_positions, eos_token_ids=eos)

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "layers": copy.deepcopy(list(self.layers)), "norm": {"eps": self.norm_eps}}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out


def _norm(width, eps, name):
    return PartSpec("rmsnorm", {"width": width, "eps": eps}, {"weight": name})


def _rotation(m, pairing: str):
    rot = m.get("rot")
    if not rot:
        return {"kind": "none", "params": {}}
    # angle = position * base^(-2i / dims): the frequencies once in 64-bit, the step's angles as 32-bit products
    return {"kind": "blended_rotary", "params": {"rope_dim": rot["dims"], "base": rot["base"], "pairing": pairing,
                                                 "scaling": None}}


def _window(m):
    return (m.get("mask") or {}).get("size")


def _attention_spec(width, eps, m, prefix):
    own = m.get("kv_from") is None
    params = {"width": width, "n_heads": m["heads"], "n_kv_heads": m["kv_heads"], "head_dim": m["dim"],
              "v_head_dim": m["vdim"], "qk_norm": "whole", "eps": eps, "window": _window(m), "scale": m["scale"],
              "sink": SINK_SCORE, "own_kv": own, "position": _rotation(m, "split_half")}
    names = {"q": prefix + "q", "o": prefix + "o", "q_norm": prefix + "q.norm"}
    if own:
        names.update({"k": prefix + "k", "v": prefix + "v", "k_norm": prefix + "k.norm"})
    return PartSpec("attention", params, names)


def _latent_spec(width, eps, m, prefix):
    params = {"width": width, "n_heads": m["heads"], "head_dim": m["dim"], "rot_dim": m["rot_dim"],
              "v_head_dim": m["vdim"], "kv_rank": m["kv_rank"], "eps": eps, "window": _window(m), "scale": m["scale"],
              "position": _rotation(m, "interleaved")}
    names = {"q": prefix + "q", "down": prefix + "dkv", "down_norm": prefix + "dkv.norm", "up_k": prefix + "uk",
             "up_v": prefix + "uv", "o": prefix + "o"}
    return PartSpec("latent_attention", params, names)


def _experts_spec(width, mlp, prefix):
    router = mlp["router"]
    groups = router.get("groups") or {"count": 1, "keep": 1}
    n = router["experts"]
    names = {"router": prefix + "router"}
    for i in range(n):
        names.update({f"up{i}": f"{prefix}e{i}.up", f"down{i}": f"{prefix}e{i}.down"})
    return PartSpec("routed_experts", {"width": width, "inner": mlp["expert"]["ff"], "experts": n, "top": router["top"],
                                       "activation": "gelu", "routing": "scores", "groups": groups["count"],
                                       "keep_groups": groups["keep"], "router_bias": False}, names)


def build_spec(cfg: ZogevikConfig) -> ModelSpec:
    d, eps = cfg.width, cfg.norm_eps
    layers, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer["mixer"]
        mixer = (_attention_spec if layer["type"] == "attention" else _latent_spec)(d, eps, m, p + "mix.")
        parts = {"mixer": ("mixer", mixer), "mixer_post": ("norm", _norm(d, eps, p + "norm1"))}
        if layer.get("mlp"):
            parts.update({"ffn": ("feed_forward", _experts_spec(d, layer["mlp"], p + "mlp.")),
                          "ffn_post": ("norm", _norm(d, eps, p + "norm2"))})
        layers.append(LayerSpec(parts, "postnorm_residual"))
        # a layer that reads another's keys and values is a place that reads that place's cache (places = layers here)
        schedule.append(SchedulePlace(i, cache_from=m.get("kv_from") if layer["type"] == "attention" else None,
                                      before="embed_norm" if i == 0 else None))
    return ModelSpec(
        vocab_size=cfg.vocab, hidden_size=d, max_positions=cfg.max_positions,
        embedding=PartSpec("token", {"vocab_size": cfg.vocab, "width": d}, {"weight": "embed"}),
        layers=layers, schedule=schedule, final_norm=_norm(d, eps, "final.norm"),
        lm_head=PartSpec("linear", {"vocab_size": cfg.vocab, "width": d}, {"weight": "head"}),
        stop_ids=tuple(cfg.eos_token_ids),
        ignorable_tensors=tuple(f"l{i}.norm2" for i, layer in enumerate(cfg.layers) if not layer.get("mlp")),
        stream_parts={"embed_norm": PartSpec("rmsnorm", {"width": d, "eps": eps}, {"weight": "embed.norm"})})


register_architecture("Zogevik", ZogevikConfig, build_spec)
