"""Sofunex: a decoder whose layers norm every sublayer before and after it and scale what they add,
x <- x + m * RMSNorm(mixer(shift(RMSNorm(x)))), then, where the layer has a feed-forward, x <- x + m * RMSNorm(ff(RMSNorm(x))).
``shift`` blends what the mixer reads with what it read for the token before, channel by channel.  The mixer
("parallel") is two mixers side by side that read the same input and are added with a weight each: grouped-query
attention (biases on q, k, v and o; a short causal convolution over time on every channel of q, k and v; q and k
RMS-normed over the whole projection; a rotation of split-half pairs over the first dims of a head whose frequencies
are divided by a factor; values divided by their root mean square a head; a score scale of its own; a window of the
most recent keys), and a delta rule with a decay and a removal rate per key channel (``parts/state_mixers.py:
DecayRemovalRule``).  A feed-forward is dense (gated, tanh gelu) or a mixture of gated silu experts routed by sigmoid
scores: a correction that only the choice sees, groups that count by their two best experts, weights that sum to a
scale, and a shared expert.  The embedding is multiplied by a number.  A stretch of layers (``loop``) runs several
times in a row with the same weights and a cache of its own each time; every pass begins by adding a row of
``loop.step`` to the stream.  The logits are the final RMSNorm times the head matrix.

config.json keys: ``architecture`` "Sofunex", ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``,
``residual_mult``, ``layers`` (a list of ``{"type": "parallel", "mixer", "mlp"}``), ``loop`` (``start``, ``stop``,
``times``; optional), ``max_positions`` (optional).  A mixer: ``left`` (``heads``, ``kv_heads``, ``dim``, ``vdim``,
``scale``, optional ``conv`` (taps), ``rot`` (``dims``, ``base``, optional ``scaling.factor``), ``mask.size``), ``right``
(``heads``, ``dim``), ``left_scale``, ``right_scale``.  ``mlp``: null, ``{"kind": "dense", "ff"}`` or ``{"kind": "moe",
"expert": {"ff"}, "router": {"experts", "top", "scale", "groups": {"count", "keep"}}, "shared": {"ff"}}`` (groups and
shared optional).  The rank of the decay's low-rank product is a size of tensors only: it is read from the model
file's shapes at load, or from the optional key ``decay_rank`` of ``right`` where there is no file (random weights).
"""
from __future__ import annotations

import copy
import dataclasses
import math
from dataclasses import dataclass

from ..config import ModelConfig, register_architecture
from ..core import ConfigError
from ..parts import LayerSpec, ModelSpec, PartSpec, SchedulePlace
from .givopel import DEFAULT_MAX_POSITIONS, _positive, _positive_int
from .zogevik import _check_window

# constants that the design fixes
DECAY_RATE = math.exp(-0.5)  # the decay of a key channel is exp(-DECAY_RATE * sigmoid(.))
UNIT_KEY_EPS = 1e-6          # inside the root of the delta rule's unit key
WEIGHT_SUM_EPS = 1e-20       # added to the sum of the chosen experts' scores
GROUP_BEST = 2               # a group of experts counts by the sum of so many of its largest choice scores


def _check_left(problems, where, m):
    heads, kv = _positive_int(problems, where, m, "heads"), _positive_int(problems, where, m, "kv_heads")
    dim = _positive_int(problems, where, m, "dim")
    _positive_int(problems, where, m, "vdim")
    _positive(problems, where, m, "scale")
    if heads % kv:
        problems.append(f"{where}: {heads} heads are not a multiple of {kv} kv_heads")
    if m.get("conv") not in (None, 0) or isinstance(m.get("conv"), bool):  # no key, null and 0 all mean no convolution
        _positive_int(problems, where, m, "conv")
    rot = m.get("rot")
    if rot is not None:
        dims = _positive_int(problems, where + ".rot", rot, "dims")
        _positive(problems, where + ".rot", rot, "base")
        if dims % 2 or dims > dim:
            problems.append(f"{where}.rot.dims {dims} must be even and at most dim {dim}")
        scaling = rot.get("scaling") if isinstance(rot, dict) else None
        if scaling is not None:
            _positive(problems, where + ".rot.scaling", scaling, "factor")
    _check_window(problems, where, m)


def _check_right(problems, where, m):
    _positive_int(problems, where, m, "heads")
    _positive_int(problems, where, m, "dim")
    if m.get("decay_rank") is not None:
        _positive_int(problems, where, m, "decay_rank")


def _check_mlp(problems, where, mlp):
    kind = mlp.get("kind") if isinstance(mlp, dict) else None
    if kind == "dense":
        _positive_int(problems, where, mlp, "ff")
        return
    if kind != "moe":
        problems.append(f"{where}.kind {kind!r} is not one of dense, moe")
        return
    _positive_int(problems, where + ".expert", mlp.get("expert"), "ff")
    router = mlp.get("router")
    experts = _positive_int(problems, where + ".router", router, "experts")
    top = _positive_int(problems, where + ".router", router, "top")
    _positive(problems, where + ".router", router, "scale")
    count, keep = 1, 1
    groups = router.get("groups") if isinstance(router, dict) else None
    if groups is not None:
        count = _positive_int(problems, where + ".router.groups", groups, "count")
        keep = _positive_int(problems, where + ".router.groups", groups, "keep")
    if experts % count or keep > count:
        problems.append(f"{where}.router: {experts} experts do not form {count} equal groups of which {keep} are kept")
    elif top > experts // count * keep:
        problems.append(f"{where}.router: top {top} exceeds the experts of the {keep} kept groups")
    if mlp.get("shared") is not None:
        _positive_int(problems, where + ".shared", mlp.get("shared"), "ff")


@dataclass(frozen=True)
class SofunexConfig(ModelConfig):
    architecture: str
    vocab: int
    width: int
    layers: tuple          # of dicts as config.json writes them (checked)
    loop: tuple | None     # (start, stop, times)
    norm_eps: float
    embedding_scale: float
    residual_mult: float
    max_positions: int
    eos_token_ids: tuple = ()

    @classmethod
    def from_dict(cls, raw: dict) -> "SofunexConfig":
        problems: list[str] = []
        vocab = _positive_int(problems, "config", raw, "vocab")
        width = _positive_int(problems, "config", raw, "width")
        eps = _positive(problems, "norm", raw.get("norm"), "eps")
        scale = (raw.get("embedding") or {}).get("scale", 1.0) if isinstance(raw.get("embedding", {}), dict) else None
        if isinstance(scale, bool) or not isinstance(scale, (int, float)) or scale == 0:
            problems.append(f"embedding.scale must be a number other than 0, got {scale!r}")
        mult = raw.get("residual_mult", 1.0)
        if isinstance(mult, bool) or not isinstance(mult, (int, float)) or mult == 0:
            problems.append(f"residual_mult must be a number other than 0, got {mult!r}")
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            problems.append("'layers' must be a non-empty list")
            layers = []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict) or not isinstance(layer.get("mixer"), dict):
                problems.append(f"{where} must be an object with a 'mixer'")
                continue
            m = layer["mixer"]
            if layer.get("type") != "parallel":
                problems.append(f"{where}.type {layer.get('type')!r} is not parallel")
                continue
            for side, check in (("left", _check_left), ("right", _check_right)):
                if not isinstance(m.get(side), dict):
                    problems.append(f"{where}.mixer.{side} is missing")
                else:
                    check(problems, f"{where}.mixer.{side}", m[side])
                weight = m.get(side + "_scale", 1.0)
                if isinstance(weight, bool) or not isinstance(weight, (int, float)):
                    problems.append(f"{where}.mixer.{side}_scale must be a number, got {weight!r}")
            if layer.get("mlp") is not None:
                _check_mlp(problems, where + ".mlp", layer["mlp"])
        loop = raw.get("loop")
        if loop is not None:
            start, stop, times = (loop.get(k) if isinstance(loop, dict) else None for k in ("start", "stop", "times"))
            ok = all(isinstance(v, int) and not isinstance(v, bool) for v in (start, stop, times))
            if not ok or not (0 <= start < stop <= len(layers)) or times < 1:
                problems.append(f"loop {loop!r} must give 0 <= start < stop <= {len(layers)} layers and times >= 1")
                loop = None
            else:
                loop = (start, stop, times)
        max_positions = raw.get("max_positions", DEFAULT_MAX_POSITIONS)
        if isinstance(max_positions, bool) or not isinstance(max_positions, int) or max_positions <= 0:
            problems.append(f"max_positions must be a positive integer, got {max_positions!r}")
        if problems:
            raise ConfigError("config.json: " + "; ".join(problems))
        eos = raw.get("eos_token_id")
        eos = () if eos is None else ((eos,) if isinstance(eos, int) else tuple(eos))
        return cls(architecture="Sofunex", vocab=vocab, width=width, layers=tuple(copy.deepcopy(layers)), loop=loop,
                   norm_eps=eps, embedding_scale=float(scale), residual_mult=float(mult), max_positions=max_positions,
                   eos_token_ids=eos)

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "layers": copy.deepcopy(list(self.layers)), "norm": {"eps": self.norm_eps},
               "embedding": {"scale": self.embedding_scale}, "residual_mult": self.residual_mult}
        if self.loop is not None:
            out["loop"] = dict(zip(("start", "stop", "times"), self.loop))
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out

    def with_tensor_shapes(self, shapes: dict) -> "SofunexConfig":
        """The same configuration with the size that only tensors give (the rank of the decay's low-rank product)
        taken from ``shapes`` ({tensor name: shape}) wherever the configuration does not name it."""
        layers = copy.deepcopy(list(self.layers))
        for i, layer in enumerate(layers):
            right = layer["mixer"]["right"]
            shape = shapes.get(f"l{i}.mix.right.w1")
            if "decay_rank" not in right and shape is not None and len(shape) == 2:
                right["decay_rank"] = int(shape[0])
        return dataclasses.replace(self, layers=tuple(layers))

    def order(self) -> list:
        """[(layer, the number of the pass that begins with it, or None)] in the order the layers run."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, None) for i in range(n)]
        start, stop, times = self.loop
        order = [(i, None) for i in range(start)]
        for t in range(times):
            order += [(i, t if i == start else None) for i in range(start, stop)]
        return order + [(i, None) for i in range(stop, n)]


def _norm(width, eps, name, gain=None):
    params = {"width": width, "eps": eps}
    if gain is not None:
        params["gain"] = gain
    return PartSpec("rmsnorm", params, {"weight": name})


def _left(width, eps, m, prefix):
    position = {"kind": "none", "params": {}}
    if m.get("rot"):
        rot = m["rot"]
        position = {"kind": "blended_rotary", "params": {
            "rope_dim": rot["dims"], "base": rot["base"], "pairing": "split_half", "scaling": None,
            "divide": (rot.get("scaling") or {}).get("factor", 1.0)}}
    params = {"width": width, "n_heads": m["heads"], "n_kv_heads": m["kv_heads"], "head_dim": m["dim"],
              "v_head_dim": m["vdim"], "qk_norm": "whole", "eps": eps, "window": (m.get("mask") or {}).get("size"),
              "scale": m["scale"], "bias": True, "o_bias": True, "conv": m.get("conv") or None, "v_norm": "unit",
              "position": position}
    names = {"q": prefix + "q", "k": prefix + "k", "v": prefix + "v", "o": prefix + "o", "q_norm": prefix + "q.norm",
             "k_norm": prefix + "k.norm", "q_bias": prefix + "q.b", "k_bias": prefix + "k.b", "v_bias": prefix + "v.b",
             "o_bias": prefix + "o.b"}
    if m.get("conv"):
        names.update({"q_conv": prefix + "q.conv", "k_conv": prefix + "k.conv", "v_conv": prefix + "v.conv"})
    return "attention", params, names


def _right(width, eps, m, prefix):
    if "decay_rank" not in m:
        raise ConfigError(f"{prefix}w1: decay_rank is not known: it is neither in the configuration nor in a model "
                          f"file's shapes")
    params = {"width": width, "n_heads": m["heads"], "dim": m["dim"], "decay_rank": int(m["decay_rank"]), "eps": eps,
              "decay_rate": DECAY_RATE, "unit_eps": UNIT_KEY_EPS}
    names = {r: prefix + r for r in ("r", "k", "v", "g", "a", "w1", "w2", "w0", "norm", "o")}
    names["a_bias"] = prefix + "a.b"
    return "decay_removal_rule", params, names


def _feed_forward(width, mlp, prefix):
    if mlp["kind"] == "dense":
        return PartSpec("swiglu", {"width": width, "inner": mlp["ff"], "activation": "gelu_tanh"},
                        {r: prefix + r for r in ("gate", "up", "down")})
    router = mlp["router"]
    groups = router.get("groups") or {"count": 1, "keep": 1}
    n = router["experts"]
    names = {"router": prefix + "router", "correction": prefix + "correction"}
    for i in range(n):
        names.update({f"gate{i}": f"{prefix}e{i}.gate", f"up{i}": f"{prefix}e{i}.up", f"down{i}": f"{prefix}e{i}.down"})
    params = {"width": width, "inner": mlp["expert"]["ff"], "experts": n, "top": router["top"],
              "activation": "gated_silu", "routing": "scores", "scores": "sigmoid", "correction": True,
              "groups": groups["count"], "keep_groups": groups["keep"], "group_best": GROUP_BEST, "normalize": True,
              "sum_eps": WEIGHT_SUM_EPS, "weight_scale": router["scale"], "router_bias": False}
    if mlp.get("shared"):
        params["shared"] = mlp["shared"]["ff"]
        names.update({"shared_" + r: f"{prefix}shared.{r}" for r in ("gate", "up", "down")})
    return PartSpec("routed_experts", params, names)


def build_spec(cfg: SofunexConfig) -> ModelSpec:
    d, eps, mult = cfg.width, cfg.norm_eps, cfg.residual_mult
    layers = []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer["mixer"]
        branches, names = [], {}
        for side, make in (("left", _left), ("right", _right)):
            kind, params, own = make(d, eps, m[side], f"{p}mix.{side}.")
            branches.append({"name": side, "kind": kind, "params": params, "scale": m.get(side + "_scale", 1.0)})
            names.update({f"{side}.{role}": tensor for role, tensor in own.items()})
        mixer = PartSpec("side_by_side", {"width": d, "combine": "weighted", "branches": branches}, names)
        parts = {"mixer_norm": ("norm", _norm(d, eps, p + "norm1")),
                 "mixer_shift": ("shift", PartSpec("token_shift", {"width": d}, {"weight": p + "shift"})),
                 "mixer": ("mixer", mixer),
                 "mixer_post": ("norm", _norm(d, eps, p + "norm1b", mult))}
        if layer.get("mlp"):
            parts.update({"ffn_norm": ("norm", _norm(d, eps, p + "norm2")),
                          "ffn": ("feed_forward", _feed_forward(d, layer["mlp"], p + "mlp.")),
                          "ffn_post": ("norm", _norm(d, eps, p + "norm2b", mult))})
        layers.append(LayerSpec(parts, "sandwich_residual"))
    stream_parts, schedule = {}, []
    times = cfg.loop[2] if cfg.loop else 0
    for i, begins in cfg.order():
        before = None
        if begins is not None:
            before = f"loop_step_{begins}"
            stream_parts[before] = PartSpec("add_row", {"width": d, "rows": times, "row": begins}, {"weight": "loop.step"})
        schedule.append(SchedulePlace(i, before=before))
    ignorable = tuple(f"l{i}.{n}" for i, layer in enumerate(cfg.layers) if not layer.get("mlp") for n in ("norm2", "norm2b"))
    return ModelSpec(
        vocab_size=cfg.vocab, hidden_size=d, max_positions=cfg.max_positions,
        embedding=PartSpec("token", {"vocab_size": cfg.vocab, "width": d, "scale": cfg.embedding_scale}, {"weight": "embed"}),
        layers=layers, schedule=schedule, final_norm=_norm(d, eps, "final.norm"),
        lm_head=PartSpec("linear", {"vocab_size": cfg.vocab, "width": d}, {"weight": "head"}),
        stop_ids=tuple(cfg.eos_token_ids), ignorable_tensors=ignorable, stream_parts=stream_parts)


register_architecture("Sofunex", SofunexConfig, build_spec)
