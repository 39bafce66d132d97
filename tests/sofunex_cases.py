"""Small Sofunex configurations and weights for the tests.  Tensor names and shapes are written down here from the
design, not taken from the package, so that a wrong name or shape in the package shows.

The cases differ from one another in every size and option: the order of the layers; layers with a dense feed-forward,
with experts and with none; key and value sizes that differ, that are no multiple of 16, that reach 128; as many kv
heads as heads, and one; a rotation over a part of the head, over all of it and none; frequencies divided and not;
convolutions of one to four taps and none; windows shorter and longer than a cache block, a window of one key and no
window; delta-rule heads of 12 to 128 channels and low ranks that are no multiple of 8; a loop in the middle, one
that begins with the first layer, one pass only, and none; experts in one group, in as many groups as experts, all
groups kept, one expert a token, with and without a shared expert; factors of 1 and others; widths and vocabularies
that are no multiple of 8.
"""
from __future__ import annotations

import json
import os

import numpy as np


def left(heads, kv, dim, vdim, scale, conv=None, rot=None, factor=None, size=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if conv is not None:
        m["conv"] = conv
    if rot is not None:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
        if factor is not None:
            m["rot"]["scaling"] = {"factor": factor}
    if size is not None:
        m["mask"] = {"size": size}
    return m


def right(heads, dim, rank):
    return {"heads": heads, "dim": dim, "decay_rank": rank}


def mixer(l, r, left_scale=1.0, right_scale=1.0):
    return {"left": l, "right": r, "left_scale": left_scale, "right_scale": right_scale}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, scale, groups=None, shared=None):
    mlp = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale}}
    if groups is not None:
        mlp["router"]["groups"] = {"count": groups[0], "keep": groups[1]}
    if shared is not None:
        mlp["shared"] = {"ff": shared}
    return mlp


def layer(m, mlp):
    return {"type": "parallel", "mixer": m, "mlp": mlp}


CASE_MIXED = {
    "architecture": "Sofunex", "vocab": 101, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.5},
    "residual_mult": 0.8, "loop": {"start": 1, "stop": 3, "times": 3},
    "layers": [
        layer(mixer(left(4, 2, 16, 16, 0.3, conv=3, rot=(8, 10000.0), factor=4.0, size=40), right(2, 32, 8), 0.7, 1.1),
              dense(96)),
        layer(mixer(left(3, 3, 8, 24, 0.5, conv=2, rot=(8, 500.0), size=70), right(4, 16, 12), 1.3, 0.6),
              moe(8, 2, 24, 1.5, groups=(4, 2), shared=40)),
        layer(mixer(left(2, 1, 32, 16, 0.2, conv=4, size=5), right(1, 64, 8), 0.9, 0.9), None),
        layer(mixer(left(4, 1, 16, 32, 0.25, conv=4, rot=(4, 10000.0), factor=2.0, size=90), right(2, 32, 16), 0.5, 1.0),
              moe(6, 3, 16, 2.5)),
    ],
}

CASE_ODD = {
    "architecture": "Sofunex", "vocab": 50, "width": 36, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
    "residual_mult": 1.0,
    "layers": [
        layer(mixer(left(3, 3, 12, 20, 0.4, conv=1, rot=(12, 300.0), factor=1.5, size=1), right(3, 12, 5)),
              moe(40, 1, 12, 1.0, groups=(5, 5), shared=20)),
        layer(mixer(left(2, 2, 24, 8, 0.3, rot=(6, 2000.0)), right(1, 36, 7), 1.0, 0.8), dense(52)),
        layer(mixer(left(6, 3, 8, 8, 0.6, conv=2, size=130), right(2, 20, 4), 0.4, 1.0),
              moe(6, 2, 20, 0.7, groups=(6, 3))),
    ],
}

# heads of 128 and a width of 256: with prompts of more than 128 tokens the tiled tensor-core products run too
CASE_WIDE = {
    "architecture": "Sofunex", "vocab": 300, "width": 256, "norm": {"eps": 1e-5}, "embedding": {"scale": 16.0},
    "residual_mult": 0.65, "loop": {"start": 0, "stop": 2, "times": 2},
    "layers": [
        layer(mixer(left(4, 2, 128, 128, 0.09, conv=4, rot=(64, 100000.0), factor=6.0, size=130), right(2, 128, 16), 0.55, 0.95),
              dense(448)),
        layer(mixer(left(8, 1, 64, 64, 0.12, conv=3, rot=(64, 10000.0), size=200), right(4, 64, 32), 1.0, 1.0),
              moe(8, 3, 48, 1.8, groups=(2, 1), shared=64)),
        layer(mixer(left(2, 2, 128, 64, 0.1, conv=2, rot=(32, 10000.0), factor=2.0), right(8, 32, 8), 0.8, 0.5), None),
    ],
}

CASES = {"mixed": (CASE_MIXED, 41), "odd": (CASE_ODD, 42), "wide": (CASE_WIDE, 43)}


def tensor_shapes(config: dict) -> dict:
    """{name: shape} of every tensor of a model of this configuration."""
    d = config["width"]
    shapes = {"embed": (config["vocab"], d), "final.norm": (d,), "head": (config["vocab"], d)}
    if config.get("loop"):
        shapes["loop.step"] = (config["loop"]["times"], d)
    for i, spec in enumerate(config["layers"]):
        p = f"l{i}."
        shapes.update({p + "norm1": (d,), p + "norm1b": (d,), p + "shift": (d,)})
        l, r = spec["mixer"]["left"], spec["mixer"]["right"]
        q = p + "mix.left."
        H, G, kd, vd = l["heads"], l["kv_heads"], l["dim"], l["vdim"]
        for name, rows in (("q", H * kd), ("k", G * kd), ("v", G * vd)):
            shapes.update({q + name: (rows, d), q + name + ".b": (rows,)})
            if l.get("conv"):
                shapes[q + name + ".conv"] = (rows, l["conv"])
        shapes.update({q + "q.norm": (H * kd,), q + "k.norm": (G * kd,), q + "o": (d, H * vd), q + "o.b": (d,)})
        q = p + "mix.right."
        w = r["heads"] * r["dim"]
        for name in ("r", "k", "v", "g", "a"):
            shapes[q + name] = (w, d)
        shapes.update({q + "a.b": (w,), q + "w1": (r["decay_rank"], d), q + "w2": (w, r["decay_rank"]), q + "w0": (w,),
                       q + "norm": (w,), q + "o": (d, w)})
        mlp = spec.get("mlp")
        if not mlp:
            continue
        shapes.update({p + "norm2": (d,), p + "norm2b": (d,)})
        q = p + "mlp."
        if mlp["kind"] == "dense":
            shapes.update({q + "gate": (mlp["ff"], d), q + "up": (mlp["ff"], d), q + "down": (d, mlp["ff"])})
            continue
        n, f = mlp["router"]["experts"], mlp["expert"]["ff"]
        shapes.update({q + "router": (n, d), q + "correction": (n,)})
        for e in range(n):
            shapes.update({f"{q}e{e}.gate": (f, d), f"{q}e{e}.up": (f, d), f"{q}e{e}.down": (d, f)})
        if mlp.get("shared"):
            f = mlp["shared"]["ff"]
            shapes.update({q + "shared.gate": (f, d), q + "shared.up": (f, d), q + "shared.down": (d, f)})
    return shapes


def _bf16(x: np.ndarray) -> np.ndarray:
    """Rounded to bfloat16 (to nearest even) and back, so that file and oracle hold the same numbers."""
    bits = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint32) << 16
    return rounded.view(np.float32).reshape(np.shape(x))


def random_weights(config: dict, seed: int) -> dict:
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        leaf = name.split(".")[-1]
        if name.endswith(".conv"):
            w = rng.normal(0.0, 0.6, shape)
        elif leaf in ("norm", "norm1", "norm2", "norm1b", "norm2b"):
            w = 1.0 + rng.normal(0.0, 0.15, shape)
        elif leaf == "shift":
            w = rng.uniform(0.0, 1.0, shape)
        elif leaf == "correction":
            w = rng.normal(0.0, 0.3, shape)     # large enough to change which experts win, and to go below zero
        elif leaf in ("b", "w0"):
            w = rng.normal(0.0, 0.5, shape)
        elif leaf == "step":
            w = rng.normal(0.0, 0.5, shape)
        elif leaf == "embed":
            w = rng.normal(0.0, 1.0, shape)
        elif leaf == "router":
            w = rng.normal(0.0, 2.0 / np.sqrt(shape[1]), shape)
        elif leaf in ("w1", "w2"):
            w = rng.normal(0.0, 2.0 / np.sqrt(shape[1]), shape)
        else:
            w = rng.normal(0.0, 1.0 / np.sqrt(shape[1]), shape)
        out[name] = _bf16(np.asarray(w, dtype=np.float32))
    return out


def stored(config: dict) -> dict:
    """The configuration as a model folder holds it: the rank of the decay's product is a size of tensors only."""
    out = json.loads(json.dumps(config))
    for spec in out["layers"]:
        spec["mixer"]["right"].pop("decay_rank", None)
    return out


def write_folder(path: str, config: dict, weights: dict) -> str:
    """config.json and model.safetensors (bfloat16) in ``path``."""
    import torch
    from xeno_rt_b200.weights import write_safetensors
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as fh:
        json.dump(stored(config), fh)
    write_safetensors(os.path.join(path, "model.safetensors"),
                      {k: torch.from_numpy(np.array(v, dtype=np.float32)).reshape(np.shape(v)).to(torch.bfloat16)
                       for k, v in weights.items()})
    return path


def make_case(tmp_path, name: str):
    """(folder, config, weights) of a named case."""
    config, seed = CASES[name]
    weights = random_weights(config, seed)
    return write_folder(os.path.join(str(tmp_path), name), config, weights), config, weights


def random_config(rng) -> dict:
    """A configuration drawn at random: any order of layers, any of the sizes and options the cases above use and
    more."""
    pick = lambda *values: values[int(rng.integers(len(values)))]
    width = pick(32, 36, 64, 96, 128, 200, 320)
    layers = []
    for _ in range(int(rng.integers(1, 6))):
        kv = pick(1, 2, 3, 4)
        dim = pick(8, 12, 16, 24, 32, 48, 64, 72, 96, 128)
        rot = pick(None, *[(r, pick(100.0, 10000.0, 5e5)) for r in (2, 4, 8, 12, 16, 24, 32, 64, 96, 128) if r <= dim])
        l = left(kv * pick(1, 2, 3, 4, 6, 8, 12), kv, dim, pick(8, 16, 20, 24, 40, 64, 96, 128), float(pick(0.5, 1.0, 2.0, 4.0)) / np.sqrt(dim),
                 conv=pick(None, 1, 2, 3, 4, 5), rot=rot, factor=pick(None, 1.0, 2.0, 6.0) if rot else None,
                 size=pick(None, 1, 5, 33, 64, 70, 80, 130, 400))
        r = right(pick(1, 2, 3, 4, 6), pick(8, 12, 16, 20, 32, 48, 64, 96, 128), pick(4, 5, 8, 16, 24, 32))
        m = mixer(l, r, pick(1.0, 0.5, 1.4), pick(1.0, 0.75, 0.3))
        kind = pick("dense", "moe", "moe", None)
        if kind == "dense":
            mlp = dense(pick(24, 52, 96, 160))
        elif kind == "moe":
            count = pick(1, 2, 4, 8)
            size = pick(1, 2, 3, 4, 10)
            keep = pick(*range(1, count + 1))
            mlp = moe(count * size, pick(*[t for t in (1, 2, 3, keep * size) if t <= keep * size]), pick(8, 12, 32, 64),
                      pick(1.0, 2.0, 0.5), groups=pick(None, (count, keep)) if keep == count else (count, keep),
                      shared=pick(None, 16, 40))
        else:
            mlp = None
        layers.append(layer(m, mlp))
    config = {"architecture": "Sofunex", "vocab": pick(50, 101, 256), "width": width, "norm": {"eps": pick(1e-5, 1e-6)},
              "embedding": {"scale": pick(1.0, 4.0, float(np.sqrt(width)))}, "residual_mult": pick(1.0, 0.8, 0.5),
              "layers": layers}
    if rng.random() < 0.7:
        start = int(rng.integers(0, len(layers)))
        stop = int(rng.integers(start + 1, len(layers) + 1))
        config["loop"] = {"start": start, "stop": stop, "times": pick(1, 2, 3, 4)}
    return config
