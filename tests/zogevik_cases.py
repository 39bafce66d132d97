"""Small Zogevik configurations and weights for the tests.  Tensor names and shapes are written down here from the
design, not taken from the package, so that a wrong name or shape in the package shows.

The cases differ from one another in every size and option: the order of the layers; layers with experts and with no
feed-forward; key and value sizes that differ, that are no multiple of 16, that reach 128; as many kv heads as heads,
and one; a rotation over a part of the head and over all of it; windows shorter and longer than a cache block and a
window of one key; a layer that reads another layer's keys and values right after it, two layers that read the same
one, a reader whose window is wider and one whose window is narrower than the owner's; latent sizes whose cached row
is no multiple of 16, and one that fills the largest head the kernels take; one group of experts, as many groups as
experts, all groups kept, one expert a token, all experts of the kept groups a token, more than 32 experts; widths
that are no multiple of 8.
"""
from __future__ import annotations

import json
import os

import numpy as np


def attn(heads, kv, dim, vdim, rot_dims, base, size, scale, kv_from=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "rot": {"dims": rot_dims, "base": base},
         "mask": {"size": size}, "scale": scale}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def latent(heads, dim, rot_dim, vdim, rank, base, size, scale):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank,
            "rot": {"dims": rot_dim, "base": base}, "mask": {"size": size}, "scale": scale}


def moe(experts, top, ff, count, keep):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top,
                                                             "groups": {"count": count, "keep": keep}}}


CASE_MIXED = {
    "architecture": "Zogevik", "vocab": 101, "width": 64, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "attention", "mixer": attn(4, 2, 16, 16, 8, 10000.0, 40, 0.6), "mlp": moe(8, 2, 24, 4, 2)},
        {"type": "latent_attention", "mixer": latent(3, 8, 8, 16, 24, 5000.0, 70, 0.4), "mlp": None},
        {"type": "attention", "mixer": attn(4, 2, 16, 16, 8, 10000.0, 90, 0.3, kv_from=0), "mlp": moe(6, 3, 16, 1, 1)},
        {"type": "latent_attention", "mixer": latent(2, 16, 4, 8, 12, 100.0, 33, 0.25), "mlp": moe(8, 2, 24, 4, 2)},
    ],
}

CASE_ODD = {
    "architecture": "Zogevik", "vocab": 50, "width": 36, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "latent_attention", "mixer": latent(1, 12, 6, 20, 13, 300.0, 5, 0.5), "mlp": moe(40, 1, 12, 5, 5)},
        {"type": "attention", "mixer": attn(3, 3, 24, 40, 24, 2000.0, 70, 0.25), "mlp": None},
        {"type": "attention", "mixer": attn(3, 3, 24, 40, 24, 2000.0, 20, 0.4, kv_from=1), "mlp": moe(3, 3, 16, 1, 1)},
        {"type": "attention", "mixer": attn(2, 1, 8, 24, 2, 50.0, 1, 1.0), "mlp": moe(6, 2, 20, 3, 1)},
        {"type": "attention", "mixer": attn(6, 3, 24, 40, 24, 2000.0, 130, 0.3, kv_from=1), "mlp": moe(4, 2, 8, 4, 4)},
    ],
}

# heads of 128 and a width of 256: with prompts of more than 128 tokens the tiled tensor-core products run too
CASE_WIDE = {
    "architecture": "Zogevik", "vocab": 300, "width": 256, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "latent_attention", "mixer": latent(4, 64, 64, 64, 192, 10000.0, 200, 0.09), "mlp": moe(8, 3, 64, 2, 2)},
        {"type": "attention", "mixer": attn(4, 2, 128, 128, 64, 100000.0, 130, 0.08), "mlp": moe(8, 3, 64, 4, 3)},
        {"type": "attention", "mixer": attn(8, 2, 128, 128, 64, 100000.0, 260, 0.1, kv_from=1), "mlp": None},
    ],
}

CASES = {"mixed": (CASE_MIXED, 31), "odd": (CASE_ODD, 32), "wide": (CASE_WIDE, 33)}


def tensor_shapes(config: dict) -> dict:
    """{name: shape} of every tensor of a model of this configuration."""
    d = config["width"]
    shapes = {"embed": (config["vocab"], d), "embed.norm": (d,), "final.norm": (d,), "head": (config["vocab"], d)}
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        shapes[p + "norm1"] = (d,)
        q = p + "mix."
        if layer["type"] == "attention":
            H, G, kd, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            shapes.update({q + "q": (H * kd, d), q + "q.norm": (H * kd,), q + "o": (d, H * vd)})
            if m.get("kv_from") is None:
                shapes.update({q + "k": (G * kd, d), q + "k.norm": (G * kd,), q + "v": (G * vd, d)})
        else:
            H, kd, rd, vd, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            shapes.update({q + "q": (H * (kd + rd), d), q + "dkv": (r + rd, d), q + "dkv.norm": (r,),
                           q + "uk": (H * kd, r), q + "uv": (H * vd, r), q + "o": (d, H * vd)})
        mlp = layer.get("mlp")
        if mlp:
            shapes[p + "norm2"] = (d,)
            n, f = mlp["router"]["experts"], mlp["expert"]["ff"]
            shapes[p + "mlp.router"] = (n, d)
            for e in range(n):
                shapes.update({f"{p}mlp.e{e}.up": (f, d), f"{p}mlp.e{e}.down": (d, f)})
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
        if len(shape) == 1:
            w = 1.0 + rng.normal(0.0, 0.15, shape)  # norm weights
        elif leaf == "embed":
            w = rng.normal(0.0, 1.0, shape)
        elif leaf == "router":
            w = rng.normal(0.0, 2.0 / np.sqrt(shape[1]), shape)
        else:
            w = rng.normal(0.0, 1.0 / np.sqrt(shape[1]), shape)
        out[name] = _bf16(np.asarray(w, dtype=np.float32))
    return out


def write_folder(path: str, config: dict, weights: dict) -> str:
    """config.json and model.safetensors (bfloat16) in ``path``."""
    import torch
    from xeno_rt_b200.weights import write_safetensors
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as fh:
        json.dump(config, fh)
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
    width = pick(32, 36, 64, 96, 128, 200)
    layers, owners = [], []
    for i in range(int(rng.integers(2, 7))):
        if rng.random() < 0.4:
            rot = pick(2, 4, 8, 16, 32, 64)
            m = latent(pick(1, 2, 3, 4, 8), pick(4, 8, 12, 16, 32, 64), rot, pick(4, 8, 16, 20, 32, 64),
                       pick(5, 12, 16, 24, 40, 64, 128), pick(100.0, 10000.0, 1e6), pick(1, 5, 33, 64, 70, 130, 400),
                       float(pick(0.5, 1.0, 2.0)) / np.sqrt(16))
            layer = {"type": "latent_attention", "mixer": m}
        elif owners and rng.random() < 0.4:
            j = pick(*owners)
            o = layers[j]["mixer"]
            heads = o["kv_heads"] * pick(1, 2, 3, 4)
            m = attn(heads, o["kv_heads"], o["dim"], o["vdim"], o["rot"]["dims"], o["rot"]["base"],
                     pick(1, 5, 33, 64, 70, 130, 400), float(pick(0.5, 1.0, 2.0, 4.0)) / np.sqrt(o["dim"]), kv_from=j)
            layer = {"type": "attention", "mixer": m}
        else:
            kv = pick(1, 2, 3)
            dim = pick(8, 16, 24, 32, 48, 64, 128)
            m = attn(kv * pick(1, 2, 3, 4, 8), kv, dim, pick(8, 16, 24, 40, 64, 128),
                     pick(*[r for r in (2, 4, 8, 16, 24, 32, 64, 128) if r <= dim]), pick(100.0, 10000.0, 5e5),
                     pick(1, 5, 33, 64, 70, 130, 400), float(pick(0.5, 1.0, 2.0, 4.0)) / np.sqrt(dim))
            layer = {"type": "attention", "mixer": m}
            owners.append(i)
        if rng.random() < 0.75:
            count = pick(1, 2, 4)
            size = pick(1, 2, 3, 4, 10)
            keep = pick(*range(1, count + 1))
            layer["mlp"] = moe(count * size, pick(*[t for t in (1, 2, 3, keep * size) if t <= keep * size]),
                               pick(8, 12, 32, 64), count, keep)
        else:
            layer["mlp"] = None
        layers.append(layer)
    return {"architecture": "Zogevik", "vocab": pick(50, 101, 256), "width": width, "norm": {"eps": pick(1e-5, 1e-6)},
            "layers": layers}
