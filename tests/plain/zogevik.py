"""Plain, slow restatement of the Zogevik decoder, one function per mechanism.

The oracle of the Zogevik tests.  It shares no code with the product package: whole sequences, no cache, numpy
float64 throughout, every head and every query by itself.

The design in short.  x = RMSNorm(E[token]).  Every layer norms what a sublayer GIVES, not what it reads:
x <- x + RMSNorm_1(mixer(x)), then, if it has a feed-forward, x <- x + RMSNorm_2(ff(x)).  A mixer is
  * grouped-query attention whose q and k are RMS-normed over the whole projection (all heads at once), rotated in
    the split-half layout over the first dims of every head, with a score scale of its own, a window of the most
    recent keys and a softmax whose denominator holds one more term of score 0 that has no value; a layer may take
    keys and values from an earlier layer instead of projecting its own; or
  * latent attention: keys and values of all heads are read out of ONE small normed vector a token, and one rotated
    key part (interleaved pairs) is shared by all heads; plain softmax over a window.
A feed-forward is a mixture of small two-matrix experts with the exact gelu; the router's softmax runs over all
experts, only experts of the best groups can be chosen, and the chosen scores are used as they are.
The logits are the final RMSNorm times the head matrix.
"""
from __future__ import annotations

import math

import numpy as np

F64 = np.float64


# ----------------------------------------------------------------------------- small functions
def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis."""
    x = np.asarray(x, F64)
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps) * np.asarray(weight, F64)


def gelu_erf(z):
    z = np.asarray(z, F64)
    return 0.5 * z * (1.0 + np.vectorize(math.erf)(z / math.sqrt(2.0)))


def angles(position: int, dims: int, base: float):
    """a_i = position * base^(-2 i / dims), i < dims / 2."""
    i = np.arange(dims // 2, dtype=F64)
    return position * np.power(F64(base), -2.0 * i / dims)


def rotate_split_half(vec, position: int, dims: int, base: float):
    """The first ``dims`` entries of ``vec``: entry i pairs with entry i + dims / 2; the rest stays."""
    out = np.array(vec, F64)
    half = dims // 2
    a = angles(position, dims, base)
    u, v = out[:half].copy(), out[half:dims].copy()
    out[:half] = u * np.cos(a) - v * np.sin(a)
    out[half:dims] = v * np.cos(a) + u * np.sin(a)
    return out


def rotate_interleaved(vec, position: int, dims: int, base: float):
    """The first ``dims`` entries of ``vec``: entry 2i pairs with entry 2i + 1; the rest stays."""
    out = np.array(vec, F64)
    a = angles(position, dims, base)
    u, v = out[0:dims:2].copy(), out[1:dims:2].copy()
    out[0:dims:2] = u * np.cos(a) - v * np.sin(a)
    out[1:dims:2] = v * np.cos(a) + u * np.sin(a)
    return out


def visible(i: int, window):
    """Keys that query i sees: itself and the window - 1 before it (every earlier key without a window)."""
    return range(max(0, i - window + 1) if window else 0, i + 1)


def softmax_weights(scores, sink: bool):
    """exp(s_j) / (sum exp(s) [+ 1 with a sink of score 0])."""
    s = np.asarray(scores, F64)
    m = max(s.max(), 0.0) if sink else s.max()
    e = np.exp(s - m)
    return e / (e.sum() + (math.exp(-m) if sink else 0.0))


# ----------------------------------------------------------------------------- attention with a sink
def attention_keys_values(h, w, m, eps):
    """What a layer keeps of every token: keys [T, kv heads, dim] after the whole-projection norm and the rotation,
    values [T, kv heads, vdim]."""
    n = h.shape[0]
    g, dim, vdim = m["kv_heads"], m["dim"], m["vdim"]
    k = rms_norm(h @ w["k"].T, w["k.norm"], eps).reshape(n, g, dim)
    for t in range(n):
        for j in range(g):
            k[t, j] = rotate_split_half(k[t, j], t, m["rot"]["dims"], m["rot"]["base"])
    return k, (h @ w["v"].T).reshape(n, g, vdim)


def attention(h, w, m, eps, keys_values):
    """The mixer's result [T, width]; ``keys_values`` from this layer or from the one it shares with."""
    n = h.shape[0]
    heads, g, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    k, v = keys_values
    q = rms_norm(h @ w["q"].T, w["q.norm"], eps).reshape(n, heads, dim)
    window = (m.get("mask") or {}).get("size")
    out = np.zeros((n, heads, vdim), F64)
    for t in range(n):
        for a in range(heads):
            qa = rotate_split_half(q[t, a], t, m["rot"]["dims"], m["rot"]["base"])
            kv = a // (heads // g)
            js = list(visible(t, window))
            p = softmax_weights([qa @ k[j, kv] * m["scale"] for j in js], sink=True)
            out[t, a] = sum(pj * v[j, kv] for pj, j in zip(p, js))
    return out.reshape(n, heads * vdim) @ w["o"].T


# ----------------------------------------------------------------------------- latent attention
def latent_attention(h, w, m, eps):
    n = h.shape[0]
    heads, dim, rot, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    base = m["rot"]["base"]
    q = (h @ w["q"].T).reshape(n, heads, dim + rot)
    down = h @ w["dkv"].T
    c = rms_norm(down[:, :rank], w["dkv.norm"], eps)
    shared = np.stack([rotate_interleaved(down[t, rank:], t, rot, base) for t in range(n)])
    k_plain = (c @ w["uk"].T).reshape(n, heads, dim)
    v = (c @ w["uv"].T).reshape(n, heads, vdim)
    window = (m.get("mask") or {}).get("size")
    out = np.zeros((n, heads, vdim), F64)
    for t in range(n):
        for a in range(heads):
            q_rot = rotate_interleaved(q[t, a, dim:], t, rot, base)
            js = list(visible(t, window))
            p = softmax_weights([(q[t, a, :dim] @ k_plain[j, a] + q_rot @ shared[j]) * m["scale"] for j in js], sink=False)
            out[t, a] = sum(pj * v[j, a] for pj, j in zip(p, js))
    return out.reshape(n, heads * vdim) @ w["o"].T


# ----------------------------------------------------------------------------- mixture of experts
def router_scores(h, router):
    z = np.asarray(h, F64) @ router.T
    e = np.exp(z - z.max(axis=-1, keepdims=True))
    return e / e.sum(axis=-1, keepdims=True)


def choose(scores, top: int, groups: int, keep: int):
    """Experts of one token: those of the ``keep`` groups with the largest best score are allowed, of those the
    ``top`` with the largest scores (a lower number wins a tie)."""
    n = len(scores)
    size = n // groups
    best = [max(scores[g * size:(g + 1) * size]) for g in range(groups)]
    kept = sorted(range(groups), key=lambda g: (-best[g], g))[:keep]
    allowed = [e for e in range(n) if e // size in kept]
    return sorted(allowed, key=lambda e: (-scores[e], e))[:top]


def route_margins(h, router, top, groups, keep):
    """For every token, how close its routing was to another outcome, as a difference of log scores (which is the
    difference of the router's logits): the smallest of (a) the last chosen score against the best allowed one that
    was not chosen, (b) the last kept group's best against the best dropped group's best.  inf where nothing else
    could have happened."""
    s = router_scores(h, router)
    n = s.shape[1]
    size = n // groups
    out = []
    for row in s:
        logs = np.log(np.maximum(row, 1e-300))
        best = sorted((max(logs[g * size:(g + 1) * size]) for g in range(groups)), reverse=True)
        margin = best[keep - 1] - best[keep] if keep < groups else math.inf
        chosen = choose(row, top, groups, keep)
        kept = {e // size for e in chosen} | set(sorted(range(groups), key=lambda g: (-max(row[g * size:(g + 1) * size]), g))[:keep])
        rest = [logs[e] for e in range(n) if e // size in kept and e not in chosen]
        if rest:
            margin = min(margin, logs[chosen[-1]] - max(rest))
        out.append(margin)
    return np.array(out)


def expert(x, up, down):
    return down @ gelu_erf(up @ x)


def moe_ff(h, w, mlp):
    h = np.asarray(h, F64)
    r = mlp["router"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    s = router_scores(h, w["router"])
    out = np.zeros((h.shape[0], w["e0.down"].shape[0]), F64)
    for t in range(h.shape[0]):
        for e in choose(s[t], r["top"], groups["count"], groups["keep"]):
            out[t] += s[t, e] * expert(h[t], w[f"e{e}.up"], w[f"e{e}.down"])
    return out


# ----------------------------------------------------------------------------- the model
def _sub(tensors, prefix):
    return {k[len(prefix):]: np.asarray(v, F64) for k, v in tensors.items() if k.startswith(prefix)}


def forward(config, tensors, tokens, layers_out=None, margins_out=None):
    """Logits [T, vocab] of one whole sequence.  ``layers_out``: a list that receives the stream after every layer;
    ``margins_out``: a list that receives every routed layer's ``route_margins``."""
    eps = config["norm"]["eps"]
    x = rms_norm(np.asarray(tensors["embed"], F64)[list(tokens)], tensors["embed.norm"], eps)
    kept = {}
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        w = _sub(tensors, p + "mix.")
        if layer["type"] == "attention":
            if m.get("kv_from") is None:
                kept[i] = attention_keys_values(x, w, m, eps)
            y = attention(x, w, m, eps, kept[i if m.get("kv_from") is None else m["kv_from"]])
        elif layer["type"] == "latent_attention":
            y = latent_attention(x, w, m, eps)
        else:
            raise ValueError(layer["type"])
        x = x + rms_norm(y, tensors[p + "norm1"], eps)
        if layer.get("mlp"):
            w = _sub(tensors, p + "mlp.")
            r = layer["mlp"]["router"]
            if margins_out is not None:
                groups = r.get("groups") or {"count": 1, "keep": 1}
                margins_out.append(route_margins(x, w["router"], r["top"], groups["count"], groups["keep"]))
            x = x + rms_norm(moe_ff(x, w, layer["mlp"]), tensors[p + "norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.copy())
    return rms_norm(x, tensors["final.norm"], eps) @ np.asarray(tensors["head"], F64).T
