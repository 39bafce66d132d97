"""Plain, slow restatement of the Sofunex decoder, one function per mechanism.

The oracle of the Sofunex tests.  It shares no code with the product package: whole sequences, no cache, numpy
float64 throughout, every head by itself, the recurrence token by token.

The design in short.  x = E[token] * c.  A layer norms every sublayer before and after it and scales what it adds:
x <- x + m * RMSNorm_1b(mixer(shift(RMSNorm_1(x)))), then, if it has a feed-forward, x <- x + m * RMSNorm_2b(ff(RMSNorm_2(x))).
``shift`` blends what the mixer reads with what it read for the token before, channel by channel.  The mixer is two
mixers side by side that read the same input, added with a weight each:
  * grouped-query attention with biases, a short causal convolution over time on every channel of q, k and v, q and k
    RMS-normed over the whole projection, a rotation of split-half pairs over the first dims of every head whose
    frequencies are divided by a factor, values divided by their root mean square a head, a score scale of its own, a
    window of the most recent keys, plain softmax;
  * a delta rule with a decay and a removal rate per key channel: the matrix state of a head loses diag(w) and what it
    answers along the unit key, and gains k v^T; read out with r, normed a head, gated, projected.
A feed-forward is dense (gated, tanh gelu) or a mixture of gated silu experts routed by sigmoid scores with a
correction that only the choice sees, groups that count by their two best experts, and a shared expert.
A stretch of layers may run several times with the same weights; every pass begins by adding a vector of its own.
The logits are the final RMSNorm times the head matrix.
"""
from __future__ import annotations

import math

import numpy as np

F64 = np.float64

UNIT_KEY_EPS = 1e-6          # inside the root of the delta rule's unit key
DECAY_RATE = math.exp(-0.5)  # w = exp(-DECAY_RATE * sigmoid(.))
WEIGHT_SUM_EPS = 1e-20       # added to the sum of the chosen experts' scores
GROUP_BEST = 2               # a group of experts counts by the sum of so many of its largest choice scores


# ----------------------------------------------------------------------------- small functions
def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) [* w] over the last axis."""
    x = np.asarray(x, F64)
    y = x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)
    return y if weight is None else y * np.asarray(weight, F64)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-np.asarray(z, F64)))


def silu(z):
    z = np.asarray(z, F64)
    return z * sigmoid(z)


def gelu_tanh(z):
    z = np.asarray(z, F64)
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def token_shift(h, shift):
    """Row t becomes h_t + (h_(t-1) - h_t) * shift with the rows as they came in; zeros stand before the first."""
    h = np.asarray(h, F64)
    before = np.vstack([np.zeros((1, h.shape[1])), h[:-1]])
    return h + (before - h) * np.asarray(shift, F64)


def short_convolution(u, taps_weight):
    """y_t[c] = sum_j w[c, j] * u_(t - taps + 1 + j)[c], zeros before the start.  u [T, C], w [C, taps]."""
    u, w = np.asarray(u, F64), np.asarray(taps_weight, F64)
    taps = w.shape[1]
    out = np.zeros_like(u)
    for t in range(u.shape[0]):
        for j in range(taps):
            src = t - taps + 1 + j
            if src >= 0:
                out[t] += w[:, j] * u[src]
    return out


def rotate_split_half(vec, position: int, dims: int, base: float, factor: float):
    """The first ``dims`` entries of ``vec``: entry i pairs with entry i + dims / 2; the angle of pair i is
    position * base^(-2 i / dims) / factor; the rest stays."""
    out = np.array(vec, F64)
    half = dims // 2
    i = np.arange(half, dtype=F64)
    a = position * (np.power(F64(base), -2.0 * i / dims) / factor)
    u, v = out[:half].copy(), out[half:dims].copy()
    out[:half] = u * np.cos(a) - v * np.sin(a)
    out[half:dims] = v * np.cos(a) + u * np.sin(a)
    return out


# ----------------------------------------------------------------------------- the attention side
def attention_side(h, w, prefix, m, eps):
    """h [T, width] -> [T, width].  ``m`` is the side's dict of config.json."""
    H, G, kd, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    project = lambda name: h @ w[prefix + name].T.astype(F64) + w[prefix + name + ".b"].astype(F64)
    q, k, v = project("q"), project("k"), project("v")
    if m.get("conv"):
        q, k, v = (short_convolution(x, w[prefix + name + ".conv"]) for x, name in ((q, "q"), (k, "k"), (v, "v")))
    q = rms_norm(q, w[prefix + "q.norm"], eps)   # over the whole projection, all heads at once
    k = rms_norm(k, w[prefix + "k.norm"], eps)
    q, k, v = q.reshape(T, H, kd), k.reshape(T, G, kd), v.reshape(T, G, vd)
    rot = m.get("rot")
    if rot:
        factor = (rot.get("scaling") or {}).get("factor", 1.0)
        for t in range(T):
            for a in range(H):
                q[t, a] = rotate_split_half(q[t, a], t, rot["dims"], rot["base"], factor)
            for g in range(G):
                k[t, g] = rotate_split_half(k[t, g], t, rot["dims"], rot["base"], factor)
    v = rms_norm(v, None, eps)                   # a head's values over their root mean square, no weight
    window = (m.get("mask") or {}).get("size")
    heads = np.zeros((T, H, vd))
    for a in range(H):
        g = a // (H // G)
        for i in range(T):
            lo = max(0, i - window + 1) if window else 0
            s = (k[lo:i + 1, g] @ q[i, a]) * m["scale"]
            e = np.exp(s - s.max())
            heads[i, a] = (e / e.sum()) @ v[lo:i + 1, g]
    return heads.reshape(T, H * vd) @ w[prefix + "o"].T.astype(F64) + w[prefix + "o.b"].astype(F64)


# ----------------------------------------------------------------------------- the delta-rule side
def delta_step(S, r, k, v, decay, removal):
    """One token of one head.  S [key, value]; with the unit key u: S <- diag(decay) S - (removal * u)(u^T S) + k v^T,
    both of the first two terms from the state as it came; returns (S, S^T r)."""
    u = k / math.sqrt(float(k @ k) + UNIT_KEY_EPS)
    S = decay[:, None] * S - np.outer(removal * u, u @ S) + np.outer(k, v)
    return S, S.T @ r


def delta_side(h, w, prefix, m, eps):
    """h [T, width] -> [T, width]."""
    H, d = m["heads"], m["dim"]
    T = h.shape[0]
    mat = lambda name: w[prefix + name].astype(F64)
    r, k, v = (h @ mat(name).T for name in ("r", "k", "v"))
    decay = np.exp(-DECAY_RATE * sigmoid(np.tanh(h @ mat("w1").T) @ mat("w2").T + mat("w0")))
    removal = sigmoid(h @ mat("a").T + mat("a.b"))
    out = np.zeros((T, H, d))
    for a in range(H):
        cols = slice(a * d, (a + 1) * d)
        S = np.zeros((d, d))
        for t in range(T):
            S, out[t, a] = delta_step(S, r[t, cols], k[t, cols], v[t, cols], decay[t, cols], removal[t, cols])
    out = rms_norm(out, None, eps).reshape(T, H * d) * mat("norm") * sigmoid(h @ mat("g").T)
    return out @ mat("o").T


def mixer(h, w, prefix, m, eps):
    return (m.get("left_scale", 1.0) * attention_side(h, w, prefix + "left.", m["left"], eps)
            + m.get("right_scale", 1.0) * delta_side(h, w, prefix + "right.", m["right"], eps))


# ----------------------------------------------------------------------------- feed-forwards
def gated(h, w, prefix, act):
    mat = lambda name: w[prefix + name].astype(F64)
    return (act(h @ mat("gate").T) * (h @ mat("up").T)) @ mat("down").T


def route(h_row, w, prefix, mlp):
    """(experts, weights, margin) of one token; the margin is the smallest lead, in choice scores, by which a kept
    group or a chosen expert won its place (infinite where nothing was left out)."""
    router = mlp["router"]
    n, top = router["experts"], router["top"]
    scores = sigmoid(w[prefix + "router"].astype(F64) @ h_row)
    choice = scores + w[prefix + "correction"].astype(F64)
    margin = np.inf
    groups = router.get("groups")
    if groups and groups["keep"] < groups["count"]:
        size = n // groups["count"]
        worth = [np.sort(choice[g * size:(g + 1) * size])[-GROUP_BEST:].sum() for g in range(groups["count"])]
        ranked = sorted(range(groups["count"]), key=lambda g: (-worth[g], g))
        kept = ranked[:groups["keep"]]
        margin = worth[ranked[groups["keep"] - 1]] - worth[ranked[groups["keep"]]]
        choice = np.array([c if e // size in kept else -np.inf for e, c in enumerate(choice)])
    ranked = sorted(range(n), key=lambda e: (-choice[e], e))
    chosen = ranked[:top]
    if top < n and np.isfinite(choice[ranked[top]]):
        margin = min(margin, choice[ranked[top - 1]] - choice[ranked[top]])
    weights = scores[chosen] / (scores[chosen].sum() + WEIGHT_SUM_EPS) * router["scale"]
    return chosen, weights, margin


def experts(h, w, prefix, mlp, margins=None):
    out = np.zeros((h.shape[0], w[prefix + "e0.down"].shape[0]))
    for t in range(h.shape[0]):
        chosen, weights, margin = route(h[t], w, prefix, mlp)
        if margins is not None:
            margins[t] = min(margins[t], margin)
        for e, weight in zip(chosen, weights):
            out[t] += weight * gated(h[t:t + 1], w, f"{prefix}e{e}.", silu)[0]
    if mlp.get("shared"):
        out += gated(h, w, prefix + "shared.", silu)
    return out


def feed_forward(h, w, prefix, mlp, margins=None):
    return gated(h, w, prefix, gelu_tanh) if mlp["kind"] == "dense" else experts(h, w, prefix, mlp, margins)


# ----------------------------------------------------------------------------- the model
def layer_order(config):
    """[(layer, pass number or None)]: the pass number where a pass of the loop begins with the layer."""
    n, loop = len(config["layers"]), config.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    order = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        order += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return order + [(i, None) for i in range(loop["stop"], n)]


def layer(x, w, i, spec, eps, mult, margins=None):
    p = f"l{i}."
    h = token_shift(rms_norm(x, w[p + "norm1"], eps), w[p + "shift"])
    x = x + mult * rms_norm(mixer(h, w, p + "mix.", spec["mixer"], eps), w[p + "norm1b"], eps)
    if spec.get("mlp"):
        y = feed_forward(rms_norm(x, w[p + "norm2"], eps), w, p + "mlp.", spec["mlp"], margins)
        x = x + mult * rms_norm(y, w[p + "norm2b"], eps)
    return x


def forward(config, w, tokens, streams=None, margins=None):
    """Logits [T, vocab] of one sequence; ``streams`` (a list) receives the stream after every layer run; ``margins``
    (an array [T] that starts at infinity) the smallest lead of any routing decision made for each token."""
    eps, mult = config["norm"]["eps"], config.get("residual_mult", 1.0)
    x = w["embed"].astype(F64)[np.asarray(tokens)] * (config.get("embedding") or {}).get("scale", 1.0)
    for i, begins in layer_order(config):
        if begins is not None:
            x = x + w["loop.step"].astype(F64)[begins]
        x = layer(x, w, i, config["layers"][i], eps, mult, margins)
        if streams is not None:
            streams.append(x.copy())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T.astype(F64)


def forward_logits(config, w, tokens):
    return forward(config, w, tokens)
