"""Every mechanism of the state-keeping mixers and of the steps around them alone, kernel against the plain
function: the scan (plain and delta rule) over unequal sequences in portions with slots that are used again,
the short convolution across portions shorter than its reach, decays, unit heads, head norm with gate, the
layer norm, the blended rotation table, the gated attention with unequal key and value sizes, and the rest."""
import math

import numpy as np
import pytest
import torch

from plain import givopel as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def dev(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV).to(dtype)


def ints(values):
    return torch.tensor(list(values), dtype=torch.int32, device=DEV)


def close(got, want, tol=2e-5):
    got = got.float().cpu().numpy().astype(np.float64)
    assert np.abs(got - want).max() <= tol * max(1.0, np.abs(want).max()), np.abs(got - want).max()


# heads, q/k heads, key size, value size: key sizes on every lane layout of the kernel (8, 16 and 32 rows a
# lane, 1 to 8 lanes a column), value sizes below, at and above a block's columns, sizes that are no power of two
SCAN_SIZES = [(2, 2, 8, 8), (3, 1, 16, 24), (4, 2, 48, 40), (1, 1, 130, 100), (2, 1, 256, 16), (2, 2, 32, 64)]


@pytest.mark.parametrize("delta", [False, True])
@pytest.mark.parametrize("heads,qk_heads,dim,vdim", SCAN_SIZES)
def test_state_scan_in_portions_over_unequal_sequences(heads, qk_heads, dim, vdim, delta):
    from xeno_rt_b200.csrc import ops
    rng = np.random.default_rng(dim * 7 + vdim + delta)
    lengths = [37, 1, 90]
    slots = [3, 0, 2]  # of 5; slot 1 and 4 stay untouched
    total = sum(lengths)
    q = rng.normal(0, 1, (total, qk_heads, dim)) / math.sqrt(dim)
    k = rng.normal(0, 1, (total, qk_heads, dim))
    if delta:
        k /= np.linalg.norm(k, axis=-1, keepdims=True)
    v = rng.normal(0, 1, (total, heads, vdim))
    decay = rng.uniform(0.9, 1.0, (total, heads, dim))
    decay[:, :, 0] = 1.0  # a channel that never forgets: token 0 counts to the end
    beta_raw = rng.normal(0, 1.5, (total, heads))
    beta = plain.sigmoid(beta_raw)
    starts = np.concatenate([[0], np.cumsum(lengths)])
    want = np.zeros((total, heads, vdim))
    for s, n in enumerate(lengths):
        rows = slice(starts[s], starts[s] + n)
        for h in range(heads):
            g = h // (heads // qk_heads)
            want[rows, h] = plain.state_scan(q[rows, g] * 0.5, k[rows, g], v[rows, h], decay[rows, h],
                                             beta[rows, h] if delta else None)
    state = torch.full((5, heads, vdim, dim), 7.0, device=DEV)  # what a slot's last user left
    for slot in slots:
        state[slot].zero_()  # the cache zeroes a slot when it opens
    # wide rows with the operands as column slices, as the mixers hand them over
    packed = dev(np.concatenate([q.reshape(total, -1), k.reshape(total, -1), v.reshape(total, -1)], axis=1))
    qw = qk_heads * dim
    got = np.zeros((total, heads * vdim))
    # three steps: the first tokens of every sequence (2 at most), then a portion, then the rest one by one for one
    at = [0, 0, 0]
    for portion in ([2, 1, 2], [30, 0, 3], [5, 0, 85]):
        rows, cu, step_slots = [], [0], []
        for s, take in enumerate(portion):
            if take == 0:
                continue
            rows += list(range(starts[s] + at[s], starts[s] + at[s] + take))
            cu.append(cu[-1] + take)
            step_slots.append(slots[s])
            at[s] += take
        step_slots.append(-1)  # a padding row of the step: no tokens, no slot
        cu.append(cu[-1])
        idx = torch.tensor(rows, device=DEV)
        out = torch.zeros((len(rows), heads * vdim), device=DEV)
        p = packed[idx].contiguous()
        ops.state_scan(out, p, p[:, qw:], p[:, 2 * qw:], dev(decay.reshape(total, -1))[idx].contiguous(),
                       dev(beta_raw)[idx].contiguous() if delta else None, state, ints(cu), ints(step_slots),
                       heads, qk_heads, dim, vdim, q_scale=0.5, delta=delta)
        got[rows] = out.cpu().numpy()
    close(torch.from_numpy(got), want.reshape(total, -1), 3e-5)
    assert bool((state[1] == 7.0).all()) and bool((state[4] == 7.0).all())


@pytest.mark.parametrize("taps", [1, 2, 4])
def test_short_convolution_across_portions_shorter_than_its_reach(taps):
    from xeno_rt_b200.csrc import ops
    rng = np.random.default_rng(taps)
    channels, lengths, slots = 70, [9, 40], [1, 0]
    x = [rng.normal(0, 1, (n, channels)) for n in lengths]
    w = rng.normal(0, 1, (channels, taps))
    want = [plain.silu(plain.short_convolution(a, w)) for a in x]
    state = torch.full((3, max(taps - 1, 1), channels), 5.0, device=DEV)[:, :taps - 1].contiguous()
    for slot in slots:
        state[slot].zero_()
    got = [[], []]
    at = [0, 0]
    for portion in ([1, 2], [1, 1], [2, 30], [5, 7]):
        rows = [x[s][at[s]:at[s] + take] for s, take in enumerate(portion)]
        wide = np.concatenate([np.concatenate(rows), np.zeros((sum(portion), 3))], axis=1)  # rows wider than the channels
        out = torch.zeros((sum(portion), channels), device=DEV)
        ops.short_conv(out, dev(wide), dev(w), state if taps > 1 else None, ints([0, portion[0], sum(portion)]),
                       ints(slots), max(portion), "silu")
        got[0].append(out[:portion[0]].cpu().numpy())
        got[1].append(out[portion[0]:].cpu().numpy())
        at = [a + t for a, t in zip(at, portion)]
    for s in range(2):
        close(torch.from_numpy(np.concatenate(got[s])), want[s])
    if taps > 1:
        close(state[1], x[0][9 - (taps - 1):9])
        assert bool((state[2] == 5.0).all())


def test_decays_unit_heads_head_norm_and_the_small_steps():
    from xeno_rt_b200.csrc import ops
    rng = np.random.default_rng(0)
    n, heads, dim, vdim = 13, 3, 20, 36
    z = rng.normal(0, 3, (n, heads * dim))
    bias = rng.normal(0, 1, heads * dim)
    a = dev(z)
    ops.decay_from_gate(a, dev(bias), heads, dim, 7.0)
    close(a, plain.sigmoid(z + bias) ** (1 / 7.0), 1e-6)
    a_log = rng.uniform(-3, 1, heads)
    a = dev(z)
    ops.decay_from_step(a, dev(bias), dev(a_log), heads, dim)
    close(a, np.exp(-np.exp(np.repeat(a_log, dim)) * plain.softplus(z + bias)), 1e-6)

    x = rng.normal(0, 2, (n, heads * dim + 5))
    t = dev(x)
    ops.unit_heads(t, heads, dim, 1e-6, scaled_heads=2, scale=0.25)
    want = x.copy()
    for h in range(heads):
        part = x[:, h * dim:(h + 1) * dim]
        want[:, h * dim:(h + 1) * dim] = part / np.sqrt((part ** 2).sum(-1, keepdims=True) + 1e-6) * (0.25 if h < 2 else 1.0)
    close(t, want, 1e-6)

    o = rng.normal(0, 3, (n, heads, vdim))
    g = rng.normal(0, 2, (n, heads * vdim + 8))
    w = rng.normal(1, 0.2, vdim)
    for act, fn in (("silu", plain.silu), ("sigmoid", plain.sigmoid)):
        for dtype, tol in ((torch.float32, 1e-6), (torch.bfloat16, 1e-2)):
            y = torch.empty((n, heads * vdim), dtype=dtype, device=DEV)
            ops.head_norm_gate(y, dev(o.reshape(n, -1)), dev(w), dev(g), heads, vdim, 1e-5, act)
            want = (plain.rms_norm(o, w, 1e-5) * fn(g[:, :heads * vdim]).reshape(n, heads, vdim)).reshape(n, -1)
            close(y, want, tol)

    width = 52
    res, y, w = rng.normal(0, 1, (n, width)), rng.normal(0, 4, (n, width)), rng.normal(1, 0.3, width)
    r = dev(res)
    ops.rms_scale_add(r, dev(y), dev(w), 1e-5, 0.5)
    close(r, res + 0.5 * plain.rms_norm(y, w, 1e-5), 1e-6)

    att = rng.normal(0, 1, (n, width))
    t = dev(att)
    ops.gate_mul(t, dev(g[:, 3:3 + width + 2])[:, :], "sigmoid")
    close(t, att * plain.sigmoid(g[:, 3:3 + width]), 1e-6)

    both = torch.empty((n, 2 * width), dtype=torch.bfloat16, device=DEV)
    ops.concat_cast(both, dev(res), dev(y))
    close(both, np.concatenate([res, y], axis=1), 1e-2)

    logits = rng.normal(0, 30, (n, width))
    t = dev(logits)
    ops.scale_softcap(t, 0.5, 12.0)
    close(t, 12.0 * np.tanh(logits * 0.5 / 12.0), 1e-6)
    t = dev(logits)
    ops.scale_softcap(t, 0.5, None)
    close(t, logits * 0.5, 1e-6)


@pytest.mark.parametrize("width", [36, 192, 1000, 4096])
def test_layer_norm_with_gathered_rows(width):
    from xeno_rt_b200.csrc import ops
    rng = np.random.default_rng(width)
    x = rng.normal(3.0, 2.0, (9, width))  # a mean far from zero: a norm without the mean would show
    w = rng.normal(1, 0.2, width)
    out = torch.empty((9, width), device=DEV)
    ops.layernorm(out, dev(x), dev(w), 1e-5)
    close(out, plain.layer_norm(x, w, 1e-5), 1e-5)
    out = torch.empty((3, width), dtype=torch.bfloat16, device=DEV)
    ops.layernorm(out, dev(x), dev(w, torch.bfloat16), 1e-5, ints([8, 0, 4]))
    close(out, plain.layer_norm(x[[8, 0, 4]], dev(w, torch.bfloat16).float().cpu().numpy(), 1e-5), 1e-2)


@pytest.mark.parametrize("scaling", [None, {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 2.0},
                                     {"factor": 3.0, "original": 1000, "fast": 20.0, "slow": 0.5},
                                     {"factor": 16.0, "original": 4096, "fast": 1.0, "slow": 1.0}])
def test_blended_rotation_table(scaling):
    from types import SimpleNamespace
    from xeno_rt_b200.parts import part_class
    dims, base = 24, 5000.0
    part = part_class("position", "blended_rotary")({"rope_dim": dims, "base": base, "scaling": scaling}, {}, None, DEV)
    assert part.pairing == "interleaved"
    positions = [0, 1, 63, 64, 65, 700, 5000, 300001, 8000003]
    ctx = SimpleNamespace(shared={}, n_tokens=len(positions), tok_pos=ints(positions))
    table = part.tables(ctx).cpu().numpy()
    f, mult = plain.yarn_frequencies(dims, base, scaling)
    angle = np.array(positions)[:, None] * f[None, :]
    want = np.stack([np.cos(angle), np.sin(angle)], axis=-1) * mult
    # the 32-bit product's rounding error is carried along: an angle of millions of radians is as exact as a small one
    assert np.abs(table - want).max() < 3e-6
    if scaling and scaling["factor"] == 4.0:  # the blend matters: neither the plain nor the fully divided frequencies
        plain_f, _ = plain.yarn_frequencies(dims, base, None)
        assert np.abs(f - plain_f).max() > 1e-3 and np.abs(f - plain_f / 4.0).max() > 1e-3


def _one_attention_layer(dtype, width, heads, kv_heads, dim, vdim, scale, rot):
    """A model of one layer: layer norm, the gated attention alone, no feed-forward; built from a spec by hand."""
    from xeno_rt_b200.core import parse_dtype
    from xeno_rt_b200.engine import Engine
    from xeno_rt_b200.engine.model import Model
    from xeno_rt_b200.parts import LayerSpec, ModelSpec, PartSpec, SchedulePlace
    vocab = 40
    position = {"kind": "none", "params": {}} if rot is None else \
        {"kind": "blended_rotary", "params": {"rope_dim": rot["dims"], "base": rot["base"], "scaling": rot.get("scaling")}}
    norm = lambda name: PartSpec("layernorm", {"width": width, "eps": 1e-5}, {"weight": name})
    attention = PartSpec("attention", {"width": width, "n_heads": heads, "n_kv_heads": kv_heads, "head_dim": dim,
                                       "v_head_dim": vdim, "qk_norm": False, "eps": 1e-5, "window": None, "scale": scale,
                                       "gate": "sigmoid", "position": position},
                         {r: "a." + r for r in ("q", "k", "v", "g", "o")})
    spec = ModelSpec(vocab_size=vocab, hidden_size=width, max_positions=4096,
                     embedding=PartSpec("token", {"vocab_size": vocab, "width": width}, {"weight": "embed"}),
                     layers=[LayerSpec({"norm": ("norm", norm("n")), "mixer": ("mixer", attention)}, "parallel_residual")],
                     schedule=[SchedulePlace(0)], final_norm=norm("fn"),
                     lm_head=PartSpec("linear", {"vocab_size": vocab, "width": width}, {"weight": "head"}))
    rng = np.random.default_rng(5)
    w = {"embed": rng.normal(0, 1, (vocab, width)), "n": np.ones(width), "fn": np.ones(width),
         "head": rng.normal(0, 1 / math.sqrt(width), (vocab, width)),
         "a.k": rng.normal(0, 1 / math.sqrt(width), (kv_heads * dim, width)),
         "a.v": rng.normal(0, 1 / math.sqrt(width), (kv_heads * vdim, width)),
         "a.g": rng.normal(0, 1 / math.sqrt(width), (heads * vdim, width)),
         "a.o": rng.normal(0, 3 / math.sqrt(heads * vdim), (width, heads * vdim))}
    # every query head asks for its kv head's key of the SAME input with the width's channels turned round by one:
    # q(h) = 4 k(roll(h)), so a token whose embedding is another's turned back finds that token, wherever it is
    wk = w["a.k"].reshape(kv_heads, dim, width)
    w["a.q"] = 4.0 * np.roll(np.repeat(wk, heads // kv_heads, axis=0), -1, axis=2).reshape(heads * dim, width)
    w["embed"][1] = np.roll(w["embed"][0], -1)  # token 1 asks for token 0
    w = {k: dev(v, torch.bfloat16).float().cpu().numpy().astype(np.float64) for k, v in w.items()}
    dt = parse_dtype(dtype)
    tensors = {k: dev(v, torch.float32 if dtype == "float32" else torch.bfloat16) for k, v in w.items()}
    p = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": rot}

    def oracle(tokens):
        x = w["embed"][np.asarray(tokens)]
        x = x + plain.softmax_attention(p, w, "a.", plain.layer_norm(x, w["n"], 1e-5))
        return plain.layer_norm(x, w["fn"], 1e-5) @ w["head"].T

    return Engine(Model(spec, tensors, dt, DEV), 64 * 8), oracle


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,rot", [
    (4, 2, 24, 40, None),                      # key and value sizes that differ and are no multiple of 16
    (2, 1, 64, 32, {"base": 10000.0, "dims": 32}),   # a rotation over half of the head
    (2, 2, 128, 128, None),                    # the size of the tensor-core kernels
])
def test_gated_attention_alone_finds_one_far_key(dtype, heads, kv_heads, dim, vdim, rot):
    """One key among 300 answers the last token's query; it lies at the start, at a block's edges, or just behind
    the query, in a prompt and in a token decoded alone.  Losing it (or seeing one key too many) changes the logits."""
    from xeno_rt_b200.engine import StepEntry
    engine, oracle = _one_attention_layer(dtype, 72, heads, kv_heads, dim, vdim, 1.0 / math.sqrt(dim), rot)
    tol = {"float32": 2e-5, "bfloat16": 3e-2}[dtype]
    rng = np.random.default_rng(8)
    n = 300
    for place in (0, 1, 63, 64, 127, 128, 255, 256, n - 2):
        tokens = rng.integers(2, 40, size=n).tolist()
        tokens[place], tokens[-1] = 0, 1
        want = oracle(tokens)[-1]
        without = list(tokens)
        without[place] = 2
        assert np.abs(oracle(without)[-1] - want).max() > 0.1 * np.abs(want).max()  # the key decides the result
        for cut in (n, n - 1, place + 1):  # whole; the query decoded alone; the query's portion begins right after the key
            if cut == 0:
                continue
            slot = engine.open_slot()
            if cut < n:
                engine.step([StepEntry(slot, tokens[:cut], [])])
            got = engine.step([StepEntry(slot, tokens[cut:] if cut < n else tokens, [n - 1 - (cut if cut < n else 0)])])
            engine.close_slot(slot)
            got = got.cpu().numpy()[0]
            assert np.abs(got - want).max() < tol * np.abs(want).max(), (place, cut)
