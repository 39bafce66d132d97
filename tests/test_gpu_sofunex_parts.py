"""The mechanisms of the Sofunex decoder one by one, each kernel or part against the plain function of the same
mechanism (tests/plain/sofunex.py): the token shift fused with its norm (portions, single tokens, slots used again),
the convolution that adds its input's bias, value heads over their root mean square, the scan's removal form and its
gates (prompts against single tokens, a far token that the state must still hold after hundreds), sigmoid routing
with a correction and groups that count by two, gated silu experts on both of their paths with a shared expert, the
tanh-gelu gate, the norm after a sublayer with factors, a bias and a second norm, the embedding's scale and the row
that a pass begins with; then each side of the mixer alone in a model of one layer."""
import copy

import numpy as np
import pytest
import torch

from plain import sofunex as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _t(a, dtype=torch.float32):
    return torch.tensor(np.asarray(a), dtype=dtype, device=DEV).contiguous()


def _ints(a):
    return torch.tensor(np.asarray(a), dtype=torch.int32, device=DEV)


def _close(got, want, tol):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert got.shape == want.shape
    if got.size:
        assert np.abs(got - want).max() <= tol * max(1.0, np.abs(want).max()), np.abs(got - want).max()


def _step_arrays(lens, slots, starts):
    """(tok_slot, tok_pos, cu_seqlens, seq_slot) of a step whose sequences bring ``lens`` tokens."""
    tok_slot = [s for s, k in zip(slots, lens) for _ in range(k)]
    tok_pos = [b + i for b, k in zip(starts, lens) for i in range(k)]
    cu = np.concatenate([[0], np.cumsum(lens)])
    return _ints(tok_slot), _ints(tok_pos), _ints(cu), _ints(slots)


# ------------------------------------------------------------------------------------------------ token shift
@pytest.mark.parametrize("width", [36, 64, 200, 1500])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_token_shift_blends_the_norm_with_the_token_before_across_steps(width, out_dtype):
    """Three sequences of unequal lengths, cut into portions (one of them a single token, one of them two), then single
    tokens; the token before a step's first token comes from the state; a padding row changes nothing."""
    from xeno_rt_b200.csrc import ops
    rng = np.random.default_rng(width)
    eps = 1e-5
    lens = [37, 5, 12]
    x = [rng.normal(0.3, 2.0, size=(n, width)).astype(np.float32) for n in lens]
    w, shift = rng.normal(1.0, 0.2, width).astype(np.float32), rng.uniform(0, 1, width).astype(np.float32)
    want = [plain.token_shift(plain.rms_norm(a, w, eps), shift) for a in x]
    state = torch.full((6, width), 7.0, device=DEV)   # what a slot held before is not zero ...
    slots = [4, 0, 2]
    state[slots] = 0.0                                # ... the cache zeroes a slot when it opens
    got = [[] for _ in lens]
    at = [0, 0, 0]
    for cut in ([30, 1, 2], [1, 2, 9], [1, 1, 1], [5, 1, 0]):
        live = [i for i in range(3) if cut[i]]
        rows = np.concatenate([x[i][at[i]:at[i] + cut[i]] for i in live] + [np.ones((1, width), np.float32)])
        arrays = _step_arrays([cut[i] for i in live], [slots[i] for i in live], [at[i] for i in live])
        tok_slot = torch.cat([arrays[0], _ints([-1])])   # one padding row at the end
        tok_pos = torch.cat([arrays[1], _ints([0])])
        out = torch.empty(rows.shape, dtype=out_dtype, device=DEV)
        ops.rmsnorm_shift(out, _t(rows), _t(w), _t(shift), state, (tok_slot, tok_pos, arrays[2], arrays[3]), eps,
                          single_tokens=max(cut) == 1)
        out = out.float().cpu().numpy()
        assert not out[-1].any()
        o = 0
        for i in live:
            got[i].append(out[o:o + cut[i]])
            o += cut[i]
            at[i] += cut[i]
    assert at == lens
    for i in range(3):
        _close(np.concatenate(got[i]), want[i], 2e-6 if out_dtype == torch.float32 else 1e-2)
    assert bool((state[[1, 3, 5]] == 7.0).all())        # other slots' states are left alone
    _close(state[slots[1]].cpu().numpy(), plain.rms_norm(x[1][-1], w, eps), 2e-6)


# ------------------------------------------------------------------------------------------------ convolution
@pytest.mark.parametrize("taps", [1, 2, 4, 5])
def test_the_convolution_adds_its_inputs_bias_inside_the_sequence_only(taps):
    """y_t = sum_j w_j (x + b)_(t - taps + 1 + j) with zeros (not b) before the sequence's start; cut into portions."""
    from xeno_rt_b200.csrc import ops
    rng = np.random.default_rng(taps)
    channels, n = 40, 23
    x = rng.normal(size=(n, channels + 3)).astype(np.float32)   # rows are slices of wider rows
    w, b = rng.normal(size=(channels, taps)).astype(np.float32), rng.normal(size=channels).astype(np.float32)
    want = plain.short_convolution(x[:, :channels].astype(np.float64) + b, w)
    state = torch.zeros((3, max(taps - 1, 1), channels), device=DEV)
    got, at = [], 0
    for cut in (1, 2, 9, 1, 1, 9):
        arrays = _step_arrays([cut], [1], [at])
        out = torch.empty((cut, channels), device=DEV)
        ops.short_conv(out, _t(x[at:at + cut])[:, :channels], _t(w), state[:, :taps - 1] if taps > 1 else None,
                       arrays[2], arrays[3], cut, "none", in_bias=_t(b))
        got.append(out.cpu().numpy())
        at += cut
    _close(np.concatenate(got), want, 2e-6)
    if taps > 1:
        _close(state[1, :taps - 1].cpu().numpy(), (x[n - taps + 1:, :channels] + b), 1e-6)


def test_value_heads_are_divided_by_their_root_mean_square_before_they_are_cached():
    """Heads of 20 values laid out at 32: the mean runs over 20; q and k pass the whole-projection norm."""
    from xeno_rt_b200.csrc import ops
    rng = np.random.default_rng(3)
    n, heads, kv, dim, vdim, size, eps = 5, 2, 2, 12, 20, 32, 1e-5
    q, k, v = rng.normal(size=(n, heads, dim)), rng.normal(size=(n, kv, dim)), rng.normal(2.0, 3.0, size=(n, kv, vdim))
    wq, wk = rng.normal(1.0, 0.3, heads * dim), rng.normal(1.0, 0.3, kv * dim)
    row = np.zeros((n, (heads + 2 * kv) * size), np.float32)
    lay = lambda t, h, d: np.pad(t, ((0, 0), (0, 0), (0, size - d))).reshape(n, h * size)
    row[:, :heads * size], row[:, heads * size:(heads + kv) * size], row[:, (heads + kv) * size:] = lay(q, heads, dim), lay(k, kv, dim), lay(v, kv, vdim)
    pad_w = lambda t, h, d: np.pad(t.reshape(h, d), ((0, 0), (0, size - d))).reshape(-1)
    k_pool = torch.zeros((2, kv, 64, size), device=DEV)
    v_pool = torch.zeros_like(k_pool)
    q_out = torch.empty((n, heads * size), device=DEV)
    table = _ints([[1, 0]])
    ops.qkv_heads_write(q_out, k_pool, v_pool, _t(row), heads * size, (heads + kv) * size, None, False, dim, eps,
                        _ints([0] * n), _ints(range(62, 62 + n)), table, heads, kv, size, v_dim=vdim,
                        q_norm_w=_t(pad_w(wq, heads, dim)), k_norm_w=_t(pad_w(wk, kv, dim)), whole_q=heads * dim,
                        whole_k=kv * dim, v_unit=True)
    want_v = plain.rms_norm(v, None, eps)
    cached = torch.cat([v_pool[1, :, 62:], v_pool[0, :, :n - 2]], dim=1).permute(1, 0, 2).cpu().numpy()  # [n, kv, size]
    _close(cached[:, :, :vdim], want_v, 2e-6)
    assert not cached[:, :, vdim:].any()
    want_q = plain.rms_norm(q.reshape(n, -1), wq, eps).reshape(n, heads, dim)
    _close(q_out.cpu().numpy().reshape(n, heads, size)[:, :, :dim], want_q, 2e-6)


# ------------------------------------------------------------------------------------------------ the scan
def _plain_scan(r, k, v, decay, removal, heads, dim, state=None):
    n = r.shape[0]
    out = np.zeros((n, heads, dim))
    S = [np.zeros((dim, dim)) if state is None else state[a].copy() for a in range(heads)]
    for a in range(heads):
        c = slice(a * dim, (a + 1) * dim)
        for t in range(n):
            S[a], out[t, a] = plain.delta_step(S[a], r[t, c], k[t, c], v[t, c], decay[t, c], removal[t, c])
    return out.reshape(n, heads * dim), S


def _gpu_scan(r, k, v, raw_decay, w0, raw_removal, a_bias, heads, dim, cuts, slot=2):
    """The gates kernel and the scan over portions of ``cuts`` tokens; returns (out, final state [heads, key, value])."""
    from xeno_rt_b200.csrc import ops
    n, w = r.shape[0], heads * dim
    state = torch.zeros((4, heads, dim, dim), device=DEV)
    outs, at = [], 0
    for cut in cuts:
        rows = slice(at, at + cut)
        p = _t(np.concatenate([r[rows], k[rows], v[rows], raw_removal[rows]], axis=1))   # slices of one wide row
        decay, unit = _t(raw_decay[rows]), torch.empty((cut, w), device=DEV)
        removal = p[:, 3 * w:]
        ops.removal_gates(decay, _t(w0), removal, _t(a_bias), unit, p[:, w:2 * w], heads, dim, plain.DECAY_RATE,
                          plain.UNIT_KEY_EPS)
        out = torch.empty((cut, w), device=DEV)
        arrays = _step_arrays([cut], [slot], [at])
        ops.state_scan(out, p, p[:, w:], p[:, 2 * w:], decay, None, state, arrays[2], arrays[3], heads, heads, dim, dim,
                       max_new=cut, unit=unit, removal=removal)
        outs.append(out.cpu().numpy())
        at += cut
    assert at == n and not state[[0, 1, 3]].any()
    return np.concatenate(outs), state[slot].permute(0, 2, 1).cpu().numpy()   # kept [heads, value, key]


@pytest.mark.parametrize("heads,dim", [(2, 32), (3, 12), (1, 64), (4, 48), (2, 128), (1, 21)])
def test_the_removal_scan_is_the_plain_recurrence_whole_cut_and_token_by_token(heads, dim):
    rng = np.random.default_rng(dim)
    n, w = 75, heads * dim
    r, k, v = (rng.normal(size=(n, w)).astype(np.float32) for _ in range(3))
    raw_decay, raw_removal = rng.normal(0, 2, size=(n, w)).astype(np.float32), rng.normal(0, 2, size=(n, w)).astype(np.float32)
    w0, a_bias = rng.normal(size=w).astype(np.float32), rng.normal(size=w).astype(np.float32)
    decay = np.exp(-plain.DECAY_RATE * plain.sigmoid(raw_decay.astype(np.float64) + w0))
    removal = plain.sigmoid(raw_removal.astype(np.float64) + a_bias)
    want, S = _plain_scan(r.astype(np.float64), k.astype(np.float64), v.astype(np.float64), decay, removal, heads, dim)
    scale = np.abs(want).max()
    for cuts in ([n], [2, 1, 17, 16, 33, 1, 5], [1] * n):
        got, state = _gpu_scan(r, k, v, raw_decay, w0, raw_removal, a_bias, heads, dim, cuts)
        assert np.abs(got - want).max() < 2e-5 * scale, (cuts[:3], np.abs(got - want).max() / scale)
        _close(state, np.stack(S), 2e-5)


def test_a_token_far_back_still_shows_in_the_state_after_hundreds():
    """One early token is written with a large key and value; nothing decays and nothing is removed (both raw gates
    are far below zero) and the later keys are small.  The last token reads along that key: its result is that value,
    hundreds of tokens and many tiles and portions later.  Had the state been lost at a portion's start it would be
    (nearly) zero."""
    heads, dim, n, far = 2, 32, 700, 3
    rng = np.random.default_rng(5)
    w = heads * dim
    r, k, v = (rng.normal(0, 0.01, size=(n, w)).astype(np.float32) for _ in range(3))
    key = rng.normal(size=w).astype(np.float32)
    key /= np.sqrt((key.reshape(heads, dim) ** 2).sum(-1)).repeat(dim)
    k[far], v[far] = key, np.arange(w, dtype=np.float32) / 8 + 1.0
    r[-1] = key
    raw_decay = np.full((n, w), -30.0, np.float32)       # sigmoid -> 0, decay -> 1
    raw_removal = np.full((n, w), -30.0, np.float32)
    zeros = np.zeros(w, np.float32)
    decay = np.exp(-plain.DECAY_RATE * plain.sigmoid(raw_decay.astype(np.float64)))
    want, _ = _plain_scan(*(a.astype(np.float64) for a in (r, k, v)), decay, plain.sigmoid(raw_removal.astype(np.float64)), heads, dim)
    assert np.abs(want[-1] - v[far]).max() < 0.05 * np.abs(v[far]).max()     # the far token is what the answer is made of
    for cuts in ([n], [far + 1, 1, 300, 64, 1, 1, n - far - 368], [10] + [1] * (n - 10)):
        got, _ = _gpu_scan(r, k, v, raw_decay, zeros, raw_removal, zeros, heads, dim, cuts)
        assert np.abs(got[-1] - want[-1]).max() < 1e-4 * np.abs(want[-1]).max(), cuts[:3]


# ------------------------------------------------------------------------------------------------ routing and experts
@pytest.mark.parametrize("experts,top,groups,keep", [(8, 2, 4, 2), (8, 4, 2, 1), (6, 3, 1, 1), (40, 1, 5, 5), (6, 2, 6, 3),
                                                     (64, 6, 8, 3), (12, 5, 3, 2)])
def test_sigmoid_routing_with_a_correction_and_groups_that_count_by_two(experts, top, groups, keep):
    from xeno_rt_b200.csrc import ops
    rng = np.random.default_rng(experts + top)
    n, d = 50, 16
    router = rng.normal(0, 1.0, size=(experts, d))
    correction = rng.normal(0, 0.6, size=experts).astype(np.float32)   # changes who wins, and goes below zero
    h = rng.normal(size=(n, d))
    logits = (h @ router.T).astype(np.float32)
    mlp = {"router": {"experts": experts, "top": top, "scale": 2.5, "groups": {"count": groups, "keep": keep}}}
    ids = torch.empty((n, top), dtype=torch.int32, device=DEV)
    weights = torch.empty((n, top), device=DEV)
    ops.moe_route_scores(ids, weights, _t(logits), top, groups, keep, scores="sigmoid", correction=_t(correction),
                         group_best=plain.GROUP_BEST, normalize=True, sum_eps=plain.WEIGHT_SUM_EPS, scale=2.5)
    # the plain router from the same 32-bit logits: w stands in as an identity product
    w = {"m.router": np.eye(experts), "m.correction": correction}
    differ = 0
    for t in range(n):
        chosen, wts, margin = plain.route(logits[t].astype(np.float64), w, "m.", mlp)
        if margin < 1e-5:
            continue
        assert ids[t].tolist() == chosen, t
        _close(weights[t].cpu().numpy(), wts, 1e-5)
        plain_scores = sorted(range(experts), key=lambda e: -logits[t, e])[:top]
        differ += sorted(plain_scores) != sorted(chosen)
    assert differ > 0      # the correction and the groups changed some choices: the test would show a router without them


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n", [3, 200])
def test_gated_silu_experts_with_a_shared_expert_on_both_paths(dtype, n):
    """Few tokens stream every (token, choice) pair's expert; many tokens sort their rows by expert.  The part's
    result is the sum of its parts: the chosen experts' weighted results and the shared expert's."""
    from xeno_rt_b200.core import parse_dtype
    from xeno_rt_b200.parts import StepContext, part_class
    rng = np.random.default_rng(n)
    d, ff, experts, top, shared = 48, 24, 8, 3, 40
    rnd = lambda *shape: torch.tensor(rng.normal(0, 1 / np.sqrt(shape[-1]), shape), dtype=torch.float32).to(dtype).to(DEV)
    w = {"router": rnd(experts, d), "correction": torch.tensor(rng.normal(0, 0.3, experts), dtype=torch.float32).to(dtype).to(DEV),
         "shared_gate": rnd(shared, d), "shared_up": rnd(shared, d), "shared_down": rnd(d, shared)}
    for e in range(experts):
        w.update({f"gate{e}": rnd(ff, d), f"up{e}": rnd(ff, d), f"down{e}": rnd(d, ff)})
    params = {"width": d, "inner": ff, "experts": experts, "top": top, "activation": "gated_silu", "routing": "scores",
              "scores": "sigmoid", "correction": True, "groups": 4, "keep_groups": 2, "group_best": 2, "normalize": True,
              "sum_eps": 1e-20, "weight_scale": 1.7, "router_bias": False, "shared": shared}
    part = part_class("feed_forward", "routed_experts")(params, w, parse_dtype("float32" if dtype == torch.float32 else "bfloat16"), DEV)
    h = torch.tensor(rng.normal(size=(n, d)), dtype=torch.float32).to(dtype).to(DEV)
    ctx = StepContext(n_tokens=n, n_seqs=1, token_ids=None, tok_pos=None, tok_slot=None, cu_seqlens=None, seq_slot=None,
                      seq_start=None, new_lens=[n], starts=[0], all_single=False, max_new=n, max_context=n,
                      dtype=part.shared.act_dtype)
    parts = part.apply(h, ctx)
    assert tuple(parts.shape) == (top + 1, n, d)
    got = parts.sum(0).cpu().numpy()
    names = {"m.router": "router", "m.correction": "correction", "m.shared.gate": "shared_gate", "m.shared.up": "shared_up",
             "m.shared.down": "shared_down"}
    for e in range(experts):
        names.update({f"m.e{e}.{r}": f"{r}{e}" for r in ("gate", "up", "down")})
    pw = {k: w[v].float().cpu().numpy().astype(np.float64) for k, v in names.items()}
    mlp = {"kind": "moe", "router": {"experts": experts, "top": top, "scale": 1.7, "groups": {"count": 4, "keep": 2}},
           "shared": {"ff": shared}}
    margins = np.full(n, np.inf)
    want = plain.experts(h.float().cpu().numpy().astype(np.float64), pw, "m.", mlp, margins)
    sure = margins > (1e-4 if dtype == torch.float32 else 0.03)
    assert sure.sum() > n // 2
    _close(got[sure], want[sure], 1e-5 if dtype == torch.float32 else 3e-2)


def test_the_gates_activation_may_be_the_tanh_gelu():
    from xeno_rt_b200.csrc import ops
    rng = np.random.default_rng(7)
    gate_up = rng.normal(0, 3, size=(9, 2 * 20)).astype(np.float32)
    out = torch.empty((9, 20), device=DEV)
    ops.swiglu(out, _t(gate_up), "gelu_tanh")
    _close(out.cpu().numpy(), plain.gelu_tanh(gate_up[:, :20]) * gate_up[:, 20:], 2e-6)
    ops.swiglu(out, _t(gate_up))
    _close(out.cpu().numpy(), plain.silu(gate_up[:, :20]) * gate_up[:, 20:], 2e-6)


@pytest.mark.parametrize("rows", [1, 8, 40, 128, 300])
def test_the_products_that_end_in_a_gate_take_the_tanh_gelu_too(rows):
    """The few-row and the tiled bfloat16 products with the gate in their last step (1 to 16 rows, up to 128 rows, and
    more), through the feed-forward part that picks among them."""
    from xeno_rt_b200.core import parse_dtype
    from xeno_rt_b200.parts import StepContext, part_class
    rng = np.random.default_rng(rows)
    d, inner = 256, 704
    rnd = lambda *shape: torch.tensor(rng.normal(0, 1.5 / np.sqrt(shape[-1]), shape), dtype=torch.float32).to(torch.bfloat16).to(DEV)
    w = {"gate": rnd(inner, d), "up": rnd(inner, d), "down": rnd(d, inner)}
    part = part_class("feed_forward", "swiglu")({"width": d, "inner": inner, "activation": "gelu_tanh"}, w, parse_dtype("bfloat16"), DEV)
    h = torch.tensor(rng.normal(size=(rows, d)), dtype=torch.float32).to(torch.bfloat16).to(DEV)
    ctx = StepContext(n_tokens=rows, n_seqs=1, token_ids=None, tok_pos=None, tok_slot=None, cu_seqlens=None, seq_slot=None,
                      seq_start=None, new_lens=[rows], starts=[0], all_single=False, max_new=rows, max_context=rows,
                      dtype=parse_dtype("bfloat16"))
    got = part.apply(h, ctx).cpu().numpy()
    pw = {"m." + k: v.float().cpu().numpy().astype(np.float64) for k, v in w.items()}
    want = plain.gated(h.float().cpu().numpy().astype(np.float64), pw, "m.", plain.gelu_tanh)
    other = plain.gated(h.float().cpu().numpy().astype(np.float64), pw, "m.", plain.silu)
    _close(got, want, 1.5e-2)
    assert np.abs(other - want).max() > 0.05 * np.abs(want).max()   # the silu gate would be another answer


# ------------------------------------------------------------------------------------------------ small steps
@pytest.mark.parametrize("width", [36, 200, 1500])
def test_the_norm_after_a_sublayer_takes_factors_a_bias_and_a_second_norm(width):
    from xeno_rt_b200.csrc import ops
    rng = np.random.default_rng(width)
    n = 6
    parts = rng.normal(0.5, 2.0, size=(2, n, width)).astype(np.float32)
    scales, bias = np.array([0.4, 1.3], np.float32), rng.normal(size=width).astype(np.float32)
    w1, w2 = rng.normal(1, 0.2, width).astype(np.float32), rng.normal(1, 0.2, width).astype(np.float32)
    residual = rng.normal(size=(n, width)).astype(np.float32)
    y = np.float64(np.float32(0.4)) * parts[0].astype(np.float64) + np.float64(np.float32(1.3)) * parts[1] + bias
    want = residual + 0.8 * plain.rms_norm(y, w1, 1e-5)
    for then_dtype in (torch.float32, torch.bfloat16):
        r, then_out = _t(residual), torch.empty((n, width), dtype=then_dtype, device=DEV)
        ops.rmsnorm_add(r, _t(parts), _t(w1), 1e-5, factor=0.8, part_scales=_t(scales), bias=_t(bias),
                        then=(_t(w2), 1e-6, then_out))
        _close(r.cpu().numpy(), want, 3e-6)
        _close(then_out.float().cpu().numpy(), plain.rms_norm(want, w2, 1e-6), 3e-6 if then_dtype == torch.float32 else 1e-2)


def test_the_embedding_is_scaled_and_a_pass_begins_with_its_row():
    from xeno_rt_b200.csrc import ops
    rng = np.random.default_rng(9)
    table = rng.normal(size=(20, 40)).astype(np.float32)
    out, flag = torch.empty((3, 40), device=DEV), torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.embedding(out, _t(table), _ints([4, 19, 0]), flag, 13.5)
    _close(out.cpu().numpy(), table[[4, 19, 0]] * 13.5, 1e-6)
    row = rng.normal(size=40).astype(np.float32)
    ops.add_row(out, _t(row))
    _close(out.cpu().numpy(), table[[4, 19, 0]] * 13.5 + row, 1e-6)
    assert int(flag[0]) == 0


# ------------------------------------------------------------------------------------------------ each side alone
def _one_layer(left_scale, right_scale, **left_options):
    from sofunex_cases import layer, left, mixer, right
    l = left(4, 2, 16, 24, 0.7, **left_options)
    return {"architecture": "Sofunex", "vocab": 60, "width": 48, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
            "residual_mult": 0.9, "layers": [layer(mixer(l, right(2, 24, 6), left_scale, right_scale), None)]}


@pytest.mark.parametrize("which", ["left", "right"])
def test_each_side_of_the_mixer_alone(tmp_path, which):
    """A model of one layer whose other side has the weight 0; 32-bit; whole, cut and decoded.  The attention side has
    a window of 33 keys that a prompt of 150 tokens passes, three taps and a rotation of half a head; with its q and k
    scaled up one score stands out in every row, so a key that is one place off is another answer."""
    from sofunex_cases import random_weights, write_folder
    from xeno_rt_b200.engine import Engine, StepEntry
    from xeno_rt_b200.engine.model import Model
    config = _one_layer(1.0 if which == "left" else 0.0, 0.0 if which == "left" else 1.0, conv=3, rot=(8, 1000.0),
                        factor=2.0, size=33)
    weights = random_weights(config, 77)
    for name in ("l0.mix.left.q.norm", "l0.mix.left.k.norm"):
        weights[name] = weights[name] * 4.0        # scores of a spread of 16 times the usual: sharp softmaxes
    folder = write_folder(str(tmp_path / which), config, weights)
    tokens = np.random.default_rng(1).integers(0, 60, 150).tolist()
    want = plain.forward(config, weights, tokens)
    other = copy.deepcopy(config)
    other["layers"][0]["mixer"]["left"]["mask"]["size"] = 32
    moved = np.abs(plain.forward(other, weights, tokens) - want).max() / np.abs(want).max()
    assert (moved > 1e-2) == (which == "left")     # the window matters to the attention side alone
    engine = Engine(Model.load(folder, dtype="float32"), 1024)
    for cuts in ([150], [100] + [1] * 50, [2, 31, 1, 33, 64, 19]):
        slot = engine.open_slot()
        rows, at = [], 0
        for cut in cuts:
            rows.append(engine.step([StepEntry(slot, tokens[at:at + cut], list(range(cut)))]).cpu().numpy())
            at += cut
        engine.close_slot(slot)
        err = np.abs(np.concatenate(rows) - want).max() / np.abs(want).max()
        assert err < 3e-5, (which, cuts[:2], err)
    engine.check_errors()
