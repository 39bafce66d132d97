"""The mechanisms of the Zogevik decoder one by one, each kernel or part against the plain function of the same
mechanism (tests/plain/zogevik.py): the norm that follows a sublayer, the whole-projection q/k norm with a rotation
over a part of the head and the cache write, the softmax with a sink under a window (edge keys and far keys made to
stand out, scores so low that the sink takes all), attention that reads another layer's keys, latent attention (its
preparation kernel, the per-head products, and the part in prompts, portions and single tokens across block edges and
window edges), routing by grouped scores, and the gelu experts on both of their paths."""
import numpy as np
import pytest
import torch

from plain import zogevik as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def _t(a, dtype=torch.float32):
    return torch.tensor(np.asarray(a), dtype=dtype, device=DEV).contiguous()


def _ints(a):
    return torch.tensor(np.asarray(a), dtype=torch.int32, device=DEV)


def _close(got, want, tol):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert got.shape == want.shape
    if not got.size:
        return
    assert np.abs(got - want).max() <= tol * max(1.0, np.abs(want).max()), np.abs(got - want).max()


def _bf16(a):
    return torch.tensor(np.asarray(a), dtype=torch.float32).to(torch.bfloat16).float().numpy()


# ------------------------------------------------------------------------------------------------ norms
@pytest.mark.parametrize("width", [36, 64, 320, 1500, 5000])
def test_the_norm_after_a_sublayer_adds_into_the_stream_and_leaves_a_rounded_copy(width):
    from xeno_rt_b200.csrc import ops
    rng = np.random.default_rng(1)
    y = rng.normal(0.5, 3.0, size=(3, 7, width)).astype(np.float32)
    w = rng.normal(1.0, 0.2, width).astype(np.float32)
    residual = rng.normal(size=(7, width)).astype(np.float32)
    r = _t(residual)
    ops.rmsnorm_add(r, _t(y[0]), _t(w), 1e-5)
    want = residual + plain.rms_norm(y[0], w, 1e-5)
    _close(r.cpu().numpy(), want, 2e-6)
    r, copy = _t(residual), torch.empty((7, width), dtype=torch.bfloat16, device=DEV)
    ops.rmsnorm_add(r, _t(y), _t(w), 1e-6, copy=copy)  # the parts are added in index order first
    want = residual + plain.rms_norm(y.astype(np.float64).sum(0), w, 1e-6)
    _close(r.cpu().numpy(), want, 3e-6)
    assert torch.equal(copy, r.to(torch.bfloat16))
    # eps inside the root: rows of tiny numbers are not blown up to unit size
    tiny = np.full((7, width), 1e-4, np.float32)
    r = _t(np.zeros((7, width), np.float32))
    ops.rmsnorm_add(r, _t(tiny), _t(w), 1e-6)
    _close(r.cpu().numpy(), plain.rms_norm(tiny, w, 1e-6), 2e-6)
    assert np.abs(r.cpu().numpy()).max() < 0.2


# ------------------------------------------------------------------------------------------------ attention heads
@pytest.mark.parametrize("heads,kv,dim,vdim,size,rot", [(4, 2, 16, 16, 16, 8), (3, 3, 24, 40, 48, 24), (2, 1, 8, 24, 32, 2),
                                                        (8, 2, 64, 64, 64, 64), (5, 1, 128, 32, 128, 48)])
def test_heads_are_normed_over_the_whole_projection_then_rotated_and_cached(heads, kv, dim, vdim, size, rot):
    """The q and k norms run over all heads of a token at once (with one head larger than the others a per-head norm
    would give other numbers); the rotation pairs entry i with i + rot / 2 and leaves the rest of a head alone; heads are
    laid out at ``size`` with zeros behind their true sizes."""
    from xeno_rt_b200.csrc import ops
    rng = np.random.default_rng(2)
    n, eps, base = 9, 1e-5, 700.0
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "rot": {"dims": rot, "base": base}}
    q, k, v = rng.normal(size=(n, heads, dim)), rng.normal(size=(n, kv, dim)), rng.normal(size=(n, kv, vdim))
    q[:, 0] *= 5.0   # one head is larger: the whole-projection norm shares ONE root mean square among the heads
    k[:, -1] *= 4.0
    wq, wk = rng.normal(1.0, 0.3, heads * dim), rng.normal(1.0, 0.3, kv * dim)
    pos = list(range(60, 60 + n))  # across a block's edge
    row = (heads + 2 * kv) * size
    qkv = np.zeros((n, row + 3))
    for name, at, x, count, d in (("q", 0, q, heads, dim), ("k", heads * size, k, kv, dim), ("v", (heads + kv) * size, v, kv, vdim)):
        for h in range(count):
            qkv[:, at + h * size: at + h * size + d] = x[:, h]
    pad = lambda w, count: np.concatenate([np.concatenate([w[h * dim:(h + 1) * dim], np.zeros(size - dim)]) for h in range(count)])
    freq = base ** (-2.0 * np.arange(rot // 2) / rot)
    ang = (np.asarray(pos, np.float32)[:, None] * freq.astype(np.float32)[None]).astype(np.float64)
    cos_sin = _t(np.stack([np.cos(ang), np.sin(ang)], -1))
    pools = [torch.zeros((2, kv, 64, size), device=DEV) for _ in range(2)]
    table = _ints([[1, 0]])
    q_out = torch.empty((n, heads * size), device=DEV)
    ops.qkv_heads_write(q_out, pools[0], pools[1], _t(qkv), heads * size, (heads + kv) * size, None, False, dim, eps,
                        _ints([0] * n), _ints(pos), table, heads, kv, size, v_dim=vdim, q_norm_w=_t(pad(wq, heads)),
                        k_norm_w=_t(pad(wk, kv)), whole_q=heads * dim, whole_k=kv * dim, cos_sin=cos_sin, pairing="split_half")
    want_q = plain.rms_norm(q.reshape(n, -1), wq, eps).reshape(n, heads, dim)
    want_k = plain.rms_norm(k.reshape(n, -1), wk, eps).reshape(n, kv, dim)
    got_q = q_out.cpu().numpy().reshape(n, heads, size)
    assert not got_q[:, :, dim:].any()
    for i, p in enumerate(pos):
        blk = [1, 0][p // 64]
        for h in range(heads):
            _close(got_q[i, h, :dim], plain.rotate_split_half(want_q[i, h], p, rot, base), 3e-6)
        for g in range(kv):
            _close(pools[0][blk, g, p % 64, :dim].cpu().numpy(), plain.rotate_split_half(want_k[i, g], p, rot, base), 3e-6)
            _close(pools[1][blk, g, p % 64, :vdim].cpu().numpy(), v[i, g], 1e-6)
    # a per-head norm is another function: the test would see it
    per_head = plain.rms_norm(q, wq.reshape(heads, dim), eps)
    assert np.abs(per_head - want_q).max() > 0.3
    # a reader of another layer's keys prepares its queries only and leaves the pools alone
    before = [p.clone() for p in pools]
    q_only = torch.empty_like(q_out)
    ops.qkv_heads_write(q_only, pools[0], pools[1], _t(qkv[:, :heads * size]), 0, 0, None, False, dim, eps, _ints([0] * n),
                        _ints(pos), table, heads, kv, size, v_dim=vdim, write_kv=False, q_norm_w=_t(pad(wq, heads)),
                        whole_q=heads * dim, cos_sin=cos_sin, pairing="split_half")
    assert torch.equal(q_only, q_out) and all(torch.equal(a, b) for a, b in zip(before, pools))


# ------------------------------------------------------------------------------------------------ scores with a sink
def _cache_of(k, v, heads_kv, size, dtype, blocks_order):
    """Pools [blocks, kv heads, 64, size] holding k, v [T, kv heads, size] of ONE sequence in the given blocks."""
    n = k.shape[0]
    n_blocks = max(blocks_order) + 1
    kp = torch.zeros((n_blocks, heads_kv, 64, size), dtype=dtype, device=DEV)
    vp = torch.zeros_like(kp)
    for pos in range(n):
        blk = blocks_order[pos // 64]
        kp[blk, :, pos % 64] = _t(k[pos]).to(dtype)
        vp[blk, :, pos % 64] = _t(v[pos]).to(dtype)
    return kp, vp


def _plain_attend(q, k, v, scale, window, sink):
    n, heads, _ = q.shape
    kv = k.shape[1]
    out = np.zeros((n, heads, v.shape[2]))
    for t in range(n):
        for a in range(heads):
            js = list(plain.visible(t, window))
            p = plain.softmax_weights([q[t, a] @ k[j, a // (heads // kv)] * scale for j in js], sink=sink)
            out[t, a] = sum(pj * v[j, a // (heads // kv)] for pj, j in zip(p, js))
    return out.reshape(n, -1)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,kv,size,window", [(4, 2, 16, 40), (6, 2, 32, 90), (3, 3, 48, 5), (2, 1, 64, 64),
                                                  (6, 1, 96, 130), (4, 1, 128, 1), (2, 2, 32, 0)])
def test_softmax_with_a_sink_under_a_window(dtype, heads, kv, size, window):
    """Random q and k of unit size would give flat weights that hide a key that is wrongly seen or missed.  So at chosen
    query positions the key just inside the window and the key just outside it are given a key that lines up with the
    query (a score that stands out) and a value of their own: a window that is one token off moves the result by far
    more than the tolerance.  Other queries are turned away from all their keys (every score far below 0): there the
    sink holds nearly all of the weight and the result is close to zero, which a softmax without a sink cannot give.
    Window 0 = every key: a key 300 tokens back stands out instead."""
    from xeno_rt_b200.csrc import ops
    rng = np.random.default_rng(5)
    n = 330
    tdt = DT[dtype]
    scale = 6.0 / np.sqrt(size)
    unit = lambda a: a / np.sqrt((a * a).mean(-1, keepdims=True))
    q, k = unit(rng.normal(size=(n, heads, size))), unit(rng.normal(size=(n, kv, size)))
    v = rng.normal(size=(n, kv, size))
    reach = window if window else n
    for i in (reach + 7, 200, 329):  # queries whose edge keys stand out
        for j in (i - reach + 1, i - reach, 3):
            if 0 <= j < i:
                k[j] = q[i % n, ::heads // kv] * 0.98 + 0.02 * k[j]
    # every key gets one common part u (a kv head's own); a lonely query points against it, so far that every key it
    # sees scores -30 or less
    u = unit(rng.normal(size=(kv, size)))
    k = k + 2.0 * u
    lonely = [150, 151, 328]
    for i in lonely:
        js = list(plain.visible(i, window))
        least = min(float(u[g] @ k[j, g]) for j in js for g in range(kv))
        assert least > 0
        q[i] = np.repeat(-u * (30.0 / (least * scale)), heads // kv, axis=0)
    if dtype == "bfloat16":
        q, k, v = _bf16(q), _bf16(k), _bf16(v)
    want = _plain_attend(q, k, v, scale, window, sink=True)
    without = _plain_attend(q, k, v, scale, window, sink=False)
    for i in lonely:
        if np.abs(want[i]).max() < 0.05:
            break
    else:
        raise AssertionError("the inputs do not show the sink")
    assert np.abs(without[i]).max() > 0.2
    blocks_order = [5, 1, 4, 0, 2, 7]  # the sequence's blocks are scattered over the pool
    kp, vp = _cache_of(k, v, kv, size, tdt, blocks_order)
    table = torch.full((3, 8), -1, dtype=torch.int32, device=DEV)
    table[2, :6] = _ints(blocks_order)
    qd = _t(q.reshape(n, heads * size)).to(tdt)
    tol = 3e-5 if dtype == "float32" else 2e-2
    out = torch.empty_like(qd)
    ops.attention_reference(out, qd, kp, vp, _ints([2] * n), _ints(range(n)), table, heads, kv, size, scale, window, sink=0.0)
    _close(out.float().cpu().numpy(), want, tol)
    if dtype == "bfloat16":
        # the tensor-core kernel: the whole sequence as one step, and its tail as a step that continues it
        for start in (0, 150, 327):
            out = torch.empty((n - start, heads * size), dtype=tdt, device=DEV)
            ops.attention_prefill(out, qd[start:].contiguous(), kp, vp, _ints([0, n - start]), _ints([2]), _ints([start]),
                                  table, n - start, heads, kv, size, scale, window, sink=0.0)
            _close(out.float().cpu().numpy(), want[start:], tol)
        # single tokens: every position as a step's one new token, the visible keys cut into stretches or not
        for chunk, splits in ((32, 11), (128, 3), (352, 1)):
            if chunk * splits >= reach + 64:
                out = torch.empty_like(qd)
                slots = _ints([2] * (n - 1) + [-1])  # the last row belongs to no sequence: zeros
                ops.attention_decode_scored(out, qd, kp, vp, slots, _ints(range(n)), table, heads, kv, size, scale, window,
                                            0, 0.0, 0.0, chunk, splits, sink=0.0)
                got = out.float().cpu().numpy()
                _close(got[:-1], want[:-1], tol)
                assert not got[-1].any()
    # the sink's score is a parameter: another value gives the plain weights with exp(s) in the denominator
    out = torch.empty_like(qd)
    ops.attention_reference(out, qd, kp, vp, _ints([2] * n), _ints(range(n)), table, heads, kv, size, scale, window, sink=1.5)
    t = 200
    for a in range(heads):
        js = list(plain.visible(t, window))
        s = np.array([q[t, a] @ k[j, a // (heads // kv)] * scale for j in js])
        mx = max(s.max(), 1.5)
        p = np.exp(s - mx) / (np.exp(s - mx).sum() + np.exp(1.5 - mx))
        _close(out[t].float().cpu().numpy().reshape(heads, size)[a], sum(pj * v[j, a // (heads // kv)] for pj, j in zip(p, js)), tol)


# ------------------------------------------------------------------------------------------------ parts with a cache
def _run_mixer(part, cache, dt, hs, plan, store_of=lambda cache: cache.store(0), owns=True, slots=None):
    """Runs ``part.mix`` over sequences whose inputs are ``hs`` (one [T_i, width] array each); ``plan`` lists for every
    step how many tokens each sequence brings.  Returns the results a sequence and the slots (left open)."""
    from xeno_rt_b200.engine import StepEntry, build_context
    tdt = DT["float32" if dt.name == "F32" else "bfloat16"]
    slots = [cache.open_slot() for _ in hs] if slots is None else slots
    at = [0] * len(hs)
    got = [[] for _ in hs]
    for step in plan:
        live = [(i, k) for i, k in enumerate(step) if k]
        ctx, _ = build_context([StepEntry(slots[i], [0] * k) for i, k in live], cache, 10, dt, DEV)
        cache.flush_tables()
        h = torch.cat([_t(hs[i][at[i]:at[i] + k]) for i, k in live]).to(tdt)
        out = part.mix(h, ctx, store_of(cache), owns).float().cpu().numpy()
        row = 0
        for i, k in live:
            got[i].append(out[row:row + k])
            row += k
            at[i] += k
            if owns:
                cache.advance(slots[i], k)
    return [np.concatenate(g) if g else np.zeros((0, hs[0].shape[1])) for g in got], slots


def _latent_part(dtype, width, m, eps, rng):
    from xeno_rt_b200.core import parse_dtype
    from xeno_rt_b200.parts import part_class
    H, dim, rot, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    mk = lambda rows, cols, s=1.0: _bf16(rng.normal(0, s / np.sqrt(cols), (rows, cols)))
    w = {"q": mk(H * (dim + rot), width, 2.0), "dkv": mk(rank + rot, width, 2.0), "dkv.norm": _bf16(rng.normal(1.0, 0.3, rank)),
         "uk": mk(H * dim, rank), "uv": mk(H * vdim, rank), "o": mk(width, H * vdim)}
    params = {"width": width, "n_heads": H, "head_dim": dim, "rot_dim": rot, "v_head_dim": vdim, "kv_rank": rank, "eps": eps,
              "window": m["mask"]["size"], "scale": m["scale"],
              "position": {"kind": "blended_rotary", "params": {"rope_dim": rot, "base": m["rot"]["base"],
                                                                "pairing": "interleaved", "scaling": None}}}
    names = {"q": "q", "down": "dkv", "down_norm": "dkv.norm", "up_k": "uk", "up_v": "uv", "o": "o"}
    dt = parse_dtype(dtype)
    tensors = {role: _t(w[name]).to(torch.float32 if w[name].ndim == 1 else DT[dtype]) for role, name in names.items()}
    return part_class("mixer", "latent_attention")(params, tensors, dt, DEV), w, dt


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,dim,rot,vdim,rank,window", [(3, 8, 8, 16, 24, 70), (1, 12, 6, 20, 13, 5), (4, 64, 64, 64, 192, 200),
                                                            (2, 16, 4, 8, 12, 1), (8, 32, 16, 32, 48, 64), (2, 24, 2, 40, 5, 129),
                                                            (2, 16, 32, 16, 300, 50), (20, 8, 4, 8, 12, 40)])
def test_latent_attention_in_prompts_portions_and_single_tokens(dtype, heads, dim, rot, vdim, rank, window):
    """The part keeps one row [latent | rotated shared key part] a token and attends in the latent space; the plain
    function builds every head's keys and values from the latent.  Prompts longer than the window and than two cache
    blocks, portions down to two tokens, a second sequence of one token beside it, and the tail token by token."""
    from xeno_rt_b200.cache import Cache
    rng = np.random.default_rng(11)
    width, eps = 72, 1e-5
    m = {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": rank, "rot": {"dims": rot, "base": 300.0},
         "mask": {"size": window}, "scale": 1.5 / np.sqrt(dim + rot)}
    part, w, dt = _latent_part(dtype, width, m, eps, rng)
    lens = [235, 1, 70]
    hs = [_bf16(rng.normal(size=(n, width))) for n in lens]
    wants = [plain.latent_attention(h, w, m, eps) for h in hs]
    need = part.cache_need()
    assert need.n_kv_heads == 1 and need.values_in_keys and need.head_dim == -(-(rank + rot) // 16) * 16
    tol = 3e-5 if dtype == "float32" else 3e-2
    for plan in ([lens], [[2, 1, 3], [1, 0, 2], [60, 0, 59], [3, 0, 6], [150, 0, 0]] + [[1, 0, 0]] * 19,
                 [[200, 0, 64]] + [[1, 0, 1]] * 6 + [[1, 0, 0]] * 29):
        cache = Cache([need], 64 * 8, 1024, dt, DEV)
        got, slots = _run_mixer(part, cache, dt, hs, plan)
        for g, want in zip(got, wants):
            _close(g, want[:len(g)], tol)
        for s in slots:
            cache.close_slot(s)
        cache.check()
        assert cache.blocks_free() == cache.n_blocks


def test_latent_rows_in_the_cache_are_the_normed_latent_and_the_rotated_shared_part():
    from xeno_rt_b200.csrc import ops
    rng = np.random.default_rng(12)
    n, heads, dim, rot, rank, size, eps, base = 7, 3, 8, 6, 13, 32, 1e-5, 50.0
    qd = rng.normal(size=(n, heads * (dim + rot) + 2 + rank + rot))
    down_at = heads * (dim + rot) + 2
    wn = rng.normal(1.0, 0.3, rank)
    pos = list(range(61, 61 + n))
    freq = base ** (-2.0 * np.arange(rot // 2) / rot)
    ang = (np.asarray(pos, np.float32)[:, None] * freq.astype(np.float32)[None]).astype(np.float64)
    pool = torch.full((2, 1, 64, size), 9.0, device=DEV)
    q_rows = torch.full((n, heads * size), 7.0, device=DEV)
    ops.latent_prepare(q_rows, pool, _t(qd), down_at, _t(wn), eps, _t(np.stack([np.cos(ang), np.sin(ang)], -1)),
                       _ints([0] * (n - 1) + [-1]), _ints(pos), _ints([[1, 0]]), heads, dim, rot, rank, size)
    got_q = q_rows.cpu().numpy().reshape(n, heads, size)
    for i, p in enumerate(pos[:-1]):
        row = pool[[1, 0][p // 64], 0, p % 64].cpu().numpy()
        _close(row[:rank], plain.rms_norm(qd[i, down_at:down_at + rank], wn, eps), 2e-6)
        _close(row[rank:rank + rot], plain.rotate_interleaved(qd[i, down_at + rank:down_at + rank + rot], p, rot, base), 3e-6)
        assert not row[rank + rot:].any()
        for h in range(heads):
            part = qd[i, h * (dim + rot) + dim:(h + 1) * (dim + rot)]
            _close(got_q[i, h, rank:rank + rot], plain.rotate_interleaved(part, p, rot, base), 3e-6)
            assert not got_q[i, h, rank + rot:].any() and (got_q[i, h, :rank] == 7.0).all()  # the head product's to write
    assert not got_q[-1].any()                                           # a row of no sequence: zero queries
    p = pos[-1]
    assert (pool[[1, 0][p // 64], 0, p % 64] == 9.0).all()               # and no cache row


@pytest.mark.parametrize("n,heads,rows,k", [(5, 3, 13, 8), (130, 4, 192, 64), (67, 1, 70, 33), (1, 8, 16, 100)])
def test_one_small_product_a_head_inside_wider_rows(n, heads, rows, k):
    from xeno_rt_b200.csrc import ops
    rng = np.random.default_rng(13)
    x_head, out_head, x_off, out_off = k + 5, rows + 3, 2, 1
    x, w = rng.normal(size=(n, heads * x_head)), rng.normal(size=(heads, rows, k))
    want = np.einsum("thk,hnk->thn", x.reshape(n, heads, x_head)[:, :, x_off:x_off + k], w)
    out = torch.full((n, heads * out_head), 5.0, device=DEV)
    ops.head_product(out, out_head, out_off, _t(x), x_head, x_off, _t(w), heads)
    got = out.cpu().numpy().reshape(n, heads, out_head)
    _close(got[:, :, out_off:out_off + rows], want, 3e-6)
    assert (got[:, :, :out_off] == 5.0).all() and (got[:, :, out_off + rows:] == 5.0).all()
    # a 32-bit input under bfloat16 matrices is rounded first, the sums stay 32-bit
    out = torch.zeros((n, heads * out_head), dtype=torch.bfloat16, device=DEV)
    ops.head_product(out, out_head, out_off, _t(x), x_head, x_off, _t(w).to(torch.bfloat16), heads)
    want = np.einsum("thk,hnk->thn", _bf16(x).reshape(n, heads, x_head)[:, :, x_off:x_off + k], _bf16(w))
    _close(out.float().cpu().numpy().reshape(n, heads, out_head)[:, :, out_off:out_off + rows], want, 1e-2)


@pytest.mark.parametrize("x_dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n,heads,rows,k,pad,x_off", [(8, 3, 192, 128, 8, 4), (16, 2, 40, 264, 0, 0), (17, 2, 72, 48, 4, 0),
                                                      (200, 5, 100, 320, 12, 8), (3, 2, 9, 24, 3, 1), (70, 1, 64, 16, 0, 0)])
def test_the_product_a_head_on_the_tensor_cores(x_dtype, n, heads, rows, k, pad, x_off):
    """bfloat16 matrices and results: few rows and many, pieces on 16-byte boundaries (whole vectors) and off them, k
    beyond one stretch of shared memory, outputs that end inside a tile; rows of a step alone give the same bits."""
    from xeno_rt_b200.csrc import ops
    rng = np.random.default_rng(15)
    x_head, out_head, out_off = k + pad, rows + 2, 1
    x, w = _bf16(rng.normal(size=(n, heads * x_head))), _bf16(rng.normal(size=(heads, rows, k)))
    xt = _t(x) if x_dtype == "float32" else _t(x).to(torch.bfloat16)
    wt = _t(w).to(torch.bfloat16)
    want = np.einsum("thk,hnk->thn", x.reshape(n, heads, x_head)[:, :, x_off:x_off + k], w)
    out = torch.full((n, heads * out_head), 5.0, dtype=torch.bfloat16, device=DEV)
    ops.head_product(out, out_head, out_off, xt, x_head, x_off, wt, heads)
    got = out.float().cpu().numpy().reshape(n, heads, out_head)
    _close(got[:, :, out_off:out_off + rows], want, 6e-3)
    assert (got[:, :, :out_off] == 5.0).all() and (got[:, :, out_off + rows:] == 5.0).all()
    alone = torch.zeros((1, heads * out_head), dtype=torch.bfloat16, device=DEV)
    ops.head_product(alone, out_head, out_off, xt[n - 1:].contiguous(), x_head, x_off, wt, heads)
    piece = lambda row: row.reshape(heads, out_head)[:, out_off:out_off + rows]
    assert torch.equal(piece(alone[0]), piece(out[n - 1]))


# ------------------------------------------------------------------------------------------------ shared keys
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("own_window,reader_window,reader_heads", [(70, 20, 3), (40, 130, 6), (64, 64, 3)])
def test_a_layer_reads_the_keys_and_values_another_layer_cached(dtype, own_window, reader_window, reader_heads):
    """The owner writes keys (after norm and rotation) and values; the reader has queries, a window and a scale of its
    own and must leave the cache alone.  The storage keeps the wider of the two windows."""
    from xeno_rt_b200.cache import Cache
    from xeno_rt_b200.core import parse_dtype
    from xeno_rt_b200.parts import part_class
    import dataclasses
    rng = np.random.default_rng(14)
    width, kv, dim, vdim, eps = 40, 3, 24, 40, 1e-6
    rot = {"dims": 12, "base": 900.0}
    dt = parse_dtype(dtype)
    mk = lambda rows, cols, s=1.0: _bf16(rng.normal(0, s / np.sqrt(cols), (rows, cols)))

    def build(heads, window, scale, own):
        w = {"q": mk(heads * dim, width), "q.norm": _bf16(rng.normal(1.0, 0.3, heads * dim)), "o": mk(width, heads * vdim)}
        names = {"q": "q", "q_norm": "q.norm", "o": "o"}
        if own:
            w.update({"k": mk(kv * dim, width), "k.norm": _bf16(rng.normal(1.0, 0.3, kv * dim)), "v": mk(kv * vdim, width)})
            names.update({"k": "k", "k_norm": "k.norm", "v": "v"})
        params = {"width": width, "n_heads": heads, "n_kv_heads": kv, "head_dim": dim, "v_head_dim": vdim, "qk_norm": "whole",
                  "eps": eps, "window": window, "scale": scale, "sink": 0.0, "own_kv": own,
                  "position": {"kind": "blended_rotary", "params": {"rope_dim": rot["dims"], "base": rot["base"],
                                                                    "pairing": "split_half", "scaling": None}}}
        tensors = {role: _t(w[name]).to(torch.float32 if w[name].ndim == 1 else DT[dtype]) for role, name in names.items()}
        m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "rot": rot, "mask": {"size": window}, "scale": scale}
        return part_class("mixer", "attention")(params, tensors, dt, DEV), w, m

    owner, w_own, m_own = build(3, own_window, 0.3, True)
    reader, w_read, m_read = build(reader_heads, reader_window, 0.5, False)
    n = 200
    h_own, h_read = _bf16(rng.normal(size=(n, width))), _bf16(rng.normal(size=(n, width)))
    kept = plain.attention_keys_values(h_own, w_own, m_own, eps)
    want_own = plain.attention(h_own, w_own, m_own, eps, kept)
    want_read = plain.attention(h_read, w_read, m_read, eps, kept)
    need = dataclasses.replace(owner.cache_need(), window=max(own_window, reader_window))
    cache = Cache([need], 64 * 6, 1024, dt, DEV)
    tol = 3e-5 if dtype == "float32" else 3e-2
    from xeno_rt_b200.engine import StepEntry, build_context
    slot = cache.open_slot()
    got_own, got_read, at = [], [], 0
    for k in [131, 2, 3] + [1] * 64:
        ctx, _ = build_context([StepEntry(slot, [0] * k)], cache, 10, dt, DEV)
        cache.flush_tables()
        got_own.append(owner.mix(_t(h_own[at:at + k]).to(DT[dtype]), ctx, cache.store(0), True).float().cpu().numpy())
        snapshot = cache.store(0).k.clone()
        got_read.append(reader.mix(_t(h_read[at:at + k]).to(DT[dtype]), ctx, cache.store(0), False).float().cpu().numpy())
        assert torch.equal(snapshot, cache.store(0).k)
        cache.advance(slot, k)
        at += k
    _close(np.concatenate(got_own), want_own, tol)
    _close(np.concatenate(got_read), want_read, tol)
    cache.check()


# ------------------------------------------------------------------------------------------------ experts
@pytest.mark.parametrize("experts,top,groups,keep", [(8, 2, 4, 2), (40, 1, 5, 5), (3, 3, 1, 1), (6, 2, 3, 1), (16, 4, 2, 1),
                                                     (70, 7, 10, 3), (4, 2, 4, 4), (64, 8, 8, 4)])
def test_routing_by_scores_among_the_best_groups(experts, top, groups, keep):
    from xeno_rt_b200.csrc import ops
    rng = np.random.default_rng(7)
    n = 60
    logits = rng.normal(0, 2, size=(n, experts)).astype(np.float32)
    logits[3, :] = 0.25  # all equal: the lower numbers win, among groups and among experts
    size = experts // groups
    if groups > keep:    # the best expert overall sits in a group whose other experts are poor, and still decides
        logits[4, :] = -1.0
        logits[4, size * (groups - 1)] = 3.0
    ids = torch.empty((n, top), dtype=torch.int32, device=DEV)
    weights = torch.empty((n, top), device=DEV)
    ops.moe_route_scores(ids, weights, _t(logits), top, groups, keep)
    scores = plain.router_scores(logits, np.eye(experts))
    got_ids, got_w = ids.cpu().numpy(), weights.cpu().numpy()
    for t in range(n):
        want = plain.choose(scores[t], top, groups, keep)
        assert got_ids[t].tolist() == want, (t, got_ids[t], want)
        _close(got_w[t], scores[t][want], 2e-6)   # the scores as they are: they do not add up to one
    if top < experts:
        assert got_w.sum(-1).max() < 1.0 - 1e-4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width,ff,experts,top", [(36, 12, 5, 2), (64, 24, 6, 6), (200, 33, 40, 1)])
def test_gelu_experts_against_the_plain_experts(dtype, width, ff, experts, top):
    from xeno_rt_b200.csrc import ops
    rng = np.random.default_rng(8)
    n = 21
    rnd = (lambda a: a) if dtype == "float32" else _bf16
    h = rnd(rng.normal(size=(n, width)))
    up = rnd(rng.normal(0, 2 / np.sqrt(width), (experts, ff, width)))
    down = rnd(rng.normal(0, 1 / np.sqrt(ff), (experts, width, ff)))
    ids = np.stack([rng.permutation(experts)[:top] for _ in range(n)]).astype(np.int32)
    weights = rng.uniform(0.05, 0.6, size=(n, top)).astype(np.float32)
    want = np.zeros((n, width))
    for t in range(n):
        for e, p in zip(ids[t], weights[t]):
            want[t] += p * plain.expert(h[t].astype(np.float64), up[e], down[e])
    out = torch.empty((top, n, width), device=DEV)
    ops.moe_experts(out, _t(h).to(DT[dtype]), _t(up.reshape(experts * ff, width)).to(DT[dtype]),
                    _t(down.reshape(experts * width, ff)).to(DT[dtype]), _ints(ids), _t(weights), ff, act="gelu")
    _close(out.sum(0).cpu().numpy(), want, 2e-5)  # the kernels keep 32-bit inside in both dtypes
    # the tanh form of the gelu is another function: the test would see it
    z = np.linspace(-3, 3, 13)
    tanh_form = 0.5 * z * (1 + np.tanh(np.sqrt(2 / np.pi) * (z + 0.044715 * z ** 3)))
    assert np.abs(tanh_form - plain.gelu_erf(z)).max() > 1e-4


@pytest.mark.parametrize("width,ff,experts,top,n", [(64, 24, 6, 2, 230), (200, 72, 40, 1, 150), (256, 64, 8, 3, 333),
                                                     (72, 136, 3, 3, 70)])
def test_gelu_experts_of_many_tokens_sorted_by_expert(width, ff, experts, top, n):
    from xeno_rt_b200.csrc import ops
    rng = np.random.default_rng(9)
    h = _bf16(rng.normal(size=(n, width)))
    up = _bf16(rng.normal(0, 2 / np.sqrt(width), (experts, ff, width)))
    down = _bf16(rng.normal(0, 1 / np.sqrt(ff), (experts, width, ff)))
    usable = [e for e in range(experts) if e != 1] if experts > top + 1 else list(range(experts))  # expert 1 gets no row
    ids = np.stack([rng.permutation(usable)[:top] for _ in range(n)]).astype(np.int32)
    weights = rng.uniform(0.05, 0.6, size=(n, top)).astype(np.float32)
    want = np.zeros((n, width))
    for t in range(n):
        for e, p in zip(ids[t], weights[t]):
            want[t] += p * plain.expert(h[t].astype(np.float64), up[e], down[e])
    bf = torch.bfloat16
    w_in, w_out = _t(up.reshape(experts * ff, width)).to(bf), _t(down.reshape(experts * width, ff)).to(bf)
    offsets = torch.empty((experts + 1,), dtype=torch.int32, device=DEV)
    pos = torch.empty((n * top,), dtype=torch.int32, device=DEV)
    row_token = torch.empty((n * top,), dtype=torch.int32, device=DEV)
    ops.moe_group(offsets, pos, row_token, _ints(ids), experts)
    rows = torch.empty((n * top, width), dtype=bf, device=DEV)
    ops.moe_gather(rows, _t(h).to(bf), row_token)
    act = torch.empty((n * top, ff), dtype=bf, device=DEV)
    y = torch.empty((n * top, width), device=DEV)
    ops.moe_grouped_product(act, rows, w_in, offsets, experts, ff, act="gelu")
    ops.moe_grouped_product(y, act, w_out, offsets, experts)
    out = torch.empty((top, n, width), device=DEV)
    ops.moe_combine(out, y, pos, _t(weights))
    _close(out.sum(0).cpu().numpy(), want, 1.5e-2)  # the hidden units are rounded to bfloat16 between the products


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_experts_part_routes_and_weighs_as_the_plain_mixture(dtype):
    """The part from router to weighted sum, few tokens (every pair by itself) and many (rows sorted by expert).
    Tokens whose routing is a close call in the compute dtype are left out of the comparison."""
    from xeno_rt_b200.core import parse_dtype
    from xeno_rt_b200.parts import part_class
    rng = np.random.default_rng(10)
    width, ff, experts, top, groups, keep = 64, 24, 12, 3, 4, 2
    w = {"router": _bf16(rng.normal(0, 3 / np.sqrt(width), (experts, width)))}
    tensors = {"router": _t(w["router"]).to(DT[dtype])}
    for e in range(experts):
        w[f"e{e}.up"], w[f"e{e}.down"] = _bf16(rng.normal(0, 2 / np.sqrt(width), (ff, width))), _bf16(rng.normal(0, 1 / np.sqrt(ff), (width, ff)))
        tensors[f"up{e}"], tensors[f"down{e}"] = _t(w[f"e{e}.up"]).to(DT[dtype]), _t(w[f"e{e}.down"]).to(DT[dtype])
    params = {"width": width, "inner": ff, "experts": experts, "top": top, "activation": "gelu", "routing": "scores",
              "groups": groups, "keep_groups": keep, "router_bias": False}
    part = part_class("feed_forward", "routed_experts")(params, tensors, parse_dtype(dtype), DEV)
    mlp = {"router": {"experts": experts, "top": top, "groups": {"count": groups, "keep": keep}}}

    class Ctx:
        all_single, captured = False, False
    for n in (5, 300):
        h = _bf16(rng.normal(size=(n, width)))
        want = plain.moe_ff(h, w, mlp)
        sure = plain.route_margins(h, w["router"], top, groups, keep) > (1e-4 if dtype == "float32" else 2e-2)
        assert sure.sum() > n // 2
        got = part.apply(_t(h).to(DT[dtype]), Ctx()).sum(0).cpu().numpy()
        _close(got[sure], want[sure], 3e-5 if dtype == "float32" else 2e-2)
