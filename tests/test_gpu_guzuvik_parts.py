"""The mechanisms of the Guzuvik decoder one by one, each kernel against the plain function of the same mechanism
(tests/plain/guzuvik.py): the token-pair embedding and its state, layer norms with a bias (alone and added into the
stream), the short convolution with a bias, the scalar-decay state-space scan (prompts against single tokens, odd
sizes), the gated group norm, the preparation of attention heads (biases, unit norms, blended values), the scores'
options (window edges, kept first tokens, far keys made to stand out, the cap, the distance slope) in the 32-bit and
the tensor-core kernel, the router and the experts."""
import numpy as np
import pytest
import torch

from plain import guzuvik as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _t(a, dtype=torch.float32):
    return torch.tensor(np.asarray(a), dtype=dtype, device=DEV).contiguous()


def _ints(a):
    return torch.tensor(np.asarray(a), dtype=torch.int32, device=DEV)


def _close(got, want, tol):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert got.shape == want.shape
    assert np.abs(got - want).max() <= tol * max(1.0, np.abs(want).max()), np.abs(got - want).max()


def _bf16(a):
    return torch.tensor(np.asarray(a), dtype=torch.float32).to(torch.bfloat16).float().numpy()


# ------------------------------------------------------------------------------------------------ embedding
@pytest.mark.parametrize("buckets,mul_prev,mul_cur", [(17, 1, 50), (211, 13, 5), (1, 3, 3)])
def test_pair_embedding_in_portions_with_its_state_and_a_slot_used_again(buckets, mul_prev, mul_cur):
    from xeno_rt_b200.csrc import ops
    rng = np.random.default_rng(1)
    vocab, width = 40, 24
    table, pairs = rng.normal(size=(vocab, width)), rng.normal(size=(buckets + 1, width))
    seqs = {3: rng.integers(0, vocab, 11).tolist(), 0: rng.integers(0, vocab, 5).tolist()}
    want = {s: plain.embed(t, table, pairs, buckets, mul_prev, mul_cur) for s, t in seqs.items()}
    state = torch.full((5,), 7, dtype=torch.int32, device=DEV)  # what an earlier user of the slots left there
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    got = {3: [], 0: []}
    # portions: slot 3 brings 4, 1, 6 tokens; slot 0 brings 2, 3 tokens and rides along in the first two steps
    plan = [[(3, 0, 4), (0, 0, 2)], [(0, 2, 5), (3, 4, 5)], [(3, 5, 11)]]
    for step in plan:
        ids, slots, pos, cu, seq_slot = [], [], [], [0], []
        for slot, lo, hi in step:
            ids += seqs[slot][lo:hi]
            slots += [slot] * (hi - lo)
            pos += list(range(lo, hi))
            cu.append(len(ids))
            seq_slot.append(slot)
        ids += [0]            # a padding row: no sequence, zeros, no state touched
        slots += [-1]
        pos += [0]
        out = torch.empty((len(ids), width), device=DEV)
        ops.embedding_pair(out, _t(table), _t(pairs), _ints(ids), _ints(slots), _ints(pos), state, _ints(cu), _ints(seq_slot),
                           mul_prev, mul_cur, flag)
        out = out.cpu().numpy()
        assert not out[-1].any()
        for (slot, lo, hi), a, b in zip(step, cu[:-1], cu[1:]):
            got[slot].append(out[a:b])
    for s in seqs:
        _close(np.concatenate(got[s]), want[s], 1e-6)
    assert int(flag.item()) == 0 and int(state[3]) == seqs[3][-1] and int(state[0]) == seqs[0][-1]


# ------------------------------------------------------------------------------------------------ norms
@pytest.mark.parametrize("width", [36, 320, 1500, 3000, 5000])
def test_layer_norm_with_a_bias_alone_and_added_to_the_stream(width):
    from xeno_rt_b200.csrc import ops
    rng = np.random.default_rng(2)
    x = rng.normal(2.0, 3.0, size=(3, 7, width)).astype(np.float32)
    w, b = rng.normal(1.0, 0.2, width).astype(np.float32), rng.normal(0.0, 0.5, width).astype(np.float32)
    out = torch.empty((7, width), device=DEV)
    ops.layernorm_affine(_t(x[0]), _t(w), _t(b), 1e-5, out=out)
    _close(out.cpu().numpy(), plain.layer_norm(x[0], w, b, 1e-5), 2e-6)
    rows = [5, 0, 5]
    out = torch.empty((3, width), dtype=torch.bfloat16, device=DEV)
    ops.layernorm_affine(_t(x[0]), _t(w), _t(b), 1e-5, out=out, rows=_ints(rows))
    _close(out.float().cpu().numpy(), plain.layer_norm(x[0][rows], w, b, 1e-5), 1e-2)
    residual = rng.normal(size=(7, width)).astype(np.float32)
    r = _t(residual)
    ops.layernorm_affine(_t(x), _t(w), _t(b), 1e-6, residual=r, n_parts=3)  # the parts are added first
    _close(r.cpu().numpy(), residual + plain.layer_norm(x.astype(np.float64).sum(0), w, b, 1e-6), 3e-6)


# ------------------------------------------------------------------------------------------------ state space
def _ssd_inputs(rng, n, heads, vdim, state, groups):
    x = rng.normal(size=(n, heads * vdim))
    b, c = rng.normal(size=(n, groups * state)), rng.normal(size=(n, groups * state))
    raw = rng.normal(size=(n, heads))
    return x, b, c, raw, rng.normal(size=heads), rng.uniform(-4, -1, heads), rng.normal(1.0, 0.5, heads)


@pytest.mark.parametrize("heads,vdim,state,groups", [(3, 8, 16, 1), (4, 20, 5, 2), (2, 64, 128, 2), (6, 4, 48, 6),
                                                     (1, 40, 200, 1)])
def test_scan_of_a_prompt_equals_single_tokens_and_the_plain_recurrence(heads, vdim, state, groups):
    from xeno_rt_b200.csrc import ops
    rng = np.random.default_rng(3)
    lens = [37, 1, 50]
    slots = [4, 0, 2]
    data = [_ssd_inputs(rng, n, heads, vdim, state, groups) for n in lens]
    dt_bias, a_log, d_skip = data[0][4:]
    want = [plain.ssd_scan(x, b, c, plain.softplus(raw + dt_bias), a_log, d_skip, heads, vdim, state, groups)
            for x, b, c, raw, *_ in data]

    def run(portions):
        """``portions``: for every step, how many tokens each sequence brings."""
        st = torch.zeros((5, heads, vdim, state), device=DEV)
        st[1] = 9.0  # a slot that no sequence of the step uses stays as it is
        got, at = [[] for _ in lens], [0] * len(lens)
        for step in portions:
            rows, cu, seq_slot, who = [], [0], [], []
            for i, k in enumerate(step):
                if k:
                    rows.append(np.concatenate([data[i][j][at[i]:at[i] + k] for j in range(4)], axis=1))
                    cu.append(cu[-1] + k)
                    seq_slot.append(slots[i])
                    who.append((i, k))
            cu.append(cu[-1])        # a padding sequence: no slot, no tokens
            seq_slot.append(-1)
            packed = _t(np.concatenate(rows))
            inner, gn = heads * vdim, groups * state
            out = torch.zeros((packed.shape[0], inner), device=DEV)
            ops.ssd_scan(out, packed, packed[:, inner:], packed[:, inner + gn:], packed[:, inner + 2 * gn:], _t(dt_bias),
                         _t(a_log), _t(d_skip), st, _ints(cu), _ints(seq_slot), heads, groups, state, vdim,
                         max_new=max(step))
            out = out.cpu().numpy()
            for (i, k), a in zip(who, cu):
                got[i].append(out[a:a + k])
                at[i] += k
        assert float(st[1].min()) == 9.0
        return [np.concatenate(g) for g in got], st

    whole, st_whole = run([lens])
    for g, w in zip(whole, want):
        _close(g, w, 2e-5)
    cut, st_cut = run([[20, 1, 2], [2, 0, 31], [15, 0, 17]])
    single, st_single = run([[1 if t < n else 0 for n in lens] for t in range(max(lens))])
    for a, b_, c_ in zip(whole, cut, single):  # how the tokens are cut changes nothing at all: the same arithmetic a token
        assert np.array_equal(a, b_) and np.array_equal(a, c_)
    assert torch.equal(st_whole, st_cut) and torch.equal(st_whole, st_single)


def test_convolution_with_a_bias_and_gated_group_norm():
    from xeno_rt_b200.csrc import ops
    rng = np.random.default_rng(4)
    n, channels, taps = 23, 44, 3
    x, w, b = rng.normal(size=(n, channels + 5)), rng.normal(size=(channels, taps)), rng.normal(size=channels)
    want = plain.silu(plain.causal_conv(x[:, 5:], w, b))
    state = torch.zeros((2, taps - 1, channels), device=DEV)
    got = []
    for lo, hi in ((0, 1), (1, 3), (3, 23)):  # portions shorter than the convolution reaches
        out = torch.empty((hi - lo, channels), device=DEV)
        ops.short_conv(out, _t(x[lo:hi])[:, 5:], _t(w), state, _ints([0, hi - lo]), _ints([1]), hi - lo, "silu", bias=_t(b))
        got.append(out.cpu().numpy())
    _close(np.concatenate(got), want, 2e-6)
    for width, groups in ((48, 3), (40, 1), (36, 36)):
        y, z, g = rng.normal(size=(n, width)), rng.normal(size=(n, width + 3)), rng.normal(1.0, 0.3, width)
        out = torch.empty((n, width), device=DEV)
        ops.gated_group_norm(out, _t(y), _t(z)[:, :width], _t(g), groups, 1e-5)
        _close(out.cpu().numpy(), plain.gated_group_norm(y, z[:, :width], g, groups, 1e-5), 3e-6)


# ------------------------------------------------------------------------------------------------ attention
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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,kv,size,window,keep,cap", [(4, 2, 16, 40, 3, 20.0), (6, 2, 32, 90, 70, 4.0),
                                                           (3, 3, 48, 5, 0, 2.0), (2, 1, 64, 64, 64, 30.0),
                                                           (4, 1, 128, 130, 66, 50.0)])
def test_scores_with_a_window_kept_first_tokens_a_cap_and_a_distance_slope(dtype, heads, kv, size, window, keep, cap):
    """Unit-length random q and k would give flat weights that hide a key that is wrongly seen or missed.  So at
    chosen query positions the key just inside the window, the key just outside it, the last kept token and the
    first token that is not kept are each given a key that lines up with the query (a score that stands out) and a
    value of their own; a key seen or missed by one position moves the result by far more than the tolerance.  The
    same holds for a key hundreds of tokens back that only the kept-first rule lets through."""
    from xeno_rt_b200.csrc import ops
    rng = np.random.default_rng(5)
    n = 330
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    m = {"mask": {"size": window, "keep_first": keep}, "scale": 6.0 / np.sqrt(size), "softcap": cap}
    unit = lambda a: a / np.sqrt((a * a).mean(-1, keepdims=True))
    q, k = unit(rng.normal(size=(n, heads, size))), unit(rng.normal(size=(n, kv, size)))
    v = rng.normal(size=(n, kv, size))
    for i in (window + 7, 200, 329):  # queries whose edge keys stand out
        for j in (i - window + 1, i - window, keep - 1, keep):
            if 0 <= j < i:
                k[j] = q[i, ::heads // kv] * 0.98 + 0.02 * k[j]
    if dtype == "bfloat16":
        q, k, v = _bf16(q), _bf16(k), _bf16(v)
    want = plain.attend(q, k, v, m).reshape(n, heads * size)
    blocks_order = [5, 1, 4, 0, 2, 7]  # the sequence's blocks are scattered over the pool
    kp, vp = _cache_of(k, v, kv, size, tdt, blocks_order)
    table = torch.full((3, 8), -1, dtype=torch.int32, device=DEV)
    table[2, :6] = _ints(blocks_order)
    qd = _t(q.reshape(n, heads * size)).to(tdt)
    options = dict(keep_first=keep, softcap=cap, distance_rate=8.0)
    tol = 3e-5 if dtype == "float32" else 2e-2
    out = torch.empty_like(qd)
    ops.attention_reference(out, qd, kp, vp, _ints([2] * n), _ints(range(n)), table, heads, kv, size, m["scale"], window,
                            **options)
    _close(out.float().cpu().numpy(), want, tol)
    if dtype == "bfloat16":
        # the tensor-core kernel: the whole sequence as one step, and its tail as a step that continues it
        for start in (0, 150, 327):
            out = torch.empty((n - start, heads * size), dtype=tdt, device=DEV)
            ops.attention_prefill(out, qd[start:].contiguous(), kp, vp, _ints([0, n - start]), _ints([2]), _ints([start]),
                                  table, n - start, heads, kv, size, m["scale"], window, **options)
            _close(out.float().cpu().numpy(), want[start:], tol)
        # single tokens: every position as a step's one new token, the visible keys cut into stretches or not
        for chunk, splits in ((32, 11), (128, 3), (352, 1)):
            if chunk * splits >= (window + keep if window < n else n):
                out = torch.empty_like(qd)
                slots = _ints([2] * (n - 1) + [-1])  # the last row belongs to no sequence: zeros
                ops.attention_decode_scored(out, qd, kp, vp, slots, _ints(range(n)), table, heads, kv, size, m["scale"],
                                            window, keep, cap, 8.0, chunk, splits)
                got = out.float().cpu().numpy()
                _close(got[:-1], want[:-1], tol)
                assert not got[-1].any()
    # without the options the window alone decides: the kept first tokens must then be gone
    if keep and window + keep < n:
        plain_m = {"mask": {"size": window, "keep_first": 0}, "scale": m["scale"], "softcap": cap}
        assert np.abs(plain.attend(q, k, v, plain_m).reshape(n, -1)[-1] - want[-1]).max() > 1e-3


def test_heads_are_prepared_with_biases_unit_norms_and_blended_values():
    from xeno_rt_b200.csrc import ops
    rng = np.random.default_rng(6)
    n, heads, kv, dim, vdim, size = 9, 4, 2, 24, 40, 48  # heads laid out at 48: dims beyond the true sizes are zero
    row = heads * size + 2 * kv * size
    qkv = np.zeros((n, row + 3))
    bias = np.zeros(row)
    true = {}
    for name, at, count, d in (("q", 0, heads, dim), ("k", heads * size, kv, dim), ("v", (heads + kv) * size, kv, vdim)):
        x, b = rng.normal(size=(n, count, d)), rng.normal(size=(count, d))
        true[name] = x + b
        for h in range(count):
            qkv[:, at + h * size: at + h * size + d] = x[:, h]
            bias[at + h * size: at + h * size + d] = b[h]
    first = rng.normal(size=(n, kv * vdim))
    lam = 0.37
    pools = [torch.zeros((2, kv, 64, size), device=DEV) for _ in range(2)]
    table = _ints([[1, 0]])
    q_out = torch.empty((n, heads * size), device=DEV)
    keep = torch.zeros((n, kv * vdim), device=DEV)
    pos = list(range(60, 60 + n))  # across a block's edge
    ops.qkv_heads_write(q_out, pools[0], pools[1], _t(qkv), heads * size, (heads + kv) * size, _t(bias), True, dim, 1e-5,
                        _ints([0] * n), _ints(pos), table, heads, kv, size, v_keep=keep, v_first=_t(first), v_blend=lam,
                        v_dim=vdim)
    _close(q_out.cpu().numpy().reshape(n, heads, size)[:, :, :dim], plain.unit_rms(true["q"], 1e-5), 2e-6)
    assert not q_out.cpu().numpy().reshape(n, heads, size)[:, :, dim:].any()
    _close(keep.cpu().numpy(), true["v"].reshape(n, -1), 1e-6)
    for i, p in enumerate(pos):
        blk = [1, 0][p // 64]
        _close(pools[0][blk, :, p % 64, :dim].cpu().numpy(), plain.unit_rms(true["k"][i], 1e-5), 2e-6)
        _close(pools[1][blk, :, p % 64, :vdim].cpu().numpy(),
               (1 - lam) * true["v"][i] + lam * first[i].reshape(kv, vdim), 2e-6)


# ------------------------------------------------------------------------------------------------ experts
@pytest.mark.parametrize("experts,top", [(6, 2), (40, 1), (3, 3), (70, 40), (16, 3)])
def test_router_picks_the_largest_logits_and_weighs_them_alone(experts, top):
    from xeno_rt_b200.csrc import ops
    rng = np.random.default_rng(7)
    n = 50
    logits, bias = rng.normal(0, 2, size=(n, experts)).astype(np.float32), rng.normal(size=experts).astype(np.float32)
    logits[3, :] = 0.25  # all equal: the lower numbers win
    ids = torch.empty((n, top), dtype=torch.int32, device=DEV)
    weights = torch.empty((n, top), device=DEV)
    ops.moe_route(ids, weights, _t(logits), _t(bias), top)
    z = logits.astype(np.float64) + bias
    order = np.argsort(-z, axis=-1, kind="stable")[:, :top]
    assert np.array_equal(ids.cpu().numpy(), order)
    zc = np.take_along_axis(z, order, -1)
    e = np.exp(zc - zc.max(-1, keepdims=True))
    _close(weights.cpu().numpy(), e / e.sum(-1, keepdims=True), 2e-6)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width,ff,experts,top,limit", [(36, 12, 5, 2, 0.7), (64, 24, 6, 6, 7.0), (200, 33, 40, 1, 2.0)])
def test_experts_against_the_plain_experts(dtype, width, ff, experts, top, limit):
    from xeno_rt_b200.csrc import ops
    rng = np.random.default_rng(8)
    n = 21
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    rnd = (lambda a: a) if dtype == "float32" else _bf16
    h = rnd(rng.normal(size=(n, width)))
    gate, up = rnd(rng.normal(0, 2 / np.sqrt(width), (experts, ff, width))), rnd(rng.normal(0, 2 / np.sqrt(width), (experts, ff, width)))
    down = rnd(rng.normal(0, 1 / np.sqrt(ff), (experts, width, ff)))
    ids = np.stack([rng.permutation(experts)[:top] for _ in range(n)]).astype(np.int32)
    weights = rng.uniform(0.1, 1.0, size=(n, top)).astype(np.float32)
    want = np.zeros((n, width))
    for t in range(n):
        for e, p in zip(ids[t], weights[t]):
            want[t] += p * plain.expert(h[t].astype(np.float64), gate[e], up[e], down[e], limit)
    w_in = np.concatenate([np.concatenate([gate[e], up[e]]) for e in range(experts)])
    out = torch.empty((top, n, width), device=DEV)
    ops.moe_experts(out, _t(h).to(tdt), _t(w_in).to(tdt), _t(down.reshape(experts * width, ff)).to(tdt), _ints(ids),
                    _t(weights), ff, limit, 1.702)
    _close(out.sum(0).cpu().numpy(), want, 2e-5)  # the kernels keep 32-bit inside in both dtypes


@pytest.mark.parametrize("width,ff,experts,top,n", [(64, 24, 6, 2, 230), (200, 72, 40, 1, 150), (256, 64, 8, 3, 333),
                                                     (72, 136, 3, 3, 70)])
def test_experts_of_many_tokens_sorted_by_expert_in_one_launch_a_product(width, ff, experts, top, n):
    """The path of long steps in bfloat16: rows sorted by expert, both products for all experts in one launch each
    (experts without a row, row counts that are no multiple of the tile, widths that are no multiple of the K step)."""
    from xeno_rt_b200.csrc import ops
    rng = np.random.default_rng(9)
    limit = 1.5
    h = _bf16(rng.normal(size=(n, width)))
    gate, up = _bf16(rng.normal(0, 2 / np.sqrt(width), (experts, ff, width))), _bf16(rng.normal(0, 2 / np.sqrt(width), (experts, ff, width)))
    down = _bf16(rng.normal(0, 1 / np.sqrt(ff), (experts, width, ff)))
    usable = [e for e in range(experts) if e != 1] if experts > top + 1 else list(range(experts))  # expert 1 gets no row
    ids = np.stack([rng.permutation(usable)[:top] for _ in range(n)]).astype(np.int32)
    weights = rng.uniform(0.1, 1.0, size=(n, top)).astype(np.float32)
    want = np.zeros((n, width))
    for t in range(n):
        for e, p in zip(ids[t], weights[t]):
            want[t] += p * plain.expert(h[t].astype(np.float64), gate[e], up[e], down[e], limit)
    bf = torch.bfloat16
    w_in = _t(np.concatenate([np.concatenate([gate[e], up[e]]) for e in range(experts)])).to(bf)
    w_out = _t(down.reshape(experts * width, ff)).to(bf)
    offsets = torch.empty((experts + 1,), dtype=torch.int32, device=DEV)
    pos = torch.empty((n * top,), dtype=torch.int32, device=DEV)
    row_token = torch.empty((n * top,), dtype=torch.int32, device=DEV)
    ops.moe_group(offsets, pos, row_token, _ints(ids), experts)
    counts = np.bincount(ids.reshape(-1), minlength=experts)
    assert offsets.cpu().tolist() == [0] + np.cumsum(counts).tolist()
    assert sorted(pos.cpu().tolist()) == list(range(n * top))
    assert (row_token.cpu().numpy()[pos.cpu().numpy()] == np.repeat(np.arange(n), top)).all()
    rows = torch.empty((n * top, width), dtype=bf, device=DEV)
    ops.moe_gather(rows, _t(h).to(bf), row_token)
    act = torch.empty((n * top, ff), dtype=bf, device=DEV)
    y = torch.empty((n * top, width), device=DEV)
    ops.moe_grouped_product(act, rows, w_in, offsets, experts, ff, limit, 1.702)
    ops.moe_grouped_product(y, act, w_out, offsets, experts)
    out = torch.empty((top, n, width), device=DEV)
    ops.moe_combine(out, y, pos, _t(weights))
    _close(out.sum(0).cpu().numpy(), want, 1.5e-2)  # the hidden units are rounded to bfloat16 between the products
    # and the kernels of few tokens give the same up to that rounding
    few = torch.empty((top, n, width), device=DEV)
    ops.moe_experts(few, _t(h).to(bf), w_in, w_out, _ints(ids), _t(weights), ff, limit, 1.702)
    _close(out.sum(0).cpu().numpy(), few.sum(0).cpu().numpy(), 1.5e-2)
