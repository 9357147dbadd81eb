"""The kernels behind the Neruzen parts, each alone against a plain float64 restatement written here, at other sizes
than the engine tests': latent attention through a scrambled cache with one key made to dominate far away, just inside
and just outside the window, in prompts and in decoding with the keys in one and in several slices; the latents' norms,
rotation and cache rows; group-limited top-k routing; the decayed outer-product recurrence from states that are not
zero; the token shift and the pair embedding across steps and reused slots; the sigmoid-gated norm."""
from __future__ import annotations

import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


def i32(values):
    return torch.tensor(values, dtype=torch.int32, device=DEV)


def status():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


def rotate_plain(x, pos, inv_freq, dims):
    """x [..., n] float64 at one position: halves of the first ``dims`` numbers paired."""
    half = dims // 2
    angle = (torch.tensor(float(pos), dtype=torch.float32) * inv_freq.cpu().float()[:half]).double()
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * angle.cos() - v * angle.sin(), v * angle.cos() + u * angle.sin(), x[..., dims:]], dim=-1)


def scrambled_cache(lengths, row, dtype, seed, spare=3):
    """A pool [blocks, 1, 64, row] and a table whose rows name blocks in a shuffled order; returns also rows[b][pos]."""
    g = torch.Generator().manual_seed(seed)
    need = [-(-n // 64) for n in lengths]
    total = sum(need) + spare
    order = torch.randperm(total, generator=g).tolist()
    width = max(need)
    table = torch.full((len(lengths), width), -1, dtype=torch.int32)
    at = 0
    for b, n in enumerate(need):
        for i in range(n):
            table[b, i] = order[at]
            at += 1
    pool = torch.zeros(total, 1, 64, row, dtype=dtype, device=DEV)
    return pool, table.to(DEV)


def fill_cache(pool, table, b, rows):
    """rows [n, row] (float64) into sequence b's cache rows; returns what the cache holds (after its dtype's rounding)."""
    stored = rows.to(pool.dtype)
    for pos in range(rows.shape[0]):
        pool[int(table[b, pos // 64]), 0, pos % 64] = stored[pos].to(DEV)
    return stored.double()


def latent_plain(q, w_key, w_value, cached, pos, heads, dim, rot, vdim, rank, inv_freq, rotary_dim, scale, window):
    """One query token (q float64 [heads * (dim + rot)]) over cached rows [n, rank + rot] (n > pos)."""
    q = q.reshape(heads, dim + rot)
    out = []
    lo = 0 if window <= 0 else max(0, pos - window + 1)
    c, kr = cached[lo:pos + 1, :rank], cached[lo:pos + 1, rank:]
    for h in range(heads):
        k_plain = c @ w_key[h * dim:(h + 1) * dim].T
        q_rot = rotate_plain(q[h, dim:], pos, inv_freq, rotary_dim)
        s = (k_plain @ q[h, :dim] + kr @ q_rot) * scale
        p = torch.softmax(s, dim=0)
        out.append((p @ c) @ w_value[h * vdim:(h + 1) * vdim].T)
    return torch.cat(out)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,dim,rot,vdim,rank,window", [(3, 16, 8, 24, 32, 0), (2, 40, 16, 8, 72, 37), (5, 8, 32, 48, 16, 64), (1, 24, 8, 40, 136, 1),
                                                            (2, 12, 6, 10, 18, 5), (3, 20, 4, 12, 20, 0), (4, 32, 16, 24, 64, 200), (18, 8, 16, 8, 48, 0)])
def test_latent_attention_marked_keys(dtype, heads, dim, rot, vdim, rank, window):
    """Sequences of unequal lengths, prompts (several new tokens) and decoding (one), through a scrambled table.  In every
    sequence one key is made to dominate a head's scores: without a window far back or at a cache block's border; with a
    window just inside the last token's window for one prompt and one decoding sequence, just outside it for the other two."""
    from thintensor_b200.kernels import api

    g = torch.Generator().manual_seed(heads * 100 + rank)
    row = rank + rot
    rotary_dim = rot if rank % 3 else rot // 4 * 2
    inv_freq = (10000.0 ** (-torch.arange(0, max(rotary_dim, 2), 2, dtype=torch.float64) / max(rotary_dim, 2))).float().to(DEV)
    scale = 0.2
    totals, new = [300, 410, 70, 131], [5, 1, 70, 1]
    w_key = torch.randn(heads * dim, rank, generator=g, dtype=torch.float64) * 0.3
    w_value = torch.randn(heads * vdim, rank, generator=g, dtype=torch.float64) * 0.3
    w_key_d, w_value_d = w_key.to(dtype).to(DEV), w_value.to(dtype).to(DEV)
    w_key, w_value = w_key_d.double().cpu(), w_value_d.double().cpu()
    pool, table = scrambled_cache(totals, row, dtype, 7)
    cached, queries = [], []
    for b, n in enumerate(totals):
        rows = torch.randn(n, row, generator=g, dtype=torch.float64)
        q = torch.randn(new[b], heads * (dim + rot), generator=g, dtype=torch.float64)
        last = n - 1
        # without a window: far back, at the last row of a cache block and the first of the next; with one: just inside the last
        # token's window (the first prompt, the second decoding sequence) or just outside it (the others)
        marked = [3, 63, 64, 127][b] if window <= 0 else (last - window + 1 if b in (0, 3) else last - window)
        marked = min(max(marked, 0), last)
        a = w_key[:dim].T @ q[-1].reshape(heads, dim + rot)[0, :dim]                       # head 0 of the last query, folded
        rows[marked, :rank] = a / a.norm() * 25.0 / (scale * a.norm()) * a.norm()           # score of about 25 before the others' noise
        cached.append(fill_cache(pool, table, b, rows))
        queries.append(q)
    q_all = torch.cat(queries).float()
    tokens = q_all.shape[0]
    cu = [0]
    for n in new:
        cu.append(cu[-1] + n)
    before = [t - n for t, n in zip(totals, new)]
    want = []
    for b, n in enumerate(totals):
        for i in range(new[b]):
            want.append(latent_plain(queries[b][i].float().double(), w_key, w_value, cached[b], before[b] + i, heads, dim, rot, vdim, rank,
                                     inv_freq, rotary_dim, scale, window))
    want = torch.stack(want)
    # the marked key matters where it is visible: dropping it from the plain computation moves the first sequence's last token
    shadow = cached[0].clone()
    shadow[3 if window <= 0 else max(totals[0] - window, 0)] = 0.0
    moved = latent_plain(queries[0][-1].float().double(), w_key, w_value, shadow, totals[0] - 1, heads, dim, rot, vdim, rank, inv_freq,
                         rotary_dim, scale, window)
    assert float((moved - want[cu[1] - 1]).abs().max()) > 0.05
    mma = dtype == torch.bfloat16 and api.latent_decode_tensor_cores(dtype, rank, rot)
    for splits in (1, 3) + ((-1,) if mma else ()):
        tensor_cores = splits < 0                               # decoding with the heads as the rows of tensor-core products
        if tensor_cores:
            reach = max(totals) if window <= 0 else min(window, max(totals))
            splits = -(-reach // api.LATENT_DECODE_SLICE)
        if splits > 1 or tensor_cores:
            # slices are for steps of one token per sequence: run the two decoding sequences alone
            pick = [b for b in range(len(new)) if new[b] == 1]
        else:
            pick = list(range(len(new)))
        rows_of = [r for b in pick for r in range(cu[b], cu[b + 1])]
        q_step = q_all[rows_of].unsqueeze(0).contiguous().to(DEV)
        cu_step = [0]
        for b in pick:
            cu_step.append(cu_step[-1] + new[b])
        out = torch.zeros(len(rows_of), heads * vdim, dtype=dtype, device=DEV)
        absorbed = torch.zeros(len(rows_of) * heads * (rank + rot), dtype=torch.float32, device=DEV)
        part_acc = torch.zeros(len(rows_of) * heads * splits * rank, dtype=torch.float32, device=DEV)
        part_ml = torch.zeros(len(rows_of) * heads * splits * 2, dtype=torch.float32, device=DEV)
        word = status()
        api.latent_attention(q_step, w_key_d, w_value_d, pool, table[pick].contiguous(), i32(cu_step), i32([before[b] for b in pick]), len(pick),
                             len(rows_of), heads, dim, rot, vdim, rank, inv_freq, rotary_dim, scale, window, splits, out, absorbed, part_acc, part_ml, word, tensor_cores)
        assert int(word.item()) == 0
        err = (out.double().cpu() - want[rows_of]).abs().max()
        bound = (1e-5 if dtype == torch.float32 else 0.03) * max(1.0, float(want.abs().max()))
        assert float(err) <= bound, f"splits {splits}, tensor cores {tensor_cores}: {float(err):.3e} against logits up to {float(want.abs().max()):.2f}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_prepare_norms_rotates_and_appends(dtype):
    from thintensor_b200.kernels import api

    g = torch.Generator().manual_seed(5)
    q_rank, rank, rot, rotary_dim, eps = 24, 40, 16, 12, 1e-5
    new, before = [3, 1, 66], [62, 130, 0]
    totals = [a + b for a, b in zip(new, before)]
    tokens = sum(new)
    down = torch.randn(3, tokens, q_rank + rank + rot, generator=g)          # three k-slices
    qw, kw = torch.rand(q_rank, generator=g) + 0.5, torch.rand(rank, generator=g) + 0.5
    inv_freq = (500.0 ** (-torch.arange(0, rotary_dim, 2, dtype=torch.float64) / rotary_dim)).float()
    pool, table = scrambled_cache(totals, rank + rot, dtype, 9)
    pool.fill_(7.0)
    q_latent = torch.zeros(tokens, q_rank, dtype=dtype, device=DEV)
    cu = [0, 3, 4, 70]
    word = status()
    api.latent_prepare(down.to(DEV), q_rank, rank, rot, qw.to(DEV), kw.to(DEV), eps, inv_freq.to(DEV), rotary_dim, q_latent, pool, table,
                       i32(cu), i32(before), 3, tokens, word)
    assert int(word.item()) == 0
    x = down.double().sum(0)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    touched = set()
    for b in range(3):
        for i in range(new[b]):
            t, pos = cu[b] + i, before[b] + i
            cq = x[t, :q_rank]
            cq = cq / torch.sqrt((cq * cq).mean() + eps) * qw.double()
            c = x[t, q_rank:q_rank + rank]
            c = c / torch.sqrt((c * c).mean() + eps) * kw.double()
            kr = rotate_plain(x[t, q_rank + rank:], pos, inv_freq, rotary_dim)
            assert float((q_latent[t].double().cpu() - cq).abs().max()) <= tol * float(cq.abs().max())
            block = int(table[b, pos // 64])
            got = pool[block, 0, pos % 64].double().cpu()
            assert float((got - torch.cat([c, kr])).abs().max()) <= tol * 4.0
            touched.add((block, pos % 64))
    for block in range(pool.shape[0]):                                        # nothing else was written
        for r in range(64):
            if (block, r) not in touched:
                assert float((pool[block, 0, r].float() - 7.0).abs().max()) == 0.0


def route_plain(scores, top, groups, keep):
    experts = scores.numel()
    size = experts // groups
    best = scores.reshape(groups, size).max(dim=1).values
    kept = sorted(range(groups), key=lambda gi: (-float(best[gi]), gi))[:keep]
    allowed = [e for e in range(experts) if e // size in kept]
    chosen = sorted(allowed, key=lambda e: (-float(scores[e]), e))[:top]
    w = torch.stack([scores[e] for e in chosen])
    return chosen, w / (w.sum() + 1e-20)


@pytest.mark.parametrize("experts,top,groups,keep", [(12, 3, 3, 2), (7, 7, 1, 1), (64, 6, 8, 3), (5, 1, 5, 1), (40, 2, 4, 4), (130, 9, 2, 1)])
def test_routing(experts, top, groups, keep):
    from thintensor_b200.kernels import api

    g = torch.Generator().manual_seed(experts)
    tokens = 150
    logits = torch.randn(2, tokens, experts, generator=g) * 2.0              # two k-slices
    gates = torch.full((tokens, experts), -1.0, device=DEV)
    chosen = torch.zeros(tokens, top, dtype=torch.int32, device=DEV)
    weights = torch.zeros(tokens, top, device=DEV)
    api.route_topk(logits.to(DEV), top, groups, keep, gates, chosen, weights)
    scores = torch.softmax(logits.sum(0).double(), dim=-1)
    for t in range(tokens):
        ids, w = route_plain(scores[t], top, groups, keep)
        assert chosen[t].tolist() == ids, f"token {t}"
        assert float((weights[t].double().cpu() - w).abs().max()) <= 1e-6
        dense = torch.zeros(experts, dtype=torch.float64)
        dense[ids] = w
        assert float((gates[t].double().cpu() - dense).abs().max()) <= 1e-6
    # the same with the router's product in front, from rows and a matrix in either dtype
    for dtype in (torch.float32, torch.bfloat16):
        x = torch.randn(tokens, 72, generator=g).to(dtype)
        w = (torch.randn(experts, 72, generator=g) * 0.5).to(dtype)
        gates.fill_(-1.0)
        api.route_rows(x.to(DEV), w.to(DEV), top, groups, keep, gates, chosen, weights)
        scores = torch.softmax(x.double() @ w.double().T, dim=-1)
        for t in range(tokens):
            ids, wt = route_plain(scores[t], top, groups, keep)
            assert chosen[t].tolist() == ids, f"token {t}"
            assert float((weights[t].double().cpu() - wt).abs().max()) <= 1e-5
            assert float(gates[t].sum()) == pytest.approx(1.0, abs=1e-5)


def test_expert_columns_are_scaled_and_the_shared_ones_left():
    from thintensor_b200.kernels import api

    g = torch.Generator().manual_seed(2)
    tokens, experts, width, shared = 9, 5, 12, 20
    for dtype in (torch.float32, torch.bfloat16):
        act = torch.randn(tokens, experts * width + shared, generator=g).to(dtype).to(DEV)
        gates = torch.rand(tokens, experts, generator=g).to(DEV)
        want = act.float().clone()
        want[:, :experts * width] = (want[:, :experts * width].reshape(tokens, experts, width) * gates[:, :, None]).reshape(tokens, -1)
        api.scale_expert_columns(act, width, gates)
        assert float((act.float() - want.to(dtype).float()).abs().max()) == 0.0


@pytest.mark.parametrize("heads,key_dim,value_dim", [(2, 24, 40), (1, 136, 8), (3, 72, 72), (4, 8, 36)])
@pytest.mark.parametrize("form", ["narrow", "wide"])
@pytest.mark.parametrize("rotary_dim,activation", [(0, True), (8, False)])
def test_decayed_recurrence_continues_from_states(heads, key_dim, value_dim, form, rotary_dim, activation):
    """Sequences of 1, 2, 17 and 50 new tokens whose states are not zero and whose slots are not in order."""
    from thintensor_b200.kernels import api

    if form == "wide" and key_dim > 128:
        pytest.skip("the form with four columns per lane group holds up to 128 rows")
    g = torch.Generator().manual_seed(heads + key_dim)
    new, before, slots = [1, 17, 2, 50], [9, 0, 300, 64], [5, 0, 3, 1]
    tokens = sum(new)
    qk, hv = heads * key_dim, heads * value_dim
    proj = torch.randn(2, tokens, 2 * qk + 2 * hv + 3, generator=g)          # [q | k | v | gate | something else], two k-slices
    decay = torch.tensor([0.5, 0.97, 1.0, 0.9][:heads])
    state = torch.randn(7, heads, value_dim, key_dim, generator=g)
    inv_freq = (100.0 ** (-torch.arange(0, max(rotary_dim, 2), 2, dtype=torch.float64) / max(rotary_dim, 2))).float()
    k_scale = key_dim ** -0.5 if rotary_dim else 1.0
    cu = [0]
    for n in new:
        cu.append(cu[-1] + n)
    vkq = torch.zeros(tokens, hv + 2 * qk, device=DEV)
    api.linear_attention_prepare(proj.to(DEV), heads, key_dim, value_dim, activation, inv_freq.to(DEV) if rotary_dim else None, rotary_dim,
                                 k_scale, vkq, i32(cu), i32(before), len(new), tokens)
    state_d = state.clone().to(DEV)
    out = torch.zeros(tokens, hv, device=DEV)
    api.decay_scan(vkq, decay.to(DEV), state_d, out, i32(cu), i32(slots), len(new), heads, key_dim, value_dim, form)
    x = proj.double().sum(0)
    act = (lambda z: z / (1.0 + torch.exp(-z))) if activation else (lambda z: z)
    for b in range(len(new)):
        S = state[slots[b]].double().transpose(1, 2).clone()                 # [heads, key_dim, value_dim]
        for i in range(new[b]):
            t, pos = cu[b] + i, before[b] + i
            q = act(x[t, :qk]).reshape(heads, key_dim)
            k = act(x[t, qk:2 * qk]).reshape(heads, key_dim)
            v = act(x[t, 2 * qk:2 * qk + hv]).reshape(heads, value_dim)
            if rotary_dim:
                q, k = rotate_plain(q, pos, inv_freq, rotary_dim), rotate_plain(k, pos, inv_freq, rotary_dim)
            k = k * k_scale
            S = decay.double()[:, None, None] * S + k[:, :, None] * v[:, None, :]
            o = torch.einsum("hdv,hd->hv", S, q).reshape(-1)
            assert float((out[t].double().cpu() - o).abs().max()) <= 2e-4 * max(1.0, float(o.abs().max())), f"sequence {b} token {i}"
        assert float((state_d[slots[b]].double().cpu().transpose(1, 2) - S).abs().max()) <= 2e-4 * max(1.0, float(S.abs().max()))
    for slot in set(range(7)) - set(slots):                                   # other sequences' states are untouched
        assert torch.equal(state_d[slot].cpu(), state[slot])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_token_shift_across_steps_and_slots(dtype):
    from thintensor_b200.kernels import api

    g = torch.Generator().manual_seed(3)
    hidden = 40
    mix = torch.rand(hidden, generator=g)
    state = torch.zeros(4, hidden, device=DEV)
    x1 = torch.randn(6, hidden, generator=g).to(dtype)                        # sequences of 4 and 2 tokens in slots 2 and 0
    x2 = torch.randn(4, hidden, generator=g).to(dtype)                        # then 1 and 3 more
    out1, out2 = torch.zeros(6, hidden, dtype=dtype, device=DEV), torch.zeros(4, hidden, dtype=dtype, device=DEV)
    api.token_shift(x1.to(DEV), mix.to(DEV), state, out1, i32([0, 4, 6]), i32([2, 0]), 2)
    api.token_shift(x2.to(DEV), mix.to(DEV), state, out2, i32([0, 1, 4]), i32([2, 0]), 2)
    first = torch.cat([x1[:4], x2[:1]]).double()
    second = torch.cat([x1[4:], x2[1:]]).double()
    for rows, got in ((first, torch.cat([out1[:4], out2[:1]])), (second, torch.cat([out1[4:], out2[1:]]))):
        before = torch.cat([torch.zeros(1, hidden, dtype=torch.float64), rows[:-1]])
        want = rows + (before - rows) * mix.double()
        assert float((got.double().cpu() - want).abs().max()) <= (1e-6 if dtype == torch.float32 else 2e-2)
    assert float((state[2].cpu().double() - first[-1]).abs().max()) == 0.0 and float(state[1].abs().max()) == 0.0


def test_pair_embedding_across_steps_and_slots():
    from thintensor_b200.kernels import api

    g = torch.Generator().manual_seed(4)
    vocab, hidden, buckets, mul_prev, mul_cur = 50, 24, 13, 1000003, 99991
    table, pairs = torch.randn(vocab, hidden, generator=g).to(DEV), torch.randn(buckets + 1, hidden, generator=g).to(DEV)
    last = torch.zeros(3, dtype=torch.int32, device=DEV)
    first, second = [7, 49, 0, 0, 12], [3, 3, 49]
    word = status()

    def run(tokens, cu, slots):
        out = torch.zeros(len(tokens), hidden, device=DEV)
        api.embed_pair_gather(table, pairs, i32(tokens), i32(cu), i32(slots), len(slots), last, out, buckets, mul_prev, mul_cur, 1.0, word)
        return out.cpu()

    got1 = run(first[:3] + second[:1], [0, 3, 4], [1, 2])
    got2 = run(first[3:] + second[1:], [0, 2, 4], [1, 2])
    assert int(word.item()) == 0
    for tokens, got in ((first, torch.cat([got1[:3], got2[:2]])), (second, torch.cat([got1[3:], got2[2:]]))):
        for t, token in enumerate(tokens):
            row = buckets if t == 0 else (tokens[t - 1] * mul_prev + token * mul_cur) % buckets
            assert float((got[t] - (table[token] + pairs[row]).cpu()).abs().max()) <= 1e-6
    assert last.tolist() == [0, first[-1] + 1, second[-1] + 1]
    last[1] = 0                                                               # the slot is handed out again: a first token once more
    again = run([5], [0, 1], [1])
    assert float((again[0] - (table[5] + pairs[buckets]).cpu()).abs().max()) <= 1e-6


def test_normed_read_out_with_a_sigmoid_gate():
    from thintensor_b200.kernels import api

    g = torch.Generator().manual_seed(6)
    tokens, width, eps = 11, 72, 1e-5
    y = torch.randn(tokens, width, generator=g)
    proj = torch.randn(2, tokens, 10 + width, generator=g)
    weight = torch.rand(width, generator=g) + 0.5
    out = torch.zeros(tokens, width, device=DEV)
    api.gated_group_norm(y.to(DEV), width, proj.to(DEV), 10, weight.to(DEV), eps, False, out, "sigmoid")
    yd = y.double()
    want = yd / torch.sqrt((yd * yd).mean(-1, keepdim=True) + eps) * weight.double() / (1.0 + torch.exp(-proj.double().sum(0)[:, 10:]))
    assert float((out.double().cpu() - want).abs().max()) <= 1e-5
