"""Each mechanism of the recurrent and sink-attention layers alone: the kernel against a float64
restatement, at sizes of its own, with inputs made so that a fault shows (a far key that dominates,
a sink that takes most of the weight, states that are not zero, sequences shorter than the
convolution's memory)."""
from __future__ import annotations

import math

import pytest
import torch

import plain_famalorn as plain

pytestmark = pytest.mark.gpu

DEV = "cuda"


def randn(*shape, seed, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed), dtype=torch.float32) * scale


def slices(x: torch.Tensor, n: int, seed: int) -> torch.Tensor:
    """x as n partial sums [n, ...] that add up to it (up to float32 rounding of the last one)."""
    parts = [randn(*x.shape, seed=seed + i) for i in range(n - 1)]
    return torch.stack(parts + [x - sum(parts)] if parts else [x])


def cu_of(news):
    return torch.tensor([0] + torch.tensor(news).cumsum(0).tolist(), dtype=torch.int32, device=DEV)


# ---------------------------------------------------------------------------------- norms
@pytest.mark.parametrize("hidden", [72, 96, 333, 4100])
@pytest.mark.parametrize("splits", [0, 1, 3])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_layer_norm_with_residual_add(hidden, splits, out_dtype):
    from thintensor_b200.kernels import api

    rows = 7
    residual = randn(rows, hidden, seed=1) + 3.0            # a mean far from zero: forgetting to take it off shows
    delta = randn(splits, rows, hidden, seed=2) if splits else None
    weight, bias = 1.0 + randn(hidden, seed=3, scale=0.2), randn(hidden, seed=4, scale=0.3)
    total = residual.double() + (delta.double().sum(0) if splits else 0.0)
    for use_bias in (False, True):
        res = residual.clone().to(DEV)
        out = torch.empty(rows, hidden, dtype=out_dtype, device=DEV)
        api.add_layernorm(res, delta.to(DEV) if splits else None, weight.to(DEV), bias.to(DEV) if use_bias else None, 1e-5, out)
        want = plain.layer_norm(total, weight.double(), 1e-5) + (bias.double() if use_bias else 0.0)
        tol = 2e-5 if out_dtype == torch.float32 else 2e-2
        assert float((out.double().cpu() - want).abs().max()) <= tol * float(want.abs().max())
        assert float((res.double().cpu() - total).abs().max()) <= 1e-5
    # wanted rows only: the stream stays as it is
    res = residual.clone().to(DEV)
    pick = torch.tensor([5, 0, 5], dtype=torch.int32, device=DEV)
    out = torch.empty(3, hidden, dtype=out_dtype, device=DEV)
    api.add_layernorm(res, delta.to(DEV) if splits else None, weight.to(DEV), None, 1e-5, out, pick)
    want = plain.layer_norm(total[[5, 0, 5]], weight.double(), 1e-5)
    assert float((out.double().cpu() - want).abs().max()) <= (2e-5 if out_dtype == torch.float32 else 2e-2) * float(want.abs().max())
    assert torch.equal(res.cpu(), residual)


@pytest.mark.parametrize("activation", ["silu", "relu", "gelu_tanh"])
def test_gate_activations(activation):
    from thintensor_b200.kernels import api

    tokens, inter = 5, 77
    gate_up = randn(2, tokens, 2 * inter, seed=5, scale=2.0)
    act = torch.empty(tokens, inter, dtype=torch.float32, device=DEV)
    api.swiglu(gate_up.to(DEV), act, activation)
    g, u = gate_up.double().sum(0)[:, :inter], gate_up.double().sum(0)[:, inter:]
    f = {"silu": plain.silu, "relu": torch.relu,
         "gelu_tanh": lambda z: 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))}[activation]
    assert float((act.double().cpu() - f(g) * u).abs().max()) <= 1e-5


def test_weighted_pair():
    from thintensor_b200.kernels import api

    a, b = randn(3, 6, 50, seed=6), randn(1, 6, 50, seed=7)
    out = torch.empty(1, 6, 50, dtype=torch.float32, device=DEV)
    api.weighted_pair(a.to(DEV), 0.8, b.to(DEV), -1.7, out)
    assert float((out[0].double().cpu() - (0.8 * a.double().sum(0) - 1.7 * b.double()[0])).abs().max()) <= 1e-5


# ---------------------------------------------------------------------------- convolution
@pytest.mark.parametrize("taps", [1, 2, 4, 5])
@pytest.mark.parametrize("splits", [1, 3])
def test_causal_conv_carries_its_inputs(taps, splits):
    """Three steps of a batch whose sequences bring fewer tokens than the convolution remembers, exactly as many, and
    many more; then one token each.  The state of a slot that another test run left is not zero, slot order is mixed."""
    from thintensor_b200.kernels import api

    channels, before, off = 150, 9, 9
    cols = before + channels + 4
    weight, bias = randn(channels, taps, seed=10), randn(channels, seed=11)
    slot_ids = [4, 0, 2]
    state = torch.zeros(6, taps - 1, channels, dtype=torch.float32, device=DEV)
    history = {s: randn(taps - 1, channels, seed=20 + s) for s in slot_ids}
    for s in slot_ids:
        state[s] = history[s].to(DEV)
    slots = torch.tensor(slot_ids, dtype=torch.int32, device=DEV)
    for step, news in enumerate([[1, taps - 1 or 1, 40], [2, 1, 3], [1, 1, 1], [1, 1, 1]]):
        tokens = sum(news)
        x = randn(tokens, cols, seed=30 + step)
        out = torch.empty(tokens, channels, dtype=torch.float32, device=DEV)
        one_each = step >= 2
        api.causal_conv(slices(x, splits, 40 + step).to(DEV), off, channels, weight.to(DEV), bias.to(DEV), True, state, out, cu_of(news),
                        slots, len(news), tokens, one_each)
        at = 0
        for s, n in zip(slot_ids, news):
            full = torch.cat([history[s], x[at: at + n, off: off + channels]]).double()
            want = plain.silu(plain.causal_conv(full, weight.double(), bias.double()))[taps - 1:]
            assert float((out[at: at + n].double().cpu() - want).abs().max()) <= 2e-5, (taps, step, s)
            history[s] = full[full.shape[0] - (taps - 1):].float()
            at += n
    if taps > 1:
        for s in slot_ids:
            assert float((state[s].cpu() - history[s]).abs().max()) <= 1e-5
        assert float(state[[1, 3, 5]].abs().max()) == 0.0        # other slots are not touched


# ----------------------------------------------------------------------------- recurrences
def mamba2_plain(x, B, C, dt, a_log, d_skip, S0):
    """x [T, H, P], B and C [T, G, N], dt [T, H] (after softplus), S0 [H, N, P] -> y [T, H, P], S."""
    T, H, P = x.shape
    G = B.shape[1]
    y = torch.zeros(T, H, P, dtype=torch.float64)
    S = S0.clone()
    for h in range(H):
        g = h // (H // G)
        for t in range(T):
            S[h] = torch.exp(-torch.exp(a_log[h]) * dt[t, h]) * S[h] + dt[t, h] * torch.outer(B[t, g], x[t, h])
            y[t, h] = S[h].T @ C[t, g] + d_skip[h] * x[t, h]
    return y, S


@pytest.mark.parametrize("form", ["narrow", "wide"])
@pytest.mark.parametrize("heads,P,N,groups", [(4, 16, 24, 2), (2, 40, 72, 1), (3, 8, 136, 3), (6, 33, 5, 2), (2, 70, 128, 2)])
def test_mamba2_scan(heads, P, N, groups, form):
    """Both forms of the kernel (one column per lane group, or four; more than 128 state rows always run the first)."""
    from thintensor_b200.kernels import api

    inner, news, slot_ids = heads * P, [37, 1, 16], [3, 1, 0]
    tokens = sum(news)
    xbc = randn(tokens, inner + 2 * groups * N, seed=50)
    cols, dt_col = heads + 5, 3
    raw = randn(tokens, cols, seed=51, scale=2.0)
    dt_bias, a_log, d_skip = randn(heads, seed=52), randn(heads, seed=53), randn(heads, seed=54)
    state = randn(5, heads, P, N, seed=55).to(DEV)
    before = state.clone()
    y = torch.empty(tokens, inner, dtype=torch.float32, device=DEV)
    api.mamba2_scan(xbc.to(DEV), slices(raw, 2, 56).to(DEV), dt_col, dt_bias.to(DEV), a_log.to(DEV), d_skip.to(DEV), state, y, cu_of(news),
                    torch.tensor(slot_ids, dtype=torch.int32, device=DEV), len(news), heads, P, N, groups, form)
    at = 0
    for s, n in zip(slot_ids, news):
        rows = xbc[at: at + n].double()
        x = rows[:, :inner].reshape(n, heads, P)
        B = rows[:, inner: inner + groups * N].reshape(n, groups, N)
        C = rows[:, inner + groups * N:].reshape(n, groups, N)
        dt = plain.softplus(raw[at: at + n, dt_col: dt_col + heads].double() + dt_bias.double())
        want, S = mamba2_plain(x, B, C, dt, a_log.double(), d_skip.double(), before[s].double().cpu().transpose(1, 2))
        assert float((y[at: at + n].double().cpu().reshape(n, heads, P) - want).abs().max()) <= 2e-5 * max(1.0, float(want.abs().max()))
        assert float((state[s].double().cpu().transpose(1, 2) - S).abs().max()) <= 2e-5 * max(1.0, float(S.abs().max()))
        at += n
    assert torch.equal(state[[2, 4]], before[[2, 4]])


@pytest.mark.parametrize("form", ["narrow", "wide"])
@pytest.mark.parametrize("heads,qk_heads,D,V", [(4, 2, 24, 40), (3, 1, 136, 8), (2, 2, 16, 16), (6, 3, 72, 33), (2, 1, 128, 70)])
def test_delta_scan(heads, qk_heads, D, V, form):
    from thintensor_b200.kernels import api

    news, slot_ids = [29, 1, 16], [2, 0, 1]
    tokens = sum(news)
    qkv = randn(tokens, 2 * qk_heads * D + heads * V, seed=60)
    cols, b_col, a_col = 2 * heads + 7, 2, heads + 4
    raw = randn(tokens, cols, seed=61, scale=2.0)
    dt_bias, a_log = randn(heads, seed=62), randn(heads, seed=63) - 1.0
    state = randn(4, heads, V, D, seed=64).to(DEV)
    before = state.clone()
    out = torch.empty(tokens, heads * V, dtype=torch.float32, device=DEV)
    api.delta_scan(qkv.to(DEV), slices(raw, 3, 65).to(DEV), b_col, a_col, dt_bias.to(DEV), a_log.to(DEV), state, out, cu_of(news),
                   torch.tensor(slot_ids, dtype=torch.int32, device=DEV), len(news), heads, qk_heads, D, V, form)
    at = 0
    for s, n in zip(slot_ids, news):
        rows = qkv[at: at + n].double()
        q = rows[:, : qk_heads * D].reshape(n, qk_heads, D)
        k = rows[:, qk_heads * D: 2 * qk_heads * D].reshape(n, qk_heads, D)
        v = rows[:, 2 * qk_heads * D:].reshape(n, heads, V)
        q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
        k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
        beta = torch.sigmoid(raw[at: at + n, b_col: b_col + heads].double())
        decay = torch.exp(-torch.exp(a_log.double()) * plain.softplus(raw[at: at + n, a_col: a_col + heads].double() + dt_bias.double()))
        S = before[s].double().cpu().transpose(1, 2).clone()            # [heads, D, V]
        want = torch.zeros(n, heads, V, dtype=torch.float64)
        for h in range(heads):
            g = h // (heads // qk_heads)
            for t in range(n):
                S[h] = decay[t, h] * S[h]
                u = beta[t, h] * (v[t, h] - S[h].T @ k[t, g])
                S[h] = S[h] + torch.outer(k[t, g], u)
                want[t, h] = S[h].T @ q[t, g]
        assert float((out[at: at + n].double().cpu().reshape(n, heads, V) - want).abs().max()) <= 2e-5 * max(1.0, float(want.abs().max()))
        assert float((state[s].double().cpu().transpose(1, 2) - S).abs().max()) <= 2e-5 * max(1.0, float(S.abs().max()))
        at += n
    assert torch.equal(state[3], before[3])


@pytest.mark.parametrize("gate_first", [True, False])
@pytest.mark.parametrize("width,group,weight_len", [(96, 96, 96), (96, 24, 96), (120, 40, 40), (4096, 2048, 4096)])
def test_gated_group_norm(gate_first, width, group, weight_len):
    from thintensor_b200.kernels import api

    tokens, gate_col = 6, 3
    y = randn(tokens, width, seed=70, scale=3.0)
    raw = randn(tokens, width + 9, seed=71, scale=2.0)
    weight = 1.0 + randn(weight_len, seed=72, scale=0.3)
    for out_dtype in (torch.float32, torch.bfloat16):
        out = torch.empty(tokens, width, dtype=out_dtype, device=DEV)
        api.gated_group_norm(y.to(DEV), group, slices(raw, 2, 73).to(DEV), gate_col, weight.to(DEV), 1e-5, gate_first, out)
        gate = plain.silu(raw[:, gate_col: gate_col + width].double())
        w = weight.double().repeat(width // weight_len)
        v = y.double() * gate if gate_first else y.double()
        want = plain.rms(v.reshape(tokens, width // group, group), 1e-5).reshape(tokens, width) * w
        if not gate_first:
            want = want * gate
        tol = 3e-5 if out_dtype == torch.float32 else 2e-2
        assert float((out.double().cpu() - want).abs().max()) <= tol * float(want.abs().max())


# ------------------------------------------------------------------- attention with a sink
def build_cache(totals, kv_heads, dim, vdim, dtype, seed):
    """Block pools whose blocks are handed out in a scrambled order, and the keys / values they hold."""
    blocks_per = [-(-n // 64) for n in totals]
    pool = sum(blocks_per) + 3
    order = torch.randperm(pool, generator=torch.Generator().manual_seed(seed)).tolist()
    k_pool = torch.zeros(pool, kv_heads, 64, dim, dtype=dtype, device=DEV)
    v_pool = torch.zeros(pool, kv_heads, vdim, 64, dtype=dtype, device=DEV)
    table = torch.full((len(totals), max(blocks_per)), -1, dtype=torch.int32)
    at = 0
    for b, blocks in enumerate(blocks_per):
        for j in range(blocks):
            table[b, j] = order[at]
            at += 1
    return k_pool, v_pool, table.to(DEV)


def sink_attention_plain(q, k, v, sinks, scale, group):
    """q [H, D] at the last position over k [n, G, D], v [n, G, V] -> [H, V]."""
    out = []
    for h in range(q.shape[0]):
        s = (k[:, h // group] @ q[h]) * scale
        m = torch.maximum(s.max(), sinks[h]) if sinks is not None else s.max()
        e = torch.exp(s - m)
        out.append((e[:, None] * v[:, h // group]).sum(0) / (e.sum() + (torch.exp(sinks[h] - m) if sinks is not None else 0.0)))
    return torch.stack(out)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("unit_norm", [False, True])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,rot,interleaved", [(4, 2, 32, 24, 16, True), (6, 1, 20, 36, 0, True), (3, 3, 16, 16, 16, True),
                                                                     (6, 2, 96, 40, 48, True), (2, 1, 24, 24, 12, False),
                                                                     (8, 2, 64, 64, 32, True), (4, 1, 128, 128, 128, True)])
@pytest.mark.parametrize("kernels", ["exact", "tensor"])
def test_norm_rotation_append_and_sink_attention(dtype, unit_norm, heads, kv_heads, dim, vdim, rot, interleaved, kernels):
    """Prompts go through the norm / rotation / append kernel into a scrambled cache and then attend; afterwards one token
    each is decoded with the keys cut into slices.  Head 1's sink is made to take nearly all of its weight.  With
    ``unit_norm`` (norm weights of one, under which norm and rotation commute) the key at position 3 of the longest
    sequence is made the decoded token's query of head 0 turned back by 697 positions, so that after both rotations the
    two coincide and that one far key out of 700 dominates the head."""
    from thintensor_b200.kernels import api

    if kernels == "tensor" and not (dim == vdim and api.attention_tcgen05_supports(dtype, heads, kv_heads, dim)):
        pytest.skip("the tensor-core kernels take bfloat16 with key and value heads of 64 or 128")
    totals = [700, 1, 65, 128]
    eps, scale, base = 1e-5, min(1.0, 32.0 / dim), 10000.0       # scores of up to 32: the aligned far key stands out of 700 others
    group = heads // kv_heads
    k_pool, v_pool, table = build_cache([t + 1 for t in totals], kv_heads, dim, vdim, dtype, seed=80)
    q_norm = torch.ones(dim) if unit_norm else 1.0 + randn(dim, seed=81, scale=0.2)
    k_norm = torch.ones(dim) if unit_norm else 1.0 + randn(dim, seed=82, scale=0.2)
    sinks = randn(heads, seed=83)
    sinks[1] = 60.0
    inv_freq = (base ** (-torch.arange(0, rot, 2, dtype=torch.float64) / rot)).float() if rot else torch.zeros(1)
    cols = heads * dim + kv_heads * (dim + vdim)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)

    def rotate(t, positions):
        if not rot:
            return t
        if interleaved:
            return plain.rotate_interleaved(t, positions, rot, base)
        a = (positions[:, None, None].float() * inv_freq).double()              # angles are float32 by definition
        lo, hi = t[..., : rot // 2], t[..., rot // 2: rot]
        return torch.cat([lo * torch.cos(a) - hi * torch.sin(a), hi * torch.cos(a) + lo * torch.sin(a), t[..., rot:]], -1)

    def prepared(x, first_position):
        """The plain q, k, v of rows x [n, cols] at positions first_position ..."""
        n = x.shape[0]
        q = x[:, : heads * dim].reshape(n, heads, dim).double()
        k = x[:, heads * dim: (heads + kv_heads) * dim].reshape(n, kv_heads, dim).double()
        v = x[:, (heads + kv_heads) * dim:].reshape(n, kv_heads, vdim).double()
        positions = torch.arange(first_position, first_position + n)
        return rotate(plain.rms(q, eps) * q_norm.double(), positions), rotate(plain.rms(k, eps) * k_norm.double(), positions), v

    def run(x, news, befores, decode):
        tokens = x.shape[0]
        q_out = torch.empty(tokens, heads * dim, dtype=dtype, device=DEV)
        cu, before = cu_of(news), torch.tensor(befores, dtype=torch.int32, device=DEV)
        cos_sin = where = None
        if rot and not decode:          # prompts look positions, cosines and sines up in the step's table; decoding computes them
            cos_sin = torch.empty(tokens, rot // 2, 2, dtype=torch.float32, device=DEV)
            where = torch.empty(tokens, 2, dtype=torch.int32, device=DEV)
            api.rope_table(inv_freq.to(DEV), rot, cu, before, len(news), tokens, cos_sin, where)
        api.qk_norm_rope_append(slices(x, 2, 84).to(DEV), q_norm.to(DEV), k_norm.to(DEV), eps, inv_freq.to(DEV), rot, interleaved, 1.0, q_out,
                                k_pool, v_pool, table, cu, before, len(news), tokens, heads, kv_heads, dim, vdim, status, cos_sin, where)
        out = torch.empty(tokens, heads * vdim, dtype=dtype, device=DEV)
        if kernels == "tensor" and not decode:              # prompts: both products on the tcgen05 tensor cores
            api.attention_tcgen05(q_out, k_pool, v_pool, table, cu, before, len(news), tokens, heads, kv_heads, dim, scale, 0, out, status,
                                  sinks=sinks.to(DEV))
            return out.double().cpu().reshape(tokens, heads, vdim)
        results = []
        for splits in ((1, 5, 11) if decode else (1,)):     # 11 slices: more than a cluster combines, so by tickets
            part_acc = torch.empty(tokens * heads * splits * vdim, dtype=torch.float32, device=DEV)
            part_ml = torch.empty(tokens * heads * splits * 2, dtype=torch.float32, device=DEV)
            if kernels == "tensor":
                tickets = torch.zeros(64, dtype=torch.int32, device=DEV) if splits > 8 else None
                api.attention_mma(q_out, k_pool, v_pool, table, cu, before, len(news), tokens, heads, kv_heads, dim, scale, 0, splits, out,
                                  part_acc, part_ml, status, one_token_each=True, tickets=tickets, sinks=sinks.to(DEV))
            else:
                api.attention(q_out, k_pool, v_pool, table, cu, before, len(news), tokens, heads, kv_heads, dim, scale, 0, splits, out,
                              part_acc, part_ml, status, value_dim=vdim, sinks=sinks.to(DEV))
            results.append(out.double().cpu().reshape(tokens, heads, vdim))
        for other in results[1:]:                            # however the keys are cut, the sink counts once
            assert float((other - results[0]).abs().max()) <= (1e-5 if dtype == torch.float32 else 2e-2)
        return results[-1]

    x = randn(sum(totals), cols, seed=85)
    last = randn(len(totals), cols, seed=86)
    if unit_norm:
        turned = rotate(last[0, :dim].double().reshape(1, 1, dim), torch.tensor([totals[0] - 3]))
        x[3, heads * dim: heads * dim + dim] = turned.reshape(dim).float()
    got = run(x, totals, [0] * len(totals), decode=False)
    tol = 3e-5 if dtype == torch.float32 else 4e-2
    keys, values, at = [], [], 0
    for b, n in enumerate(totals):
        q, k, v = prepared(x[at: at + n], 0)
        keys.append(k), values.append(v)
        for t in (0, n // 2, n - 1):
            want = sink_attention_plain(q[t], k[: t + 1], v[: t + 1], sinks.double(), scale, group)
            assert float((got[at + t] - want).abs().max()) <= tol * max(1.0, float(want.abs().max())), (b, t)
        at += n
    got = run(last, [1] * len(totals), totals, decode=True)
    for b, n in enumerate(totals):
        q, k, v = prepared(last[b: b + 1], n)
        k, v = torch.cat([keys[b], k]), torch.cat([values[b], v])
        want = sink_attention_plain(q[0], k, v, sinks.double(), scale, group)
        assert float((got[b] - want).abs().max()) <= tol * max(1.0, float(want.abs().max())), b
        assert float(want[1].abs().max()) < 1e-6             # head 1: the sink has it all
        if unit_norm and b == 0:                              # head 0: the far key has most of it
            assert float((want[0] - values[0][3, 0]).abs().max()) < 0.5 * float(values[0][3, 0].abs().max())
    assert int(status.item()) == 0
