"""Plain, slow implementation of the Neruzen decoder, used only as the test oracle.

Neruzen is a decoder whose layers are *parallel*: one RMS norm per layer, and the token mixer and the
feed-forward both read its output and both add into the residual stream.  The mixer reads a *shifted*
input: a learned per-channel blend of this token's normed vector with the previous token's.  The
mixer is one of three: softmax attention over a compressed latent (a low-rank query path, one cached
latent per token that all heads expand into keys and values, one rotated key part shared by all heads,
a sliding window), or one of two linear attentions with a fixed decay per head (``lightning``: silu on
q, k and v, a norm over all heads together, a sigmoid gate; ``retention``: rotated q and k, a norm per
head, a silu gate).  The feed-forward is a mixture of experts with group-limited top-k routing and an
always-on shared expert.  The embedding adds a hashed row for the (previous token, token) pair.

Everything here works on one whole sequence at a time, token by token where the mechanism is a
recurrence, with no cache and no batching.  It shares no code with the package under test: own config
reading, own safetensors reader, one function per mechanism.  Arithmetic is float64 except for the
rotation's angles, which are float32 products of float32 factors like an engine's.
"""
from __future__ import annotations

import json
import struct
from pathlib import Path

import numpy as np
import torch

# What stands in for the narrowing of activations: None (exact), or a function applied wherever an engine that
# multiplies bfloat16 matrices narrows its operand (the input of every projection, cached latents, the read-outs before
# the output projections).  ``forward(..., narrow=f)`` sets it.
_narrow = None


def nar(x):
    return x if _narrow is None else _narrow(x)


_NP = {"F32": np.float32, "F64": np.float64, "F16": np.float16, "I32": np.int32, "I64": np.int64}


def read_safetensors(path) -> dict[str, torch.Tensor]:
    """name -> float64 (or int64) tensor; bfloat16 is widened exactly."""
    data = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", data[:8])
    header = json.loads(data[8:8 + n].decode("utf-8"))
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        raw = data[8 + n + lo:8 + n + hi]
        shape = tuple(meta["shape"])
        if meta["dtype"] == "BF16":
            words = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            array = words.view(np.float32).astype(np.float64)
        else:
            array = np.frombuffer(raw, dtype=np.dtype(_NP[meta["dtype"]]).newbyteorder("<"))
            array = array.astype(np.int64 if meta["dtype"].startswith("I") else np.float64)
        out[name] = torch.from_numpy(array.reshape(shape).copy())
    return out


def read_model(folder):
    folder = Path(folder)
    return json.loads((folder / "config.json").read_text()), read_safetensors(folder / "model.safetensors")


# ------------------------------------------------------------------------- small pieces
def silu(x):
    return x / (1.0 + torch.exp(-x))


def sigmoid(x):
    return 1.0 / (1.0 + torch.exp(-x))


def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) (* w) over the last axis."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def rotate_halves(x, positions, dims, base):
    """Rotate the first ``dims`` numbers of the last axis of x [tokens, ..., n]: number i is paired with number
    i + dims / 2, the pair (u, v) at position p becomes (u cos a - v sin a, v cos a + u sin a), a = p * base^(-2i/dims).
    The angle is a float32 product."""
    half = dims // 2
    freq = (float(base) ** (-torch.arange(0, dims, 2, dtype=torch.float64) / dims)).to(torch.float32)
    angle = (positions.to(torch.float32)[:, None] * freq[None, :]).to(torch.float64)
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    cos, sin = torch.cos(angle).reshape(shape), torch.sin(angle).reshape(shape)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], dim=-1)


# ---------------------------------------------------------------------------- embedding
def embed(tokens, table, bigram, spec):
    """Row ``token`` of the table plus the pair's hashed row of ``bigram``; a sequence's first token takes the last row."""
    x = table[tokens].clone()
    if spec is None:
        return x
    buckets, a, b = spec["buckets"], spec["mul_prev"], spec["mul_cur"]
    for t in range(len(tokens)):
        row = buckets if t == 0 else (int(tokens[t - 1]) * a + int(tokens[t]) * b) % buckets
        x[t] += bigram[row]
    return x


def token_shift(h, mix):
    """h_t + (h_(t-1) - h_t) * mix, with zeros before the first token."""
    before = torch.cat([torch.zeros_like(h[:1]), h[:-1]], dim=0)
    return h + (before - h) * mix


# ------------------------------------------------------------------------------- mixers
def latent_attention(h, w, p, m, eps):
    """Softmax attention whose keys and values are expansions of one latent per token."""
    T = h.shape[0]
    H, D, R, V, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    h = nar(h)
    cq = nar(rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps))
    q = (cq @ w[p + "uq"].T).reshape(T, H, D + R)
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    q_plain, q_rot = q[..., :D], rotate_halves(q[..., D:], pos, rot["dims"], rot["base"])
    down = h @ w[p + "dkv"].T
    c = nar(rms_norm(down[:, :rank], w[p + "dkv.norm"], eps))
    k_rot = nar(rotate_halves(down[:, rank:], pos, rot["dims"], rot["base"]))      # one for all heads
    k_plain = (c @ w[p + "uk"].T).reshape(T, H, D)
    v = (c @ w[p + "uv"].T).reshape(T, H, V)
    window = (m.get("mask") or {}).get("size")
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for t in range(T):
        lo = 0 if not window else max(0, t - window + 1)
        s = (torch.einsum("hd,jhd->hj", q_plain[t], k_plain[lo:t + 1]) + q_rot[t] @ k_rot[lo:t + 1].T) * m["scale"]
        a = torch.softmax(s, dim=-1)
        out[t] = torch.einsum("hj,jhv->hv", a, v[lo:t + 1])
    return nar(out.reshape(T, H * V)) @ w[p + "o"].T


def decayed_outer_product_scan(q, k, v, decay):
    """Per head: S_t = decay * S_(t-1) + k_t v_t^T, o_t = S_t^T q_t.  q, k [T, H, D], v [T, H, V]."""
    T, H, D = q.shape
    S = torch.zeros(H, D, v.shape[-1], dtype=q.dtype)
    out = torch.zeros_like(v)
    g = torch.tensor(decay, dtype=q.dtype)[:, None, None]
    for t in range(T):
        S = g * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return out


def lightning(h, w, p, m, eps):
    T = h.shape[0]
    h = nar(h)
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[p + "q"].T).reshape(T, H, D)
    k = silu(h @ w[p + "k"].T).reshape(T, H, D)
    v = silu(h @ w[p + "v"].T).reshape(T, H, V)
    o = decayed_outer_product_scan(q, k, v, m["decay"]).reshape(T, H * V)
    o = rms_norm(o, w[p + "norm"], eps) * sigmoid(h @ w[p + "g"].T)
    return nar(o) @ w[p + "o"].T


def retention(h, w, p, m, eps):
    T = h.shape[0]
    h = nar(h)
    H, D, V = m["heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = (h @ w[p + "q"].T).reshape(T, H, D)
    k = (h @ w[p + "k"].T).reshape(T, H, D)
    if m.get("rot"):
        q = rotate_halves(q, pos, m["rot"]["dims"], m["rot"]["base"])
        k = rotate_halves(k, pos, m["rot"]["dims"], m["rot"]["base"])
    k = k * D ** -0.5
    v = (h @ w[p + "v"].T).reshape(T, H, V)
    o = rms_norm(decayed_outer_product_scan(q, k, v, m["decay"]), None, eps).reshape(T, H * V)
    return nar(o * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


MIXERS = {"latent_attention": latent_attention, "lightning": lightning, "retention": retention}


# ------------------------------------------------------------------------- feed-forward
def gated_expert(h, w, p):
    return nar(silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(scores, top, groups, keep):
    """The chosen experts of one token and their weights: experts outside the ``keep`` groups with the largest best
    score are out; of the rest the ``top`` largest; weights are the scores over their sum (+ 1e-20)."""
    E = scores.numel()
    size = E // groups
    best = scores.reshape(groups, size).max(dim=1).values
    kept = torch.topk(best, keep).indices.tolist()
    allowed = [e for e in range(E) if e // size in kept]
    chosen = sorted(allowed, key=lambda e: (-float(scores[e]), e))[:top]
    weights = torch.stack([scores[e] for e in chosen])
    return chosen, weights / (weights.sum() + 1e-20)


def mixture(h, w, p, mlp):
    r = mlp["router"]
    h = nar(h)
    groups = r.get("groups") or {"count": 1, "keep": 1}
    scores = torch.softmax(h @ w[p + "router"].T, dim=-1)
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        chosen, weights = route(scores[t], r["top"], groups["count"], groups["keep"])
        for e, g in zip(chosen, weights):
            out[t] += g * gated_expert(h[t:t + 1], w, f"{p}e{e}.")[0]
    if mlp.get("shared"):
        out = out + gated_expert(h, w, p + "shared.")
    return out


# -------------------------------------------------------------------------------- model
def forward(config, w, tokens, dtype=torch.float64, layers_out=None, narrow=None):
    """Logits [tokens, vocab] of one whole sequence.  ``layers_out``: a list that receives the stream after each layer."""
    global _narrow
    _narrow = narrow
    try:
        return _forward(config, w, tokens, dtype, layers_out)
    finally:
        _narrow = None


def _forward(config, w, tokens, dtype, layers_out):
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    eps = config["norm"]["eps"]
    tokens = torch.as_tensor(tokens, dtype=torch.int64)
    x = embed(tokens, w["embed"], w.get("bigram"), (config.get("embedding") or {}).get("bigram"))
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        h = nar(rms_norm(x, w[p + "norm1"], eps))
        add = MIXERS[layer["type"]](token_shift(h, w[p + "shift"]), w, p + "mix.", layer["mixer"], eps)
        if layer.get("mlp") is not None:
            add = add + mixture(h, w, p + "mlp.", layer["mlp"])
        x = x + add
        if layers_out is not None:
            layers_out.append(x.clone())
    return nar(rms_norm(x, w["final.norm"], eps)) @ w["head"].T
