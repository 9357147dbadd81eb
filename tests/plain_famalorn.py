"""Plain, slow implementation of the Famalorn decoder, used only as the test oracle.

Famalorn is a pre-norm decoder whose layers each carry one of three token mixers: a
gated delta-rule recurrence, a Mamba-2 state-space recurrence, or softmax attention
(grouped heads, per-head query/key norm, interleaved partial rotary encoding, a learned
sink in the softmax denominator) running side by side with a Mamba-2 branch.  A layer may
or may not have a dense feed-forward ``down(relu(gate x) * up x)``.  Norms around the
sublayers are weight-only layer norms.

Everything here works on one whole sequence at a time, token by token where the
mechanism is a recurrence, with no cache and no batching.  It shares no code with the
package under test: own config reading, own safetensors reader, one function per
mechanism.  Arithmetic is float64 throughout (``dtype``) except for the rotation's angles
(see ``rotate_interleaved``), so what it returns is the design's value up to the rounding of
the stored weights.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch

# What stands in for the narrowing of activations: None (exact), or a function applied wherever an engine that
# multiplies bfloat16 matrices has to narrow its operand (the input of every projection, queries, keys and values on
# their way to the scores, the read-outs before the output projections).  ``forward(..., narrow=f)`` sets it.
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


def softplus(x):
    return torch.where(x > 30.0, x, torch.log1p(torch.exp(torch.clamp(x, max=30.0))))


def layer_norm(x, w, eps):
    """(x - mean) / sqrt(var + eps) * w over the last axis, var the mean squared deviation."""
    mean = x.mean(-1, keepdim=True)
    var = ((x - mean) ** 2).mean(-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * w


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def causal_conv(x, w, bias=None):
    """x [T, C], w [C, taps]: y[t, c] = sum_j w[c, j] * x[t - (taps - 1) + j, c], zeros before t = 0."""
    T, C = x.shape
    taps = w.shape[1]
    y = torch.zeros_like(x)
    for t in range(T):
        for j in range(taps):
            s = t - (taps - 1) + j
            if s >= 0:
                y[t] += w[:, j] * x[s]
    if bias is not None:
        y = y + bias
    return y


# --------------------------------------------------------------------------- mixers
def mamba2(h, p, w, prefix, eps):
    """h [T, width] -> [T, width].  p: heads, vdim, state, groups, norm_groups, conv."""
    H, P, N, G = p["heads"], p["vdim"], p["state"], p["groups"]
    inner = H * P
    T = h.shape[0]
    proj = nar(h) @ w[prefix + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[prefix + "conv"], w[prefix + "conv.b"]))
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + w[prefix + "dt_bias"])
    decay = torch.exp(-torch.exp(w[prefix + "A_log"]) * dt)              # [T, H]
    y = torch.zeros(T, H, P, dtype=h.dtype)
    for head in range(H):
        g = head // (H // G)
        S = torch.zeros(N, P, dtype=h.dtype)
        for t in range(T):
            S = decay[t, head] * S + dt[t, head] * torch.outer(B[t, g], x[t, head])
            y[t, head] = S.T @ C[t, g] + w[prefix + "D"][head] * x[t, head]
    y = y.reshape(T, inner) * silu(z)
    parts = p["norm_groups"]
    y = rms(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * w[prefix + "norm"]
    return nar(y) @ w[prefix + "o"].T


def rotate_interleaved(x, positions, dims, base):
    """x [T, heads, dim]: pairs (2i, 2i+1) of the first ``dims`` numbers turn by p * base^(-2i/dims).  The design
    computes positions and angles in 32-bit floats, and at a far position an angle rounded there differs from the
    exact one by more than the tests allow; so the frequency is rounded to float32 and so is its product with the
    position, the one place where this file does not work in ``x.dtype``."""
    out = x.clone()
    for i in range(dims // 2):
        a = (positions.to(torch.float32) * torch.tensor(base ** (-2.0 * i / dims), dtype=torch.float32)).to(x.dtype)
        c, s = torch.cos(a)[:, None], torch.sin(a)[:, None]
        u, v = x[:, :, 2 * i], x[:, :, 2 * i + 1]
        out[:, :, 2 * i] = u * c - v * s
        out[:, :, 2 * i + 1] = v * c + u * s
    return out


def sink_attention(h, p, w, prefix, eps):
    H, G, D, V = p["heads"], p["kv_heads"], p["dim"], p["vdim"]
    T = h.shape[0]
    h = nar(h)
    q = (h @ w[prefix + "q"].T).reshape(T, H, D)
    k = (h @ w[prefix + "k"].T).reshape(T, G, D)
    v = nar((h @ w[prefix + "v"].T).reshape(T, G, V))
    q = rms(q, eps) * w[prefix + "q.norm"]
    k = rms(k, eps) * w[prefix + "k.norm"]
    rot = p.get("rot")
    if rot and rot["dims"]:
        pos = torch.arange(T)
        q = rotate_interleaved(q, pos, rot["dims"], rot["base"])
        k = rotate_interleaved(k, pos, rot["dims"], rot["base"])
    q, k = nar(q), nar(k)
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for head in range(H):
        g = head // (H // G)
        sink = w[prefix + "sink"][head]
        for t in range(T):
            s = (k[:t + 1, g] @ q[t, head]) * p["scale"]
            m = torch.maximum(s.max(), sink)
            e = torch.exp(s - m)
            out[t, head] = (e[:, None] * v[:t + 1, g]).sum(0) / (e.sum() + torch.exp(sink - m))
    return nar(out.reshape(T, H * V)) @ w[prefix + "o"].T


def parallel(h, p, w, prefix, eps):
    return (p["left_scale"] * sink_attention(h, p["left"], w, prefix + "left.", eps)
            + p["right_scale"] * mamba2(h, p["right"], w, prefix + "right.", eps))


def gated_delta(h, p, w, prefix, eps):
    H, G, D, V = p["heads"], p["kv_heads"], p["dim"], p["vdim"]
    T = h.shape[0]
    h = nar(h)
    q = silu(causal_conv(h @ w[prefix + "q"].T, w[prefix + "q.conv"])).reshape(T, G, D)
    k = silu(causal_conv(h @ w[prefix + "k"].T, w[prefix + "k.conv"])).reshape(T, G, D)
    v = silu(causal_conv(h @ w[prefix + "v"].T, w[prefix + "v.conv"])).reshape(T, H, V)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[prefix + "b"].T)
    decay = torch.exp(-torch.exp(w[prefix + "A_log"]) * softplus(h @ w[prefix + "a"].T + w[prefix + "dt_bias"]))
    gate = silu(h @ w[prefix + "g"].T).reshape(T, H, V)
    o = torch.zeros(T, H, V, dtype=h.dtype)
    for head in range(H):
        g = head // (H // G)
        S = torch.zeros(D, V, dtype=h.dtype)
        for t in range(T):
            S = decay[t, head] * S
            u = beta[t, head] * (v[t, head] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            o[t, head] = S.T @ q[t, g]
    o = rms(o, eps) * w[prefix + "norm"] * gate
    return nar(o.reshape(T, H * V)) @ w[prefix + "o"].T


def dense_ffn(h, w, prefix):
    h = nar(h)
    return nar(torch.relu(h @ w[prefix + "gate"].T) * (h @ w[prefix + "up"].T)) @ w[prefix + "down"].T


MIXERS = {"mamba2": mamba2, "parallel": parallel, "delta": gated_delta}


# ------------------------------------------------------------------------ whole model
def forward(cfg, w, tokens, dtype=torch.float64, layers_out: list | None = None, narrow=None):
    """Logits [T, vocab] for one whole sequence; ``layers_out`` collects the stream after each layer.  ``narrow``: see
    ``_narrow`` (for measuring how far the rounding of activations alone moves a position's logits)."""
    global _narrow
    _narrow = narrow
    try:
        return _forward(cfg, w, tokens, dtype, layers_out)
    finally:
        _narrow = None


def _forward(cfg, w, tokens, dtype, layers_out):
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    for i, layer in enumerate(cfg["layers"]):
        pre = f"l{i}."
        x = x + MIXERS[layer["type"]](layer_norm(x, w[pre + "norm1"], eps), layer["mixer"], w, pre + "mix.", eps)
        if layer.get("mlp") is not None:
            x = x + dense_ffn(layer_norm(x, w[pre + "norm2"], eps), w, pre + "mlp.")
        if layers_out is not None:
            layers_out.append(x.clone())
    return nar(layer_norm(x, w["final.norm"], eps)) @ w["head"].T
