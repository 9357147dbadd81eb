"""Recurrent token mixers: a state of fixed size per sequence instead of keys and values.

Both mixers here share one skeleton.  One matrix product makes everything that is linear in the
normed hidden state; a short causal convolution over time with silu follows on part of it; a
recurrence walks each sequence's tokens and reads out one vector per head; the read-out is gated
and divided by its root mean square in groups; the output projection follows.  What a sequence
carries from step to step are the recurrence's matrix per head (float32) and the last ``conv - 1``
inputs of the convolution (float32), both declared as states, so the cache hands them out per slot,
zeroed for a new sequence, and prompts cut into steps, decoding and batches all continue from them.

``mamba2``: the state-space recurrence of Mamba-2 (Dao and Gu, "Transformers are SSMs").  The input
projection is laid out [z | x | B | C | dt] (z and x ``heads * head_dim`` wide, B and C ``groups *
state`` wide, dt one number per head); x, B and C pass the convolution (with bias) and silu;
``dt = softplus(dt + dt_bias)``; per head, with S of shape state x head_dim,
``S <- exp(-exp(A_log) dt) S + dt B x^T`` and ``y = S^T C + D x``; then ``y * silu(z)`` is divided by
its root mean square in ``norm_groups`` equal parts and multiplied by the norm weight.

``gated_delta``: the gated delta rule (Yang, Kautz and Hatamizadeh, "Gated Delta Networks").  Queries
and keys (``qk_heads`` heads of ``key_dim``) and values (``heads`` heads of ``value_dim``) pass
convolutions of their own (no bias) and silu; q and k become unit vectors per head
(``x / sqrt(sum x^2 + 1e-6)``, q also times ``key_dim ** -0.5``); per head, with S of shape key_dim x
value_dim, ``S <- g S``, ``u = beta (v - S^T k)``, ``S <- S + k u^T``, ``o = S^T q`` with
``beta = sigmoid(W_b h)`` and ``g = exp(-exp(A_log) softplus(W_a h + dt_bias))``; each head's o is
divided by its root mean square, multiplied by a weight of ``value_dim`` numbers that the heads
share, and by ``silu(W_g h)``.

``decay_linear_attention``: linear attention with a fixed decay per head and neither softmax nor
denominator: per head, with S of shape key_dim x value_dim, ``S <- decay_h S + k v^T`` and ``o = S^T q``.
Two published forms are parameter sets of it.  Lightning attention: ``activation="silu"`` on q, k and v,
the read-out of all heads RMS-normed together with a weight (``norm="all"``) and gated by
``sigmoid(W_g h)``.  Retention: q and k rotated by the position (``position``), k times
``key_dim ** -0.5`` (``key_scale``), every head's read-out divided by its own root mean square without a
weight (``norm="head"``) and gated by ``silu(W_g h)``.  There is no convolution; the only state is S.

Decays, step sizes, gates of the recurrence, unit norms and the states are float32 whatever the
model's dtype; only the normed read-out that feeds the output projection is narrowed.
"""
from __future__ import annotations

import torch

from ..kernels import api
from .base import MIXERS, POSITION_ENCODINGS, Delta, Mixer, RotaryTable, StateNeed, WeightDecl
from .linear import Linear
from .spec import PartSpec


def _f32(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.float32).contiguous()


@MIXERS.register("mamba2")
class Mamba2(Mixer):
    NAMES = {"in": "in_proj.weight", "conv": "conv1d.weight", "conv_bias": "conv1d.bias", "dt_bias": "dt_bias", "A_log": "A_log",
             "D": "D", "norm": "norm.weight", "out": "out_proj.weight"}

    def __init__(self, hidden: int, heads: int, head_dim: int, state: int, groups: int = 1, norm_groups: int = 1, conv: int = 4,
                 eps: float = 1e-6, names: dict | None = None):
        self.hidden, self.heads, self.head_dim, self.state = int(hidden), int(heads), int(head_dim), int(state)
        self.groups, self.norm_groups, self.conv, self.eps = int(groups), int(norm_groups), int(conv), float(eps)
        self.inner = self.heads * self.head_dim
        self.channels = self.inner + 2 * self.groups * self.state          # what passes the convolution: x, B, C
        if self.heads % self.groups:
            raise ValueError(f"{heads} heads are not a multiple of {groups} groups")
        if self.inner % self.norm_groups:
            raise ValueError(f"the inner width {self.inner} is not a multiple of {norm_groups} norm groups")
        if not 1 <= self.conv <= 8 or not 1 <= self.state <= 256:
            raise ValueError("the recurrent kernels take 1 to 8 convolution taps and states of up to 256")
        self.names = {**self.NAMES, **(names or {})}
        self.proj: Linear | None = None
        self.out: Linear | None = None

    def weights(self) -> dict[str, WeightDecl]:
        n = self.names
        return {
            n["in"]: WeightDecl((2 * self.inner + 2 * self.groups * self.state + self.heads, self.hidden)),
            n["conv"]: WeightDecl((self.channels, self.conv)),
            n["conv_bias"]: WeightDecl((self.channels,)),
            n["dt_bias"]: WeightDecl((self.heads,)),
            n["A_log"]: WeightDecl((self.heads,)),
            n["D"]: WeightDecl((self.heads,), init="norm"),
            n["norm"]: WeightDecl((self.inner,), init="norm"),
            n["out"]: WeightDecl((self.hidden, self.inner)),
        }

    def state_needs(self) -> list[StateNeed]:
        return [StateNeed((self.heads, self.head_dim, self.state), torch.float32),
                StateNeed((self.conv - 1, self.channels), torch.float32)]

    def bind(self, tensors, dtype, device) -> None:
        n = self.names
        self.proj = Linear(tensors[n["in"]])
        self.out = Linear(tensors[n["out"]])
        self.conv_weight, self.conv_bias = _f32(tensors[n["conv"]]), _f32(tensors[n["conv_bias"]])
        self.dt_bias, self.a_log, self.d_skip = _f32(tensors[n["dt_bias"]]), _f32(tensors[n["A_log"]]), _f32(tensors[n["D"]])
        self.norm = _f32(tensors[n["norm"]])

    def projections(self) -> list:
        return [self.proj, self.out]

    def vectors(self) -> list[torch.Tensor]:
        return [self.conv_weight, self.conv_bias, self.dt_bias, self.a_log, self.d_skip, self.norm]

    def device_driven(self) -> bool:
        return True

    def forward(self, ctx, x, cache, states) -> Delta:
        recurrent, tail = states
        tokens = ctx.n_tokens
        proj = self.proj(ctx, x, "mamba2.in")
        xbc = ctx.scratch("mamba2.xbc", (tokens, self.channels), torch.float32)
        api.causal_conv(proj, self.inner, self.channels, self.conv_weight, self.conv_bias, True, tail, xbc, ctx.cu, ctx.slots,
                        ctx.sequences, tokens, ctx.decode)
        y = ctx.scratch("mamba2.y", (tokens, self.inner), torch.float32)
        api.mamba2_scan(xbc, proj, self.inner + self.channels, self.dt_bias, self.a_log, self.d_skip, recurrent, y, ctx.cu, ctx.slots,
                        ctx.sequences, self.heads, self.head_dim, self.state, self.groups)
        gated = ctx.scratch("mamba2.gated", (tokens, self.inner))
        api.gated_group_norm(y, self.inner // self.norm_groups, proj, 0, self.norm, self.eps, True, gated)
        return self.out.delta(ctx, gated, "mamba2.out")


@MIXERS.register("gated_delta")
class GatedDelta(Mixer):
    NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "q_conv": "q_conv1d.weight", "k_conv": "k_conv1d.weight",
             "v_conv": "v_conv1d.weight", "b": "b_proj.weight", "a": "a_proj.weight", "g": "g_proj.weight", "dt_bias": "dt_bias",
             "A_log": "A_log", "norm": "o_norm.weight", "out": "o_proj.weight"}

    def __init__(self, hidden: int, heads: int, qk_heads: int, key_dim: int, value_dim: int, conv: int = 4, eps: float = 1e-6,
                 names: dict | None = None):
        self.hidden, self.heads, self.qk_heads = int(hidden), int(heads), int(qk_heads)
        self.key_dim, self.value_dim, self.conv, self.eps = int(key_dim), int(value_dim), int(conv), float(eps)
        if self.heads % self.qk_heads:
            raise ValueError(f"{heads} heads are not a multiple of {qk_heads} query/key heads")
        if not 1 <= self.conv <= 8 or not 1 <= self.key_dim <= 256:
            raise ValueError("the recurrent kernels take 1 to 8 convolution taps and key sizes of up to 256")
        self.qk, self.v = self.qk_heads * self.key_dim, self.heads * self.value_dim
        self.channels = 2 * self.qk + self.v                               # what passes the convolutions: q, k, v
        self.names = {**self.NAMES, **(names or {})}
        self.proj: Linear | None = None
        self.out: Linear | None = None

    def weights(self) -> dict[str, WeightDecl]:
        n = self.names
        return {
            n["q"]: WeightDecl((self.qk, self.hidden)),
            n["q_conv"]: WeightDecl((self.qk, self.conv)),
            n["k"]: WeightDecl((self.qk, self.hidden)),
            n["k_conv"]: WeightDecl((self.qk, self.conv)),
            n["v"]: WeightDecl((self.v, self.hidden)),
            n["v_conv"]: WeightDecl((self.v, self.conv)),
            n["b"]: WeightDecl((self.heads, self.hidden)),
            n["A_log"]: WeightDecl((self.heads,)),
            n["norm"]: WeightDecl((self.value_dim,), init="norm"),
            n["a"]: WeightDecl((self.heads, self.hidden)),
            n["dt_bias"]: WeightDecl((self.heads,)),
            n["g"]: WeightDecl((self.v, self.hidden)),
            n["out"]: WeightDecl((self.hidden, self.v)),
        }

    def state_needs(self) -> list[StateNeed]:
        return [StateNeed((self.heads, self.value_dim, self.key_dim), torch.float32),
                StateNeed((self.conv - 1, self.channels), torch.float32)]

    def bind(self, tensors, dtype, device) -> None:
        n = self.names
        # one product for everything linear in the input: [q | k | v | gate | b | a]
        self.proj = Linear(torch.cat([tensors[n[key]] for key in ("q", "k", "v", "g", "b", "a")], dim=0))
        self.out = Linear(tensors[n["out"]])
        self.conv_weight = torch.cat([_f32(tensors[n[key]]) for key in ("q_conv", "k_conv", "v_conv")], dim=0).contiguous()
        self.dt_bias, self.a_log, self.norm = _f32(tensors[n["dt_bias"]]), _f32(tensors[n["A_log"]]), _f32(tensors[n["norm"]])

    def projections(self) -> list:
        return [self.proj, self.out]

    def vectors(self) -> list[torch.Tensor]:
        return [self.conv_weight, self.dt_bias, self.a_log, self.norm]

    def device_driven(self) -> bool:
        return True

    def forward(self, ctx, x, cache, states) -> Delta:
        recurrent, tail = states
        tokens = ctx.n_tokens
        proj = self.proj(ctx, x, "delta.in")
        qkv = ctx.scratch("delta.qkv", (tokens, self.channels), torch.float32)
        api.causal_conv(proj, 0, self.channels, self.conv_weight, None, True, tail, qkv, ctx.cu, ctx.slots, ctx.sequences, tokens, ctx.decode)
        gate_col = self.channels
        read = ctx.scratch("delta.read", (tokens, self.v), torch.float32)
        api.delta_scan(qkv, proj, gate_col + self.v, gate_col + self.v + self.heads, self.dt_bias, self.a_log, recurrent, read, ctx.cu,
                       ctx.slots, ctx.sequences, self.heads, self.qk_heads, self.key_dim, self.value_dim)
        gated = ctx.scratch("delta.gated", (tokens, self.v))
        api.gated_group_norm(read, self.value_dim, proj, gate_col, self.norm, self.eps, False, gated)
        return self.out.delta(ctx, gated, "delta.out")


@MIXERS.register("decay_linear_attention")
class DecayLinearAttention(Mixer):
    NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "g": "g_proj.weight", "norm": "norm.weight",
             "out": "o_proj.weight"}

    def __init__(self, hidden: int, heads: int, key_dim: int, value_dim: int, decay, activation: str | None = None,
                 position: PartSpec | None = None, key_scale: float = 1.0, norm: str = "head", norm_weight: bool = False,
                 gate: str = "silu", eps: float = 1e-6, names: dict | None = None):
        self.hidden, self.heads, self.key_dim, self.value_dim = int(hidden), int(heads), int(key_dim), int(value_dim)
        self.decay = tuple(float(d) for d in decay)
        if len(self.decay) != self.heads:
            raise ValueError(f"{len(self.decay)} decays for {self.heads} heads")
        if activation not in (None, "silu"):
            raise ValueError(f"q, k and v pass silu or nothing, not {activation!r}")
        if norm not in ("head", "all"):
            raise ValueError(f"the read-out is normed per head or over all heads, not {norm!r}")
        if gate not in api.NORM_GATES:
            raise ValueError(f"the gate is one of {sorted(api.NORM_GATES)}, not {gate!r}")
        if not 1 <= self.key_dim <= 256:
            raise ValueError("the recurrent kernels take key sizes of up to 256")
        self.activation, self.key_scale, self.norm, self.norm_weight = activation, float(key_scale), norm, bool(norm_weight)
        self.gate, self.eps = gate, float(eps)
        self.qk, self.v = self.heads * self.key_dim, self.heads * self.value_dim
        self.names = {**self.NAMES, **(names or {})}
        position = position or PartSpec("none", {"head_dim": self.key_dim})
        self.position = POSITION_ENCODINGS.build(position.kind, dict(position.params))
        if self.position.kind not in ("rotary", "none"):
            raise ValueError(f"linear attention applies rotary position encodings or none, not one of kind {self.position.kind!r}")
        self.rot: RotaryTable | None = None
        self.proj: Linear | None = None
        self.out: Linear | None = None

    def weights(self) -> dict[str, WeightDecl]:
        n = self.names
        out = {
            n["q"]: WeightDecl((self.qk, self.hidden)),
            n["k"]: WeightDecl((self.qk, self.hidden)),
            n["v"]: WeightDecl((self.v, self.hidden)),
            n["g"]: WeightDecl((self.v, self.hidden)),
            n["out"]: WeightDecl((self.hidden, self.v)),
        }
        if self.norm_weight:
            out[n["norm"]] = WeightDecl((self.v if self.norm == "all" else self.value_dim,), init="norm")
        return out

    def state_needs(self) -> list[StateNeed]:
        return [StateNeed((self.heads, self.value_dim, self.key_dim), torch.float32)]

    def bind(self, tensors, dtype, device) -> None:
        n = self.names
        self.position.bind({}, dtype, device)
        self.rot = None
        if self.position.kind == "rotary":
            self.rot = self.position.rotary()
            if self.rot.interleaved or self.rot.attention_scaling != 1.0 or self.rot.rotary_dim % 2 or self.rot.rotary_dim > self.key_dim:
                raise ValueError("linear attention rotates halves of an even part of the head and does not scale the rotation")
        # one product for everything linear in the input: [q | k | v | gate]
        self.proj = Linear(torch.cat([tensors[n[key]] for key in ("q", "k", "v", "g")], dim=0))
        self.out = Linear(tensors[n["out"]])
        self.decays = torch.tensor(self.decay, dtype=torch.float32, device=device)
        count = self.v if self.norm == "all" else self.value_dim
        self.norm_w = _f32(tensors[n["norm"]]) if self.norm_weight else torch.ones(count, dtype=torch.float32, device=device)

    def projections(self) -> list:
        return [self.proj, self.out]

    def vectors(self) -> list[torch.Tensor]:
        return [self.norm_w] if self.norm_weight else []

    def device_driven(self) -> bool:
        return True

    def forward(self, ctx, x, cache, states) -> Delta:
        (recurrent,) = states
        tokens = ctx.n_tokens
        proj = self.proj(ctx, x, "linear_attention.in")
        vkq = ctx.scratch("linear_attention.vkq", (tokens, self.v + 2 * self.qk), torch.float32)
        rotary_dim = self.rot.rotary_dim if self.rot is not None else 0
        api.linear_attention_prepare(proj, self.heads, self.key_dim, self.value_dim, self.activation == "silu",
                                     self.rot.inv_freq if rotary_dim else None, rotary_dim, self.key_scale, vkq, ctx.cu, ctx.len_before,
                                     ctx.sequences, tokens)
        read = ctx.scratch("linear_attention.read", (tokens, self.v), torch.float32)
        api.decay_scan(vkq, self.decays, recurrent, read, ctx.cu, ctx.slots, ctx.sequences, self.heads, self.key_dim, self.value_dim)
        gated = ctx.scratch("linear_attention.gated", (tokens, self.v))
        api.gated_group_norm(read, self.v if self.norm == "all" else self.value_dim, proj, 2 * self.qk + self.v, self.norm_w, self.eps,
                             False, gated, self.gate)
        return self.out.delta(ctx, gated, "linear_attention.out")
