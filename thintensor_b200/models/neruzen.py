"""The Neruzen decoder as a description: which parts each layer has, with what numbers, and what the
checkpoint calls their tensors.

Layers are parallel: one RMS norm (``l<i>.norm1``) whose output the mixer (through a token shift with the blend
weights ``l<i>.shift``) and the feed-forward both read.  The mixer's tensors lie under ``l<i>.mix.``, the mixture of
experts' under ``l<i>.mlp.`` (``e<k>.gate`` / ``up`` / ``down``, ``router``, ``shared.gate`` / ...).  The token table
is ``embed``, the hashed pair table ``bigram``, the last norm ``final.norm`` and the output matrix ``head``.

``lightning`` and ``retention`` are two parameter sets of the linear attention with a fixed decay per head:
lightning passes q, k and v through silu, norms all heads together with a weight and gates with a sigmoid; retention
rotates q and k, scales k by ``dim ** -0.5``, norms each head alone without a weight and gates with silu.
"""
from __future__ import annotations

from ..config.neruzen import ARCHITECTURE, LatentAttentionSizes, LinearAttentionSizes, MoeSizes, NeruzenConfig, Rotation
from ..config.registry import Architecture, register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, Run

LATENT_NAMES = {"dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv", "o": "o"}
LINEAR_NAMES = {"q": "q", "k": "k", "v": "v", "g": "g", "norm": "norm", "out": "o"}
MOE_NAMES = {"router": "router", "expert": "e{}.", "shared": "shared.", "gate": "gate", "up": "up", "down": "down"}


def rope_part(rot: Rotation | None, head_dim: int) -> PartSpec | None:
    if rot is None:
        return None
    return PartSpec("rope", {"head_dim": head_dim, "theta": rot.base, "rotary_dim": rot.dims, "table_precision": "float64"})


def latent_attention_part(config: NeruzenConfig, sizes: LatentAttentionSizes, prefix: str) -> PartSpec:
    return PartSpec("latent_attention", {
        "hidden": config.width, "heads": sizes.heads, "dim": sizes.dim, "rot_dim": sizes.rot_dim, "value_dim": sizes.vdim,
        "q_rank": sizes.q_rank, "kv_rank": sizes.kv_rank, "scale": sizes.scale, "eps": config.eps, "window": sizes.window,
        "position": rope_part(sizes.rot, sizes.rot_dim), "names": LATENT_NAMES}, prefix)


def linear_attention_part(config: NeruzenConfig, kind: str, sizes: LinearAttentionSizes, prefix: str) -> PartSpec:
    params = {"hidden": config.width, "heads": sizes.heads, "key_dim": sizes.dim, "value_dim": sizes.vdim, "decay": sizes.decay,
              "eps": config.eps, "names": LINEAR_NAMES}
    if kind == "lightning":
        params.update({"activation": "silu", "norm": "all", "norm_weight": True, "gate": "sigmoid"})
    else:
        params.update({"position": rope_part(sizes.rot, sizes.dim), "key_scale": sizes.dim ** -0.5, "norm": "head", "norm_weight": False,
                       "gate": "silu"})
    return PartSpec("decay_linear_attention", params, prefix)


def moe_part(config: NeruzenConfig, sizes: MoeSizes, prefix: str) -> PartSpec:
    return PartSpec("moe", {"hidden": config.width, "experts": sizes.experts, "top": sizes.top, "inter": sizes.ff, "groups": sizes.groups,
                            "keep": sizes.keep, "shared_inter": sizes.shared_ff, "activation": "silu", "names": MOE_NAMES}, prefix)


def describe_neruzen(config: NeruzenConfig) -> ModelSpec:
    def norm(prefix: str, name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"dim": config.width, "eps": config.eps, "name": name}, prefix)

    layers = []
    for index, layer in enumerate(config.layers):
        prefix = f"l{index}."
        parts = {"norm": norm(prefix, "norm1"), "shift": PartSpec("token_shift", {"dim": config.width, "name": "shift"}, prefix)}
        if layer.type == "latent_attention":
            parts["mixer"] = latent_attention_part(config, layer.mixer, prefix + "mix.")
        else:
            parts["mixer"] = linear_attention_part(config, layer.type, layer.mixer, prefix + "mix.")
        if layer.mlp is not None:
            parts["ffn"] = moe_part(config, layer.mlp, prefix + "mlp.")
        layers.append(LayerSpec("parallel", parts))
    if config.bigram is not None:
        embedding = PartSpec("table_pair_hash", {"vocab": config.vocab, "hidden": config.width, "buckets": config.bigram.buckets,
                                                 "mul_prev": config.bigram.mul_prev, "mul_cur": config.bigram.mul_cur, "name": "embed",
                                                 "pair_name": "bigram"}, "")
    else:
        embedding = PartSpec("table", {"vocab": config.vocab, "hidden": config.width, "name": "embed"}, "")
    return ModelSpec(
        hidden_size=config.width,
        vocab_size=config.vocab,
        embedding=embedding,
        layers=tuple(layers),
        schedule=tuple(Run(i) for i in range(len(layers))),
        final_norm=norm("final.", "norm"),
        head=PartSpec("linear", {"hidden": config.width, "vocab": config.vocab, "name": "head"}, ""),
    )


register_architecture(Architecture(
    name=ARCHITECTURE,
    model_types=("neruzen",),
    config_class=NeruzenConfig,
    describe=describe_neruzen,
))
