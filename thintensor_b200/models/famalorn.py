"""The Famalorn decoder as a description: which parts each layer has, with what numbers, and what the
checkpoint calls their tensors.

Layer ``i``'s tensors start with ``l<i>.``: ``norm1`` (and ``norm2`` where the layer has a feed-forward),
the mixer's under ``mix.`` and the feed-forward's under ``mlp.``; a ``parallel`` mixer keeps its attention
branch under ``mix.left.`` and its Mamba-2 branch under ``mix.right.``.  The table is ``embed``, the last
norm ``final.norm`` and the output matrix ``head``.  Norms are weight-only layer norms; the feed-forward
is ``down(relu(gate x) * up x)``.
"""
from __future__ import annotations

from ..config.famalorn import ARCHITECTURE, AttentionSizes, DeltaSizes, FamalornConfig, Mamba2Sizes
from ..config.registry import Architecture, register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, Run

MAMBA2_NAMES = {"in": "in", "conv": "conv", "conv_bias": "conv.b", "dt_bias": "dt_bias", "A_log": "A_log", "D": "D", "norm": "norm",
                "out": "o"}
DELTA_NAMES = {"q": "q", "k": "k", "v": "v", "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv", "b": "b", "a": "a", "g": "g",
               "dt_bias": "dt_bias", "A_log": "A_log", "norm": "norm", "out": "o"}
ATTENTION_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm", "sink": "sink"}
FFN_NAMES = {"gate": "gate", "up": "up", "down": "down"}


def mamba2_part(config: FamalornConfig, sizes: Mamba2Sizes, prefix: str) -> PartSpec:
    return PartSpec("mamba2", {"hidden": config.width, "heads": sizes.heads, "head_dim": sizes.vdim, "state": sizes.state,
                               "groups": sizes.groups, "norm_groups": sizes.norm_groups, "conv": sizes.conv, "eps": config.eps,
                               "names": MAMBA2_NAMES}, prefix)


def delta_part(config: FamalornConfig, sizes: DeltaSizes, prefix: str) -> PartSpec:
    return PartSpec("gated_delta", {"hidden": config.width, "heads": sizes.heads, "qk_heads": sizes.kv_heads, "key_dim": sizes.dim,
                                    "value_dim": sizes.vdim, "conv": sizes.conv, "eps": config.eps, "names": DELTA_NAMES}, prefix)


def attention_part(config: FamalornConfig, sizes: AttentionSizes, prefix: str) -> PartSpec:
    position = None
    if sizes.rot_dims:
        position = PartSpec("rope", {"head_dim": sizes.dim, "theta": sizes.rot_base, "rotary_dim": sizes.rot_dims, "interleaved": True,
                                     "table_precision": "float64"})
    return PartSpec("attention", {"hidden": config.width, "heads": sizes.heads, "kv_heads": sizes.kv_heads, "head_dim": sizes.dim,
                                  "value_dim": sizes.vdim, "position": position, "scale": sizes.scale, "qk_norm_eps": config.eps,
                                  "sink": True, "names": ATTENTION_NAMES}, prefix)


def describe_famalorn(config: FamalornConfig) -> ModelSpec:
    def norm(prefix: str, name: str) -> PartSpec:
        return PartSpec("layernorm", {"dim": config.width, "eps": config.eps, "name": name}, prefix)

    layers = []
    for index, layer in enumerate(config.layers):
        prefix = f"l{index}."
        parts = {"mixer_norm": norm(prefix, "norm1")}
        params = {}
        if layer.type == "parallel":
            arrangement = "pre_norm_pair"
            parts["left"] = attention_part(config, layer.mixer.left, prefix + "mix.left.")
            parts["right"] = mamba2_part(config, layer.mixer.right, prefix + "mix.right.")
            params = {"left_scale": layer.mixer.left_scale, "right_scale": layer.mixer.right_scale}
        else:
            arrangement = "pre_norm"
            make = mamba2_part if layer.type == "mamba2" else delta_part
            parts["mixer"] = make(config, layer.mixer, prefix + "mix.")
        if layer.ff is not None:
            parts["ffn_norm"] = norm(prefix, "norm2")
            parts["ffn"] = PartSpec("swiglu", {"hidden": config.width, "inter": layer.ff, "activation": "relu", "names": FFN_NAMES},
                                    prefix + "mlp.")
        layers.append(LayerSpec(arrangement, parts, params))
    return ModelSpec(
        hidden_size=config.width,
        vocab_size=config.vocab,
        embedding=PartSpec("table", {"vocab": config.vocab, "hidden": config.width, "name": "embed"}, ""),
        layers=tuple(layers),
        schedule=tuple(Run(i) for i in range(len(layers))),
        final_norm=norm("final.", "norm"),
        head=PartSpec("linear", {"hidden": config.width, "vocab": config.vocab, "name": "head"}, ""),
    )


register_architecture(Architecture(
    name=ARCHITECTURE,
    model_types=("famalorn",),
    config_class=FamalornConfig,
    describe=describe_famalorn,
))
