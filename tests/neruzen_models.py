"""Tiny Neruzen configurations with random weights for the tests, and the plain implementation's outputs for them.
The configurations differ from one another in every size; between them they cover: one head and several, key, value
and rotated sizes that differ, latents smaller and larger than the heads they expand into, windows shorter than a
cache block, longer than one and none at all, a rotation of part of a retention head and of all of it and none,
decays from fast to very slow, experts in one group and in several of which one or two stay, one choice per token and
several, layers with and without a shared expert and without any feed-forward, a model without the pair table, a model
without any attention layer, and one whose attention heads have the sizes that prompts expand for the tensor cores."""
from __future__ import annotations

import json
from pathlib import Path

import torch


def _moe(experts, top, ff, groups=None, shared=None):
    router = {"experts": experts, "top": top}
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    out = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared:
        out["shared"] = {"ff": shared}
    return out


CONFIGS = {
    # every kind of mixer; the window (21) ends inside the first cache block
    "a": {
        "architecture": "Neruzen", "vocab": 211, "width": 96, "norm": {"eps": 1e-5},
        "embedding": {"bigram": {"buckets": 97, "mul_prev": 7, "mul_cur": 13}},
        "layers": [
            {"type": "latent_attention", "mlp": _moe(6, 2, 40, (3, 2), 56), "mixer": {
                "heads": 3, "dim": 24, "rot_dim": 16, "vdim": 40, "q_rank": 48, "kv_rank": 64, "scale": 0.21, "mask": {"size": 21},
                "rot": {"dims": 16, "base": 10000.0}}},
            {"type": "lightning", "mlp": None, "mixer": {"heads": 3, "dim": 24, "vdim": 40, "decay": [0.5, 0.9, 0.995]}},
            {"type": "retention", "mlp": _moe(4, 1, 72, None, None), "mixer": {
                "heads": 2, "dim": 40, "vdim": 24, "decay": [0.97, 0.999], "rot": {"dims": 16, "base": 500.0}}},
        ],
    },
    # no attention anywhere and no pair table: the cache holds states only
    "b": {
        "architecture": "Neruzen", "vocab": 130, "width": 64, "norm": {"eps": 1e-6},
        "layers": [
            {"type": "retention", "mlp": _moe(8, 3, 24, (2, 1), 32), "mixer": {"heads": 1, "dim": 136, "vdim": 8, "decay": [0.9375]}},
            {"type": "lightning", "mlp": _moe(5, 5, 16, (1, 1), None), "mixer": {"heads": 4, "dim": 8, "vdim": 36, "decay": [0.3, 0.8, 0.99, 1.0]}},
        ],
    },
    # two attention layers of different shapes (two cache groups): a window of more than two blocks and none; one head;
    # a latent smaller than the head it expands into; odd width and vocabulary
    "c": {
        "architecture": "Neruzen", "vocab": 97, "width": 72, "norm": {"eps": 1e-6},
        "embedding": {"bigram": {"buckets": 31, "mul_prev": 1, "mul_cur": 1}},
        "layers": [
            {"type": "latent_attention", "mlp": None, "mixer": {
                "heads": 1, "dim": 48, "rot_dim": 8, "vdim": 16, "q_rank": 24, "kv_rank": 32, "scale": 0.3, "mask": {"size": 150},
                "rot": {"dims": 8, "base": 100.0}}},
            {"type": "latent_attention", "mlp": _moe(4, 2, 32, (4, 2), 8), "mixer": {
                "heads": 5, "dim": 8, "rot_dim": 24, "vdim": 12, "q_rank": 80, "kv_rank": 40, "scale": 0.11,
                "rot": {"dims": 24, "base": 1000000.0}}},
            {"type": "retention", "mlp": None, "mixer": {"heads": 3, "dim": 16, "vdim": 16, "decay": [0.8, 0.9, 0.99],
                                                         "rot": {"dims": 16, "base": 10000.0}}},
        ],
    },
    # heads of 64 and of 128 numbers for keys and values alike: the sizes whose prompts are expanded for the tensor-core
    # attention kernel in bfloat16 (a window that ends inside the second block, and none)
    "d": {
        "architecture": "Neruzen", "vocab": 160, "width": 128, "norm": {"eps": 1e-6},
        "embedding": {"bigram": {"buckets": 61, "mul_prev": 3, "mul_cur": 5}},
        "layers": [
            {"type": "latent_attention", "mlp": _moe(4, 2, 48, (2, 1), 64), "mixer": {
                "heads": 2, "dim": 32, "rot_dim": 32, "vdim": 64, "q_rank": 40, "kv_rank": 48, "scale": 0.13, "mask": {"size": 100},
                "rot": {"dims": 32, "base": 10000.0}}},
            {"type": "lightning", "mlp": None, "mixer": {"heads": 2, "dim": 32, "vdim": 32, "decay": [0.9, 0.99]}},
            {"type": "latent_attention", "mlp": None, "mixer": {
                "heads": 3, "dim": 96, "rot_dim": 32, "vdim": 128, "q_rank": 64, "kv_rank": 72, "scale": 0.09,
                "rot": {"dims": 32, "base": 100000.0}}},
        ],
    },
}
SEEDS = {"a": 3, "b": 4, "c": 6, "d": 8}


def shape_weights(tensors: dict[str, torch.Tensor], seed: int) -> dict[str, torch.Tensor]:
    """Rescale the drawn weights so that every mechanism moves the logits: hidden states and logits of order one, peaked
    attention, gates and routers away from their middle, a token shift that takes a visible share of the row before."""
    g = torch.Generator().manual_seed(seed + 1000)
    out = {}
    for name, t in tensors.items():
        leaf = name.split(".", 1)[1] if name.startswith("l") and "." in name else name
        if name in ("embed", "head", "bigram"):
            t = t * 30.0
        elif leaf == "shift":
            t = torch.rand(t.shape, generator=g)
        elif leaf in ("mix.uq", "mix.dkv"):
            t = t * 25.0
        elif leaf.endswith("router"):
            t = t * 40.0
        elif "norm" in leaf:
            pass
        elif leaf.startswith("mix.") or leaf.startswith("mlp."):
            t = t * 10.0
        out[name] = t
    return out


def write_model(folder: Path, name: str, stored: str = "float32") -> Path:
    from thintensor_b200.config.registry import load_config
    from thintensor_b200.engine.model import DecoderModel
    from thintensor_b200.weights.random_init import STORED_DTYPES, random_tensors
    from thintensor_b200.weights.safetensors_io import write_safetensors

    arch, config = load_config(CONFIGS[name])
    declared = DecoderModel(arch.describe(config), torch.float32, None).weight_declarations()
    tensors = shape_weights(random_tensors(declared, SEEDS[name], torch.float32), SEEDS[name])
    tensors = {k: v.to(STORED_DTYPES[stored]) for k, v in tensors.items()}
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(CONFIGS[name], indent=1))
    write_safetensors(folder / "model.safetensors", tensors)
    return folder


_oracle: dict = {}


def oracle_logits(folder: Path, tokens: list[int]) -> torch.Tensor:
    """float64 logits [T, vocab] of the plain implementation for one whole sequence."""
    import plain_neruzen

    model_key = ("model", str(folder))
    if model_key not in _oracle:
        _oracle[model_key] = plain_neruzen.read_model(folder)
    key = (str(folder), tuple(tokens))
    if key not in _oracle:
        cfg, weights = _oracle[model_key]
        with torch.no_grad():
            _oracle[key] = plain_neruzen.forward(cfg, weights, tokens)
    return _oracle[key]


def oracle_sensitivity(folder: Path, tokens: list[int]) -> torch.Tensor:
    """Per position, one minus the cosine between the plain implementation's logits and its logits with every operand of
    a matrix product narrowed to bfloat16 on the way, everything else as exact as before: how far the rounding of
    activations alone carries that position (a router's close call that rounding decides the other way shows here)."""
    import plain_neruzen

    key = ("sensitivity", str(folder), tuple(tokens))
    if key not in _oracle:
        want = oracle_logits(folder, tokens)
        cfg, weights = _oracle[("model", str(folder))]
        with torch.no_grad():
            other = plain_neruzen.forward(cfg, weights, tokens, narrow=lambda x: x.to(torch.bfloat16).to(x.dtype))
        _oracle[key] = 1.0 - torch.nn.functional.cosine_similarity(want, other, dim=-1)
    return _oracle[key]
