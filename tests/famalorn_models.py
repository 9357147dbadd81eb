"""Tiny Famalorn configurations with random weights for the tests, and the plain implementation's
outputs for them.  The configurations differ from one another in every size; between them they
cover: heads per query/key head and per group above one and equal to one, key and value sizes that
differ and that are equal, states smaller and larger than a head, one to five convolution taps,
norm groups different from the groups, a rotation of the whole head, of a part of it and none at
all, layers with and without a feed-forward, and a model without any attention layer."""
from __future__ import annotations

import json
from pathlib import Path

import torch

CONFIGS = {
    # attention first; a Mamba-2 layer whose heads are wider than one CTA's columns and whose state needs two registers' rounds
    "p": {
        "architecture": "Famalorn", "vocab": 211, "width": 96, "norm": {"eps": 1e-5},
        "layers": [
            {"type": "parallel", "mlp": {"kind": "dense", "ff": 160}, "mixer": {
                "left": {"heads": 4, "kv_heads": 2, "dim": 32, "vdim": 24, "scale": 0.21, "rot": {"dims": 16, "base": 10000.0}},
                "right": {"heads": 3, "vdim": 16, "state": 24, "groups": 3, "norm_groups": 1, "conv": 4},
                "left_scale": 0.7, "right_scale": 1.3}},
            {"type": "delta", "mlp": None, "mixer": {"heads": 4, "kv_heads": 2, "dim": 24, "vdim": 40, "conv": 3}},
            {"type": "mamba2", "mlp": {"kind": "dense", "ff": 72}, "mixer": {"heads": 4, "vdim": 40, "state": 72, "groups": 2,
                                                                             "norm_groups": 4, "conv": 2}},
        ],
    },
    # no attention anywhere: the cache holds states only
    "r": {
        "architecture": "Famalorn", "vocab": 130, "width": 64, "norm": {"eps": 1e-6},
        "layers": [
            {"type": "mamba2", "mlp": None, "mixer": {"heads": 2, "vdim": 8, "state": 136, "groups": 1, "norm_groups": 2, "conv": 5}},
            {"type": "delta", "mlp": {"kind": "dense", "ff": 96}, "mixer": {"heads": 3, "kv_heads": 1, "dim": 136, "vdim": 8, "conv": 1}},
            {"type": "delta", "mlp": None, "mixer": {"heads": 2, "kv_heads": 2, "dim": 16, "vdim": 16, "conv": 4}},
        ],
    },
    # two attention layers of different shapes (two cache groups): a head rotated whole with one key/value head per query
    # head and equal key and value sizes, and a head that is not rotated at all; odd width and vocabulary
    "s": {
        "architecture": "Famalorn", "vocab": 97, "width": 72, "norm": {"eps": 1e-6},
        "layers": [
            {"type": "parallel", "mlp": None, "mixer": {
                "left": {"heads": 3, "kv_heads": 3, "dim": 16, "vdim": 16, "scale": 0.25, "rot": {"dims": 16, "base": 500.0}},
                "right": {"heads": 2, "vdim": 12, "state": 8, "groups": 1, "norm_groups": 2, "conv": 3},
                "left_scale": 1.0, "right_scale": 1.0}},
            {"type": "parallel", "mlp": {"kind": "dense", "ff": 100}, "mixer": {
                "left": {"heads": 6, "kv_heads": 1, "dim": 20, "vdim": 36, "scale": 0.4},
                "right": {"heads": 4, "vdim": 6, "state": 20, "groups": 2, "norm_groups": 1, "conv": 2},
                "left_scale": 1.5, "right_scale": 0.5}},
        ],
    },
    # key and value heads of 64 and of 128 numbers: the sizes the tensor-core attention kernels take in bfloat16
    "t": {
        "architecture": "Famalorn", "vocab": 160, "width": 128, "norm": {"eps": 1e-6},
        "layers": [
            {"type": "parallel", "mlp": {"kind": "dense", "ff": 192}, "mixer": {
                "left": {"heads": 4, "kv_heads": 2, "dim": 64, "vdim": 64, "scale": 0.125, "rot": {"dims": 32, "base": 100000.0}},
                "right": {"heads": 2, "vdim": 32, "state": 16, "groups": 1, "norm_groups": 1, "conv": 4},
                "left_scale": 0.9, "right_scale": 1.1}},
            {"type": "parallel", "mlp": None, "mixer": {
                "left": {"heads": 2, "kv_heads": 1, "dim": 128, "vdim": 128, "scale": 0.09, "rot": {"dims": 128, "base": 10000.0}},
                "right": {"heads": 4, "vdim": 16, "state": 32, "groups": 4, "norm_groups": 2, "conv": 3},
                "left_scale": 1.2, "right_scale": 0.8}},
        ],
    },
}
SEEDS = {"p": 3, "r": 4, "s": 6, "t": 8}


def shape_weights(tensors: dict[str, torch.Tensor], seed: int, slow_decay: bool = False) -> dict[str, torch.Tensor]:
    """Rescale the drawn weights so that every mechanism moves the logits: hidden states and logits of order
    one, peaked attention, sinks that take a visible share, decays spread between fast and slow, write strengths
    and gates away from their middle.  ``slow_decay``: the recurrences forget slowly, so the first tokens of a
    long sequence still show at its end."""
    g = torch.Generator().manual_seed(seed + 1000)
    out = {}
    for name, t in tensors.items():
        leaf = name.split(".", 1)[1] if name.startswith("l") and "." in name else name
        if name in ("embed", "head"):
            t = t * 30.0
        elif leaf in ("mix.left.q", "mix.left.k"):
            t = t * 20.0
        elif leaf.endswith("sink"):
            t = torch.randn(t.shape, generator=g) * 2.0
        elif leaf.endswith("A_log"):
            t = torch.rand(t.shape, generator=g) * (1.0 if slow_decay else 2.5) - (4.0 if slow_decay else 1.0)
        elif leaf.endswith("dt_bias"):
            t = torch.rand(t.shape, generator=g) * 3.0 - 2.0
        elif leaf.endswith(".D"):
            t = 1.0 + 0.5 * torch.randn(t.shape, generator=g)
        elif leaf.endswith("conv.b"):
            t = torch.randn(t.shape, generator=g) * 0.3
        elif leaf.endswith("conv"):
            t = torch.randn(t.shape, generator=g) * 0.6
        elif "norm" in leaf:
            pass
        elif leaf.startswith("mix.") or leaf.startswith("mlp."):
            t = t * 10.0
        out[name] = t
    return out


def write_model(folder: Path, name: str, stored: str = "float32", slow_decay: bool = False) -> Path:
    from thintensor_b200.config.registry import load_config
    from thintensor_b200.engine.model import DecoderModel
    from thintensor_b200.weights.random_init import STORED_DTYPES, random_tensors
    from thintensor_b200.weights.safetensors_io import write_safetensors

    arch, config = load_config(CONFIGS[name])
    declared = DecoderModel(arch.describe(config), torch.float32, None).weight_declarations()
    tensors = shape_weights(random_tensors(declared, SEEDS[name], torch.float32), SEEDS[name], slow_decay)
    tensors = {k: v.to(STORED_DTYPES[stored]) for k, v in tensors.items()}
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(CONFIGS[name], indent=1))
    write_safetensors(folder / "model.safetensors", tensors)
    return folder


_oracle: dict = {}


def oracle_logits(folder: Path, tokens: list[int]) -> torch.Tensor:
    """float64 logits [T, vocab] of the plain implementation for one whole sequence."""
    import plain_famalorn

    model_key = ("model", str(folder))
    if model_key not in _oracle:
        _oracle[model_key] = plain_famalorn.read_model(folder)
    key = (str(folder), tuple(tokens))
    if key not in _oracle:
        cfg, weights = _oracle[model_key]
        with torch.no_grad():
            _oracle[key] = plain_famalorn.forward(cfg, weights, tokens)
    return _oracle[key]


def oracle_sensitivity(folder: Path, tokens: list[int]) -> torch.Tensor:
    """Per position, one minus the cosine between the plain implementation's logits and its logits with every operand of
    a matrix product (and queries, keys and values) narrowed to bfloat16 on the way, everything else as exact as before:
    how far the rounding of activations alone carries that position.  Positions where a norm divides by a nearly
    vanishing vector, or a gate sits at its kink, move a hundred times further than the others."""
    import plain_famalorn

    key = ("sensitivity", str(folder), tuple(tokens))
    if key not in _oracle:
        want = oracle_logits(folder, tokens)
        cfg, weights = _oracle[("model", str(folder))]
        with torch.no_grad():
            other = plain_famalorn.forward(cfg, weights, tokens, narrow=lambda x: x.to(torch.bfloat16).to(x.dtype))
        _oracle[key] = 1.0 - torch.nn.functional.cosine_similarity(want, other, dim=-1)
    return _oracle[key]
