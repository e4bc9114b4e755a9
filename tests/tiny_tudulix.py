"""Small Tudulix configurations for the tests, and a writer of model folders whose tensor names and shapes are spelled
out here from the configuration (not taken from the package), with weights large enough that every mechanism matters
in the logits."""

from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch

from lalamo_b200.weights.safetensors_io import write_safetensors


def attention(heads=4, kv_heads=2, dim=16, vdim=16, window=8, rot_dims=8, base=10000.0, scale=0.25):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": window}, "rot": {"dims": rot_dims, "base": base}}


def latent(heads=4, dim=16, rot_dim=8, vdim=16, kv_rank=32, window=8, base=10000.0, scale=0.2):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale, "mask": {"size": window},
            "rot": {"dims": rot_dim, "base": base}}


def moe(ff, experts, top, limit=2.0, shared_ff=None, shared_limit=2.0):
    mlp = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared_ff is not None:
        mlp["shared"] = {"ff": shared_ff, "limit": shared_limit}
    return mlp


def layer(kind, mix, mlp):
    return {"type": kind, "mixer": mix, "mlp": mlp}


def model(vocab, width, layers, eps=1e-6, embedding_scale=1.0, logit_scale=1.0, loop=None):
    config = {"architecture": "Tudulix", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": embedding_scale},
              "logit_scale": logit_scale, "layers": layers}
    if loop is not None:
        config["loop"] = dict(zip(("start", "stop", "times"), loop))
    return config


# A: a latent layer first, value heads wider and narrower than key heads, rotation over part of a head and over all of it, a layer
# without a feed-forward, windows that differ between layers, limits that differ between the experts and the shared expert, the
# middle two layers three times.
CONFIG_A = model(160, 64, [
    layer("latent_attention", latent(heads=4, dim=16, rot_dim=8, vdim=24, kv_rank=32, window=11, base=500.0), moe(32, 6, 2, 1.5, 40, 3.0)),
    layer("attention", attention(heads=4, kv_heads=2, dim=16, vdim=32, window=8, rot_dims=8), moe(24, 5, 3, 2.5, 16, 1.0)),
    layer("attention", attention(heads=2, kv_heads=1, dim=32, vdim=16, window=5, rot_dims=32, base=77.0), None),
    layer("latent_attention", latent(heads=2, dim=8, rot_dim=16, vdim=8, kv_rank=24, window=20), moe(32, 6, 2, 1.5, 40, 3.0)),
], eps=1e-5, embedding_scale=4.0, logit_scale=0.25, loop=(1, 3, 3))

# B: sizes that fit no kernel's favourite shape (a width and a vocabulary that are multiples of nothing much), no rotation at all in
# the attention, a window of one token, one head, every expert chosen, one expert chosen, no shared expert, no repeated stretch,
# scales of one.
CONFIG_B = model(131, 72, [
    layer("attention", attention(heads=3, kv_heads=3, dim=24, vdim=8, window=1, rot_dims=0, scale=0.5), moe(20, 4, 4)),
    layer("latent_attention", latent(heads=1, dim=10, rot_dim=6, vdim=12, kv_rank=20, window=3, scale=0.4), moe(30, 3, 1, 0.7)),
    layer("attention", attention(heads=2, kv_heads=1, dim=12, vdim=20, window=23, rot_dims=2, scale=0.3), moe(16, 5, 2, 2.0, 28, 0.5)),
])

# C: the sizes the tensor-core kernels take (heads of 64 with keys and values of one size, widths in multiples of 64), windows wider
# than a page and no multiples of one, the whole model twice.
CONFIG_C = model(256, 128, [
    layer("attention", attention(heads=4, kv_heads=2, dim=64, vdim=64, window=40, rot_dims=64, scale=0.125), moe(64, 8, 2, 2.0, 128, 2.0)),
    layer("latent_attention", latent(heads=4, dim=64, rot_dim=32, vdim=64, kv_rank=64, window=50, scale=0.1), moe(64, 4, 1, 2.0, 64, 2.0)),
], embedding_scale=8.0, logit_scale=0.5, loop=(0, 2, 2))

# D, E: one layer of each kind without a feed-forward: the mixers alone.
CONFIG_D = model(96, 64, [layer("attention", attention(heads=4, kv_heads=1, dim=32, vdim=16, window=13, rot_dims=20, base=300.0, scale=0.2), None)])
CONFIG_E = model(96, 64, [layer("latent_attention", latent(heads=3, dim=24, rot_dim=12, vdim=20, kv_rank=40, window=13, base=300.0, scale=0.15), None)], loop=(0, 1, 2))

CONFIGS = {"A": CONFIG_A, "B": CONFIG_B, "C": CONFIG_C, "D": CONFIG_D, "E": CONFIG_E}


def tensor_shapes(config: dict) -> dict[str, tuple[int, ...]]:
    width = config["width"]
    shapes: dict[str, tuple[int, ...]] = {"embed": (config["vocab"], width), "head": (config["vocab"], width), "final.norm": (width,)}
    for index, entry in enumerate(config["layers"]):
        root = f"l{index}."
        shapes[root + "norm1"] = shapes[root + "norm1b"] = (width,)
        mix, p = entry["mixer"], root + "mix."
        if entry["type"] == "attention":
            shapes[p + "q"] = (mix["heads"] * mix["dim"], width)
            shapes[p + "k"] = (mix["kv_heads"] * mix["dim"], width)
            shapes[p + "v"] = (mix["kv_heads"] * mix["vdim"], width)
        else:
            shapes[p + "q"] = (mix["heads"] * (mix["dim"] + mix["rot_dim"]), width)
            shapes[p + "dkv"] = (mix["kv_rank"] + mix["rot_dim"], width)
            shapes[p + "dkv.norm"] = (mix["kv_rank"],)
            shapes[p + "uk"] = (mix["heads"] * mix["dim"], mix["kv_rank"])
            shapes[p + "uv"] = (mix["heads"] * mix["vdim"], mix["kv_rank"])
            shapes[p + "g"] = (mix["heads"] * mix["vdim"], width)
        shapes[p + "o"] = (width, mix["heads"] * mix["vdim"])
        mlp = entry["mlp"]
        if mlp is None:
            continue
        shapes[root + "norm2"] = shapes[root + "norm2b"] = (width,)
        p = root + "mlp."
        shapes[p + "router"] = (mlp["router"]["experts"], width)
        shapes[p + "router.b"] = (mlp["router"]["experts"],)
        blocks = [(f"e{e}", mlp["expert"]["ff"]) for e in range(mlp["router"]["experts"])]
        if "shared" in mlp:
            blocks.append(("shared", mlp["shared"]["ff"]))
        for name, ff in blocks:
            shapes[f"{p}{name}.gate"] = shapes[f"{p}{name}.up"] = (ff, width)
            shapes[f"{p}{name}.down"] = (width, ff)
    return shapes


def random_weights(config: dict, seed: int) -> dict[str, torch.Tensor]:
    """bfloat16 tensors: matrices N(0, 1/in) (gates and ups twice that, so that the limits bite), the layers' norm weights around
    zero, the latent's around one, router biases of a size that changes choices."""
    generator = np.random.default_rng(seed)
    tensors: dict[str, torch.Tensor] = {}
    for name, shape in tensor_shapes(config).items():
        last = name.rsplit(".", 1)[-1]
        if name.endswith("dkv.norm"):
            values = 1.0 + 0.2 * generator.standard_normal(shape)
        elif last in ("norm", "norm1", "norm1b", "norm2", "norm2b"):
            values = 0.2 * generator.standard_normal(shape)
        elif name.endswith("router.b"):
            values = 0.7 * generator.standard_normal(shape)
        elif last == "embed":
            values = generator.standard_normal(shape)
        elif last == "router":
            # small beside the biases: a logit's rounding error grows with the logit, so close calls that bfloat16 turns stay rare
            values = 0.5 * generator.standard_normal(shape) / np.sqrt(shape[1])
        elif last in ("gate", "up"):
            values = 2.0 * generator.standard_normal(shape) / np.sqrt(shape[1])
        else:
            values = generator.standard_normal(shape) / np.sqrt(shape[1])
        tensors[name] = torch.from_numpy(values).to(torch.bfloat16)
    return tensors


def write_model(directory: Path, config: dict, seed: int) -> tuple[Path, dict[str, np.ndarray]]:
    """Writes the folder; returns it and the weights as float64 arrays (the bfloat16 values) for the plain implementation."""
    directory = Path(directory)
    directory.mkdir(parents=True, exist_ok=True)
    tensors = random_weights(config, seed)
    (directory / "config.json").write_text(json.dumps(config, indent=1))
    write_safetensors(directory / "model.safetensors", tensors)
    return directory, {name: tensor.to(torch.float64).numpy() for name, tensor in tensors.items()}
