"""Small Vuvulorn configurations for the tests, and a writer of model folders whose tensor names and shapes are
spelled out here from the configuration (not taken from the package), with weights large enough that every
mechanism matters in the logits."""

from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch

from lalamo_b200.weights.safetensors_io import write_safetensors


def mixer(heads=4, kv_heads=2, dim=16, vdim=16, window=8, keep_first=2, rot_dims=8, base=10000.0, scale=0.25,
          r_heads=2, r_kv_heads=1, r_dim=16, r_vdim=32, conv=3, left_scale=0.7, right_scale=1.1, decay_rank=6, gate_rank=5):
    return {
        "left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
                 "mask": {"size": window, "keep_first": keep_first}, "rot": {"dims": rot_dims, "base": base}},
        "right": {"heads": r_heads, "kv_heads": r_kv_heads, "dim": r_dim, "vdim": r_vdim, "conv": conv,
                  "decay_rank": decay_rank, "gate_rank": gate_rank},
        "left_scale": left_scale,
        "right_scale": right_scale,
    }


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, top, count, keep):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "groups": {"count": count, "keep": keep}}}


def layer(mix, mlp):
    return {"type": "parallel", "mixer": mix, "mlp": mlp}


# P: a routed layer first, a layer without a feed-forward, grouped heads on both sides, value heads wider and narrower
# than key heads, rotation over part of a head, windows that differ between layers (two cache groups).
CONFIG_P = {
    "architecture": "Vuvulorn", "vocab": 160, "width": 64, "norm": {"eps": 1e-5},
    "layers": [
        layer(mixer(heads=4, kv_heads=2, dim=16, vdim=32, window=8, keep_first=3, rot_dims=8), moe(32, 6, 2, 3, 2)),
        layer(mixer(heads=2, kv_heads=2, dim=32, vdim=16, window=5, keep_first=1, rot_dims=32, r_heads=4, r_kv_heads=2, r_dim=8, r_vdim=16, conv=4), None),
        layer(mixer(heads=4, kv_heads=1, dim=16, vdim=16, window=8, keep_first=3, rot_dims=4, r_heads=2, r_kv_heads=2, r_dim=24, r_vdim=40, conv=2), dense(96)),
    ],
}

# Q: a width that is no multiple of 32, one head, nothing kept, a window of one token, no rotation at all, one tap (no
# convolution state), every expert chosen from one group, groups of one expert, an odd vocabulary.
CONFIG_Q = {
    "architecture": "Vuvulorn", "vocab": 131, "width": 72, "norm": {"eps": 1e-6},
    "layers": [
        layer(mixer(heads=1, kv_heads=1, dim=24, vdim=8, window=1, keep_first=0, rot_dims=0, scale=0.5, r_heads=1, r_kv_heads=1, r_dim=40, r_vdim=24, conv=1), dense(40)),
        layer(mixer(heads=3, kv_heads=3, dim=16, vdim=16, window=20, keep_first=4, rot_dims=16, r_heads=3, r_kv_heads=1, r_dim=16, r_vdim=8, conv=3), moe(24, 4, 4, 1, 1)),
        layer(mixer(heads=2, kv_heads=1, dim=16, vdim=24, window=3, keep_first=7, rot_dims=2, r_heads=2, r_kv_heads=2, r_dim=72, r_vdim=16, conv=5), moe(16, 5, 1, 5, 2)),
    ],
}

# R: head size 64 on the left with keys and values of one size (the sizes the tensor-core attention kernels take), a
# window wider than a page and kept tokens that fill more than one page, widths that the tensor-core products take.
CONFIG_R = {
    "architecture": "Vuvulorn", "vocab": 256, "width": 128, "norm": {"eps": 1e-6},
    "layers": [
        layer(mixer(heads=4, kv_heads=2, dim=64, vdim=64, window=40, keep_first=19, rot_dims=32, scale=0.125, r_heads=2, r_kv_heads=2, r_dim=64, r_vdim=64), dense(256)),
        layer(mixer(heads=2, kv_heads=1, dim=64, vdim=64, window=17, keep_first=5, rot_dims=64, scale=0.125, r_heads=2, r_kv_heads=1, r_dim=128, r_vdim=32), moe(64, 8, 2, 4, 2)),
    ],
}

# S: sizes that fit no kernel's favourite shape: a width and a vocabulary that are multiples of nothing, heads of 12, 20 and 10
# channels, three experts, a feed-forward of 30 columns.
CONFIG_S = {
    "architecture": "Vuvulorn", "vocab": 97, "width": 100, "norm": {"eps": 1e-6},
    "layers": [
        layer(mixer(heads=2, kv_heads=1, dim=24, vdim=12, window=6, keep_first=2, rot_dims=10, scale=0.3, r_heads=2, r_kv_heads=1, r_dim=20, r_vdim=12, conv=3,
                    decay_rank=7, gate_rank=3), moe(30, 3, 2, 1, 1)),
        layer(mixer(heads=3, kv_heads=3, dim=10, vdim=10, window=9, keep_first=0, rot_dims=6, scale=0.4, r_heads=3, r_kv_heads=3, r_dim=10, r_vdim=6, conv=2,
                    decay_rank=33, gate_rank=40), dense(30)),
    ],
}

CONFIGS = {"P": CONFIG_P, "Q": CONFIG_Q, "R": CONFIG_R, "S": CONFIG_S}


def tensor_shapes(config: dict) -> dict[str, tuple[int, ...]]:
    width = config["width"]
    shapes: dict[str, tuple[int, ...]] = {"embed": (config["vocab"], width), "head": (config["vocab"], width), "final.norm": (width,)}
    for index, entry in enumerate(config["layers"]):
        root = f"l{index}."
        shapes[root + "norm1"] = (width,)
        left, right = entry["mixer"]["left"], entry["mixer"]["right"]
        p = root + "mix.left."
        sizes = {"q": left["heads"] * left["dim"], "k": left["kv_heads"] * left["dim"], "v": left["kv_heads"] * left["vdim"]}
        for name, rows in sizes.items():
            shapes[p + name] = (rows, width)
            shapes[p + name + ".b"] = (rows,)
        shapes[p + "q.norm"] = shapes[p + "k.norm"] = (left["dim"],)
        shapes[p + "o"] = (width, left["heads"] * left["vdim"])
        shapes[p + "o.b"] = (width,)
        p = root + "mix.right."
        heads, groups, dim, vdim = right["heads"], right["kv_heads"], right["dim"], right["vdim"]
        for name, rows in {"q": groups * dim, "k": groups * dim, "v": heads * vdim}.items():
            shapes[p + name] = (rows, width)
            shapes[p + name + ".conv"] = (rows, right["conv"])
        shapes[p + "b"] = (heads, width)
        shapes[p + "A_log"] = (heads,)
        shapes[p + "dt_bias"] = (heads * dim,)
        shapes[p + "a1"] = (right["decay_rank"], width)
        shapes[p + "a2"] = (heads * dim, right["decay_rank"])
        shapes[p + "g1"] = (right["gate_rank"], width)
        shapes[p + "g2"] = (heads * vdim, right["gate_rank"])
        shapes[p + "norm"] = (vdim,)
        shapes[p + "o"] = (width, heads * vdim)
        mlp = entry["mlp"]
        if mlp is None:
            continue
        shapes[root + "norm2"] = (width,)
        p = root + "mlp."
        if mlp["kind"] == "dense":
            shapes[p + "gate"] = shapes[p + "up"] = (mlp["ff"], width)
            shapes[p + "down"] = (width, mlp["ff"])
        else:
            shapes[p + "router"] = (mlp["router"]["experts"], width)
            for e in range(mlp["router"]["experts"]):
                shapes[f"{p}e{e}.gate"] = shapes[f"{p}e{e}.up"] = (mlp["expert"]["ff"], width)
                shapes[f"{p}e{e}.down"] = (width, mlp["expert"]["ff"])
    return shapes


def random_weights(config: dict, seed: int) -> dict[str, torch.Tensor]:
    """bfloat16 tensors: matrices N(0, 1/in), scales near one, biases and taps of a size that shows."""
    generator = np.random.default_rng(seed)
    tensors: dict[str, torch.Tensor] = {}
    for name, shape in tensor_shapes(config).items():
        last = name.rsplit(".", 1)[-1]
        if name.endswith("norm") or last in ("norm1", "norm2"):
            values = 1.0 + 0.2 * generator.standard_normal(shape)
        elif last == "b" and len(shape) == 1:
            values = 0.3 * generator.standard_normal(shape)
        elif last == "conv":
            values = 0.6 * generator.standard_normal(shape)
        elif last == "A_log":
            values = 0.5 * generator.standard_normal(shape)
        elif last == "dt_bias":
            values = generator.standard_normal(shape)
        elif last == "embed":
            values = generator.standard_normal(shape)
        elif last == "router":
            values = 2.0 * generator.standard_normal(shape) / np.sqrt(shape[1])
        else:
            values = generator.standard_normal(shape) / np.sqrt(shape[1])
        tensors[name] = torch.from_numpy(values).to(torch.bfloat16)
    return tensors


def write_model(directory: Path, config: dict, seed: int, strip_ranks: bool = True) -> tuple[Path, dict[str, np.ndarray]]:
    """Writes the folder; returns it and the weights as float64 arrays (the bfloat16 values) for the plain implementation.
    ``strip_ranks``: ``config.json`` does not say the bottleneck ranks, which the loader then takes from the tensors."""
    directory = Path(directory)
    directory.mkdir(parents=True, exist_ok=True)
    tensors = random_weights(config, seed)
    written = json.loads(json.dumps(config))
    if strip_ranks:
        for entry in written["layers"]:
            entry["mixer"]["right"].pop("decay_rank", None)
            entry["mixer"]["right"].pop("gate_rank", None)
    (directory / "config.json").write_text(json.dumps(written, indent=1))
    write_safetensors(directory / "model.safetensors", tensors)
    return directory, {name: tensor.to(torch.float64).numpy() for name, tensor in tensors.items()}
