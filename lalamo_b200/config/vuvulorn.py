"""Typed configuration of the Vuvulorn architecture (``"architecture": "Vuvulorn"`` in ``config.json``).

A decoder whose layers each run two mixers side by side on the residual stream itself, a softmax
attention under a sliding window that keeps a request's first tokens and a gated-delta-rule
recurrence, then a dense or routed feed-forward, with RMS norms on the sublayers' *outputs*:
``x <- x + norm1(mixer(x)); x <- x + norm2(ff(x))``.

``config.json``: ``vocab``, ``width``, ``norm.eps`` and ``layers``, a list with one entry per layer:
``type`` (``"parallel"``), ``mixer`` (``left``: ``heads, kv_heads, dim, vdim, scale, rot.dims,
rot.base, mask.size, mask.keep_first``; ``right``: ``heads, kv_heads, dim, vdim, conv``; ``left_scale``,
``right_scale``) and ``mlp`` (``null``, ``{"kind": "dense", "ff"}`` or ``{"kind": "moe", "expert.ff",
"router.experts", "router.top", "router.groups.count", "router.groups.keep"}``).  The ranks of the
recurrence's two bottlenecks are not in ``config.json``: they are the checkpoint's ``a1`` and ``g1``
row counts, read from the tensors' shapes when a folder is loaded (``decay_rank`` / ``gate_rank`` in a
layer's ``right`` entry say them where there is no checkpoint, as for random weights).

Checkpoint names: ``embed``, ``head``, ``final.norm``, and per layer ``l<i>.norm1``, ``l<i>.norm2``,
``l<i>.mix.left.{q,k,v,o}`` with ``.b`` biases and ``.q.norm`` / ``.k.norm``,
``l<i>.mix.right.{q,k,v}`` with ``.conv``, ``.b``, ``.A_log``, ``.dt_bias``, ``.a1``, ``.a2``, ``.g1``,
``.g2``, ``.norm``, ``.o``, and ``l<i>.mlp.{gate,up,down}`` or ``l<i>.mlp.router`` with
``l<i>.mlp.e<j>.{gate,up,down}``.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Mapping

from .errors import ConfigError
from .plan import (
    AttentionSpec,
    GatedDeltaSpec,
    GatedMLPSpec,
    ModelPlan,
    OutputNormBlockSpec,
    ParallelMixerSpec,
    RMSNormSpec,
    RopeSpec,
    RoutedMLPSpec,
)

__all__ = ["VuvulornConfig"]

UNIT_EPS = 1e-6  # the design fixes the epsilon under the root that makes q and k unit vectors
DEFAULT_RANK = 16  # bottleneck rank of random-weight models that name none


def _get(raw: Mapping[str, Any], path: str, kind: type | tuple[type, ...], where: str) -> Any:
    value: Any = raw
    for key in path.split("."):
        if not isinstance(value, Mapping) or key not in value or value[key] is None:
            raise ConfigError(f"{where}.{path}", "is required but missing")
        value = value[key]
    if isinstance(value, bool) or not isinstance(value, kind):
        raise ConfigError(f"{where}.{path}", f"has the wrong type: {value!r}")
    return value


def _positive(raw: Mapping[str, Any], path: str, where: str) -> int:
    value = _get(raw, path, int, where)
    if value < 1:
        raise ConfigError(f"{where}.{path}", f"must be positive, got {value}")
    return value


@dataclass(frozen=True)
class VuvulornConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: tuple[OutputNormBlockSpec, ...]
    raw: dict

    architecture = "Vuvulorn"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], ranks: Mapping[int, tuple[int, int]] | None = None) -> "VuvulornConfig":
        """``ranks``: per layer the (decay, gate) bottleneck ranks found in a checkpoint."""
        name = raw.get("architecture")
        if name is not None and name != "Vuvulorn":
            raise ConfigError("architecture", f"expected 'Vuvulorn', got {name!r}")
        vocab = _positive(raw, "vocab", "config")
        width = _positive(raw, "width", "config")
        eps = float(_get(raw, "norm.eps", (int, float), "config"))
        layer_list = raw.get("layers")
        if not isinstance(layer_list, list) or not layer_list:
            raise ConfigError("layers", "must be a non-empty list")
        layers = tuple(cls._layer(entry, index, width, eps, (ranks or {}).get(index)) for index, entry in enumerate(layer_list))
        return cls(vocab=vocab, width=width, norm_eps=eps, layers=layers, raw=copy.deepcopy(dict(raw)))

    @classmethod
    def from_model_dir(cls, model_dir: str | Path, raw: Mapping[str, Any]) -> "VuvulornConfig":
        """The configuration of a model folder: what ``config.json`` leaves to the tensors' shapes is read there."""
        from ..weights.safetensors_io import open_checkpoint

        ranks: dict[int, tuple[int, int]] = {}
        try:
            checkpoint = open_checkpoint(model_dir)
        except (FileNotFoundError, OSError):
            checkpoint = None
        if checkpoint is not None:
            for index in range(len(raw.get("layers") or [])):
                decay, gate = f"l{index}.mix.right.a1", f"l{index}.mix.right.g1"
                if decay in checkpoint and gate in checkpoint:
                    ranks[index] = (checkpoint[decay].shape[0], checkpoint[gate].shape[0])
        return cls.from_dict(raw, ranks)

    @staticmethod
    def _layer(entry: Any, index: int, width: int, eps: float, ranks: tuple[int, int] | None) -> OutputNormBlockSpec:
        where = f"layers[{index}]"
        if not isinstance(entry, Mapping):
            raise ConfigError(where, "must be an object")
        kind = entry.get("type")
        if kind != "parallel":
            raise ConfigError(f"{where}.type", f"unknown layer type {kind!r}; known: ['parallel']")
        mixer = _get(entry, "mixer", Mapping, where)
        left, right = _get(mixer, "left", Mapping, where + ".mixer"), _get(mixer, "right", Mapping, where + ".mixer")
        norm = RMSNormSpec(dim=width, eps=eps)

        at = where + ".mixer.left"
        heads, groups, dim = _positive(left, "heads", at), _positive(left, "kv_heads", at), _positive(left, "dim", at)
        if heads % groups:
            raise ConfigError(f"{at}.kv_heads", f"{groups} does not divide heads={heads}")
        rot_dims = _get(left, "rot.dims", int, at)
        if rot_dims < 0 or rot_dims % 2 or rot_dims > dim:
            raise ConfigError(f"{at}.rot.dims", f"must be even and at most dim={dim}, got {rot_dims}")
        keep_first = _get(left, "mask.keep_first", int, at) if isinstance(left.get("mask"), Mapping) and left["mask"].get("keep_first") is not None else 0
        if keep_first < 0:
            raise ConfigError(f"{at}.mask.keep_first", f"must not be negative, got {keep_first}")
        attention = AttentionSpec(
            model_dim=width,
            num_heads=heads,
            num_groups=groups,
            head_dim=dim,
            qk_norm=RMSNormSpec(dim=dim, eps=eps),
            position=RopeSpec(rotary_dim=rot_dims, theta=float(_get(left, "rot.base", (int, float), at))) if rot_dims else None,
            window=_positive(left, "mask.size", at),
            scale=float(_get(left, "scale", (int, float), at)),
            value_dim=_positive(left, "vdim", at),
            keep_first=keep_first,
            has_bias=True,
        )

        at = where + ".mixer.right"
        heads, groups = _positive(right, "heads", at), _positive(right, "kv_heads", at)
        if heads % groups:
            raise ConfigError(f"{at}.kv_heads", f"{groups} does not divide heads={heads}")
        decay_rank = ranks[0] if ranks else (_positive(right, "decay_rank", at) if right.get("decay_rank") is not None else DEFAULT_RANK)
        gate_rank = ranks[1] if ranks else (_positive(right, "gate_rank", at) if right.get("gate_rank") is not None else DEFAULT_RANK)
        recurrence = GatedDeltaSpec(
            model_dim=width,
            num_heads=heads,
            num_groups=groups,
            key_dim=_positive(right, "dim", at),
            value_dim=_positive(right, "vdim", at),
            conv_taps=_positive(right, "conv", at),
            decay_rank=decay_rank,
            gate_rank=gate_rank,
            norm_eps=eps,
            unit_eps=UNIT_EPS,
        )
        parallel = ParallelMixerSpec(branches=(
            ("left", attention, float(_get(mixer, "left_scale", (int, float), where + ".mixer"))),
            ("right", recurrence, float(_get(mixer, "right_scale", (int, float), where + ".mixer"))),
        ))

        mlp = entry.get("mlp")
        if mlp is None:
            return OutputNormBlockSpec(mixer=parallel, mixer_norm=norm)
        at = where + ".mlp"
        if not isinstance(mlp, Mapping):
            raise ConfigError(at, "must be an object or null")
        mlp_kind = mlp.get("kind")
        if mlp_kind == "dense":
            ffn: Any = GatedMLPSpec(model_dim=width, hidden_dim=_positive(mlp, "ff", at), activation="silu")
        elif mlp_kind == "moe":
            experts, top = _positive(mlp, "router.experts", at), _positive(mlp, "router.top", at)
            grouped = isinstance(mlp.get("router"), Mapping) and mlp["router"].get("groups") is not None   # no groups: one group, kept
            count = _positive(mlp, "router.groups.count", at) if grouped else 1
            keep = _positive(mlp, "router.groups.keep", at) if grouped else 1
            if experts % count:
                raise ConfigError(f"{at}.router.groups.count", f"{count} does not divide experts={experts}")
            if keep > count:
                raise ConfigError(f"{at}.router.groups.keep", f"{keep} exceeds groups.count={count}")
            if top > keep * (experts // count):
                raise ConfigError(f"{at}.router.top", f"{top} exceeds the {keep * (experts // count)} experts of the kept groups")
            ffn = RoutedMLPSpec(model_dim=width, hidden_dim=_positive(mlp, "expert.ff", at), num_experts=experts, top=top, group_count=count,
                                group_keep=keep, score="sigmoid", renormalize=False, activation="silu")
        else:
            raise ConfigError(f"{at}.kind", f"unknown feed-forward kind {mlp_kind!r}; known: ['dense', 'moe']")
        return OutputNormBlockSpec(mixer=parallel, mixer_norm=norm, ffn=ffn, ffn_norm=norm)

    # --------------------------------------------------------------------- plan
    def to_plan(self) -> ModelPlan:
        return ModelPlan(
            vocab_size=self.vocab,
            model_dim=self.width,
            layers=self.layers,
            final_norm=RMSNormSpec(dim=self.width, eps=self.norm_eps),
            tie_embeddings=False,
        )

    # ---------------------------------------------------------- checkpoint names
    _LEFT = {
        "q_proj": "q", "k_proj": "k", "v_proj": "v", "out_proj": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b", "out_bias": "o.b",
        "q_norm": "q.norm", "k_norm": "k.norm",
    }
    _RIGHT = {
        "q_proj": "q", "k_proj": "k", "v_proj": "v", "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv", "beta_proj": "b", "a_log": "A_log",
        "dt_bias": "dt_bias", "decay_down": "a1", "decay_up": "a2", "gate_down": "g1", "gate_up": "g2", "out_norm": "norm", "out_proj": "o",
    }
    _MLP = {"gate_proj": "gate", "up_proj": "up", "down_proj": "down"}

    def checkpoint_names(self, path: tuple, local: str) -> list[str]:
        if path == ("embedding",):
            return ["embed"]
        if path == ("lm_head",):
            return ["head"]
        if path == ("final_norm",):
            return ["final.norm"]
        if path[0] == "layers":
            index, role = path[1], path[2]
            root = f"l{index}"
            if role == "mixer_norm":
                return [f"{root}.norm1"]
            if role == "ffn_norm":
                return [f"{root}.norm2"]
            if role == "mixer":
                branch, _, name = local.partition(".")
                table = self._LEFT if branch == "left" else self._RIGHT if branch == "right" else None
                if table is not None and name in table:
                    return [f"{root}.mix.{branch}.{table[name]}"]
            if role == "ffn":
                if local == "router":
                    return [f"{root}.mlp.router"]
                if local.startswith("experts."):
                    _, expert, name = local.split(".")
                    return [f"{root}.mlp.e{expert}.{self._MLP[name]}"]
                if local in self._MLP:
                    return [f"{root}.mlp.{self._MLP[local]}"]
        raise KeyError(f"Vuvulorn has no tensor {local!r} at {path!r}")

    def to_json_dict(self) -> dict[str, Any]:
        """A ``config.json`` from which :meth:`from_dict` rebuilds this configuration (the bottleneck ranks written
        out, so that a folder of random weights says them)."""
        raw = copy.deepcopy(self.raw)
        raw["architecture"] = "Vuvulorn"
        for entry, layer in zip(raw["layers"], self.layers):
            recurrence = layer.mixer.branches[1][1]
            entry["mixer"]["right"]["decay_rank"] = recurrence.decay_rank
            entry["mixer"]["right"]["gate_rank"] = recurrence.gate_rank
        return raw
