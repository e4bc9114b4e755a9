"""Typed configuration of the Tudulix architecture (``"architecture": "Tudulix"`` in ``config.json``).

A decoder whose layers have a norm before and after each sublayer, ``x <- x + norm1b(mixer(norm1(x)));
x <- x + norm2b(ff(norm2(x)))``, the norms' weights kept as offsets from one (``1 + w``).  A layer's mixer is
softmax attention with grouped key/value heads, pairwise ("interleaved") rotation of part of each head and
a sliding window, or latent attention: keys and values made from one normed latent vector per token plus
one rotated key part shared by all heads, under a sliding window, with a sigmoid gate on the heads'
outputs.  The feed-forward is a mixture of experts (biased router, the largest logits chosen, softmax over
the chosen ones; experts with a clamped sigmoid gate) plus a shared expert.  A stretch of the layers may
run several times in a row with the same weights, each pass with a cache of its own and the embedding's
output added to the stream before every pass but the first.  The embedding is scaled, and so are the logits.

``config.json``: ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``, ``logit_scale``, ``loop`` (``start``,
``stop``, ``times``; optional) and ``layers``, one entry per layer: ``type`` (``"attention"`` with ``mixer``:
``heads, kv_heads, dim, vdim, scale, rot.dims, rot.base, mask.size``; or ``"latent_attention"`` with
``mixer``: ``heads, dim, rot_dim, vdim, kv_rank, scale, rot.base, mask.size``) and ``mlp`` (``null`` or
``{"kind": "moe", "expert": {ff, limit}, "router": {experts, top}, "shared": {ff, limit}}``).

Checkpoint names: ``embed``, ``head``, ``final.norm``, and per layer ``l<i>.norm1``, ``l<i>.norm1b``,
``l<i>.norm2``, ``l<i>.norm2b``, ``l<i>.mix.{q,k,v,o}`` or ``l<i>.mix.{q,dkv,dkv.norm,uk,uv,g,o}``,
``l<i>.mlp.router``, ``l<i>.mlp.router.b``, ``l<i>.mlp.e<j>.{gate,up,down}``, ``l<i>.mlp.shared.{gate,up,down}``.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Mapping

from .errors import ConfigError
from .plan import (
    AttentionSpec,
    EmbeddingSpec,
    GatedMLPSpec,
    HeadSpec,
    LatentAttentionSpec,
    ModelPlan,
    RMSNormSpec,
    RopeSpec,
    RoutedMLPSpec,
    SandwichBlockSpec,
    ScheduleEntry,
)

__all__ = ["TudulixConfig"]

EXPERT_ACTIVATION = "sigmoid_limit"


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


def _number(raw: Mapping[str, Any], path: str, where: str) -> float:
    return float(_get(raw, path, (int, float), where))


@dataclass(frozen=True)
class TudulixConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    logit_scale: float
    layers: tuple[SandwichBlockSpec, ...]
    loop: tuple[int, int, int]  # start, stop, times: layers start .. stop - 1 run `times` times in a row
    raw: dict

    architecture = "Tudulix"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "TudulixConfig":
        name = raw.get("architecture")
        if name is not None and name != "Tudulix":
            raise ConfigError("architecture", f"expected 'Tudulix', got {name!r}")
        vocab = _positive(raw, "vocab", "config")
        width = _positive(raw, "width", "config")
        eps = _number(raw, "norm.eps", "config")
        layer_list = raw.get("layers")
        if not isinstance(layer_list, list) or not layer_list:
            raise ConfigError("layers", "must be a non-empty list")
        layers = tuple(cls._layer(entry, index, width, eps) for index, entry in enumerate(layer_list))
        loop = (0, 0, 1)
        if raw.get("loop") is not None:
            start, stop = _get(raw, "loop.start", int, "config"), _get(raw, "loop.stop", int, "config")
            times = _positive(raw, "loop.times", "config")
            if not 0 <= start <= stop <= len(layers):
                raise ConfigError("loop", f"start={start} and stop={stop} must satisfy 0 <= start <= stop <= {len(layers)} layers")
            loop = (start, stop, times)
        return cls(
            vocab=vocab,
            width=width,
            norm_eps=eps,
            embedding_scale=_number(raw, "embedding.scale", "config") if raw.get("embedding") is not None else 1.0,
            logit_scale=_number(raw, "logit_scale", "config") if raw.get("logit_scale") is not None else 1.0,
            layers=layers,
            loop=loop,
            raw=copy.deepcopy(dict(raw)),
        )

    @staticmethod
    def _norm(width: int, eps: float) -> RMSNormSpec:
        return RMSNormSpec(dim=width, eps=eps, scale_offset=1.0, exact=True)

    @classmethod
    def _layer(cls, entry: Any, index: int, width: int, eps: float) -> SandwichBlockSpec:
        where = f"layers[{index}]"
        if not isinstance(entry, Mapping):
            raise ConfigError(where, "must be an object")
        kind = entry.get("type")
        mixer = _get(entry, "mixer", Mapping, where)
        at = where + ".mixer"
        heads = _positive(mixer, "heads", at)
        window = min(_positive(mixer, "mask.size", at), 1 << 30)   # wider than any context: the kernels count in 32 bits
        scale = _number(mixer, "scale", at)
        if kind == "attention":
            groups, dim = _positive(mixer, "kv_heads", at), _positive(mixer, "dim", at)
            if heads % groups:
                raise ConfigError(f"{at}.kv_heads", f"{groups} does not divide heads={heads}")
            rot_dims = _get(mixer, "rot.dims", int, at)
            if rot_dims < 0 or rot_dims % 2 or rot_dims > dim:
                raise ConfigError(f"{at}.rot.dims", f"must be even and at most dim={dim}, got {rot_dims}")
            mixer_spec: Any = AttentionSpec(
                model_dim=width,
                num_heads=heads,
                num_groups=groups,
                head_dim=dim,
                position=RopeSpec(rotary_dim=rot_dims, theta=_number(mixer, "rot.base", at), pairing="interleaved") if rot_dims else None,
                window=window,
                scale=scale,
                value_dim=_positive(mixer, "vdim", at),
            )
        elif kind == "latent_attention":
            rot_dim = _positive(mixer, "rot_dim", at)
            if rot_dim % 2:
                raise ConfigError(f"{at}.rot_dim", f"must be even, got {rot_dim}")
            declared = mixer.get("rot", {}).get("dims") if isinstance(mixer.get("rot"), Mapping) else None
            if declared is not None and declared != rot_dim:
                raise ConfigError(f"{at}.rot.dims", f"the rotated part has rot_dim={rot_dim} channels, got {declared}")
            rank = _positive(mixer, "kv_rank", at)
            mixer_spec = LatentAttentionSpec(
                model_dim=width,
                num_heads=heads,
                head_dim=_positive(mixer, "dim", at),
                rope_dim=rot_dim,
                value_dim=_positive(mixer, "vdim", at),
                latent_dim=rank,
                latent_norm=RMSNormSpec(dim=rank, eps=eps, exact=True),
                position=RopeSpec(rotary_dim=rot_dim, theta=_number(mixer, "rot.base", at), pairing="half"),
                window=window,
                scale=scale,
                gated=True,
            )
        else:
            raise ConfigError(f"{where}.type", f"unknown layer type {kind!r}; known: ['attention', 'latent_attention']")

        norm = cls._norm(width, eps)
        mlp = entry.get("mlp")
        if mlp is None:
            return SandwichBlockSpec(mixer_norm=norm, mixer=mixer_spec, mixer_out_norm=norm)
        at = where + ".mlp"
        if not isinstance(mlp, Mapping):
            raise ConfigError(at, "must be an object or null")
        if mlp.get("kind") != "moe":
            raise ConfigError(f"{at}.kind", f"unknown feed-forward kind {mlp.get('kind')!r}; known: ['moe']")
        experts, top = _positive(mlp, "router.experts", at), _positive(mlp, "router.top", at)
        if top > experts:
            raise ConfigError(f"{at}.router.top", f"{top} exceeds experts={experts}")
        shared = None
        if mlp.get("shared") is not None:
            shared = GatedMLPSpec(model_dim=width, hidden_dim=_positive(mlp, "shared.ff", at), activation=EXPERT_ACTIVATION,
                                  limit=_number(mlp, "shared.limit", at))
        ffn = RoutedMLPSpec(
            model_dim=width,
            hidden_dim=_positive(mlp, "expert.ff", at),
            num_experts=experts,
            top=top,
            score="logits",
            chosen_softmax=True,
            router_bias=True,
            activation=EXPERT_ACTIVATION,
            limit=_number(mlp, "expert.limit", at),
            shared=shared,
        )
        return SandwichBlockSpec(mixer_norm=norm, mixer=mixer_spec, mixer_out_norm=norm, ffn_norm=norm, ffn=ffn, ffn_out_norm=norm)

    # --------------------------------------------------------------------- plan
    def schedule(self) -> tuple[ScheduleEntry, ...]:
        """Layers before the repeated stretch once, the stretch ``times`` times (every pass but the first begins by
        adding the embedding's output to the stream; every execution owns its cache), then the rest."""
        start, stop, times = self.loop
        entries = [ScheduleEntry(index) for index in range(start)]
        for turn in range(times):
            entries += [ScheduleEntry(index, add_embedding=turn > 0 and index == start) for index in range(start, stop)]
        entries += [ScheduleEntry(index) for index in range(stop, len(self.layers))]
        return tuple(entries)

    def to_plan(self) -> ModelPlan:
        return ModelPlan(
            vocab_size=self.vocab,
            model_dim=self.width,
            layers=self.layers,
            final_norm=self._norm(self.width, self.norm_eps),
            tie_embeddings=False,
            schedule=self.schedule(),
            embedding=EmbeddingSpec(self.vocab, self.width, self.embedding_scale),
            head=HeadSpec(self.vocab, self.width, tied=False, scale=self.logit_scale),
        )

    # ---------------------------------------------------------- checkpoint names
    _ATTENTION = {"q_proj": "q", "k_proj": "k", "v_proj": "v", "out_proj": "o"}
    _LATENT = {"q_proj": "q", "down_proj": "dkv", "latent_norm": "dkv.norm", "key_up_proj": "uk", "value_up_proj": "uv", "gate_proj": "g", "out_proj": "o"}
    _MLP = {"gate_proj": "gate", "up_proj": "up", "down_proj": "down"}
    _NORMS = {"mixer_norm": "norm1", "mixer_out_norm": "norm1b", "ffn_norm": "norm2", "ffn_out_norm": "norm2b"}

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
            if role in self._NORMS:
                return [f"{root}.{self._NORMS[role]}"]
            if role == "mixer":
                table = self._LATENT if isinstance(self.layers[index].mixer, LatentAttentionSpec) else self._ATTENTION
                if local in table:
                    return [f"{root}.mix.{table[local]}"]
            if role == "ffn":
                if local == "router":
                    return [f"{root}.mlp.router"]
                if local == "router_bias":
                    return [f"{root}.mlp.router.b"]
                if local.startswith("experts."):
                    _, expert, name = local.split(".")
                    return [f"{root}.mlp.e{expert}.{self._MLP[name]}"]
                if local.startswith("shared."):
                    return [f"{root}.mlp.shared.{self._MLP[local.split('.', 1)[1]]}"]
        raise KeyError(f"Tudulix has no tensor {local!r} at {path!r}")

    def to_json_dict(self) -> dict[str, Any]:
        raw = copy.deepcopy(self.raw)
        raw["architecture"] = "Tudulix"
        return raw
