"""A routed feed-forward (mixture of experts): the router's scores in 32-bit, the choice of experts under a
limit on groups of experts, the chosen experts' gated feed-forwards, and their weighted sum."""

from __future__ import annotations

from typing import Mapping

import torch

from .. import ops
from ..config.plan import RoutedMLPSpec
from .base import FeedForward, Part, Runtime, StepInputs, TensorDecl, build_part, part_type, register_part

__all__ = ["RoutedMLP"]


@register_part(RoutedMLPSpec)
class RoutedMLP(FeedForward):
    def __init__(self, spec: RoutedMLPSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        super().__init__(spec, tensors, runtime)
        if not (1 <= spec.top <= spec.num_experts and spec.num_experts % spec.group_count == 0 and 1 <= spec.group_keep <= spec.group_count):
            raise ValueError(f"top {spec.top} of {spec.num_experts} experts in {spec.group_count} groups of which {spec.group_keep} are kept is not a valid choice")
        if spec.top > spec.group_keep * (spec.num_experts // spec.group_count):
            raise ValueError("the kept groups hold fewer experts than a token uses")
        self.router = runtime.vector(tensors["router"])  # the router's logits are 32-bit
        self.router_bias = runtime.vector(tensors["router_bias"]) if spec.router_bias else None
        self.shared: FeedForward | None = None
        if spec.shared is not None:
            self.shared = build_part(spec.shared, {local[len("shared."):]: tensor for local, tensor in tensors.items() if local.startswith("shared.")}, runtime)  # type: ignore[assignment]
        experts = range(spec.num_experts)
        self.gate = runtime.matrix(torch.stack([tensors[f"experts.{e}.gate_proj"] for e in experts]))
        self.up = runtime.matrix(torch.stack([tensors[f"experts.{e}.up_proj"] for e in experts]))
        self.down = runtime.matrix(torch.stack([tensors[f"experts.{e}.down_proj"] for e in experts]))

    @classmethod
    def tensor_decls(cls, spec: RoutedMLPSpec) -> dict[str, TensorDecl]:
        decls = {"router": TensorDecl((spec.num_experts, spec.model_dim))}
        if spec.router_bias:
            decls["router_bias"] = TensorDecl((spec.num_experts,), role="vector")
        if spec.shared is not None:
            for local, decl in part_type(spec.shared).tensor_decls(spec.shared).items():
                decls[f"shared.{local}"] = decl
        for e in range(spec.num_experts):
            decls[f"experts.{e}.gate_proj"] = TensorDecl((spec.hidden_dim, spec.model_dim))
            decls[f"experts.{e}.up_proj"] = TensorDecl((spec.hidden_dim, spec.model_dim))
            decls[f"experts.{e}.down_proj"] = TensorDecl((spec.model_dim, spec.hidden_dim))
        return decls

    def sub_parts(self) -> list[Part]:
        return [self.shared] if self.shared is not None else []

    def forward(self, x: torch.Tensor, step: StepInputs | None = None) -> "torch.Tensor | ops.ScaledSum":
        """The experts' weighted sum; with a shared feed-forward the two terms are handed on un-summed
        (``ops.ScaledSum``), for a consumer that adds them in 32-bit."""
        spec = self.spec
        chosen, weights = ops.moe_route(x, self.router, top=spec.top, group_count=spec.group_count, group_keep=spec.group_keep, score=spec.score,
                                        renormalize=spec.renormalize, bias=self.router_bias, chosen_softmax=spec.chosen_softmax)
        # with a shared feed-forward the consumer adds two terms anyway: the experts' weighted sum is left to it as well
        routed = ops.moe_experts(x, self.gate, self.up, self.down, chosen, weights, spec.activation, limit=spec.limit, combine=self.shared is None)
        if self.shared is None:
            return routed
        everyone = self.shared.forward(x, step)
        if isinstance(everyone, ops.SlicedSum):
            everyone = everyone.sum()
        return ops.ScaledSum([(routed, 1.0, None), (everyone, 1.0, None)])
