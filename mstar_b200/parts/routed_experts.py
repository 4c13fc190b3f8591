"""Routed experts feed-forward: a float router chooses ``top`` of ``experts`` small gated
feed-forwards per token; an optional shared one runs for every token and is added.

The router's logits are a product with float output; a kernel turns them into the chosen
experts and their weights (sigmoid or softmax scores, renormalised or not).  The shared
expert is the dense gated feed-forward's path (one fused gate/up product, one down
product); the routed experts' kernels add its output while they write theirs.  A few rows
(decoded tokens) each stream the matrices of their experts; many rows (prompt portions)
are sorted by expert on the device and run as tiles on the tensor cores.
"""
from __future__ import annotations

import torch

from .. import ops
from ..weights.names import ParamSpec
from .base import Runtime
from .registry import register_part


class RoutedExperts:
    graph_safe = True       # shapes are fixed by the batch; the choice stays on the device

    @classmethod
    def param_specs(cls, spec) -> dict:
        e, ff, width = spec.num_experts, spec.expert_size, spec.hidden_size
        outputs = e + spec.identity_experts
        out = {"router.weight": ParamSpec((outputs, width))}
        if spec.choice_bias:
            out["router.correction"] = ParamSpec((outputs,), role="vector", init="zeros")
        if spec.gated:
            out["experts.gate_up.weight"] = ParamSpec((e * 2 * ff, width))
        else:
            out["experts.up.weight"] = ParamSpec((e * ff, width))
        out["experts.down.weight"] = ParamSpec((e * width, ff))
        if spec.shared_size:
            out["shared.gate_up.weight"] = ParamSpec((2 * spec.shared_size, width))
            out["shared.down.weight"] = ParamSpec((width, spec.shared_size))
        return out

    def __init__(self, spec, params: dict, runtime: Runtime):
        if (spec.gated, spec.activation) not in ((True, "silu"), (False, "relu2")):
            raise ValueError(f"routed experts with gated={spec.gated} and activation "
                             f"{spec.activation!r} have no kernel (gated silu and plain relu2 have)")
        if spec.identity_experts and spec.scale_input:
            raise ValueError("identity experts go with weights on the experts' outputs")
        if spec.score not in ("sigmoid", "softmax"):
            raise ValueError(f"router score {spec.score!r} is not known (sigmoid, softmax)")
        self.spec = spec
        self.runtime = runtime
        self.router = params["router.weight"]
        self.gate_up = params["experts.gate_up.weight" if spec.gated else "experts.up.weight"]
        self.correction = None
        if spec.choice_bias:
            self.correction = params["router.correction"].float().contiguous()
        self.down = params["experts.down.weight"]
        self.shared_gate_up = params.get("shared.gate_up.weight")
        self.shared_down = params.get("shared.down.weight")

    def forward(self, x, ctx):
        s = self.spec
        logits = ops.linear(x, self.router, out_dtype=torch.float32, static_weights=True)
        chosen, weight = ops.route_topk(logits, s.top, softmax=s.score == "softmax",
                                        renormalize=s.renormalize, choice_bias=self.correction)
        shared = None
        if self.shared_gate_up is not None:
            shared = ops.linear(ops.gated_up(x, self.shared_gate_up, static_weights=True),
                                self.shared_down, static_weights=True)
        return ops.routed_experts(x, self.gate_up, self.down, chosen, weight, s.num_experts,
                                  s.expert_size, s.scale_input, add=shared, gated=s.gated,
                                  identity=s.identity_experts)


register_part("ffn", "routed_experts", RoutedExperts)
