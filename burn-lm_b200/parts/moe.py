"""The mixture-of-experts feed-forward: a router picks `top` of `n_experts` small gated feed-forwards per token.

Router logits z = W_router h in fp32, scores s = sigmoid(z); the `top` experts of largest score are chosen (the
lower index on a tie) and weighted by those scores as they are, not renormalised.  With `weight_on` "input" the
weight multiplies the expert's input, out = sum expert(s h); with "output" its result, out = sum s expert(h).
expert(x) = W_down (silu(W_gate x) * (W_up x)), without biases.  A shared feed-forward (any registered kind) may run
for every token beside them; its result is added.

Everything stays on the device: the pairs (token, expert) are grouped by expert and the experts run as grouped
products over them, so a step can be captured in a CUDA graph.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import kernels as K
from ..plan import PartPlan
from ..registry import part_class, register_part
from ..weights.loader import TensorSpec
from .base import Part


@dataclass(frozen=True)
class SigmoidMoESpec:
    hidden_size: int
    n_experts: int
    top: int
    expert_size: int                       # inner size of one expert
    weight_on: str = "input"               # "input" or "output"
    shared: Optional[PartPlan] = None      # family "feed_forward": runs for every token


@register_part("feed_forward", "sigmoid_moe")
class SigmoidMoE(Part):
    """tensors: "router"; "gate", "up", "down": the experts' stored names with {} where the expert's number stands."""
    family = "feed_forward"
    graph_safe = True
    roles = ("router", "gate", "up", "down")
    kernel_modules = ("elementwise", "moe")

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        if spec.weight_on not in ("input", "output"):
            raise ValueError(f"weight_on is 'input' or 'output', not {spec.weight_on!r}")
        if not 1 <= spec.top <= spec.n_experts:
            raise ValueError(f"top {spec.top} of {spec.n_experts} experts")
        self.shared = None
        if spec.shared is not None:
            self.shared = part_class("feed_forward", spec.shared.kind)(spec.shared.spec, spec.shared.tensors, runtime)

    def _names(self, role):
        return [self.tensor_names[role].format(e) for e in range(self.spec.n_experts)]

    def tensor_specs(self):
        s = self.spec
        specs = [TensorSpec(self.tensor_names["router"], (s.n_experts, s.hidden_size), init="normal:0.1")]
        for g, u, d in zip(self._names("gate"), self._names("up"), self._names("down")):
            specs += [TensorSpec(g, (s.expert_size, s.hidden_size)), TensorSpec(u, (s.expert_size, s.hidden_size)),
                      TensorSpec(d, (s.hidden_size, s.expert_size))]
        return specs + (self.shared.tensor_specs() if self.shared is not None else [])

    def bind(self, loaded):
        self.router = loaded[self.tensor_names["router"]].to(torch.float32).contiguous()
        dt = self.runtime.dtype
        gates, ups, downs = ([loaded[n].to(dt) for n in self._names(r)] for r in ("gate", "up", "down"))
        # one tensor for all experts: [experts, gate rows then up rows, width] and [experts, width, inner]
        self.gate_up = torch.stack([torch.cat([g, u], dim=0) for g, u in zip(gates, ups)]).contiguous()
        self.down = torch.stack(downs).contiguous()
        if self.shared is not None:
            self.shared.bind(loaded)

    def forward(self, x, step, stream=None):
        ids, weights = K.moe_route(x, self.router, self.spec.top)
        extra = None
        if self.shared is not None:
            # a shared part that can add into the stream itself does so (x is already there for both); else its result
            # rides along into the sum
            if stream is not None and getattr(self.shared, "adds_to_stream", False):
                extra = self.shared.forward(x, step, stream=stream)
            else:
                extra = self.shared.forward(x, step)
        return K.moe_experts(x, ids, weights, self.gate_up, self.down, extra=extra, weight_on_input=self.spec.weight_on == "input")

    adds_to_stream = True


@dataclass(frozen=True)
class RoutedMoESpec:
    hidden_size: int
    n_experts: int
    top: int
    expert_size: int
    scores: str = "softmax"                # "softmax" over all experts, or "sigmoid" of every logit
    correction: bool = False               # a stored number per expert joins the scores for the choice only
    renormalise: bool = True               # the chosen weights are divided by their sum + 1e-20
    clamp_limit: Optional[float] = None    # the experts' clamped unit: g = min(Wgate x, limit), u = clamp(Wup x, -limit, limit),
    clamp_alpha: float = 1.702             # y = g sigmoid(alpha g) (u + 1); None: silu(g) u
    n_groups: int = 1                      # the experts form this many equal groups of neighbours; only experts of the
    keep_groups: int = 1                   # `keep_groups` best groups can be chosen (a group's mark: its two largest choice scores)
    unit: str = "gated"                    # "gated": W_down (act(W_gate x) * W_up x); "gelu" / "gelu_tanh": W_down gelu(W_up x),
                                           # the exact (erf) form or the tanh one; such experts store no gate


@register_part("feed_forward", "routed_moe")
class RoutedMoE(SigmoidMoE):
    """The mixture of experts with the router's options spelled out: scores s = softmax(W_router h) over all experts (or
    sigmoids), the `top` experts of largest s (+ a stored correction that the weights do not see), weights s of the chosen,
    optionally divided by their sum; out = sum weight_k expert_k(h), with the plain or the clamped gated unit, or a unit
    without a gate.  The choice may be limited to the experts of the best groups.  Router logits, scores and weights are
    fp32.  tensors: "router", "correction" (when the spec says so); "gate" (gated units), "up", "down" with {} where the
    expert's number stands."""
    roles = ("router", "correction", "gate", "up", "down")
    adds_to_stream = False

    def __init__(self, spec, tensors, runtime):
        Part.__init__(self, spec, tensors, runtime)
        if spec.scores not in ("softmax", "sigmoid"):
            raise ValueError(f"scores are 'softmax' or 'sigmoid', not {spec.scores!r}")
        if not 1 <= spec.top <= spec.n_experts:
            raise ValueError(f"top {spec.top} of {spec.n_experts} experts")
        if spec.unit not in self.UNITS:
            raise ValueError(f"an expert's unit is one of {sorted(self.UNITS)}, not {spec.unit!r}")
        if spec.unit != "gated" and spec.clamp_limit:
            raise ValueError("the clamped unit is a gated one")
        if (spec.n_groups < 1 or spec.n_experts % spec.n_groups or not 1 <= spec.keep_groups <= spec.n_groups
                or spec.keep_groups * (spec.n_experts // spec.n_groups) < spec.top):
            raise ValueError(f"{spec.n_experts} experts in {spec.n_groups} groups of which {spec.keep_groups} are kept, for {spec.top} chosen")
        self.shared = None
        if spec.unit == "gelu" and runtime.dtype == torch.bfloat16:
            self.kernel_modules = ("elementwise", "moe", "gemm_tc")       # prompts run these experts' products on tcgen05

    UNITS = {"gated": K.UNIT_GATED, "gelu": K.UNIT_GELU, "gelu_tanh": K.UNIT_GELU_TANH}

    def tensor_specs(self):
        s = self.spec
        if s.unit == "gated":
            specs = super().tensor_specs()
        else:
            specs = [TensorSpec(self.tensor_names["router"], (s.n_experts, s.hidden_size), init="normal:0.1")]
            for u, d in zip(self._names("up"), self._names("down")):
                specs += [TensorSpec(u, (s.expert_size, s.hidden_size)), TensorSpec(d, (s.hidden_size, s.expert_size))]
        if self.spec.correction:
            specs.insert(1, TensorSpec(self.tensor_names["correction"], (self.spec.n_experts,), init="normal:0.05"))
        return specs

    def bind(self, loaded):
        if self.spec.unit == "gated":
            super().bind(loaded)
        else:                                  # no gate: the first product's weight holds the up rows alone
            dt = self.runtime.dtype
            self.router = loaded[self.tensor_names["router"]].to(torch.float32).contiguous()
            self.gate_up = torch.stack([loaded[n].to(dt) for n in self._names("up")]).contiguous()
            self.down = torch.stack([loaded[n].to(dt) for n in self._names("down")]).contiguous()
        self.correction = None
        if self.spec.correction:
            self.correction = loaded[self.tensor_names["correction"]].to(torch.float32).contiguous()

    def forward(self, x, step):
        s = self.spec
        ids, weights = K.moe_route(x, self.router, s.top, softmax=s.scores == "softmax", correction=self.correction,
                                   renormalise=s.renormalise, n_groups=s.n_groups, keep_groups=s.keep_groups)
        return K.moe_experts(x, ids, weights, self.gate_up, self.down, weight_on_input=False, clamp_limit=s.clamp_limit or 0.0,
                             clamp_alpha=s.clamp_alpha, out_dtype=torch.float32, unit=self.UNITS[s.unit])
