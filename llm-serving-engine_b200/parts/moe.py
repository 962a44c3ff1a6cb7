"""Routed experts: each token runs through the ``top`` of ``num_experts`` small gated feed-forward
layers that a router picks for it, and through an optional shared expert.

    s      = sigmoid(Wr h)                    router scores, computed in 32-bit
    chosen = the ``top`` experts with the largest scores; their weights are the scores themselves
    y      = sum_{e chosen} expert_e(s_e * h)            the weight multiplies the expert's input
           + sigmoid(wg . h) * shared(h)                 if there is a shared expert
    expert(z) = Wdown (act(Wgate z) * (Wup z))

The tokens' choices are sorted by expert on the device and the experts' products run as one
launch over tiles of rows that belong to one expert each, so nothing comes back to the host
between the router and the sum.
"""

from __future__ import annotations

from dataclasses import dataclass

from .base import FEED_FORWARDS, FeedForward, ParamDecl
from .feed_forward import SwiGLUSpec


@dataclass(frozen=True)
class RoutedExpertsSpec:
    hidden_size: int
    num_experts: int
    top: int
    expert_size: int  # inner size of a routed expert
    shared_size: int = 0  # inner size of the shared expert; 0: none
    activation: str = "silu"
    kind: str = "routed_experts"


@FEED_FORWARDS.register("routed_experts")
class RoutedExperts(FeedForward):
    accepts_residual = True

    def __init__(self, spec: RoutedExpertsSpec, env) -> None:
        super().__init__(spec, env)
        if not 1 <= spec.top <= spec.num_experts:
            raise ValueError("routed_experts: top must lie between 1 and the number of experts")
        self.children = {}
        if spec.shared_size:
            self.children["shared"] = FEED_FORWARDS.build(
                SwiGLUSpec(spec.hidden_size, spec.shared_size, activation=spec.activation), env)
        self.shared = self.children.get("shared")

    def param_decls(self):
        s = self.spec
        decls = {
            # one more row with a shared expert: its gate
            "router.weight": ParamDecl((s.num_experts + (1 if s.shared_size else 0), s.hidden_size), "matrix32"),
            "experts.gate_up.weight": ParamDecl((s.num_experts * 2 * s.expert_size, s.hidden_size), "matrix"),
            "experts.down.weight": ParamDecl((s.num_experts * s.hidden_size, s.expert_size), "matrix"),
        }
        if self.shared is not None:
            for name, decl in self.shared.param_decls().items():
                decls["shared." + name] = decl
        return decls

    def bind(self, params):
        s = self.spec
        self.router_weight = params["router.weight"]
        self.gate_up_weight = params["experts.gate_up.weight"].view(s.num_experts, 2 * s.expert_size, s.hidden_size)
        self.down_weight = params["experts.down.weight"].view(s.num_experts, s.hidden_size, s.expert_size)
        if self.shared is not None:
            self.shared.bind({k[len("shared."):]: v for k, v in params.items() if k.startswith("shared.")})

    def forward(self, h, step, residual=None, may_defer=False):
        s, ops = self.spec, self.ops
        idx, wts, gate = ops.moe_route(h, self.router_weight, s.num_experts, s.top, self.shared is not None)
        plan = ops.moe_sort(idx, s.num_experts, self.env.dtype, width=_gcd8(s.hidden_size, s.expert_size))
        gu = ops.expert_linear(h, self.gate_up_weight, plan, top=s.top, wts=wts)
        a = ops.silu_mul(gu, out_dtype=self.env.dtype, activation=s.activation)
        y = ops.expert_linear(a, self.down_weight, plan)
        shared = self.shared.forward(h, step) if self.shared is not None else None
        return ops.moe_combine(y, plan, s.top, shared, gate, residual)


def _gcd8(*sizes: int) -> int:
    """8 if every size is a multiple of 8 (rows of whole 16-byte vectors in bfloat16), else 1."""
    return 8 if all(n % 8 == 0 for n in sizes) else 1
