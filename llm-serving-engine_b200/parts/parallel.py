"""Mixers side by side: every branch reads the same input; their outputs are normed one by one
and summed with fixed coefficients.

    out = sum_b coefficient_b * w_b * a_b / sqrt(mean(a_b^2) + eps),      a_b = branch_b(h)

Each branch is a mixer of its own kind with its own cache need; the cache layer of the block holds
all of them (pages for one, states for others), and each branch sees its own part of it.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from .base import MIXERS, BranchMix, Mixer, ParamDecl, count_states, flatten_needs, has_pages


@dataclass(frozen=True)
class ParallelMixerSpec:
    hidden_size: int
    names: tuple[str, ...]
    branches: tuple[Any, ...]  # mixer specs
    coefficients: tuple[float, ...]
    eps: float
    kind: str = "parallel"


@MIXERS.register("parallel")
class ParallelMixer(Mixer):
    def __init__(self, spec: ParallelMixerSpec, env) -> None:
        super().__init__(spec, env)
        if not (len(spec.names) == len(spec.branches) == len(spec.coefficients)) or not spec.branches:
            raise ValueError("names, branches and coefficients must have one entry per branch")
        self.children = {n: MIXERS.build(b, env) for n, b in zip(spec.names, spec.branches)}
        self.branches = list(self.children.values())
        # which part of the shared cache layer each branch sees
        self._parts = []
        first = 0
        for b in self.branches:
            need = b.cache_need()
            self._parts.append((has_pages(need), first, count_states(need)))
            first += count_states(need)

    def param_decls(self):
        out = {}
        for name, child in self.children.items():
            for pname, decl in child.param_decls().items():
                out[f"{name}.{pname}"] = decl
            out[f"out.{name}.weight"] = ParamDecl((self.spec.hidden_size,), "scale")
        return out

    def bind(self, params):
        self.out_weights = []
        for name, child in self.children.items():
            prefix = name + "."
            child.bind({k[len(prefix):]: v for k, v in params.items() if k.startswith(prefix)})
            self.out_weights.append(params[f"out.{name}.weight"])

    def cache_need(self):
        return tuple(n for b in self.branches for n in flatten_needs(b.cache_need()))

    accepts_deferral = True

    def forward(self, h, step, cache, may_defer=False):
        outs = []
        for b, (pages, first, n) in zip(self.branches, self._parts):
            defer = may_defer and getattr(b, "accepts_deferral", False)
            a = (b.forward(h, step, cache.part(pages, first, n), may_defer=True) if defer
                 else b.forward(h, step, cache.part(pages, first, n)))
            # a branch's product that is not converted yet stays so only if the caller takes such
            outs.append(a.resolve() if hasattr(a, "resolve") and not defer else a)
        return BranchMix(self.ops, outs, self.out_weights, tuple(self.spec.coefficients), self.spec.eps)
