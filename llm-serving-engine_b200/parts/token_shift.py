"""Token shift: every row is blended with the row of the token before it.

    h_t = x_t + (x_{t-1} - x_t) * mix          element by element; x_{-1} = 0

``x`` is what the filter reads (the float32 residual stream), before any blending. The last row a
request has run is kept per request (a state of ``size`` float32 values), so that a prompt cut
into portions, or a single decoded token, finds its predecessor. A request's first token
(position 0) reads zeros whatever the state slot held before.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .base import INPUT_FILTERS, ParamDecl, Part, StateNeed


@dataclass(frozen=True)
class TokenShiftSpec:
    size: int
    kind: str = "token_shift"


@INPUT_FILTERS.register("token_shift")
class TokenShift(Part):
    """``forward(x, step, cache) -> h`` in the compute dtype; ``cache.state`` is ``[slots, size]``."""

    keeps_running_state = True  # a step changes the state for good: no step may be run twice

    def param_decls(self):
        return {"mix": ParamDecl((self.spec.size,), "mix")}

    def cache_need(self):
        return StateNeed((self.spec.size,), torch.float32)

    def forward(self, x, step, cache):
        return self.ops.token_shift(x, self.mix, cache.state, step, out_dtype=self.env.dtype)
