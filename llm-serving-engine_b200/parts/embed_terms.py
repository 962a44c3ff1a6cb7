"""Terms that are added to the embedded tokens before the first layer.

``hashed_pair``: a second table, indexed by the token and the token before it,

    row = (previous * mul_previous + token * mul_token) mod buckets,

with a row of its own (the last, number ``buckets``) for a sequence's first token. The token
before a portion's first one is kept per request: an int32 state of one number that each step
replaces by its last token.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .base import EMBED_TERMS, EmbedTerm, ParamDecl, StateNeed


@dataclass(frozen=True)
class HashedPairSpec:
    hidden_size: int
    buckets: int
    mul_previous: int
    mul_token: int
    kind: str = "hashed_pair"


@EMBED_TERMS.register("hashed_pair")
class HashedPairEmbedding(EmbedTerm):
    keeps_running_state = True  # the token before the next step's first row

    def __init__(self, spec: HashedPairSpec, env) -> None:
        super().__init__(spec, env)
        if spec.buckets < 1 or spec.mul_previous < 0 or spec.mul_token < 0:
            raise ValueError("hashed_pair: buckets must be positive and the multipliers not negative")

    def param_decls(self):
        return {"table": ParamDecl((self.spec.buckets + 1, self.spec.hidden_size), "embedding")}

    def cache_need(self):
        return StateNeed((1,), torch.int32)

    def forward(self, x, step, cache) -> None:
        s = self.spec
        self.ops.hashed_pair_add(x, self.table, cache.state, step, buckets=s.buckets,
                                 mul_previous=s.mul_previous, mul_token=s.mul_token)
