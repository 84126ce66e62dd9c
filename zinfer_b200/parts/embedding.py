"""Token embedding and output head.  x_t = E[token_t] (times a scale, 1 here:
src/model.zig:2352-2358, 466); logits = xn W_out^T in float32 with W_out the head tensor or
the embedding itself when tied (src/model.zig:595-598, 2490).

Two options other designs use: a learned position table whose row for the token's position is
added to the embedding (unscaled, float32), a soft cap on the logits,
logits <- cap * tanh(logits / cap), and a constant the logits are multiplied by (`scale`, applied last)."""
from __future__ import annotations

import torch

from .. import kernels
from .base import Part, WeightSpec
from .linear import linear


class TokenEmbedding(Part):
    def __init__(self, vocab: int, dim: int, weight_name: str, scale: float = 1.0,
                 position_name: str | None = None, max_positions: int = 0):
        """position_name: a learned table [max_positions, dim] whose row of the token's position is added."""
        self.vocab, self.dim, self.weight_name, self.scale = vocab, dim, weight_name, float(scale)
        self.position_name, self.max_positions = position_name, int(max_positions)
        if position_name is not None and self.max_positions <= 0:
            raise ValueError("a position table needs its number of positions")
        self.weight = self.positions = None

    def weight_specs(self):
        specs = [WeightSpec(self.weight_name, (self.vocab, self.dim))]
        if self.position_name is not None:
            specs.append(WeightSpec(self.position_name, (self.max_positions, self.dim)))
        return specs

    def load(self, weights, dtype, device):
        self.weight = weights[self.weight_name]
        self.positions = weights[self.position_name] if self.position_name is not None else None

    def forward(self, ctx, tokens: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        return kernels.embed(tokens, self.weight, ctx.status, self.scale, self.positions,
                             ctx.tok_pos if self.positions is not None else None, out=out)


class LMHead(Part):
    """`weight_name` None ties the head to `embedding`."""

    def __init__(self, vocab: int, dim: int, weight_name: str | None, embedding: TokenEmbedding | None = None,
                 softcap: float | None = None, scale: float = 1.0):
        if weight_name is None and embedding is None:
            raise ValueError("a tied head needs the embedding it is tied to")
        if softcap is not None and not softcap > 0:
            raise ValueError(f"a logit cap must be positive, got {softcap}")
        self.vocab, self.dim, self.weight_name, self.embedding = vocab, dim, weight_name, embedding
        self.softcap = None if softcap is None else float(softcap)
        self.scale = float(scale)
        self.weight = None

    def weight_specs(self):
        return [] if self.weight_name is None else [WeightSpec(self.weight_name, (self.vocab, self.dim))]

    def load(self, weights, dtype, device):
        self.weight = None if self.weight_name is None else weights[self.weight_name]

    takes_pending_norm = True

    def forward(self, ctx, xn, out: torch.Tensor | None = None) -> torch.Tensor:
        """float32 logits of the rows of xn (a tensor, or a norm still pending), into `out` if given."""
        w = self.weight if self.weight is not None else self.embedding.weight
        logits = linear(xn, w, out=out, out_dtype=torch.float32)
        if self.softcap is not None:
            kernels.softcap(logits, self.softcap)
        if self.scale != 1.0:
            kernels.scale_(logits, self.scale)
        return logits
