"""What a repeated stretch of layers is given at the start of each pass.

A model may run some consecutive layers several times in a row with the same weights (each pass with a
cache and state of its own: the schedule simply names those layers again).  Right before the first layer
of pass t = 0, 1, ... the residual rows x become

    x <- x + x_emb   (only for t > 0; x_emb = the rows as the embedding left them)
    x <- x + step[t]  (a learned vector per pass, `step` [passes, width])

both in float32, in this order.  `PassInput` holds the `step` table and knows before which schedule
entries a pass starts; `Model.forward` calls it between the entries.

With `in_name` the first line is a learned map of the rows and the embedding's rows together instead, in EVERY pass
(the first too):

    x <- W_in [x; x_emb]          (W_in [width, 2 width], the columns that meet x first)

W_in is cut at load into its two halves, so the step is two contractions that add into the same float32 rows;
their inputs are the rows in the run dtype."""
from __future__ import annotations

from typing import Mapping

import torch

from .. import kernels
from .base import Part, WeightSpec


class PassInput(Part):
    def __init__(self, step_name: str, passes: int, width: int, starts: Mapping[int, int], in_name: str | None = None):
        """starts: schedule index of a pass's first entry -> the pass's number."""
        self.step_name, self.passes, self.width = step_name, int(passes), int(width)
        self.in_name, self.w_rows, self.w_emb, self._emb = in_name, None, None, None
        self.starts = {int(c): int(t) for c, t in starts.items()}
        if any(not 0 <= t < self.passes for t in self.starts.values()):
            raise ValueError(f"pass numbers {sorted(self.starts.values())} outside the {self.passes} passes")
        self.step = None

    def weight_specs(self):
        specs = [WeightSpec(self.step_name, (self.passes, self.width), role="vector")]
        if self.in_name is not None:
            specs.append(WeightSpec(self.in_name, (self.width, 2 * self.width)))
        return specs

    def load(self, weights, dtype, device):
        self.step = weights[self.step_name]
        if self.in_name is not None:
            w = weights[self.in_name]
            self.w_rows, self.w_emb = w[:, :self.width].contiguous(), w[:, self.width:].contiguous()

    @property
    def needs_embedding(self) -> bool:
        return self.in_name is not None or any(t > 0 for t in self.starts.values())

    def starts_at(self, call_index: int) -> bool:
        return call_index in self.starts

    def before(self, ctx, call_index: int, x, x_emb) -> None:
        t = self.starts.get(call_index)
        if t is None:
            return
        if self.in_name is None:
            kernels.rows_add(x, self.step[t], x_emb if t > 0 else None)
            return
        from .linear import linear
        rows = kernels.cast_rows(x, ctx.dtype) if ctx.dtype != x.dtype else kernels.weighted_sum(x.unsqueeze(0), None, 1, torch.empty_like(x))
        # the embedding's rows in the run dtype, made once per step (every pass reads the same rows)
        if self._emb is None or self._emb[0] is not x_emb:
            self._emb = (x_emb, kernels.cast_rows(x_emb, ctx.dtype) if ctx.dtype != x_emb.dtype else x_emb)
        emb = self._emb[1]
        linear(rows, self.w_rows, out=x)                  # x is overwritten: `rows` is a copy of it
        linear(emb, self.w_emb, out=x, accumulate=True)
        kernels.rows_add(x, self.step[t])
