"""What a repeated stretch of layers is given at the start of each pass.

A model may run some consecutive layers several times in a row with the same weights (each pass with a
cache and state of its own: the schedule simply names those layers again).  Right before the first layer
of pass t = 0, 1, ... the residual rows x become

    x <- x + x_emb   (only for t > 0; x_emb = the rows as the embedding left them)
    x <- x + step[t]  (a learned vector per pass, `step` [passes, width])

both in float32, in this order.  `PassInput` holds the `step` table and knows before which schedule
entries a pass starts; `Model.forward` calls it between the entries."""
from __future__ import annotations

from typing import Mapping

from .. import kernels
from .base import Part, WeightSpec


class PassInput(Part):
    def __init__(self, step_name: str, passes: int, width: int, starts: Mapping[int, int]):
        """starts: schedule index of a pass's first entry -> the pass's number."""
        self.step_name, self.passes, self.width = step_name, int(passes), int(width)
        self.starts = {int(c): int(t) for c, t in starts.items()}
        if any(not 0 <= t < self.passes for t in self.starts.values()):
            raise ValueError(f"pass numbers {sorted(self.starts.values())} outside the {self.passes} passes")
        self.step = None

    def weight_specs(self):
        return [WeightSpec(self.step_name, (self.passes, self.width), role="vector")]

    def load(self, weights, dtype, device):
        self.step = weights[self.step_name]

    @property
    def needs_embedding(self) -> bool:
        return any(t > 0 for t in self.starts.values())

    def starts_at(self, call_index: int) -> bool:
        return call_index in self.starts

    def before(self, ctx, call_index: int, x, x_emb) -> None:
        t = self.starts.get(call_index)
        if t is not None:
            kernels.rows_add(x, self.step[t], x_emb if t > 0 else None)
