"""Depth-weighted average of the residual stream: what goes on to the next layer is not the layer's
result alone but a learned mix of every result so far,

    x_in(i+1) = sum_{j = 0 .. i+1} a_i[j] * X_j,      X_0 = embedding output, X_{j+1} = result of layer j

with one weight vector a_i of i+2 numbers per layer (the last layer's mix is what the final norm reads).

The model keeps the X_j of a step in ONE float32 buffer [layers + 2, tokens, width]: plane j+1 starts as
layer j's input (written by the mix of the layer before) and the layer turns it into X_{j+1} in place,
so no result is copied.  The sum is float32 and runs in the order of j."""
from __future__ import annotations

import torch

from .. import kernels
from .base import Part, WeightSpec


class DepthAverage(Part):
    def __init__(self, weight_names):
        """weight_names[i]: the vector of i + 2 weights applied after the i-th layer run."""
        self.weight_names = list(weight_names)
        self.weights: list[torch.Tensor] = []

    def weight_specs(self):
        return [WeightSpec(n, (i + 2,), role="vector", init="norm") for i, n in enumerate(self.weight_names)]

    def load(self, weights, dtype, device):
        self.weights = [weights[n] for n in self.weight_names]

    def planes(self, ctx, n_runs: int, width: int) -> torch.Tensor:
        if n_runs != len(self.weight_names):
            raise ValueError(f"{n_runs} layer runs, depth weights for {len(self.weight_names)}")
        return torch.empty((n_runs + 2, ctx.n_tokens, width), dtype=torch.float32, device=ctx.device)

    def first_input(self, planes: torch.Tensor) -> torch.Tensor:
        """Plane 0 holds X_0; the first layer works on a copy of it in plane 1."""
        return kernels.weighted_sum(planes, None, 1, planes[1])

    def after(self, planes: torch.Tensor, run: int) -> torch.Tensor:
        """Plane run + 1 now holds X_{run+1}: the mix goes to plane run + 2 and is returned."""
        return kernels.weighted_sum(planes, self.weights[run], run + 2, planes[run + 2])
