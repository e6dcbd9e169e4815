"""Mixture of small gated feed-forwards picked by a table: token id -> its `top` experts, each with
weight 1/top (no router, nothing learned at run time decides):

    y_t = (1/top) * sum_k  W_down[e_k] (silu(W_gate[e_k] x_t) * (W_up[e_k] x_t)),   e = table[token_t]

plus, optionally, a shared expert of the same form that every token takes, weighed by one number
per token: y_t += sigmoid(g . x_t) * Shared(x_t), the gate in float32 on the float32 rows.

The experts' matrices are stacked at load ([experts, rows, cols]); the kernels find a token's experts
through the table on the device, so the step needs nothing from the host and can be recorded.  The
part reads the token ids of the step from the step context (`ctx.tokens`)."""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from .base import FEED_FORWARDS, FeedForward, WeightSpec


class TableMoE(FeedForward):
    takes_residual_rows = True       # the shared expert's gate reads the float32 rows

    def __init__(self, hidden: int, ffn_dim: int, n_experts: int, top: int, vocab: int, table_name: str,
                 expert_names, shared: Optional[FeedForward] = None, shared_gate_name: Optional[str] = None):
        """expert_names(e) -> (gate name, up name, down name) of expert e.  `shared`: a feed-forward
        every token takes (built by the caller, e.g. a SwiGLU); `shared_gate_name`: the [1, hidden]
        vector of its per-token sigmoid gate (None = weight 1)."""
        if not 0 < top <= n_experts:
            raise ValueError(f"{top} experts per token out of {n_experts}")
        self.hidden, self.ffn_dim, self.n_experts, self.top, self.vocab = hidden, ffn_dim, n_experts, top, vocab
        self.table_name, self.names = table_name, [tuple(expert_names(e)) for e in range(n_experts)]
        self.shared, self.shared_gate_name = shared, shared_gate_name
        if shared is None and shared_gate_name is not None:
            raise ValueError("a shared-expert gate without a shared expert")
        self.table = self.w_gate = self.w_up = self.w_down = self.shared_gate = None

    def parts(self):
        return [self.shared] if self.shared is not None else []

    def weight_specs(self):
        F, D = self.ffn_dim, self.hidden
        specs = [WeightSpec(self.table_name, (self.vocab, self.top), role="table", bound=self.n_experts)]
        for g, u, d in self.names:
            specs += [WeightSpec(g, (F, D)), WeightSpec(u, (F, D)), WeightSpec(d, (D, F))]
        if self.shared_gate_name is not None:
            specs.append(WeightSpec(self.shared_gate_name, (1, D), role="vector"))
        return specs

    def load(self, weights, dtype, device):
        self.table = weights[self.table_name].contiguous()
        self.w_gate = torch.stack([weights[g] for g, _, _ in self.names]).contiguous()
        self.w_up = torch.stack([weights[u] for _, u, _ in self.names]).contiguous()
        self.w_down = torch.stack([weights[d] for _, _, d in self.names]).contiguous()
        if self.shared_gate_name is not None:
            self.shared_gate = weights[self.shared_gate_name].reshape(self.hidden).contiguous()

    def forward(self, ctx, xn, out, accumulate):
        rows = xn if xn.dtype == ctx.dtype else kernels.cast_rows(xn, ctx.dtype)
        kernels.moe_table(rows, ctx.tokens, self.table, self.w_gate, self.w_up, self.w_down, ctx.status, out=out,
                          accumulate=accumulate)
        if self.shared is None:
            return
        if self.shared_gate is None:
            self.shared.forward(ctx, rows, out, True)
            return
        if xn.dtype != torch.float32:
            raise ValueError("the shared expert's gate reads the float32 rows")
        branch = torch.empty_like(out)
        self.shared.forward(ctx, rows, branch, False)
        kernels.gate_add(xn, self.shared_gate, branch, out)


FEED_FORWARDS.register("table_moe", TableMoE)
