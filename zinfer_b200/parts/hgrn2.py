"""HGRN2 mixer: a gated linear recurrence over a matrix state; the gate that decays the state also sets how much
of the new value enters it (input gate = 1 - forget gate).

Per head (H heads, d query channels, e value channels) a state S [d, e] that starts at zero and is
carried from token to token:

    q_t = silu(W_q h_t)            f_t = l + (1 - l) * sigmoid(W_f h_t + b_f)         v_t = W_v h_t
    S_t = diag(f_t) S_{t-1} + (1 - f_t) v_t^T                o_t = S_t^T q_t

with l in [0, 1) a learned lower bound of the gate per head and channel (stored as it is used).  The mixer has
no key projection: 1 - f_t stands where a key would.  Each head's o_t is RMS-normalised over its e values with one weight
vector [e] shared by the heads; the heads are concatenated and projected by W_o.

The three projections are one contraction against the stacked [2*H*d + H*e, width] matrix whose result is
kept in float32; the gate, the state and all sums of the recurrence are float32 in both run dtypes
(`kernels.hgrn2_scan`), the state lives in the cache's per-sequence state.  Prompt steps and single-token
steps run the same kernel, which walks a sequence's tokens from the state the step before left."""
from __future__ import annotations

import torch

from .. import kernels
from .base import MIXERS, Mixer, StateRequest, WeightSpec
from .linear import linear


class Hgrn2(Mixer):
    capture_safe = True
    takes_pending_norm = True
    sums_through_linear = True

    def __init__(self, hidden: int, n_heads: int, dim: int, value_dim: int, q_name: str, f_name: str, f_bias_name: str,
                 lower_name: str, v_name: str, norm_name: str, out_name: str, norm_eps: float = 1e-5):
        self.hidden, self.n_heads, self.dim, self.value_dim, self.eps = hidden, n_heads, dim, value_dim, float(norm_eps)
        self.q_name, self.f_name, self.f_bias_name, self.lower_name = q_name, f_name, f_bias_name, lower_name
        self.v_name, self.norm_name, self.out_name = v_name, norm_name, out_name
        self.w_qfv = self.w_out = self.f_bias = self.lower = self.norm = None

    @property
    def gate_dim(self):
        return self.n_heads * self.dim

    @property
    def out_dim(self):
        return self.n_heads * self.value_dim

    def weight_specs(self):
        return [WeightSpec(self.q_name, (self.gate_dim, self.hidden)),
                WeightSpec(self.f_name, (self.gate_dim, self.hidden)),
                WeightSpec(self.f_bias_name, (self.gate_dim,), role="vector"),
                WeightSpec(self.lower_name, (self.gate_dim,), role="vector", init="unit_interval"),
                WeightSpec(self.v_name, (self.out_dim, self.hidden)),
                WeightSpec(self.norm_name, (self.value_dim,), role="vector", init="norm"),
                WeightSpec(self.out_name, (self.hidden, self.out_dim))]

    def load(self, weights, dtype, device):
        self.w_qfv = torch.cat([weights[self.q_name], weights[self.f_name], weights[self.v_name]], dim=0).contiguous()
        self.w_out = weights[self.out_name]
        self.f_bias, self.lower, self.norm = weights[self.f_bias_name], weights[self.lower_name], weights[self.norm_name]

    def state_request(self):
        return StateRequest((self.n_heads * self.dim * self.value_dim,), torch.float32)

    def check(self, dtype, page_size):
        if self.dim > kernels.hgrn2_max_dim():
            raise ValueError(f"hgrn2: {self.dim} channels per head exceed the supported {kernels.hgrn2_max_dim()}")

    def forward(self, ctx, call, xn, out, accumulate):
        qfv = linear(xn, self.w_qfv, out_dtype=torch.float32)
        o = kernels.hgrn2_scan(qfv, self.f_bias, self.lower, call.state, ctx.cu_q, ctx.seq_slot, ctx.n_seqs,
                               self.n_heads, self.dim, self.value_dim)
        on = kernels.rmsnorm(o.view(-1, self.value_dim), self.norm, self.eps, ctx.dtype).view(-1, self.out_dim)
        linear(on, self.w_out, out=out, accumulate=accumulate)


MIXERS.register("hgrn2", Hgrn2)
