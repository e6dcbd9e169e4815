"""Token shift on a mixer's input: every channel of row t is moved towards the same channel of row t-1 by a
learned fraction, h_t <- h_t + (h_{t-1} - h_t) * mu, where h_{t-1} is the UNSHIFTED row of the token before (a
zero row ahead of a sequence's first token).

`TokenShift` is a mixer that wraps a mixer.  It asks for the inner mixer's growing cache, and for ONE
per-sequence state that holds its own row (the last token's unshifted h, float32) followed by whatever
fixed state the inner mixer asks for; the inner mixer sees its part as a view.  So a sequence cut into
steps shifts as if it were whole.  When the block's norm is still pending the shift kernel applies it
itself (one pass over the residual rows, float32; h goes on in the run dtype); it also takes float32 rows
that are to be shifted as they are."""
from __future__ import annotations

import math
from dataclasses import replace

import torch

from .. import kernels
from .base import MIXERS, Mixer, StateRequest, WeightSpec
from .linear import NormedRows


class TokenShift(Mixer):
    takes_pending_norm = True
    takes_residual_rows = True

    def __init__(self, inner: Mixer, channels: int, weight_name: str):
        self.inner, self.channels, self.weight_name = inner, int(channels), weight_name
        self.mu = None
        inner_state = inner.state_request()
        if inner_state is not None and inner_state.dtype != torch.float32:
            raise ValueError("TokenShift keeps the call's state as float32; the inner mixer asks for another type")
        self._inner_shape = None if inner_state is None else tuple(inner_state.shape)

    @property
    def capture_safe(self):
        return self.inner.capture_safe

    @property
    def sums_through_linear(self):
        return getattr(self.inner, "sums_through_linear", False)

    def parts(self):
        return [self.inner]

    def weight_specs(self):
        return [WeightSpec(self.weight_name, (self.channels,), role="vector", init="unit_interval")]

    def load(self, weights, dtype, device):
        self.mu = weights[self.weight_name]

    def kv_request(self):
        return self.inner.kv_request()

    def state_request(self):
        extra = 0 if self._inner_shape is None else math.prod(self._inner_shape)
        return StateRequest((self.channels + extra,), torch.float32)

    def check(self, dtype, page_size):
        self.inner.check(dtype, page_size)

    def launch_key(self, n_seqs, longest):
        return self.inner.launch_key(n_seqs, longest)

    def forward(self, ctx, call, xn, out, accumulate):
        if isinstance(xn, NormedRows):
            x, w, eps = xn.x, xn.weight, xn.eps
        elif isinstance(xn, torch.Tensor) and xn.dtype == torch.float32:
            x, w, eps = xn, None, 0.0
        else:
            raise ValueError("TokenShift reads float32 rows, or a norm of them that is still pending")
        h = kernels.norm_shift(x, w, eps, self.mu, call.state, ctx.tok_seq, ctx.cu_q, ctx.seq_slot, ctx.n_seqs, ctx.dtype,
                               single_token=ctx.is_decode)
        inner_call = call
        if self._inner_shape is not None:
            inner_call = replace(call, state=call.state[:, self.channels:].unflatten(1, self._inner_shape))
        else:
            inner_call = replace(call, state=None)
        self.inner.forward(ctx, inner_call, h, out, accumulate)


MIXERS.register("token_shift", TokenShift)
