"""A causal convolution over time on what a mixer READS: h_t = x_t + sum_j w[:, j] * x_{t-K+1+j}
per channel, zeros before a sequence's start, K taps, no bias; the wrapped mixer then runs on h.

`InputConv` is itself a mixer: it asks for the inner mixer's growing cache and for a fixed-size
state of its own, the last K-1 rows x of the sequence (float32, zero at a sequence's start), so
that a sequence cut into steps convolves as if it were whole.  The convolution is float32 on the
float32 residual rows (`takes_residual_rows`); h goes on in the run dtype.  The file stores the
taps [channels, K]; they are kept [K, channels] so that a tap's channels lie side by side."""
from __future__ import annotations

import torch

from .. import kernels
from .base import MIXERS, Mixer, StateRequest, WeightSpec


class InputConv(Mixer):
    takes_residual_rows = True

    def __init__(self, inner: Mixer, channels: int, taps: int, weight_name: str, residual: bool = True):
        if taps < 1:
            raise ValueError(f"a convolution needs at least one tap, got {taps}")
        if inner.state_request() is not None:
            raise ValueError("InputConv keeps the call's state itself; the inner mixer must not ask for one")
        self.inner, self.channels, self.taps, self.weight_name, self.residual = inner, channels, int(taps), weight_name, residual
        self.weight = None

    @property
    def capture_safe(self):
        return self.inner.capture_safe

    def parts(self):
        return [self.inner]

    def weight_specs(self):
        return [WeightSpec(self.weight_name, (self.channels, self.taps), role="vector")]

    def load(self, weights, dtype, device):
        self.weight = weights[self.weight_name].t().contiguous()

    def kv_request(self):
        return self.inner.kv_request()

    def state_request(self):
        # one row at least, so that a single tap (no history) still has a tensor to point at
        return StateRequest((max(self.taps - 1, 1), self.channels), torch.float32)

    def check(self, dtype, page_size):
        if self.taps > kernels.seqconv_max_taps():
            raise ValueError(f"input convolution: {self.taps} taps exceed the supported {kernels.seqconv_max_taps()}")
        self.inner.check(dtype, page_size)

    def launch_key(self, n_seqs, longest):
        return self.inner.launch_key(n_seqs, longest)

    def forward(self, ctx, call, xn, out, accumulate):
        state = call.state[:, :self.taps - 1] if self.taps > 1 else call.state[:, :0]
        h = kernels.seqconv(xn, state, self.weight, ctx.tok_seq, ctx.cu_q, ctx.seq_slot, ctx.n_seqs, ctx.dtype,
                            residual=self.residual, single_token=ctx.is_decode)
        self.inner.forward(ctx, call, h, out, accumulate)


MIXERS.register("input_conv", InputConv)
