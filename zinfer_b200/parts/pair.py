"""Two mixers side by side: both read the same normalised rows, each result is RMS-normalised over the model width
with a weight of its own, and the pair's result is a fixed share of their sum (half by default):

    out (+)= share * (rms(A(h)) * w_a + rms(B(h)) * w_b)

The two mixers are any parts with the `Mixer` interface; at most one of them may ask for a growing cache and at most
one for a per-sequence state (the call's storage is handed to both as it is, each takes what it asked for).  Norms and
sums are float32, both norms and the sum into the rows one kernel (`kernels.rmsnorm_pair_add`)."""
from __future__ import annotations

import torch

from .. import kernels
from .base import MIXERS, Mixer, WeightSpec
from .linear import as_tensor


class MixerPair(Mixer):
    def __init__(self, hidden: int, first: Mixer, second: Mixer, first_norm_name: str, second_norm_name: str,
                 norm_eps: float = 1e-5, share: float = 0.5):
        if first.kv_request() is not None and second.kv_request() is not None:
            raise ValueError("mixer pair: both sides ask for a growing cache; a call has one")
        if first.state_request() is not None and second.state_request() is not None:
            raise ValueError("mixer pair: both sides ask for a per-sequence state; a call has one")
        self.hidden, self.first, self.second = hidden, first, second
        self.first_norm_name, self.second_norm_name = first_norm_name, second_norm_name
        self.eps, self.share = float(norm_eps), float(share)
        self.w_first = self.w_second = None

    @property
    def capture_safe(self):
        return self.first.capture_safe and self.second.capture_safe

    def parts(self):
        return [self.first, self.second]

    def weight_specs(self):
        return [WeightSpec(self.first_norm_name, (self.hidden,), role="vector", init="norm"),
                WeightSpec(self.second_norm_name, (self.hidden,), role="vector", init="norm")]

    def load(self, weights, dtype, device):
        self.w_first, self.w_second = weights[self.first_norm_name], weights[self.second_norm_name]

    def kv_request(self):
        return self.first.kv_request() or self.second.kv_request()

    def state_request(self):
        return self.first.state_request() or self.second.state_request()

    def check(self, dtype, page_size):
        self.first.check(dtype, page_size)
        self.second.check(dtype, page_size)

    def launch_key(self, n_seqs, longest):
        return (self.first.launch_key(n_seqs, longest), self.second.launch_key(n_seqs, longest))

    def forward(self, ctx, call, xn, out, accumulate):
        h = as_tensor(xn)
        rows = out.rows if hasattr(out, "rows") else out
        if not accumulate:
            rows.zero_()
        both = torch.empty((2, h.shape[0], self.hidden), dtype=torch.float32, device=h.device)
        self.first.forward(ctx, call, h, both[0], False)
        self.second.forward(ctx, call, h, both[1], False)
        kernels.rmsnorm_pair_add(both[0], both[1], self.w_first, self.w_second, self.eps, rows, self.share)


MIXERS.register("mixer_pair", MixerPair)
