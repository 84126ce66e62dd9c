"""Retention mixer: linear attention with one fixed decay per head and neither softmax nor denominator.

Per head (H heads, d query/key channels, e value channels) a state S [d, e] that starts at zero and is carried from
token to token:

    q_t = rot(W_q h_t)        k_t = rot(W_k h_t) * key_scale        v_t = W_v h_t
    S_t = decay_h S_{t-1} + k_t v_t^T                                o_t = S_t^T q_t

with decay_h a constant of the configuration and rot an optional rotary encoding (half-split pairs over the first
entries of a head).  Each head's o_t is divided by its root mean square (no weight), the heads are concatenated,
multiplied value by value with silu(W_g h_t) and projected by W_o.

The four projections are one contraction against the stacked [2*H*d + 2*H*e, width] matrix whose result is kept in
float32; rotation, scale, state and all sums of the recurrence, the unit norm and the gate are float32 in both run
dtypes (`kernels.retention_scan`, the keyed form of the recurrence kernel that also serves `Hgrn2`;
`kernels.unit_norm_gate`).  The state lives in the cache's per-sequence state.  Prompt steps and single-token steps run
the same kernels, which walk a sequence's tokens from the state the step before left."""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from .. import kernels
from .base import MIXERS, Mixer, StateRequest, WeightSpec
from .linear import linear
from .rope import RotaryEncoding


class Retention(Mixer):
    capture_safe = True
    takes_pending_norm = True
    sums_through_linear = True

    def __init__(self, hidden: int, n_heads: int, dim: int, value_dim: int, decay: Sequence[float], q_name: str, k_name: str,
                 v_name: str, gate_name: str, out_name: str, position: Optional[RotaryEncoding] = None,
                 key_scale: Optional[float] = None, norm_eps: float = 1e-5):
        if len(decay) != n_heads:
            raise ValueError(f"retention: {len(decay)} decays for {n_heads} heads")
        if position is not None and position.interleaved:
            raise ValueError("retention: the recurrence kernel rotates half-split pairs only")
        self.hidden, self.n_heads, self.dim, self.value_dim, self.eps = hidden, n_heads, dim, value_dim, float(norm_eps)
        self.decay_host = [float(g) for g in decay]
        self.key_scale = float(dim) ** -0.5 if key_scale is None else float(key_scale)
        self.q_name, self.k_name, self.v_name, self.gate_name, self.out_name = q_name, k_name, v_name, gate_name, out_name
        self.position = position
        self.w_qkvg = self.w_out = self.decay = None

    @property
    def key_dim(self):
        return self.n_heads * self.dim

    @property
    def out_dim(self):
        return self.n_heads * self.value_dim

    def parts(self):
        return [self.position] if self.position is not None else []

    def weight_specs(self):
        return [WeightSpec(self.q_name, (self.key_dim, self.hidden)), WeightSpec(self.k_name, (self.key_dim, self.hidden)),
                WeightSpec(self.v_name, (self.out_dim, self.hidden)), WeightSpec(self.gate_name, (self.out_dim, self.hidden)),
                WeightSpec(self.out_name, (self.hidden, self.out_dim))]

    def load(self, weights, dtype, device):
        self.w_qkvg = torch.cat([weights[n] for n in (self.q_name, self.k_name, self.v_name, self.gate_name)], dim=0).contiguous()
        self.w_out = weights[self.out_name]
        self.decay = torch.tensor(self.decay_host, dtype=torch.float32).to(device)

    def state_request(self):
        return StateRequest((self.n_heads * self.dim * self.value_dim,), torch.float32)

    def check(self, dtype, page_size):
        if self.dim > kernels.hgrn2_max_dim():
            raise ValueError(f"retention: {self.dim} channels per head exceed the supported {kernels.hgrn2_max_dim()}")

    def forward(self, ctx, call, xn, out, accumulate):
        H, d, e = self.n_heads, self.dim, self.value_dim
        qkvg = linear(xn, self.w_qkvg, out_dtype=torch.float32)
        rot = self.position.rotary() if self.position is not None else None
        o = kernels.retention_scan(qkvg, self.decay, rot.inv_freq if rot else None, rot.n_rot if rot else 0, self.key_scale,
                                   ctx.tok_pos, call.state, ctx.cu_q, ctx.seq_slot, ctx.n_seqs, H, d, e)
        on = kernels.unit_norm_gate(o, qkvg[:, 2 * H * d + H * e:], H, self.eps, ctx.dtype)
        linear(on, self.w_out, out=out, accumulate=accumulate)


MIXERS.register("retention", Retention)
