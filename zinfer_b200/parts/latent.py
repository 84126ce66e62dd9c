"""Attention through a latent: per token the cache holds ONE row, [c | k_rot], from which every head's keys and
values could be expanded but never are for cached tokens.

With h the mixer's input, H heads, per head d unrotated and p rotated query/key entries, values e wide, a key/value
latent of r entries and a query latent of s entries:

    c_q   = rms(W_dq h) * w_q                     [s]        q = W_uq c_q, head by head [d unrotated | p rotated]
    [a|b] = W_dkv h                               [r + p]    c = rms(a) * w_c,  k_rot = rot(b): one part for all heads
    k_h   = W_uk,h c,   v_h = W_uv,h c
    score = (q_h[:d] . k_h + rot(q_h[d:]) . k_rot) * scale,  causal softmax,  o_h = sigmoid(W_g h)_h * sum_j w_j v_h(j)
    out   = W_o [o_0 .. o_{H-1}]

Since q_h[:d] . (W_uk,h c) = (W_uk,h^T q_h[:d]) . c and sum_j w_j W_uv,h c_j = W_uv,h sum_j w_j c_j, a step carries its
queries into the latent's space (one small product per head), runs multi-query attention over the cached rows, whose
first r entries also serve as the values, and expands the result with W_uv,h afterwards: the cache costs r + p values
a token whatever H is, and nothing is expanded for the tokens of earlier steps.  Norms, angles, scores, softmax and the
gate are float32; the gate's logits and the latents leave their contraction as float32.

A prompt step that starts its sequences reads nothing cached, and there the other order is cheaper: the step's own
tokens get every head's k_h and v_h (one contraction of c against [W_uk; W_uv]), a kernel lays [k_h | k_rot] and v_h
out in rows padded to the widths the tensor-core prompt kernel takes, and ordinary attention over those rows costs
d + p multiplications a score instead of r + p.  The cache rows are written all the same, for the steps that follow.
A prompt step that CONTINUES its sequences (a later portion of a long prompt) does the same over all their tokens:
the cached latents are packed and expanded once more, and the shared key part is read back from the cache rows.

The output gate is optional (`gate_name` None = none), as is the query latent (`q_down_name` None: q = W_uq h).
Options other designs use: `gate_per_value` (the gate has a logit for every output value, W_g [H * e, width], instead of
one per head); `sink_name` (one learned number per head; exp(sink_h) is one more term of head h's softmax denominator,
with no key and no value, not scaled); `interleaved` (the rotated part pairs entry 2i with entry 2i + 1 instead of i
with i + p/2: since the rotated query and key parts only ever meet in a dot product, the rows of W_uq and W_dkv that
make them are reordered once at load, pairs (2i, 2i + 1) -> (i, i + p/2), and every kernel rotates half-split pairs)."""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from .. import kernels
from .attention import key_chunks
from .base import MIXERS, KVRequest, Mixer, WeightSpec
from .linear import as_tensor, linear


# A prompt step expands keys and values when it brings at least this share of its sequences' tokens: expanding costs a
# contraction over ALL their tokens, which a step of a few tokens behind a long prompt would not earn back.
EXPAND_MIN_SHARE = 1.0 / 16


class LatentAttention(Mixer):
    capture_safe = True
    takes_pending_norm = True
    sums_through_linear = True

    def __init__(self, hidden: int, n_heads: int, dim: int, rot_dim: int, value_dim: int, kv_rank: int, q_rank: Optional[int],
                 scale: float, rot_base: float, q_down_name: Optional[str], q_norm_name: Optional[str], q_up_name: str,
                 kv_down_name: str, kv_norm_name: str, k_up_name: str, v_up_name: str, out_name: str,
                 gate_name: Optional[str] = None, norm_eps: float = 1e-5, split_keys: int = 0, gate_per_value: bool = False,
                 sink_name: Optional[str] = None, interleaved: bool = False):
        if rot_dim <= 0 or rot_dim % 2:
            raise ValueError(f"latent attention: the rotated width {rot_dim} must be even and positive")
        if (q_down_name is None) != (q_rank is None) or (q_down_name is None) != (q_norm_name is None):
            raise ValueError("latent attention: a query latent comes with its width, its projection and its norm")
        self.hidden, self.n_heads, self.dim, self.rot_dim, self.value_dim = hidden, n_heads, dim, rot_dim, value_dim
        self.kv_rank, self.q_rank, self.scale, self.rot_base, self.eps = kv_rank, q_rank, float(scale), float(rot_base), float(norm_eps)
        self.q_down_name, self.q_norm_name, self.q_up_name = q_down_name, q_norm_name, q_up_name
        self.kv_down_name, self.kv_norm_name, self.k_up_name, self.v_up_name = kv_down_name, kv_norm_name, k_up_name, v_up_name
        self.out_name, self.gate_name, self.split_keys = out_name, gate_name, int(split_keys)
        self.gate_per_value, self.sink_name, self.interleaved = bool(gate_per_value) and gate_name is not None, sink_name, bool(interleaved)
        self.sink = None
        self.w_dq = self.w_down = self.w_uq = self.w_uk_t = self.w_uv = self.w_out = self.q_norm = self.c_norm = self.inv_freq = None
        self._sm_count = 0

    @property
    def row_dim(self) -> int:
        """Width of a token's cache row and of a query carried into the latent's space."""
        return self.kv_rank + self.rot_dim

    def weight_specs(self):
        H, d, p, e, r, D = self.n_heads, self.dim, self.rot_dim, self.value_dim, self.kv_rank, self.hidden
        specs = [WeightSpec(self.q_up_name, (H * (d + p), self.q_rank if self.q_rank is not None else D)),
                 WeightSpec(self.kv_down_name, (r + p, D)), WeightSpec(self.kv_norm_name, (r,), role="vector", init="norm"),
                 WeightSpec(self.k_up_name, (H * d, r)), WeightSpec(self.v_up_name, (H * e, r)),
                 WeightSpec(self.out_name, (D, H * e))]
        if self.q_down_name is not None:
            specs += [WeightSpec(self.q_down_name, (self.q_rank, D)),
                      WeightSpec(self.q_norm_name, (self.q_rank,), role="vector", init="norm")]
        if self.gate_name is not None:
            specs.append(WeightSpec(self.gate_name, (H * e if self.gate_per_value else H, D)))
        if self.sink_name is not None:
            specs.append(WeightSpec(self.sink_name, (H,), role="vector"))
        return specs

    def load(self, weights, dtype, device):
        H, d, e, r = self.n_heads, self.dim, self.value_dim, self.kv_rank
        # the key/value latent, the shared key part and the gate's logits are one contraction with a float32 result
        self.w_dq = weights[self.q_down_name] if self.q_down_name is not None else None
        w_uq, w_dkv = weights[self.q_up_name], weights[self.kv_down_name]
        if self.interleaved:        # pairs (2i, 2i + 1) of the rotated parts become pairs (i, i + p/2)
            p = self.rot_dim
            order = torch.cat([torch.arange(0, p, 2), torch.arange(1, p, 2)]).to(w_uq.device)
            w_uq = w_uq.reshape(H, d + p, -1)
            w_uq = torch.cat([w_uq[:, :d], w_uq[:, d:][:, order]], dim=1).reshape(H * (d + p), -1).contiguous()
            w_dkv = torch.cat([w_dkv[:r], w_dkv[r:][order]], dim=0).contiguous()
        down = [w_dkv]
        if self.gate_name is not None:
            down.append(weights[self.gate_name])
        self.w_down = torch.cat(down, dim=0).contiguous()
        self.w_uq = w_uq
        self.sink = weights[self.sink_name].contiguous() if self.sink_name is not None else None
        self.w_uk_t = weights[self.k_up_name].reshape(H, d, r).transpose(1, 2).contiguous()      # [H, r, d]
        self.w_uv = weights[self.v_up_name].reshape(H, e, r).contiguous()                         # [H, e, r]
        self.w_out = weights[self.out_name]
        # for prompt steps that expand keys and values: [W_uk; W_uv] as one weight, and W_o with zero columns where
        # the attention kernel's value rows are wider than e
        self.w_ukv = self.w_out_wide = None
        self.key_width = self.value_width = 0
        if dtype == torch.bfloat16 and d + self.rot_dim <= 128 and e <= 128:
            kw, vw = (64 if d + self.rot_dim <= 64 else 128), (64 if e <= 64 else 128)
            self.key_width, self.value_width = max(kw, vw), vw
            self.w_ukv = torch.cat([weights[self.k_up_name], weights[self.v_up_name]], dim=0).contiguous()
            self.w_out_wide = self.w_out
            if vw != e:
                wide = torch.zeros((self.hidden, H, vw), dtype=self.w_out.dtype, device=self.w_out.device)
                wide[:, :, :e] = self.w_out.reshape(self.hidden, H, e)
                self.w_out_wide = wide.reshape(self.hidden, H * vw).contiguous()
        self.q_norm = weights[self.q_norm_name] if self.q_norm_name is not None else None
        self.c_norm = weights[self.kv_norm_name]
        i = np.arange(self.rot_dim // 2, dtype=np.float64)
        inv = np.power(np.float64(self.rot_base), -2.0 * i / np.float64(self.rot_dim)).astype(np.float32)
        self.inv_freq = torch.from_numpy(inv).to(device)
        self._sm_count = kernels.sm_count(device) if torch.device(device).type == "cuda" else 0

    def kv_request(self):
        return KVRequest(1, self.row_dim, 0, 0)           # one tensor per token, one "head"

    def check(self, dtype, page_size):
        most = kernels.attn_max_head_dim()
        if self.row_dim > most:
            raise ValueError(f"latent attention: a cache row of {self.kv_rank} + {self.rot_dim} values exceeds {most}")

    def launch_key(self, n_seqs, longest):
        return key_chunks(n_seqs, 1, longest, self._sm_count, self.split_keys)

    def _per_head(self, a, a_head, w, out, o_head, gate=None):
        """out[:, h] = a[:, h] w[h]^T for every head (times the head's gate)."""
        return kernels.head_gemm(a, a_head, w, out, o_head, gate)

    def forward(self, ctx, call, xn, out, accumulate):
        kv = call.kv
        H, d, p, e, r = self.n_heads, self.dim, self.rot_dim, self.value_dim, self.kv_rank
        n = ctx.n_tokens
        x = as_tensor(xn)
        low = linear(x, self.w_down, out_dtype=torch.float32)          # [n, r + p (+ H)] float32
        cq = x
        if self.w_dq is not None:
            cq = kernels.rmsnorm(linear(x, self.w_dq, out_dtype=torch.float32), self.q_norm, self.eps, ctx.dtype)
        q = linear(cq, self.w_uq)                                      # [n, H * (d + p)]
        dkv = low[:, :r + p]
        gate = low[:, r + p:] if self.gate_name is not None else None
        head_gate = None if self.gate_per_value else gate           # what the per-head products apply in their epilogue
        if (self.w_ukv is not None and ctx.starts is not None and not ctx.is_decode and call.writes_kv
                and ctx.n_tokens >= EXPAND_MIN_SHARE * sum(s + l for s, l in zip(ctx.starts, ctx.q_lens))
                and kernels.attention_step_rows_takes(q.dtype, self.key_width, self.value_width, kv.page_size)):
            return self._forward_expanded(ctx, kv, q, dkv, gate, out, accumulate)
        q_full = torch.empty((n, H * (r + p)), dtype=q.dtype, device=q.device)
        kernels.latent_prepare(q, q_full, dkv, self.c_norm, self.inv_freq, kv.k, ctx.tok_seq, ctx.tok_pos, ctx.seq_slot,
                               kv.page_table, H, d, p, r, self.eps, ctx.status, write_kv=call.writes_kv)
        self._per_head(q, d + p, self.w_uk_t, q_full, r + p)           # the unrotated parts, carried to the latent's space
        if ctx.is_decode and kernels.attention_latent_single_takes(q.dtype, H, r + p, r, kv.page_size):
            num_splits, split_keys = key_chunks(ctx.n_seqs, 1, ctx.max_kv_len, self._sm_count, self.split_keys)
            lat = kernels.attention_latent_single(q_full, kv.k, ctx.seq_start, ctx.seq_slot, kv.page_table, H, r, self.scale,
                                                  num_splits, split_keys, sink=self.sink)
            att = torch.empty((n, H * e), dtype=q.dtype, device=q.device)
            self._per_head(lat, r, self.w_uv, att, e, head_gate)
            if self.gate_per_value:
                kernels.value_gate(att, gate, H, e)
            linear(att, self.w_out, out=out, accumulate=accumulate)
            return
        kind, tile_tokens = kernels.attention_plan(q.dtype, H, 1, r + p, kv.page_size, ctx.is_decode, 0, r, False, False, True)
        from .attention import GqaAttention
        tile_seq, tile_q0 = ctx.memo(("query tiles", tile_tokens), lambda: GqaAttention._tiles_on_device(ctx, tile_tokens))
        num_splits, split_keys = (key_chunks(ctx.n_seqs, 1, ctx.max_kv_len, self._sm_count, self.split_keys)
                                  if ctx.is_decode else (1, 0))
        lat = kernels.attention(q_full, kv.k, None, tile_seq, tile_q0, ctx.cu_q, ctx.seq_start, ctx.seq_slot, kv.page_table,
                                H, 1, r + p, self.scale, 0, num_splits, split_keys, single_token=ctx.is_decode, kind=kind,
                                value_dim=r, values_in_keys=True, sink=self.sink)   # [n, H * r]: the weighted sums of the latents
        att = torch.empty((n, H * e), dtype=q.dtype, device=q.device)
        self._per_head(lat, r, self.w_uv, att, e, head_gate)
        if self.gate_per_value:
            kernels.value_gate(att, gate, H, e)
        linear(att, self.w_out, out=out, accumulate=accumulate)


    def _forward_expanded(self, ctx, kv, q, dkv, gate, out, accumulate):
        """A prompt step whose host knows where its sequences begin: keys and values expanded for the step's own tokens
        (sequences that start at position 0) or for every token of its sequences (a later portion of a prompt)."""
        H, d, p, e, r = self.n_heads, self.dim, self.rot_dim, self.value_dim, self.kv_rank
        n, page = ctx.n_tokens, kv.page_size
        c = torch.empty((n, r), dtype=q.dtype, device=q.device) if ctx.from_start else None
        kernels.latent_prepare(q, None, dkv, self.c_norm, self.inv_freq, kv.k, ctx.tok_seq, ctx.tok_pos, ctx.seq_slot,
                               kv.page_table, H, d, p, r, self.eps, ctx.status, write_kv=True, c_out=c)
        ends = [s + l for s, l in zip(ctx.starts, ctx.q_lens)]
        pages = [-(-t // page) for t in ends]

        def tables():
            words = [np.cumsum([0] + pages[:-1])]
            if not ctx.from_start:      # every position of every sequence, in order
                words += [np.repeat(np.arange(len(ends)), ends), np.concatenate([np.arange(t) for t in ends])]
            dev = torch.from_numpy(np.concatenate(words).astype(np.int32)).to(ctx.device, non_blocking=True)
            B, m = len(ends), sum(ends)
            return (dev[:B], None, None) if ctx.from_start else (dev[:B], dev[B:B + m], dev[B + m:])

        first, kv_seq, kv_pos = ctx.memo(("step rows", page), tables)
        if ctx.from_start:
            kvx = linear(c, self.w_ukv)                                # [n, H * d + H * e]
            q_pad, k_rows, v_rows = kernels.latent_pack(q, kvx, dkv, self.inv_freq, ctx.tok_pos, ctx.tok_seq, ctx.tok_pos, first,
                                                        sum(pages), page, H, d, p, e, r, self.key_width, self.value_width)
        else:                           # the cache rows (this step's among them, just written) are expanded once more
            c_all = kernels.latent_gather(kv.k, kv_seq, kv_pos, ctx.seq_slot, kv.page_table, r)
            kvx = linear(c_all, self.w_ukv)
            q_pad, k_rows, v_rows = kernels.latent_pack(q, kvx, None, self.inv_freq, ctx.tok_pos, kv_seq, kv_pos, first,
                                                        sum(pages), page, H, d, p, e, r, self.key_width, self.value_width,
                                                        cache=kv.k, seq_slot=ctx.seq_slot, page_table=kv.page_table)
        tile_tokens = kernels.attention_step_rows_tile_tokens(H)
        from .attention import GqaAttention
        tile_seq, tile_q0 = ctx.memo(("query tiles", tile_tokens), lambda: GqaAttention._tiles_on_device(ctx, tile_tokens))
        att = kernels.attention_step_rows(q_pad, k_rows, v_rows, tile_seq, tile_q0, ctx.cu_q, ctx.seq_start, first, H, self.scale,
                                          sink=self.sink)
        if self.gate_per_value:
            kernels.value_gate(att, gate, H, e)
        elif gate is not None:
            kernels.head_gate(att, gate, H)
        linear(att, self.w_out_wide, out=out, accumulate=accumulate)


MIXERS.register("latent_attention", LatentAttention)
