"""Grouped-query attention mixer over the paged cache (src/model.zig:1715-1991).

q, k, v come from one contraction against the stacked [Q + 2KV, D] weight (the reference fuses
them in one dispatch, src/model.zig:1720-1734); then per-head RMSNorm of q and k with the
layer's eps, before the rotation (src/model.zig:1741-1744, 1760-1763); keys and values are
written to the cache at the tokens' absolute positions; every query then attends to the cache
(its own token included) under the causal mask and an optional window
(src/model.zig:1362-1363); the output projection adds into the residual stream
(src/model.zig:1988-1990).  Scores are scaled by 1/sqrt(head_dim) (src/model.zig:465).

A call that reads another call's cache (`call.writes_kv` False) computes only its queries; a
mixer built with `own_kv=False` has no key and value weights at all and can only run in such a call.

Options that other designs use: `value_dim` (values of another width than keys), `qk_norm_span`
"all" (the q norm runs over all heads of a token at once with a weight of that width, likewise k;
"head" is the per-head norm with a weight of head_dim), `distance_bias` = (name of r1, name of r2),
two numbers per query head: r1_h * ln(1 + r2_h * (i - j)) is taken off the scaled score of query
position i and key position j, in float32, before the softmax.  `unit_norm_after_rotation`: q and k
heads are divided by their root mean square (no weight, the layer's eps) after the position encoding.
`talk_name`: a matrix T [heads, heads]; after the softmax head h's weights become
sum_g T[h, g] * (weights of head g), and head h applies them to the values of its own key/value head.
`keep_first` (with a window): the first so many tokens of a sequence stay visible to every later query, at their
true positions; the cache keeps their pages.  `sink_name`: one learned number per head, [heads]; exp(sink_h) is
one more term of head h's softmax denominator, with no key and no value, and is not scaled.
`query_temperature` = (coef, every): the query at position p is multiplied by 1 + coef * ln(floor((p + 1) / every) + 1)
(positions enter through that factor alone when there is no position encoding).  `softcap`: a scaled score s becomes
softcap * tanh(s / softcap) before the softmax.
`pad_heads`: in a bfloat16 run, heads whose keys and values are not both 64 or both 128 wide (and at most 128) are
padded at load to the next of those widths, with zero rows in W_q, W_k and W_v and zero columns in W_o, so that the
tensor-core kernels take them; a padded entry adds nothing to a score and meets a zero column of W_o, the cache holds
the padded rows.  Only without q/k norms (a norm would count the padding).

How the kernels are launched is decided here, not by the engine: the table of query tiles of a
step, and for single-token steps the cut of a sequence's keys into chunks that separate blocks
walk (the reference cuts single-token attention into up to 16 chunks for its threads,
src/model.zig:1941-1955).
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import numpy as np
import torch

from .. import kernels
from .base import MIXERS, KVRequest, Mixer, PositionEncoding, WeightSpec
from .linear import linear


def query_tiles(q_lens: Sequence[int], bq: int) -> np.ndarray:
    """Query tiles of `bq` tokens: rows [tile_seq; tile_q0] as one int32 array [2, n_tiles]."""
    seq, q0 = [], []
    for b, l in enumerate(q_lens):
        for s in range(0, l, bq):
            seq.append(b)
            q0.append(s)
    return np.asarray([seq, q0], dtype=np.int32).reshape(2, len(seq))


def key_capacity(longest: int) -> int:
    """The smallest of 512, 768, 1024, 1536, 2048, 3072, ... that holds `longest` keys.  The chunks of a
    single-token step are laid out for this capacity, not for the longest sequence itself, so
    that the layout (which a recorded step bakes in) changes a few times in a sequence's life
    instead of every few hundred tokens; chunks beyond a sequence's end cost a block that exits."""
    cap = 512
    while cap < longest:
        cap = cap * 3 // 2 if cap & (cap - 1) == 0 else cap // 3 * 4
    return cap


CHUNK_ALIGN = 64            # chunk boundaries the single-token kernels take (their key tile)


def key_chunks(n_seqs: int, n_kv_heads: int, longest: int, sm_count: int, split_keys: int = 0) -> tuple[int, int]:
    """(number of key chunks, keys per chunk) for single-token attention of `n_seqs` sequences up to
    `longest` tokens long.  The cuts lie at multiples of the chunk size, whatever the batch, and
    the chunks are added in order by the merge kernel, so a sequence's result does not depend on its
    neighbours.  split_keys > 0 fixes the chunk size; otherwise it is chosen so that about four
    blocks per SM have work, between 128 and 4096 keys: with unequal sequences a longer chunk
    leaves the SMs that drew a short sequence idle (64 sequences of 1K to 32K tokens on a B200:
    3.90 ms a step with chunks of 16K keys, 3.27 ms with 4K)."""
    if longest <= 0:
        return 1, 0
    cap = key_capacity(longest)
    keys = split_keys
    if keys <= 0:
        blocks = max(1, n_seqs * n_kv_heads)
        want = max(1, -(-4 * max(sm_count, 1) // blocks))
        keys = min(4096, max(128, -(-cap // want)))
        keys = -(-keys // CHUNK_ALIGN) * CHUNK_ALIGN
    n = -(-cap // keys)
    return (n, keys) if n > 1 else (1, 0)


class GqaAttention(Mixer):
    capture_safe = True

    def __init__(self, hidden: int, n_heads: int, n_kv_heads: int, head_dim: int, q_name: str, k_name: str,
                 v_name: str, out_name: str, q_norm_name: Optional[str] = None, k_norm_name: Optional[str] = None,
                 norm_eps: float = 1e-5, position: Optional[PositionEncoding] = None, window: int = 0,
                 scale: Optional[float] = None, split_keys: int = 0, value_dim: Optional[int] = None,
                 qk_norm_span: str = "head", distance_bias: Optional[tuple[str, str]] = None, own_kv: bool = True,
                 unit_norm_after_rotation: bool = False, talk_name: Optional[str] = None, keep_first: int = 0,
                 sink_name: Optional[str] = None, query_temperature: Optional[tuple[float, int]] = None,
                 softcap: Optional[float] = None, pad_heads: bool = False):
        """split_keys: keys per chunk of single-token attention, a multiple of 64 (0 = chosen per
        step from the batch and the GPU's size)."""
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} heads are not a multiple of {n_kv_heads} KV heads")    # src/model.zig:487
        if qk_norm_span not in ("head", "all"):
            raise ValueError(f"qk_norm_span {qk_norm_span!r}: 'head' or 'all'")
        self.value_dim = head_dim if value_dim is None else int(value_dim)
        self.qk_norm_span, self.distance_bias, self.own_kv = qk_norm_span, distance_bias, bool(own_kv)
        # the kernel that prepares q and k over the whole projection takes a rotation table, no other encoding
        self.span_prepare = qk_norm_span == "all" or not own_kv
        if self.span_prepare and unit_norm_after_rotation:
            raise ValueError("attention: a norm behind the position encoding goes with per-head norms")
        if self.span_prepare and position is not None and not own_kv:
            raise ValueError("attention: a position encoding goes with key/value weights of the mixer's own")
        if keep_first < 0 or (keep_first > 0 and window <= 0):
            raise ValueError("attention: kept first tokens go with a window")
        if (keep_first > 0 or sink_name is not None) and (talk_name is not None or distance_bias is not None):
            raise ValueError("attention: no kernel takes kept first tokens or a sink together with a distance bias or "
                             "weights mixed across heads")
        self.keep_first, self.sink_name, self.sink = int(keep_first), sink_name, None
        if query_temperature is not None and (int(query_temperature[1]) <= 0 or qk_norm_span == "all" or not own_kv):
            raise ValueError("attention: a query temperature needs a positive period and goes with per-head preparation")
        self.query_temperature = None if query_temperature is None else (float(query_temperature[0]), int(query_temperature[1]))
        if softcap is not None and (not softcap > 0 or talk_name is not None):
            raise ValueError("attention: a score cap must be positive and does not go with weights mixed across heads")
        self.softcap = 0.0 if softcap is None else float(softcap)
        if pad_heads and (q_norm_name or k_norm_name or unit_norm_after_rotation or not own_kv or qk_norm_span == "all"):
            raise ValueError("attention: padded heads go with key/value weights of the mixer's own and no q/k norms")
        self.pad_heads = bool(pad_heads)
        self.run_head_dim, self.run_value_dim = head_dim, self.value_dim      # the widths the kernels see (load may pad)
        if self.span_prepare and qk_norm_span == "head" and (q_norm_name or k_norm_name):
            raise ValueError("attention: per-head norms go with key/value weights of the mixer's own")
        if talk_name is not None and distance_bias is not None:
            raise ValueError("attention: no kernel takes a distance bias together with weights mixed across heads")
        self.unit_norm_after, self.talk_name, self.talk = bool(unit_norm_after_rotation), talk_name, None
        self.bias_r1 = self.bias_r2 = None
        self.split_keys = int(split_keys)
        self._sm_count = 0
        self.hidden, self.n_heads, self.n_kv, self.head_dim = hidden, n_heads, n_kv_heads, head_dim
        self.q_name, self.k_name, self.v_name, self.out_name = q_name, k_name, v_name, out_name
        self.q_norm_name, self.k_norm_name = q_norm_name, k_norm_name
        self.eps, self.position, self.window = float(norm_eps), position, int(window)
        self.scale = 1.0 / math.sqrt(head_dim) if scale is None else float(scale)
        self.w_qkv = self.w_out = self.q_norm = self.k_norm = None

    @property
    def q_dim(self):
        return self.n_heads * self.head_dim

    @property
    def kv_dim(self):
        return self.n_kv * self.head_dim

    @property
    def v_dim(self):
        return self.n_kv * self.value_dim

    @property
    def out_dim(self):
        return self.n_heads * self.value_dim

    def parts(self):
        return [self.position] if self.position is not None else []

    def weight_specs(self):
        specs = [WeightSpec(self.q_name, (self.q_dim, self.hidden)),
                 WeightSpec(self.out_name, (self.hidden, self.out_dim))]
        if self.own_kv:
            specs += [WeightSpec(self.k_name, (self.kv_dim, self.hidden)),
                      WeightSpec(self.v_name, (self.v_dim, self.hidden))]
        whole = self.qk_norm_span == "all"
        if self.q_norm_name is not None:
            specs.append(WeightSpec(self.q_norm_name, (self.q_dim if whole else self.head_dim,), role="vector", init="norm"))
        if self.k_norm_name is not None and self.own_kv:
            specs.append(WeightSpec(self.k_norm_name, (self.kv_dim if whole else self.head_dim,), role="vector", init="norm"))
        if self.distance_bias is not None:
            specs += [WeightSpec(n, (self.n_heads,), role="vector", init="abs_normal") for n in self.distance_bias]
        if self.talk_name is not None:
            specs.append(WeightSpec(self.talk_name, (self.n_heads, self.n_heads), role="vector"))
        if self.sink_name is not None:
            specs.append(WeightSpec(self.sink_name, (self.n_heads,), role="vector"))
        return specs

    def load(self, weights, dtype, device):
        self.run_head_dim, self.run_value_dim = self.head_dim, self.value_dim
        hd, vd = self.head_dim, self.value_dim
        if (self.pad_heads and dtype == torch.bfloat16 and max(hd, vd) <= 128 and not (hd == vd and hd in (64, 128))
                and (self.position is None or hasattr(self.position, "inv_freq_host"))):
            P = 64 if max(hd, vd) <= 64 else 128
            D = self.hidden

            def rows(w, heads, width):                        # [heads * width, D] -> [heads * P, D], zero rows behind
                out = torch.zeros((heads, P, D), dtype=w.dtype, device=w.device)
                out[:, :width] = w.reshape(heads, width, D)
                return out.reshape(heads * P, D)

            w_o = torch.zeros((D, self.n_heads, P), dtype=weights[self.out_name].dtype, device=weights[self.out_name].device)
            w_o[:, :, :vd] = weights[self.out_name].reshape(D, self.n_heads, vd)
            self.w_qkv = torch.cat([rows(weights[self.q_name], self.n_heads, hd), rows(weights[self.k_name], self.n_kv, hd),
                                    rows(weights[self.v_name], self.n_kv, vd)], dim=0).contiguous()
            self.w_out = w_o.reshape(D, self.n_heads * P).contiguous()
            self.run_head_dim = self.run_value_dim = P
        elif self.own_kv:
            self.w_qkv = torch.cat([weights[self.q_name], weights[self.k_name], weights[self.v_name]], dim=0).contiguous()
            self.w_out = weights[self.out_name]
        else:
            self.w_qkv = weights[self.q_name]
            self.w_out = weights[self.out_name]
        self.q_norm = weights[self.q_norm_name] if self.q_norm_name else None
        self.k_norm = weights[self.k_norm_name] if self.k_norm_name and self.own_kv else None
        if self.distance_bias is not None:
            self.bias_r1, self.bias_r2 = (weights[n] for n in self.distance_bias)
        self.talk = weights[self.talk_name] if self.talk_name is not None else None
        self.sink = weights[self.sink_name].contiguous() if self.sink_name is not None else None
        self._sm_count = kernels.sm_count(device) if torch.device(device).type == "cuda" else 0

    def kv_request(self):
        hd, vd = self.run_head_dim, self.run_value_dim        # as load left them: padded in a bfloat16 run with `pad_heads`
        return KVRequest(self.n_kv, hd, self.window, None if vd == hd else vd, keep_first=self.keep_first)

    def check(self, dtype, page_size):
        most = kernels.attn_max_head_dim()
        if not 0 < self.head_dim <= most or not 0 < self.value_dim <= most:
            raise ValueError(f"attention: head_dim {self.head_dim} and value_dim {self.value_dim} must be at most {most}")
        if self.split_keys < 0 or self.split_keys % CHUNK_ALIGN:
            raise ValueError(f"attention: split_keys {self.split_keys} must be a multiple of {CHUNK_ALIGN}")

    def launch_key(self, n_seqs, longest):
        return key_chunks(n_seqs, self.n_kv, longest, self._sm_count, self.split_keys)

    takes_pending_norm = True
    sums_through_linear = True

    def forward(self, ctx, call, xn, out, accumulate):
        kv = call.kv
        hd, vd = self.run_head_dim, self.run_value_dim
        if not self.own_kv and call.writes_kv:
            raise ValueError("attention: a mixer without key and value weights must read another call's cache")
        # a call that reads another call's cache needs its queries only (the stacked rows start with q)
        w_qkv = self.w_qkv[:self.q_dim] if self.span_prepare and self.own_kv and not call.writes_kv else self.w_qkv
        qkv = linear(xn, w_qkv)
        rot = self.position.rotary() if self.position is not None else None
        fused = self.position is None or rot is not None
        common = dict(tok_seq=ctx.tok_seq, tok_pos=ctx.tok_pos, seq_slot=ctx.seq_slot, page_table=kv.page_table,
                      n_heads=self.n_heads, n_kv=self.n_kv, head_dim=hd, eps=self.eps, status=ctx.status)
        if self.span_prepare:
            if self.position is not None and rot is None:
                raise ValueError("attention: norms over the whole projection take a rotation table, no other encoding")
            if rot is not None and rot.interleaved:
                raise ValueError("attention: norms over the whole projection take the half-split pairing only")
            q = kernels.qk_prepare_span(qkv, kv.k, kv.v, self.q_norm, self.k_norm, value_dim=vd,
                                        write_kv=call.writes_kv, inv_freq=rot.inv_freq if rot else None,
                                        n_rot=rot.n_rot if rot else 0, **common)
        elif fused:
            q = kernels.qk_prepare(qkv, kv.k, kv.v, self.q_norm, self.k_norm, rot.inv_freq if rot else None,
                                   n_rot=rot.n_rot if rot else 0, interleaved=rot.interleaved if rot else False,
                                   write_kv=call.writes_kv, value_dim=vd,
                                   unit_norm_after=self.unit_norm_after, query_temperature=self.query_temperature, **common)
        else:
            # A position encoding that is not a rotation table runs between the norm and the
            # cache write: norm in place of a copy of qkv, the encoding's own step, then the write.
            if self.value_dim != self.head_dim or self.query_temperature is not None:
                raise ValueError("attention: a position encoding of its own needs values as wide as the keys and takes "
                                 "no query temperature")
            normed = kernels.qk_normed(qkv, self.q_norm, self.k_norm, self.n_heads, self.n_kv, self.head_dim, self.eps,
                                       ctx.tok_pos, ctx.status)
            self.position.apply(ctx, normed[:, :self.q_dim], normed[:, self.q_dim:self.q_dim + self.kv_dim])
            q = kernels.qk_prepare(normed, kv.k, kv.v, None, None, None, n_rot=0, interleaved=False,
                                   write_kv=call.writes_kv, unit_norm_after=self.unit_norm_after, **common)
        kind, tile_tokens = kernels.attention_plan(q.dtype, self.n_heads, self.n_kv, hd, kv.page_size,
                                                   ctx.is_decode, self.window, vd,
                                                   self.distance_bias is not None, self.talk_name is not None,
                                                   kept_or_sink=self.keep_first > 0 or self.sink is not None,
                                                   capped=self.softcap > 0)
        tile_seq, tile_q0 = ctx.memo(("query tiles", tile_tokens), lambda: self._tiles_on_device(ctx, tile_tokens))
        num_splits, split_keys = (key_chunks(ctx.n_seqs, self.n_kv, ctx.max_kv_len, self._sm_count, self.split_keys)
                                  if ctx.is_decode else (1, 0))
        att = kernels.attention(q, kv.k, kv.v, tile_seq, tile_q0, ctx.cu_q, ctx.seq_start, ctx.seq_slot,
                                kv.page_table, self.n_heads, self.n_kv, hd, self.scale, self.window,
                                num_splits, split_keys, single_token=ctx.is_decode, kind=kind,
                                value_dim=vd,
                                bias=(self.bias_r1, self.bias_r2) if self.distance_bias is not None else None,
                                talk=self.talk, keep_first=self.keep_first, sink=self.sink, softcap=self.softcap)
        linear(att, self.w_out, out=out, accumulate=accumulate)


    @staticmethod
    def _tiles_on_device(ctx, tile_tokens: int):
        dev = torch.from_numpy(query_tiles(ctx.q_lens, tile_tokens)).to(ctx.device, non_blocking=True)
        return dev[0].contiguous(), dev[1].contiguous()


MIXERS.register("gqa_attention", GqaAttention)
