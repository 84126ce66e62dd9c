"""Mixture of small gated feed-forwards picked by a table: token id -> its `top` experts, each with
weight 1/top (no router, nothing learned at run time decides):

    y_t = (1/top) * sum_k  W_down[e_k] (silu(W_gate[e_k] x_t) * (W_up[e_k] x_t)),   e = table[token_t]

plus, optionally, a shared expert of the same form that every token takes, weighed by one number
per token: y_t += sigmoid(g . x_t) * Shared(x_t), the gate in float32 on the float32 rows.

The experts' matrices are stacked at load (gate and up as one [experts, 2F, D] tensor in the layout of
`SwiGLU`, down as [experts, D, F]).  Two ways to run, which agree to rounding:

* few tokens (single-token steps): two weight-streaming kernels find a token's experts through the table
  on the device (`ctx.tokens`), so the step needs nothing from the host and can be recorded;
* many tokens (prompt steps): which expert a token takes is a function of its id alone, and the ids of a
  prompt step are known on the host when the step is packed (`ctx.host_tokens`).  The rows are gathered in
  the order of their experts, every expert's rows padded to whole tiles of 128, and ONE grouped tcgen05
  contraction per matrix runs all experts (each token tile against its expert's matrix; the activation is
  the first one's epilogue); a last kernel sums each token's `top` rows in the order of k.  Where the grouped
  kernel does not take the sizes or the dtype (32-bit), each expert runs as an ordinary `SwiGLU` over its
  contiguous rows instead.  No device-to-host copy is involved either way."""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from .. import kernels
from .base import FEED_FORWARDS, FeedForward, WeightSpec
from .feedforward import SwiGLU
from .linear import FUSION_GROUP, interleave_rows

# From this many tokens on a step whose ids the host knows runs expert by expert.  Below it the streaming
# kernels, which read an expert's weights once per (token, k), are faster than 2 launches per expert.
GROUPED_MIN_TOKENS = 96


def expert_rows(experts: np.ndarray, n_experts: int, top: int, tile: int = 1):
    """For the expert of every (token, k) pair, flat in the order t * top + k: (row_token [rows]: the token of each
    row when the pairs are sorted by expert, keeping their order within an expert, -1 for a padding row; pair_row
    [n * top]: the row each pair went to; bounds [experts + 1]: expert e owns rows bounds[e] .. bounds[e + 1]).
    Every expert's rows are padded to a multiple of `tile`.  An id of `n_experts` or more names an identity expert:
    such a pair gets no row (pair_row -1)."""
    experts = np.asarray(experts)
    if experts.size and experts.max() >= n_experts:
        real = np.flatnonzero(experts < n_experts)
        row_token, rows_of_real, bounds = _expert_rows(experts[real], real // top, n_experts, tile)
        pair_row = np.full(experts.size, -1, dtype=np.int32)
        pair_row[real] = rows_of_real
        return row_token, pair_row, bounds
    return _expert_rows(experts, np.arange(experts.size) // top, n_experts, tile)


def _expert_rows(experts: np.ndarray, tokens: np.ndarray, n_experts: int, tile: int):
    """`expert_rows` for pairs that all name real experts; tokens[i] is the token of pair i."""
    order = np.argsort(experts, kind="stable")
    counts = np.bincount(experts, minlength=n_experts)
    padded = -(-counts // tile) * tile
    bounds = np.zeros(n_experts + 1, dtype=np.int64)
    np.cumsum(padded, out=bounds[1:])
    starts = np.zeros(n_experts, dtype=np.int64)
    np.cumsum(counts[:-1], out=starts[1:])
    rows = np.arange(order.size) + np.repeat(bounds[:-1] - starts, counts)     # row of each pair, in sorted order
    row_token = np.full(int(bounds[-1]), -1, dtype=np.int32)
    row_token[rows] = tokens[order]
    pair_row = np.empty(order.size, dtype=np.int32)
    pair_row[order] = rows
    return row_token, pair_row, bounds


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
        self.table = self.table_host = self.w_gate_up = self.w_down = self.shared_gate = None
        self.interleave = FUSION_GROUP if ffn_dim % FUSION_GROUP == 0 else 0
        self.experts: list[SwiGLU] = []         # views of the stacked tensors, one ordinary feed-forward per expert
        # pinned host buffer through which a prompt step's row tables reach the device, and the event of the
        # copy that last read it: allocating pinned memory every step cost more than the step's kernels
        self._staging: Optional[torch.Tensor] = None
        self._staged: Optional[torch.cuda.Event] = None

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
        self.table_host = self.table.cpu().numpy()
        self._set_sort_keys()
        stack = (lambda g, u: interleave_rows([g, u])) if self.interleave else (lambda g, u: torch.cat([g, u], dim=0))
        self.w_gate_up = torch.stack([stack(weights[g], weights[u]) for g, u, _ in self.names]).contiguous()
        self.w_down = torch.stack([weights[d] for _, _, d in self.names]).contiguous()
        self.experts = []
        for e in range(self.n_experts):
            ff = SwiGLU(self.hidden, self.ffn_dim, "", "", "")
            ff.w_gate_up, ff.w_down = self.w_gate_up[e], self.w_down[e]
            self.experts.append(ff)
        if self.shared_gate_name is not None:
            self.shared_gate = weights[self.shared_gate_name].reshape(self.hidden).contiguous()

    def forward(self, ctx, xn, out, accumulate):
        rows = xn if xn.dtype == ctx.dtype else kernels.cast_rows(xn, ctx.dtype)
        host_tokens = getattr(ctx, "host_tokens", None)
        if host_tokens is not None and rows.shape[0] >= GROUPED_MIN_TOKENS:
            self._expert_by_expert(ctx, rows, host_tokens, out, accumulate)
        else:
            kernels.moe_table(rows, ctx.tokens, self.table, self.w_gate_up, self.interleave, self.w_down, ctx.status,
                              out=out, accumulate=accumulate)
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

    def _set_sort_keys(self):
        small = np.uint8 if self.n_experts <= 256 else (np.uint16 if self.n_experts <= 65536 else np.int64)
        self.table_sort_keys = np.clip(self.table_host, 0, self.n_experts - 1).astype(small)

    def routing(self, host_tokens: np.ndarray, tile: int = 1):
        """For token ids known on the host: (row_token [rows]: the token of each row when the (token, k)
        pairs are sorted by expert, keeping their order within an expert, -1 for a padding row; pair_row
        [n * top]: the row pair t * top + k went to; bounds [experts + 1]: expert e owns rows bounds[e] ..
        bounds[e + 1]).  Every expert's rows are padded to a multiple of `tile`."""
        ids = np.asarray(host_tokens)
        if ids.size and (ids.min() < 0 or ids.max() >= self.vocab):
            ids = np.clip(ids, 0, self.vocab - 1)            # a bad id is flagged by the embedding kernel
        experts = self.table_sort_keys[ids].reshape(-1)      # 8- or 16-bit keys: NumPy sorts those by radix, ten times faster
        return expert_rows(experts, self.n_experts, self.top, tile)

    def _upload(self, words: np.ndarray, device) -> torch.Tensor:
        """int32 words on the device, copied through the part's own pinned buffer (rewritten only after the
        copy that last read it has run)."""
        n = int(words.size)
        if self._staging is None or self._staging.numel() < n:
            self._staging = torch.empty(max(n, 1024) * 2, dtype=torch.int32).pin_memory()
            self._staged = None
        if self._staged is not None:
            self._staged.synchronize()
        self._staging[:n].numpy()[:] = words
        dev = torch.empty(n, dtype=torch.int32, device=device)
        dev.copy_(self._staging[:n], non_blocking=True)
        if self._staged is None:
            self._staged = torch.cuda.Event()
        self._staged.record()
        return dev

    def _expert_by_expert(self, ctx, rows, host_tokens, out, accumulate, chosen=None, weights=None):
        """`chosen` (host, flat [n * top]) names the experts when a router picked them, `weights` (device, float32
        [n, top]) their weights; without them the table decides and every expert weighs 1/top."""
        tile = kernels.GEMM_TC_GROUP_ROWS
        grouped = (self.interleave and rows.dtype == torch.bfloat16 and self.hidden % 8 == 0 and self.ffn_dim % 8 == 0
                   and rows.is_contiguous())

        def make():
            if chosen is None:
                row_token, pair_row, bounds = self.routing(host_tokens, tile if grouped else 1)
            else:
                row_token, pair_row, bounds = expert_rows(chosen, self.n_experts, self.top, tile if grouped else 1)
            tile_group = np.repeat(np.arange(self.n_experts), np.diff(bounds) // tile).astype(np.int32) if grouped \
                else np.zeros(0, dtype=np.int32)
            sizes = np.cumsum([row_token.size, pair_row.size, tile_group.size])
            dev = self._upload(np.concatenate([row_token, pair_row, tile_group]), ctx.device)
            return dev[:sizes[0]], dev[sizes[0]:sizes[1]], dev[sizes[1]:sizes[2]], bounds

        # a table's rows depend on the step's ids alone; a router's on what this very call read
        row_token, pair_row, tile_group, bounds = ctx.memo(("expert rows", id(self)), make) if chosen is None else make()
        xg = kernels.moe_gather(rows, row_token)
        if grouped:
            h = kernels.gemm_tc_grouped(xg, self.w_gate_up, tile_group, swiglu=True)
            y = kernels.gemm_tc_grouped(h, self.w_down, tile_group, out_dtype=torch.float32)
        else:
            y = torch.empty((xg.shape[0], self.hidden), dtype=torch.float32, device=xg.device)
            for e, ff in enumerate(self.experts):
                r0, r1 = int(bounds[e]), int(bounds[e + 1])
                if r1 > r0:
                    ff.forward(ctx, xg[r0:r1], y[r0:r1], False)
        kernels.moe_combine(y, pair_row, self.top, out, accumulate, weights,
                            identity_rows=rows if getattr(self, "n_identity", 0) else None)


class RoutedMoE(TableMoE):
    """Mixture of small gated feed-forwards picked by a learned router:

        z = W_router x_t (float32),  s = softmax(z) over all experts,  the `top` largest s are chosen,
        y_t = sum_k (s_k / (sum of the chosen s + 1e-20)) * W_down[e_k] (silu(W_gate[e_k] x_t) * (W_up[e_k] x_t))

    The router runs on the device (`kernels.moe_router`: ids and weights per token).  Few tokens: the two
    weight-streaming kernels read them there, so a single-token step needs nothing from the host and can be
    recorded.  Many tokens (prompt steps): a kernel sorts the rows by expert, every expert's rows padded to whole
    tiles, and the grouped tensor-core contractions of `TableMoE` run them; where those do not take the sizes, the
    chosen ids come to the host once per call and the experts run one after the other.

    Options other designs use.  `correction_name`: a vector [router outputs] that is added to the scores for the CHOICE
    only; the weights are made of the scores alone.  `n_identity`: the router has that many outputs more than there are
    experts with weights, and its last `n_identity` outputs stand for identity experts, whose result is the row they
    read (times the weight); `top` may then exceed nothing but the router's outputs.  `shared`: a feed-forward every
    token takes, added with weight 1."""

    takes_residual_rows = False
    takes_pending_norm = True

    def __init__(self, hidden: int, ffn_dim: int, n_experts: int, top: int, router_name: str, expert_names,
                 correction_name: Optional[str] = None, n_identity: int = 0, shared: Optional[FeedForward] = None):
        if n_identity < 0 or not 0 < top <= n_experts + n_identity:
            raise ValueError(f"{top} experts per token out of {n_experts} and {n_identity} identity experts")
        super().__init__(hidden, ffn_dim, n_experts, min(top, n_experts), 1, "", expert_names, shared=shared)
        self.top = top
        self.router_name, self.w_router = router_name, None
        self.correction_name, self.correction, self.n_identity = correction_name, None, int(n_identity)

    @property
    def n_router(self) -> int:
        return self.n_experts + self.n_identity

    def weight_specs(self):
        F, D = self.ffn_dim, self.hidden
        specs = [WeightSpec(self.router_name, (self.n_router, D), role="vector")]      # kept in float32
        if self.correction_name is not None:
            specs.append(WeightSpec(self.correction_name, (self.n_router,), role="vector"))
        for g, u, d in self.names:
            specs += [WeightSpec(g, (F, D)), WeightSpec(u, (F, D)), WeightSpec(d, (D, F))]
        return specs

    def load(self, weights, dtype, device):
        self.w_router = weights[self.router_name].contiguous()
        self.correction = weights[self.correction_name].contiguous() if self.correction_name is not None else None
        stack = (lambda g, u: interleave_rows([g, u])) if self.interleave else (lambda g, u: torch.cat([g, u], dim=0))
        self.w_gate_up = torch.stack([stack(weights[g], weights[u]) for g, u, _ in self.names]).contiguous()
        self.w_down = torch.stack([weights[d] for _, _, d in self.names]).contiguous()
        self.experts = []
        for e in range(self.n_experts):
            ff = SwiGLU(self.hidden, self.ffn_dim, "", "", "")
            ff.w_gate_up, ff.w_down = self.w_gate_up[e], self.w_down[e]
            self.experts.append(ff)

    def forward(self, ctx, xn, out, accumulate):
        from .linear import as_tensor
        rows = as_tensor(xn)
        if rows.dtype != ctx.dtype:
            rows = kernels.cast_rows(rows, ctx.dtype)
        self._experts(ctx, rows, out, accumulate)
        if self.shared is not None:
            self.shared.forward(ctx, rows, out, True)

    def _experts(self, ctx, rows, out, accumulate):
        ids, wts = kernels.moe_router(rows, self.w_router, self.top, self.correction)
        if ctx.is_decode or rows.shape[0] < GROUPED_MIN_TOKENS:
            kernels.moe_routed(rows, ids, wts, self.w_gate_up, self.interleave, self.w_down, ctx.status, out=out,
                               accumulate=accumulate, n_identity=self.n_identity)
            return
        tile = kernels.GEMM_TC_GROUP_ROWS
        if (self.interleave and rows.dtype == torch.bfloat16 and self.hidden % 8 == 0 and self.ffn_dim % 8 == 0
                and rows.is_contiguous() and self.n_experts <= 4096):
            # the rows are sorted by expert where the router left its choice: the step never waits for the host
            row_token, pair_row, tile_group = kernels.moe_expert_rows(ids, self.n_experts, tile, self.n_identity)
            xg = kernels.moe_gather(rows, row_token)
            h = kernels.gemm_tc_grouped(xg, self.w_gate_up, tile_group, swiglu=True)
            y = kernels.gemm_tc_grouped(h, self.w_down, tile_group, out_dtype=torch.float32)
            kernels.moe_combine(y, pair_row, self.top, out, accumulate, wts, identity_rows=rows if self.n_identity else None)
            return
        chosen = ids.cpu().numpy().reshape(-1).astype(np.int64)
        self._expert_by_expert(ctx, rows, None, out, accumulate, chosen=np.clip(chosen, 0, self.n_router - 1), weights=wts)


FEED_FORWARDS.register("table_moe", TableMoE)
FEED_FORWARDS.register("routed_moe", RoutedMoE)
