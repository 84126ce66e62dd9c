"""Pre-norm decoder block with two residual sums: x += Mixer(norm(x)); x += FFN(norm(x))
(src/model.zig:2395-2422).  The residual stream x is float32; each sum is the `accumulate`
store of the part's last contraction (src/model.zig:918-920).

A part that sets `takes_pending_norm = True` receives its input as the norm's `pending` form (a
`NormedRows`: the norm not yet applied) when the norm has one, and passes it to `linear` or a
fused kernel; any other part, and any part behind a norm without that form, receives a tensor.

A part that sets `sums_through_linear = True` uses `out` only as the `out=` of its last `linear`
call.  It may then be handed, in place of the residual rows, what the NEXT norm's `ahead`
returned (a `ResidualSink`), so that the kernel of that contraction writes the next norm's inputs
beside the sum.  The next norm is the block's own second norm for the mixer, and for the
feed-forward whatever the model says runs next (`forward_chained`).

Two options other designs use: no feed-forward at all (`ffn` and `ffn_norm` None: the block is its first
sum alone), and layer scale: a sublayer's result is multiplied by a learned vector (`mixer_scale_name`,
`ffn_scale_name`, one number per channel) before it is summed, x += s * Mixer(norm(x)).  A scaled sublayer
that sums through `linear` is handed a `ScaledSink` (rows and scale: the contraction applies the scale in its
epilogue where it can); any other writes into a float32 buffer and `kernels.scale_add` sums it in.  Nothing is
prepared for the next norm behind a scale."""
from __future__ import annotations

from .base import BLOCKS, Block, FeedForward, Mixer, Norm, WeightSpec
from .linear import ScaledSink


class PreNormBlock(Block):
    def __init__(self, mixer_norm: Norm, mixer: Mixer, ffn_norm: Norm | None = None, ffn: FeedForward | None = None,
                 mixer_scale_name: str | None = None, ffn_scale_name: str | None = None):
        if (ffn is None) != (ffn_norm is None):
            raise ValueError("a feed-forward and its norm come together")
        if ffn is None and ffn_scale_name is not None:
            raise ValueError("a scale for a feed-forward that is not there")
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn = mixer_norm, mixer, ffn_norm, ffn
        self.mixer_scale_name, self.ffn_scale_name = mixer_scale_name, ffn_scale_name
        self.mixer_scale = self.ffn_scale = None

    def parts(self):
        return [p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn) if p is not None]

    def weight_specs(self):
        names = [n for n in (self.mixer_scale_name, self.ffn_scale_name) if n is not None]
        if names and not hasattr(self.mixer_norm, "dim"):
            raise ValueError(f"layer scale: {type(self.mixer_norm).__name__} does not tell the width of the rows (`dim`)")
        return [WeightSpec(n, (self.mixer_norm.dim,), role="vector", init="norm") for n in names]

    def load(self, weights, dtype, device):
        self.mixer_scale = weights[self.mixer_scale_name] if self.mixer_scale_name is not None else None
        self.ffn_scale = weights[self.ffn_scale_name] if self.ffn_scale_name is not None else None

    def entry_norm(self):
        return self.mixer_norm

    def forward(self, ctx, call, x):
        self.forward_chained(ctx, call, x)

    def forward_chained(self, ctx, call, x, entry=None, next_norm=None):
        from .. import kernels
        import torch
        mid = None
        if self.mixer_scale is not None and getattr(self.mixer, "sums_through_linear", False):
            self.mixer.forward(ctx, call, normed_for(self.mixer, self.mixer_norm, ctx, x, entry),
                               ScaledSink(x, self.mixer_scale), True)
        elif self.mixer_scale is not None:
            m = torch.empty_like(x)
            self.mixer.forward(ctx, call, normed_for(self.mixer, self.mixer_norm, ctx, x, entry), m, False)
            kernels.scale_add(m, self.mixer_scale, x)
        else:
            mid = ahead_for(self.mixer, self.ffn_norm if self.ffn_scale is None else None, ctx, x)
            self.mixer.forward(ctx, call, normed_for(self.mixer, self.mixer_norm, ctx, x, entry),
                               x if mid is None else mid, True)
        if self.ffn is None:
            return None
        if self.ffn_scale is not None and getattr(self.ffn, "sums_through_linear", False):
            self.ffn.forward(ctx, normed_for(self.ffn, self.ffn_norm, ctx, x, mid), ScaledSink(x, self.ffn_scale), True)
            return None
        if self.ffn_scale is not None:
            m = torch.empty_like(x)
            self.ffn.forward(ctx, normed_for(self.ffn, self.ffn_norm, ctx, x, mid), m, False)
            kernels.scale_add(m, self.ffn_scale, x)
            return None
        last = ahead_for(self.ffn, next_norm, ctx, x)
        self.ffn.forward(ctx, normed_for(self.ffn, self.ffn_norm, ctx, x, mid), x if last is None else last, True)
        return last


def normed_for(consumer, norm: Norm, ctx, x, prepared=None):
    """norm(x) for `consumer`: still pending if the consumer takes that and the norm offers it.
    `prepared`: what `ahead_for` returned for this norm before the rows were last summed into."""
    if getattr(consumer, "takes_pending_norm", False):
        p = norm.pending(ctx, x) if prepared is None else norm.pending(ctx, x, prepared)
        if p is not None:
            return p
    return norm.forward(ctx, x)


def ahead_for(producer, norm, ctx, x):
    """What `producer` gets as `out` in place of `x` so that its last contraction prepares `norm`,
    or None: the producer must sum through `linear`, and the norm must offer `ahead`."""
    if norm is None or not getattr(producer, "sums_through_linear", False):
        return None
    ahead = getattr(norm, "ahead", None)
    return ahead(ctx, x) if ahead is not None else None


class SublayerNormBlock(Block):
    """x += norm1(Mixer(x)); x += norm2(FFN(x)): the norms sit on the sublayers' OUTPUTS and the
    sublayers read the residual rows as they are.  Either sublayer may be absent (`ffn` None).

    A part that sets `takes_residual_rows = True` is handed the float32 rows themselves (it may
    want them in 32-bit: a convolution with state, a gate); any other part gets them in the run
    dtype.  The part writes its result into a float32 buffer of the rows' shape (`accumulate`
    False); `Norm.add_normed` then sums its norm into the rows."""

    def __init__(self, mixer: Mixer, mixer_norm: Norm, ffn: FeedForward | None = None, ffn_norm: Norm | None = None):
        if (ffn is None) != (ffn_norm is None):
            raise ValueError("a feed-forward and its norm come together")
        for n in (mixer_norm, ffn_norm):
            if n is not None and not hasattr(n, "add_normed"):
                raise ValueError(f"{type(n).__name__} cannot sum a normalised sublayer output into the rows")
        self.mixer, self.mixer_norm, self.ffn, self.ffn_norm = mixer, mixer_norm, ffn, ffn_norm

    def parts(self):
        return [p for p in (self.mixer, self.mixer_norm, self.ffn, self.ffn_norm) if p is not None]

    @staticmethod
    def _input(part, ctx, x):
        from .. import kernels
        return x if getattr(part, "takes_residual_rows", False) else kernels.cast_rows(x, ctx.dtype)

    def forward(self, ctx, call, x):
        import torch
        m = torch.empty_like(x)
        self.mixer.forward(ctx, call, self._input(self.mixer, ctx, x), m, False)
        self.mixer_norm.add_normed(ctx, m, x)
        if self.ffn is not None:
            self.ffn.forward(ctx, self._input(self.ffn, ctx, x), m, False)
            self.ffn_norm.add_normed(ctx, m, x)


class ParallelBlock(Block):
    """x += Mixer(norm(x)) + FFN(norm(x)): ONE norm, both sublayers read its output, both results are summed into
    the float32 rows (the mixer's first, then the feed-forward's).  `ffn` None: the mixer alone.  The normalised rows
    are made once, before the mixer changes the rows they are made from, and both sublayers read that tensor."""

    def __init__(self, norm: Norm, mixer: Mixer, ffn: FeedForward | None = None):
        self.norm, self.mixer, self.ffn = norm, mixer, ffn

    def parts(self):
        return [p for p in (self.norm, self.mixer, self.ffn) if p is not None]

    def entry_norm(self):
        return self.norm

    def forward(self, ctx, call, x):
        self.forward_chained(ctx, call, x)

    def forward_chained(self, ctx, call, x, entry=None, next_norm=None):
        consumers = [p for p in (self.mixer, self.ffn) if p is not None]
        h = None
        if all(getattr(p, "takes_pending_norm", False) for p in consumers):
            h = self.norm.pending(ctx, x) if entry is None else self.norm.pending(ctx, x, entry)
        if h is None:
            h = self.norm.forward(ctx, x)
        if self.ffn is None:
            last = ahead_for(self.mixer, next_norm, ctx, x)
            self.mixer.forward(ctx, call, h, x if last is None else last, True)
            return last
        # The mixer sums into the rows that the norm reads: what the feed-forward reads must exist before it does.
        # (A pending norm is evaluated when its first consumer wants it, which may be never for a fused kernel.)
        if hasattr(h, "tensor"):
            h.tensor()
        self.mixer.forward(ctx, call, h, x, True)
        last = ahead_for(self.ffn, next_norm, ctx, x)
        self.ffn.forward(ctx, h, x if last is None else last, True)
        return last


BLOCKS.register("parallel", ParallelBlock)
BLOCKS.register("prenorm", PreNormBlock)
BLOCKS.register("sublayer_norm", SublayerNormBlock)
