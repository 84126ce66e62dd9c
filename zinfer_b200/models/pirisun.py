"""Pirisun: a decoder of parallel layers (one layer norm with weight and bias; the mixer and the feed-forward both read
it and both results are summed into the rows).  A layer's mixer is either causal attention through a latent vector per
token (interleaved rotation of a key part shared by all heads, a learned sink per head in the softmax, a sigmoid gate on
every output value) or a pair of mixers side by side whose RMS-normalised results are averaged: grouped-query softmax
attention without a rotation (a query temperature that grows with the position, scores through a tanh cap) and
retention (a linear recurrence with a fixed decay per head, rotated queries and keys, unit norm per head, silu gate).
A layer's feed-forward is none or routed experts (a correction vector for the choice, identity experts, a shared
expert).  A stretch of layers may run several times in a row, each pass with a cache and state of its own and nothing
else between the passes; the final norm is a layer norm, the head has its own matrix and the logits are multiplied by a
constant.

Per layer i the tensors are `l<i>.*`.  Every part is a general part of `parts/`; this file only names tensors and
passes the configuration's numbers on."""
from __future__ import annotations

from ..config.pirisun import PirisunConfig
from ..config.registry import register_architecture
from ..parts import (GqaAttention, LatentAttention, LayerNorm, LMHead, MixerPair, ParallelBlock, Retention, RotaryEncoding,
                     RoutedMoE, SwiGLU, TokenEmbedding)
from .model import LayerCall, Model


def build_pirisun(cfg: PirisunConfig) -> Model:
    D, eps = cfg.hidden_size, cfg.norm_eps
    embedding = TokenEmbedding(cfg.vocab_size, D, "embed")
    layers = []
    for i, L in enumerate(cfg.layers):
        p = f"l{i}."
        a = p + "mix."
        if L.type == "latent_attention":
            m = L.latent
            mixer = LatentAttention(D, m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank, None, m.scale, m.rot_base,
                                    None, None, a + "q", a + "dkv", a + "dkv.norm", a + "uk", a + "uv", a + "o",
                                    gate_name=a + "g", norm_eps=eps, gate_per_value=True, sink_name=a + "sink", interleaved=True)
        else:
            l, r = L.left, L.right
            left = GqaAttention(D, l.heads, l.kv_heads, l.dim, a + "left.q", a + "left.k", a + "left.v", a + "left.o",
                                norm_eps=eps, scale=l.scale, value_dim=l.vdim, softcap=l.softcap or None, pad_heads=True,
                                query_temperature=(l.q_temp_coef, l.q_temp_every) if l.q_temp_every else None)
            position = RotaryEncoding(r.dim, r.rot_base, n_rot=r.rot_dims) if r.rot_dims else None
            right = Retention(D, r.heads, r.dim, r.vdim, r.decay, a + "right.q", a + "right.k", a + "right.v", a + "right.g",
                              a + "right.o", position=position, norm_eps=eps)
            mixer = MixerPair(D, left, right, a + "left.out", a + "right.out", norm_eps=eps, share=0.5)
        ffn = None
        if L.mlp is not None:
            f = p + "mlp."
            shared = SwiGLU(D, L.mlp.shared_ff, f + "shared.gate", f + "shared.up", f + "shared.down") if L.mlp.shared_ff else None
            ffn = RoutedMoE(D, L.mlp.ff, L.mlp.experts, L.mlp.top, f + "router",
                            lambda e, f=f: (f"{f}e{e}.gate", f"{f}e{e}.up", f"{f}e{e}.down"),
                            correction_name=f + "correction", n_identity=L.mlp.identity, shared=shared)
        layers.append(ParallelBlock(LayerNorm(D, eps, p + "norm1", p + "norm1.b"), mixer, ffn))
    return Model(cfg, embedding, layers, LayerNorm(D, eps, "final.norm", "final.norm.b"),
                 LMHead(cfg.vocab_size, D, "head", scale=cfg.logit_scale),
                 schedule=[LayerCall(layer) for layer in cfg.layer_runs()])


register_architecture("Pirisun", PirisunConfig, build_pirisun)
