"""Kerotar: a decoder of parallel layers (one norm; the mixer and the feed-forward both read it and both results are
summed into the rows) that mixes two kinds of attention in any order -- windowed grouped-query attention that also
keeps a sequence's first tokens and has a learned sink per head in its softmax, and causal attention through a latent
vector per token with a gate per head -- each with no feed-forward, a dense gated one with clamps, or routed experts.
The token rows are scaled; a stretch of layers may run several times in a row (each pass with a cache of its own) and
is then given, at the start of every pass, a learned map of its rows together with the embedding's rows, and a learned
vector per pass; the head has its own matrix.

Per layer i the tensors are `l<i>.*`.  Every part is a general part of `parts/`; this file only names tensors and
passes the configuration's numbers on."""
from __future__ import annotations

from ..config.kerotar import KerotarConfig
from ..config.registry import register_architecture
from ..parts import (ClampedGLU, GqaAttention, LatentAttention, LMHead, ParallelBlock, PassInput, RMSNorm, RotaryEncoding,
                     RoutedMoE, TokenEmbedding)
from .model import LayerCall, Model


def build_kerotar(cfg: KerotarConfig) -> Model:
    D, eps = cfg.hidden_size, cfg.norm_eps
    embedding = TokenEmbedding(cfg.vocab_size, D, "embed", scale=cfg.embedding_scale)
    layers = []
    for i, L in enumerate(cfg.layers):
        p, m = f"l{i}.", L.mixer
        a = p + "mix."
        if L.type == "attention":
            position = RotaryEncoding(m.dim, m.rot_base, n_rot=m.rot_dims) if m.rot_dims else None
            mixer = GqaAttention(D, m.heads, m.kv_heads, m.dim, a + "q", a + "k", a + "v", a + "o",
                                 q_norm_name=a + "q.norm", k_norm_name=a + "k.norm", norm_eps=eps, position=position,
                                 window=m.window, scale=m.scale, value_dim=m.vdim, qk_norm_span="all",
                                 keep_first=m.keep_first, sink_name=a + "sink")
        else:
            mixer = LatentAttention(D, m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank, m.q_rank, m.scale, m.rot_base,
                                    a + "dq", a + "dq.norm", a + "uq", a + "dkv", a + "dkv.norm", a + "uk", a + "uv",
                                    a + "o", gate_name=a + "g", norm_eps=eps)
        ffn = None
        if L.mlp is not None and L.mlp.kind == "dense":
            ffn = ClampedGLU(D, L.mlp.ff, p + "mlp.gate", p + "mlp.up", p + "mlp.down", limit=L.mlp.limit)
        elif L.mlp is not None:
            ffn = RoutedMoE(D, L.mlp.ff, L.mlp.experts, L.mlp.top, p + "mlp.router",
                            lambda e, p=p: (f"{p}mlp.e{e}.gate", f"{p}mlp.e{e}.up", f"{p}mlp.e{e}.down"))
        layers.append(ParallelBlock(RMSNorm(D, eps, p + "norm1"), mixer, ffn))
    runs = cfg.layer_runs()
    passes = None
    if cfg.loop is not None:
        passes = PassInput("loop.step", cfg.loop.times, D, {c: t for c, (_, t) in enumerate(runs) if t is not None},
                           in_name="loop.in")
    return Model(cfg, embedding, layers, RMSNorm(D, eps, "final.norm"), LMHead(cfg.vocab_size, D, "head"),
                 schedule=[LayerCall(layer) for layer, _ in runs], pass_input=passes)


register_architecture("Kerotar", KerotarConfig, build_kerotar)
