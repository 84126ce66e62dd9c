"""Typed configuration of the Kerotar architecture, read from its own config.json keys.

The file is nested: `vocab`, `width`, `norm.eps`, `embedding.scale` (the token rows are multiplied by it; 1 if
absent), optionally `loop` {start, stop, times} (layers start .. stop-1 run `times` times in a row with the same
weights) and `layers`, a list with one entry per layer:

* `type` "attention": `mixer` {heads, kv_heads, dim, vdim, scale, rot {base, dims}, mask {size, keep_first}}:
  grouped-query softmax attention with q/k norms over the whole projection, a half-split rotation of the first
  `rot.dims` entries of every head, a window of `mask.size` tokens that also keeps the first `mask.keep_first`
  tokens of the sequence, and a learned sink per head in the softmax denominator;
* `type` "latent_attention": `mixer` {heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, rot {base, dims}}: causal
  attention whose keys and values are expanded from a latent of `kv_rank` entries per token, with `rot_dim` rotated
  entries shared by all heads, queries through a latent of `q_rank` entries and a sigmoid gate per head;
* `mlp`: null, {kind "dense", ff, limit} (a gated unit with capped gate and clamped linear branch) or {kind "moe",
  expert {ff}, router {experts, top}} (softmax router, the `top` best experts, weights renormalised).

Every size and constant comes from here; what the file does not mention (no `loop`, no `rot`, no `mask`) the model
does not have.  The design sets no longest sequence; `max_positions`, if a file has it, is only the default context
of an engine (else DEFAULT_CONTEXT)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional

from .base import ConfigError, ModelConfig, as_float, as_int, need

MIXER_TYPES = ("attention", "latent_attention")
MLP_KINDS = ("dense", "moe")
DEFAULT_CONTEXT = 8192


@dataclass(frozen=True)
class KerotarMixer:
    heads: int
    dim: int
    vdim: int
    scale: float
    rot_base: float = 0.0               # 0 with rot_dims 0 = no rotation (attention only)
    rot_dims: int = 0
    kv_heads: int = 0                   # attention
    window: int = 0                     # attention: 0 = every earlier token
    keep_first: int = 0
    rot_dim: int = 0                    # latent attention
    kv_rank: int = 0
    q_rank: int = 0


@dataclass(frozen=True)
class KerotarMlp:
    kind: str
    ff: int
    limit: float = 0.0                  # dense
    experts: int = 0                    # moe
    top: int = 0


@dataclass(frozen=True)
class KerotarLayer:
    type: str
    mixer: KerotarMixer
    mlp: Optional[KerotarMlp]


@dataclass(frozen=True)
class KerotarLoop:
    start: int
    stop: int
    times: int


def _obj(d: dict, key: str, where: str) -> dict:
    v = d.get(key)
    if v is None:
        return {}
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: '{where}{key}' must be an object")
    return v


def _mixer(kind: str, m: dict, w: str) -> KerotarMixer:
    heads = as_int(m, w + "heads", need(m, "heads"), 1)
    dim = as_int(m, w + "dim", need(m, "dim"), 1)
    vdim = as_int(m, w + "vdim", m.get("vdim", dim), 1)
    scale = as_float(w + "scale", need(m, "scale"))
    rot = _obj(m, "rot", w)
    base = as_float(w + "rot.base", need(rot, "base")) if rot else 0.0
    dims = as_int(rot, w + "rot.dims", need(rot, "dims"), 0) if rot else 0
    if kind == "attention":
        mask = _obj(m, "mask", w)
        return KerotarMixer(heads, dim, vdim, scale, base, dims,
                            kv_heads=as_int(m, w + "kv_heads", m.get("kv_heads", heads), 1),
                            window=as_int(mask, w + "mask.size", need(mask, "size"), 1) if mask else 0,
                            keep_first=as_int(mask, w + "mask.keep_first", mask.get("keep_first", 0), 0) if mask else 0)
    rot_dim = as_int(m, w + "rot_dim", need(m, "rot_dim"), 2)
    return KerotarMixer(heads, dim, vdim, scale, base, dims if rot else rot_dim, rot_dim=rot_dim,
                        kv_rank=as_int(m, w + "kv_rank", need(m, "kv_rank"), 1),
                        q_rank=as_int(m, w + "q_rank", need(m, "q_rank"), 1))


def _mlp(ml, w: str) -> Optional[KerotarMlp]:
    if ml is None:
        return None
    if not isinstance(ml, dict):
        raise ConfigError(f"config.json: '{w}' must be an object or null")
    kind = str(ml.get("kind", "dense"))
    if kind == "dense":
        return KerotarMlp("dense", as_int(ml, w + ".ff", need(ml, "ff"), 1), limit=as_float(w + ".limit", need(ml, "limit")))
    if kind == "moe":
        ex, ro = _obj(ml, "expert", w + "."), _obj(ml, "router", w + ".")
        return KerotarMlp("moe", as_int(ex, w + ".expert.ff", need(ex, "ff"), 1),
                          experts=as_int(ro, w + ".router.experts", need(ro, "experts"), 1),
                          top=as_int(ro, w + ".router.top", need(ro, "top"), 1))
    raise ConfigError(f"config.json: '{w}.kind' = {kind!r}; known kinds are {list(MLP_KINDS)}")


@dataclass
class KerotarConfig(ModelConfig):
    layers: tuple[KerotarLayer, ...] = ()
    loop: Optional[KerotarLoop] = None
    norm_eps: float = 1e-5
    embedding_scale: float = 1.0

    @classmethod
    def from_json_dict(cls, d: dict[str, Any]) -> "KerotarConfig":
        vocab = as_int(d, "vocab", need(d, "vocab"), 1)
        width = as_int(d, "width", need(d, "width"), 1)
        norm, emb = _obj(d, "norm", ""), _obj(d, "embedding", "")
        raw_layers = need(d, "layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, L in enumerate(raw_layers):
            if not isinstance(L, dict):
                raise ConfigError(f"config.json: 'layers[{i}]' must be an object")
            kind = str(need(L, "type"))
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: 'layers[{i}].type' = {kind!r}; known types are {list(MIXER_TYPES)}")
            layers.append(KerotarLayer(kind, _mixer(kind, _obj(L, "mixer", f"layers[{i}]."), f"layers[{i}].mixer."),
                                       _mlp(L.get("mlp"), f"layers[{i}].mlp")))
        loop = None
        lp = _obj(d, "loop", "")
        if lp:
            loop = KerotarLoop(as_int(lp, "loop.start", need(lp, "start"), 0), as_int(lp, "loop.stop", need(lp, "stop"), 0),
                               as_int(lp, "loop.times", need(lp, "times"), 1))
        eos = d.get("eos_token_id")
        max_pos = d.get("max_positions")
        cfg = cls(architecture=str(d.get("architecture") or (d.get("architectures") or ["Kerotar"])[0]),
                  vocab_size=vocab, hidden_size=width,
                  max_position_embeddings=DEFAULT_CONTEXT if max_pos is None else as_int(d, "max_positions", max_pos, 1),
                  eos_token_ids=() if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos])),
                  raw=dict(d), layers=tuple(layers), loop=loop, norm_eps=as_float("norm.eps", norm.get("eps", 1e-5)),
                  embedding_scale=as_float("embedding.scale", emb.get("scale", 1.0)))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.norm_eps <= 0:
            raise ConfigError(f"config.json: norm.eps must be positive, found {self.norm_eps}")
        for i, L in enumerate(self.layers):
            m, w = L.mixer, f"config.json: layers[{i}]"
            if L.type not in MIXER_TYPES:
                raise ConfigError(f"{w}.type = {L.type!r}; known types are {list(MIXER_TYPES)}")
            if L.type == "attention":
                if m.heads % m.kv_heads:
                    raise ConfigError(f"{w}: {m.heads} heads are not a multiple of {m.kv_heads} kv_heads")
                if m.rot_dims % 2 or m.rot_dims > m.dim:
                    raise ConfigError(f"{w}.mixer.rot.dims = {m.rot_dims} must be even and at most dim {m.dim}")
                if m.keep_first and not m.window:
                    raise ConfigError(f"{w}.mixer.mask: kept first tokens need a window size")
            else:
                if m.rot_dim % 2:
                    raise ConfigError(f"{w}.mixer.rot_dim = {m.rot_dim} must be even")
                if m.rot_dims != m.rot_dim:
                    raise ConfigError(f"{w}.mixer.rot.dims = {m.rot_dims} must equal rot_dim {m.rot_dim}")
            if m.rot_dims and m.rot_base <= 0:
                raise ConfigError(f"{w}.mixer.rot.base must be positive, found {m.rot_base}")
            if L.mlp is not None:
                if L.mlp.kind not in MLP_KINDS:
                    raise ConfigError(f"{w}.mlp.kind = {L.mlp.kind!r}; known kinds are {list(MLP_KINDS)}")
                if L.mlp.kind == "dense" and not L.mlp.limit > 0:
                    raise ConfigError(f"{w}.mlp.limit must be positive, found {L.mlp.limit}")
                if L.mlp.kind == "moe" and not 0 < L.mlp.top <= L.mlp.experts:
                    raise ConfigError(f"{w}.mlp.router: {L.mlp.top} experts per token out of {L.mlp.experts}")
        if self.loop is not None:
            lp = self.loop
            if not 0 <= lp.start < lp.stop <= len(self.layers):
                raise ConfigError(f"config.json: loop {lp.start}..{lp.stop} is no stretch of the {len(self.layers)} layers")

    def layer_runs(self) -> list[tuple[int, Optional[int]]]:
        """The order layers run in: (layer, pass number if this run opens a pass of the loop, else None)."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, None) for i in range(n)]
        lp = self.loop
        runs: list[tuple[int, Optional[int]]] = [(i, None) for i in range(lp.start)]
        for t in range(lp.times):
            runs += [(i, t if i == lp.start else None) for i in range(lp.start, lp.stop)]
        return runs + [(i, None) for i in range(lp.stop, n)]

    def to_json_dict(self) -> dict[str, Any]:
        layers = []
        for L in self.layers:
            m = L.mixer
            mixer: dict[str, Any] = {"heads": m.heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale}
            if m.rot_dims:
                mixer["rot"] = {"base": m.rot_base, "dims": m.rot_dims}
            if L.type == "attention":
                mixer["kv_heads"] = m.kv_heads
                if m.window:
                    mixer["mask"] = {"size": m.window, "keep_first": m.keep_first}
            else:
                mixer.update(rot_dim=m.rot_dim, kv_rank=m.kv_rank, q_rank=m.q_rank)
            mlp = None
            if L.mlp is not None and L.mlp.kind == "dense":
                mlp = {"kind": "dense", "ff": L.mlp.ff, "limit": L.mlp.limit}
            elif L.mlp is not None:
                mlp = {"kind": "moe", "expert": {"ff": L.mlp.ff}, "router": {"experts": L.mlp.experts, "top": L.mlp.top}}
            layers.append({"type": L.type, "mixer": mixer, "mlp": mlp})
        d: dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
                             "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embedding_scale}, "layers": layers}
        if self.loop is not None:
            d["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        if self.max_position_embeddings != DEFAULT_CONTEXT:
            d["max_positions"] = self.max_position_embeddings
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d
