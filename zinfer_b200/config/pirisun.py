"""Typed configuration of the Pirisun architecture, read from its own config.json keys.

The file is nested: `vocab`, `width`, `norm.eps` (of the layer norms and of every RMS norm inside the mixers),
`logit_scale` (the logits are multiplied by it; 1 if absent), optionally `loop` {start, stop, times} (layers start ..
stop-1 run `times` times in a row with the same weights, each pass with a cache and state of its own) and `layers`, a
list with one entry per layer:

* `type` "latent_attention": `mixer` {heads, dim, rot_dim, vdim, kv_rank, scale, rot {base, dims}}: causal attention
  whose keys and values are expanded from a latent of `kv_rank` entries per token, with `rot_dim` rotated entries
  (interleaved pairs) shared by all heads, queries straight from the layer's input, a learned sink per head in the
  softmax and a sigmoid gate on every output value;
* `type` "parallel": `mixer` {left, right}, two mixers side by side whose normalised results are averaged:
  `left` {heads, kv_heads, dim, vdim, scale, softcap, q_temp {coef, every}}: grouped-query softmax attention without a
  rotation, the query multiplied by a temperature that grows with the logarithm of its position, the scaled scores
  through a tanh cap; `right` {heads, dim, vdim, decay [one per head], rot {base, dims}}: retention, a linear
  recurrence with a fixed decay per head;
* `mlp`: null or {kind "moe", expert {ff}, router {experts, top, identity}, shared {ff}}: a softmax router over
  `experts` + `identity` outputs (the last `identity` stand for experts that return their input) with a correction
  vector for the choice, and optionally a shared expert every token takes.

Every size and constant comes from here; what the file does not mention (no `loop`, no `q_temp`, no `softcap`, no `rot`
of the retention, no `shared`, no `identity`) the model does not have.  The design sets no longest sequence;
`max_positions`, if a file has it, is only the default context of an engine (else DEFAULT_CONTEXT)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional

from .base import ConfigError, ModelConfig, as_float, as_int, need

MIXER_TYPES = ("latent_attention", "parallel")
DEFAULT_CONTEXT = 8192


@dataclass(frozen=True)
class PirisunLatent:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot_base: float


@dataclass(frozen=True)
class PirisunAttention:            # the left side of a parallel mixer
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float = 0.0           # 0 = no cap
    q_temp_coef: float = 0.0
    q_temp_every: int = 0          # 0 = no query temperature


@dataclass(frozen=True)
class PirisunRetention:            # the right side of a parallel mixer
    heads: int
    dim: int
    vdim: int
    decay: tuple[float, ...]
    rot_base: float = 0.0
    rot_dims: int = 0              # 0 = no rotation


@dataclass(frozen=True)
class PirisunMlp:
    ff: int
    experts: int
    top: int
    identity: int = 0
    shared_ff: int = 0             # 0 = no shared expert


@dataclass(frozen=True)
class PirisunLayer:
    type: str
    latent: Optional[PirisunLatent] = None
    left: Optional[PirisunAttention] = None
    right: Optional[PirisunRetention] = None
    mlp: Optional[PirisunMlp] = None


@dataclass(frozen=True)
class PirisunLoop:
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


def _rot(m: dict, w: str) -> tuple[float, int]:
    rot = _obj(m, "rot", w)
    if not rot:
        return 0.0, 0
    return as_float(w + "rot.base", need(rot, "base")), as_int(rot, w + "rot.dims", need(rot, "dims"), 0)


def _latent(m: dict, w: str) -> PirisunLatent:
    rot_dim = as_int(m, w + "rot_dim", need(m, "rot_dim"), 2)
    base, dims = _rot(m, w)
    if not dims:
        raise ConfigError(f"config.json: '{w}rot' is missing")
    if dims != rot_dim:
        raise ConfigError(f"config.json: '{w}rot.dims' = {dims} must equal rot_dim {rot_dim}")
    dim = as_int(m, w + "dim", need(m, "dim"), 1)
    return PirisunLatent(as_int(m, w + "heads", need(m, "heads"), 1), dim, rot_dim, as_int(m, w + "vdim", m.get("vdim", dim), 1),
                         as_int(m, w + "kv_rank", need(m, "kv_rank"), 1), as_float(w + "scale", need(m, "scale")), base)


def _left(m: dict, w: str) -> PirisunAttention:
    heads = as_int(m, w + "heads", need(m, "heads"), 1)
    dim = as_int(m, w + "dim", need(m, "dim"), 1)
    qt = _obj(m, "q_temp", w)
    cap = m.get("softcap")
    return PirisunAttention(heads, as_int(m, w + "kv_heads", m.get("kv_heads", heads), 1), dim,
                            as_int(m, w + "vdim", m.get("vdim", dim), 1), as_float(w + "scale", need(m, "scale")),
                            softcap=0.0 if cap is None else as_float(w + "softcap", cap),
                            q_temp_coef=as_float(w + "q_temp.coef", need(qt, "coef")) if qt else 0.0,
                            q_temp_every=as_int(qt, w + "q_temp.every", need(qt, "every"), 1) if qt else 0)


def _right(m: dict, w: str) -> PirisunRetention:
    dim = as_int(m, w + "dim", need(m, "dim"), 1)
    decay = need(m, "decay")
    if not isinstance(decay, (list, tuple)):
        raise ConfigError(f"config.json: '{w}decay' must be a list with one number per head")
    base, dims = _rot(m, w)
    return PirisunRetention(as_int(m, w + "heads", need(m, "heads"), 1), dim, as_int(m, w + "vdim", m.get("vdim", dim), 1),
                            tuple(as_float(w + "decay", g) for g in decay), base, dims)


def _mlp(ml, w: str) -> Optional[PirisunMlp]:
    if ml is None:
        return None
    if not isinstance(ml, dict):
        raise ConfigError(f"config.json: '{w}' must be an object or null")
    kind = str(ml.get("kind", "moe"))
    if kind != "moe":
        raise ConfigError(f"config.json: '{w}.kind' = {kind!r}; the design's feed-forward is 'moe'")
    ex, ro, sh = _obj(ml, "expert", w + "."), _obj(ml, "router", w + "."), _obj(ml, "shared", w + ".")
    return PirisunMlp(as_int(ex, w + ".expert.ff", need(ex, "ff"), 1),
                      experts=as_int(ro, w + ".router.experts", need(ro, "experts"), 1),
                      top=as_int(ro, w + ".router.top", need(ro, "top"), 1),
                      identity=as_int(ro, w + ".router.identity", ro.get("identity", 0), 0),
                      shared_ff=as_int(sh, w + ".shared.ff", need(sh, "ff"), 1) if sh else 0)


@dataclass
class PirisunConfig(ModelConfig):
    layers: tuple[PirisunLayer, ...] = ()
    loop: Optional[PirisunLoop] = None
    norm_eps: float = 1e-5
    logit_scale: float = 1.0

    @classmethod
    def from_json_dict(cls, d: dict[str, Any]) -> "PirisunConfig":
        vocab = as_int(d, "vocab", need(d, "vocab"), 1)
        width = as_int(d, "width", need(d, "width"), 1)
        norm = _obj(d, "norm", "")
        raw_layers = need(d, "layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, L in enumerate(raw_layers):
            if not isinstance(L, dict):
                raise ConfigError(f"config.json: 'layers[{i}]' must be an object")
            kind = str(need(L, "type"))
            w = f"layers[{i}].mixer."
            m = _obj(L, "mixer", f"layers[{i}].")
            mlp = _mlp(L.get("mlp"), f"layers[{i}].mlp")
            if kind == "latent_attention":
                layers.append(PirisunLayer(kind, latent=_latent(m, w), mlp=mlp))
            elif kind == "parallel":
                for side in ("left", "right"):
                    if not _obj(m, side, w):
                        raise ConfigError(f"config.json: required key '{w}{side}' is missing")
                layers.append(PirisunLayer(kind, left=_left(_obj(m, "left", w), w + "left."),
                                           right=_right(_obj(m, "right", w), w + "right."), mlp=mlp))
            else:
                raise ConfigError(f"config.json: 'layers[{i}].type' = {kind!r}; known types are {list(MIXER_TYPES)}")
        loop = None
        lp = _obj(d, "loop", "")
        if lp:
            loop = PirisunLoop(as_int(lp, "loop.start", need(lp, "start"), 0), as_int(lp, "loop.stop", need(lp, "stop"), 0),
                               as_int(lp, "loop.times", need(lp, "times"), 1))
        eos = d.get("eos_token_id")
        max_pos = d.get("max_positions")
        cfg = cls(architecture=str(d.get("architecture") or (d.get("architectures") or ["Pirisun"])[0]),
                  vocab_size=vocab, hidden_size=width,
                  max_position_embeddings=DEFAULT_CONTEXT if max_pos is None else as_int(d, "max_positions", max_pos, 1),
                  eos_token_ids=() if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos])),
                  raw=dict(d), layers=tuple(layers), loop=loop, norm_eps=as_float("norm.eps", norm.get("eps", 1e-5)),
                  logit_scale=as_float("logit_scale", d.get("logit_scale", 1.0)))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.norm_eps <= 0:
            raise ConfigError(f"config.json: norm.eps must be positive, found {self.norm_eps}")
        for i, L in enumerate(self.layers):
            w = f"config.json: layers[{i}]"
            if L.type == "latent_attention":
                if L.latent is None or L.latent.rot_dim % 2:
                    raise ConfigError(f"{w}.mixer.rot_dim must be even")
                if L.latent.rot_base <= 0:
                    raise ConfigError(f"{w}.mixer.rot.base must be positive, found {L.latent.rot_base}")
            elif L.type == "parallel":
                a, r = L.left, L.right
                if a is None or r is None:
                    raise ConfigError(f"{w}.mixer needs 'left' and 'right'")
                if a.heads % a.kv_heads:
                    raise ConfigError(f"{w}.mixer.left: {a.heads} heads are not a multiple of {a.kv_heads} kv_heads")
                if a.softcap < 0:
                    raise ConfigError(f"{w}.mixer.left.softcap must be positive, found {a.softcap}")
                if len(r.decay) != r.heads:
                    raise ConfigError(f"{w}.mixer.right: {len(r.decay)} decays for {r.heads} heads")
                if r.rot_dims % 2 or r.rot_dims > r.dim:
                    raise ConfigError(f"{w}.mixer.right.rot.dims = {r.rot_dims} must be even and at most dim {r.dim}")
                if r.rot_dims and r.rot_base <= 0:
                    raise ConfigError(f"{w}.mixer.right.rot.base must be positive, found {r.rot_base}")
            else:
                raise ConfigError(f"{w}.type = {L.type!r}; known types are {list(MIXER_TYPES)}")
            if L.mlp is not None and not 0 < L.mlp.top <= L.mlp.experts + L.mlp.identity:
                raise ConfigError(f"{w}.mlp.router: {L.mlp.top} experts per token out of {L.mlp.experts} + {L.mlp.identity}")
        if self.loop is not None:
            lp = self.loop
            if not 0 <= lp.start < lp.stop <= len(self.layers):
                raise ConfigError(f"config.json: loop {lp.start}..{lp.stop} is no stretch of the {len(self.layers)} layers")

    def layer_runs(self) -> list[int]:
        """The order layers run in, the loop unrolled."""
        n = len(self.layers)
        if self.loop is None:
            return list(range(n))
        lp = self.loop
        return list(range(lp.start)) + list(range(lp.start, lp.stop)) * lp.times + list(range(lp.stop, n))

    def to_json_dict(self) -> dict[str, Any]:
        layers = []
        for L in self.layers:
            if L.type == "latent_attention":
                m = L.latent
                mixer: dict[str, Any] = {"heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim, "kv_rank": m.kv_rank,
                                         "scale": m.scale, "rot": {"base": m.rot_base, "dims": m.rot_dim}}
            else:
                a, r = L.left, L.right
                left: dict[str, Any] = {"heads": a.heads, "kv_heads": a.kv_heads, "dim": a.dim, "vdim": a.vdim, "scale": a.scale}
                if a.softcap:
                    left["softcap"] = a.softcap
                if a.q_temp_every:
                    left["q_temp"] = {"coef": a.q_temp_coef, "every": a.q_temp_every}
                right: dict[str, Any] = {"heads": r.heads, "dim": r.dim, "vdim": r.vdim, "decay": list(r.decay)}
                if r.rot_dims:
                    right["rot"] = {"base": r.rot_base, "dims": r.rot_dims}
                mixer = {"left": left, "right": right}
            mlp = None
            if L.mlp is not None:
                mlp = {"kind": "moe", "expert": {"ff": L.mlp.ff},
                       "router": {"experts": L.mlp.experts, "top": L.mlp.top, "identity": L.mlp.identity}}
                if L.mlp.shared_ff:
                    mlp["shared"] = {"ff": L.mlp.shared_ff}
            layers.append({"type": L.type, "mixer": mixer, "mlp": mlp})
        d: dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
                             "norm": {"eps": self.norm_eps}, "logit_scale": self.logit_scale, "layers": layers}
        if self.loop is not None:
            d["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        if self.max_position_embeddings != DEFAULT_CONTEXT:
            d["max_positions"] = self.max_position_embeddings
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d
