"""Small Pirisun configurations with seeded weights, written as model folders, and the helpers that run them through
the engine and through the plain implementation.

The configurations differ from one another in every size and option: 1, 2 and 5 heads per key/value head and a single
key/value head; values wider, narrower and as wide as keys; a query temperature with short periods, one with a period
longer than any test sequence, and none; a score cap low enough to bend most scores, a high one and none; retention
with a rotation over the whole head, over a part and none, decays from 0.8 to 1, one head and several; latents narrower
and wider than the heads they expand to; routed experts with one, some and all router outputs per token, with no, one
and several identity experts, with and without a shared expert, and layers with no feed-forward; a loop over the first
layers, over the last, over the middle, of one pass and none; a logit scale and none; widths that are multiples of 64
and widths that no vectorised kernel takes.  Weights are N(0, 1/inputs) ("loud": every layer changes the stream by as
much as it holds)."""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch

import plain_pirisun as P


def _latent(heads, dim, rot_dim, vdim, kv_rank, scale, base, mlp=None):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
                      "rot": {"base": base, "dims": rot_dim}}, "mlp": mlp}


def _left(heads, kv_heads, dim, vdim, scale, softcap=None, q_temp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if softcap is not None:
        m["softcap"] = softcap
    if q_temp is not None:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return m


def _right(heads, dim, vdim, decay, rot=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}
    if rot is not None:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    return m


def _pair(left, right, mlp=None):
    return {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp}


def _moe(experts, top, ff, identity=0, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "identity": identity}}
    if shared is not None:
        m["shared"] = {"ff": shared}
    return m


CONFIGS = {
    # a loop over the first two layers; a low cap and a short temperature period; a partial rotation; one identity expert
    "pa": {"architecture": "Pirisun", "vocab": 101, "width": 48, "norm": {"eps": 1e-6}, "logit_scale": 0.5,
           "loop": {"start": 0, "stop": 2, "times": 2},
           "layers": [_pair(_left(4, 2, 16, 12, 0.3, softcap=2.0, q_temp=(0.4, 7)), _right(3, 8, 10, (0.9, 0.97, 0.995), rot=(100.0, 4)),
                            mlp=_moe(6, 2, 24, identity=1, shared=16)),
                      _latent(3, 8, 4, 10, 24, 0.3, 50.0, mlp=_moe(4, 1, 8)),
                      _pair(_left(2, 1, 24, 24, 0.2, q_temp=(1.5, 1000)), _right(1, 12, 20, (1.0,)))]},
    # no loop, no logit scale; every router output chosen, one of them an identity expert; no cap, no temperature
    "pb": {"architecture": "Pirisun", "vocab": 130, "width": 64, "norm": {"eps": 1e-5},
           "layers": [_latent(2, 16, 8, 16, 32, 0.2, 10000.0, mlp=_moe(3, 4, 16, identity=1)),
                      _pair(_left(6, 6, 8, 16, 0.35), _right(4, 16, 8, (0.8, 0.9, 0.95, 0.99), rot=(30.0, 16)),
                            mlp=_moe(2, 2, 72, shared=40))]},
    # sizes in multiples of 64 (what the tensor-core kernels take), a loop over the middle, two identity experts
    "pc": {"architecture": "Pirisun", "vocab": 512, "width": 128, "norm": {"eps": 1e-5}, "logit_scale": 2.0,
           "loop": {"start": 1, "stop": 3, "times": 2},
           "layers": [_latent(4, 32, 32, 64, 64, 0.12, 10000.0, mlp=_moe(8, 2, 64, identity=2, shared=128)),
                      _pair(_left(8, 2, 64, 64, 0.12, softcap=8.0, q_temp=(0.35, 16)), _right(4, 32, 32, (0.96, 0.98, 0.99, 0.999), rot=(300000.0, 32)),
                            mlp=_moe(8, 3, 64, identity=1)),
                      _latent(2, 64, 16, 32, 128, 0.1, 1000.0),
                      _pair(_left(4, 4, 64, 64, 0.11, softcap=50.0), _right(2, 64, 64, (0.9, 0.99), rot=(500.0, 32)), mlp=_moe(3, 1, 128))]},
    # the same kernels as "pc" with every router output chosen, so that bfloat16 runs compare at every position
    "pf": {"architecture": "Pirisun", "vocab": 256, "width": 128, "norm": {"eps": 1e-5}, "logit_scale": 2.0,
           "loop": {"start": 0, "stop": 2, "times": 2},
           "layers": [_pair(_left(8, 2, 64, 64, 0.12, softcap=6.0, q_temp=(0.25, 32)), _right(4, 32, 32, (0.96, 0.98, 0.99, 0.999), rot=(10000.0, 16)),
                            mlp=_moe(3, 5, 64, identity=2, shared=64)),
                      _latent(4, 32, 32, 64, 64, 0.12, 10000.0, mlp=_moe(4, 4, 32)),
                      _pair(_left(2, 1, 128, 128, 0.09, softcap=20.0), _right(2, 64, 64, (0.9, 0.99)))]},
    # the least there can be: one pair with one head on each side and no feed-forward, in a loop that runs once
    "pd": {"architecture": "Pirisun", "vocab": 50, "width": 32, "norm": {"eps": 1e-5}, "logit_scale": 1.0,
           "loop": {"start": 0, "stop": 1, "times": 1},
           "layers": [_pair(_left(1, 1, 4, 6, 0.4, softcap=1.0, q_temp=(0.2, 1)), _right(1, 4, 4, (0.95,), rot=(20.0, 2)))]},
    # sizes no vectorised kernel takes, five heads on one, a loop of three passes over the LAST layer
    "pe": {"architecture": "Pirisun", "vocab": 71, "width": 38, "norm": {"eps": 1e-4}, "logit_scale": 1.5,
           "loop": {"start": 1, "stop": 2, "times": 3},
           "layers": [_pair(_left(5, 1, 10, 7, 0.3, softcap=4.0, q_temp=(0.25, 3)), _right(2, 6, 5, (0.93, 0.999), rot=(20.0, 2)),
                            mlp=_moe(5, 3, 10)),
                      _latent(3, 6, 6, 5, 18, 0.3, 40.0, mlp=_moe(3, 2, 10, identity=3, shared=12))]},
}


def bf16_round(a: np.ndarray) -> np.ndarray:
    return torch.from_numpy(np.asarray(a, dtype=np.float32)).to(torch.bfloat16).float().numpy()


def make_weights(cfg: dict, seed: int) -> dict[str, np.ndarray]:
    """Seeded weights that bfloat16 holds exactly, as float32, by tensor name."""
    import zinfer_b200 as z
    from zinfer_b200.config.registry import build_model

    rng = np.random.default_rng(seed)
    model = build_model(z.config_from_dict(cfg))
    W = {}
    for name, spec in model.weight_specs().items():
        shape = spec.shape
        if name.endswith(".sink"):
            W[name] = bf16_round(rng.normal(0.5, 1.5, shape))
        elif name.endswith(".b"):
            W[name] = bf16_round(rng.normal(0, 0.2, shape))
        elif name.endswith(".correction"):
            W[name] = bf16_round(rng.normal(0, 0.1, shape))
        elif "norm" in name or name.endswith(".out"):
            W[name] = bf16_round(1.0 + rng.normal(0, 0.2, shape))
        elif name == "embed":
            W[name] = bf16_round(rng.normal(0, 1.0, shape))
        elif name.endswith(".router"):
            W[name] = bf16_round(rng.normal(0, 3.0 * shape[-1] ** -0.5, shape))
        else:
            W[name] = bf16_round(rng.normal(0, shape[-1] ** -0.5, shape))
    return W


def write_folder(folder, cfg: dict, W: dict[str, np.ndarray]) -> Path:
    from zinfer_b200.weights import write_safetensors

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    write_safetensors(folder / "model.safetensors", {n: torch.from_numpy(a).to(torch.bfloat16) for n, a in W.items()})
    return folder


CLOSE_CALL = 0.02       # a router choice whose margin (in score + correction) is below this may fall either way in bfloat16


def plain_logits(cfg: dict, W: dict[str, np.ndarray], tokens):
    """(logits [n, vocab], safe): the plain implementation's logits and the number of leading positions before the
    first token whose expert choice is a close call.  In bfloat16 such a token may take another expert, and it and
    every later position then differ by far more than rounding; positions before it cannot be affected."""
    margins = [np.inf] * len(tokens)
    logits = P.forward(cfg, {n: a.astype(np.float64) for n, a in W.items()}, list(tokens), margins=margins)
    close = [t for t, m in enumerate(margins) if m < CLOSE_CALL]
    return logits, (close[0] if close else len(tokens))


def tokens_for(cfg: dict, seed: int, n: int) -> list[int]:
    return np.random.default_rng(seed).integers(0, cfg["vocab"], size=n).tolist()


TOL = {"float32": 5e-5, "bfloat16": 4e-2}


def rel_err(got, ref) -> float:
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    scale = float(np.abs(ref).max())
    assert scale > 0 and got.shape == ref.shape, (got.shape, ref.shape)
    return float(np.abs(got - ref).max()) / scale
