"""Small Kerotar configurations with seeded weights, written as model folders, and the helpers that run them through
the engine and through the plain implementation.

The configurations differ from one another in every size and option: 1, 2 and 5 heads per key/value head and as many
key/value heads as heads; values wider, narrower and as wide as keys; rotations over a whole head and over a part;
windows shorter and longer than a cache page, with no, one, a few and more kept first tokens than the window is long,
and a layer with no window at all; latents narrower and wider than the heads they expand to, one head and several;
dense feed-forwards, routed experts with one, some and all experts per token, and layers with no feed-forward; a loop
over the first layers, over the last, over the middle, of one pass and none; an embedding scale and none; widths that
are multiples of 64 and widths that no vectorised kernel takes.  Weights are N(0, 1/inputs) ("loud": every layer
changes the stream by as much as it holds)."""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch

import plain_kerotar as P


def _attn(heads, kv_heads, dim, vdim, scale, rot=None, mask=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot is not None:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    if mask is not None:
        m["mask"] = {"size": mask[0], "keep_first": mask[1]}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def _latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base, mlp=None):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
                      "scale": scale, "rot": {"base": base, "dims": rot_dim}}, "mlp": mlp}


def _dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def _moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


CONFIGS = {
    # a loop over the first two layers; a window that crosses pages with three kept tokens; a whole-head rotation
    "ka": {"architecture": "Kerotar", "vocab": 101, "width": 48, "norm": {"eps": 1e-6}, "embedding": {"scale": 0.7},
           "loop": {"start": 0, "stop": 2, "times": 2},
           "layers": [_attn(4, 2, 16, 12, 0.3, rot=(100.0, 8), mask=(20, 3), mlp=_moe(6, 2, 24)),
                      _latent(3, 8, 4, 10, 24, 20, 0.3, 50.0, mlp=_dense(56, 2.0)),
                      _attn(2, 1, 24, 24, 0.2, rot=(10000.0, 24), mask=(40, 0))]},
    # no loop, no embedding scale; every expert chosen; more kept tokens than the window is long, in two pages
    "kb": {"architecture": "Kerotar", "vocab": 130, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
           "layers": [_latent(2, 16, 8, 16, 32, 40, 0.2, 10000.0, mlp=_moe(4, 4, 16)),
                      _attn(6, 6, 8, 16, 0.35, rot=(30.0, 4), mask=(7, 20), mlp=_dense(72, 0.5))]},
    # sizes in multiples of 64 (what the tensor-core contractions take), a loop over the middle, a layer with no
    # window, one expert per token
    "kc": {"architecture": "Kerotar", "vocab": 512, "width": 128, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
           "loop": {"start": 1, "stop": 3, "times": 2},
           "layers": [_latent(4, 32, 32, 64, 64, 64, 0.12, 10000.0, mlp=_dense(256, 1.0)),
                      _attn(8, 2, 64, 64, 0.12, rot=(300000.0, 32), mask=(112, 5), mlp=_moe(8, 2, 64)),
                      _attn(4, 4, 64, 64, 0.11, rot=(500.0, 64), mlp=_moe(3, 1, 128)),
                      _latent(2, 64, 16, 32, 128, 96, 0.1, 1000.0)]},
    # the least there can be: one latent layer with one head and no feed-forward, in a loop that runs once
    "kd": {"architecture": "Kerotar", "vocab": 50, "width": 32, "norm": {"eps": 1e-5}, "embedding": {"scale": 0.5},
           "loop": {"start": 0, "stop": 1, "times": 1},
           "layers": [_latent(1, 4, 2, 4, 8, 8, 0.4, 20.0)]},
    # sizes no vectorised kernel takes, five heads on five, one kept token, a loop of three passes over the LAST layer
    "ke": {"architecture": "Kerotar", "vocab": 71, "width": 38, "norm": {"eps": 1e-4}, "embedding": {"scale": 1.5},
           "loop": {"start": 1, "stop": 2, "times": 3},
           "layers": [_attn(5, 5, 10, 7, 0.3, rot=(20.0, 6), mask=(33, 1), mlp=_dense(50, 0.75)),
                      _latent(3, 6, 6, 5, 18, 14, 0.3, 40.0, mlp=_moe(5, 3, 10))]},
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
        elif "norm" in name:
            W[name] = bf16_round(1.0 + rng.normal(0, 0.2, shape))
        elif name == "loop.step":
            W[name] = bf16_round(rng.normal(0, 0.5, shape))
        elif name == "embed":
            W[name] = bf16_round(rng.normal(0, 1.0, shape))
        elif name.endswith(".router"):
            W[name] = bf16_round(rng.normal(0, 2.0 * shape[-1] ** -0.5, shape))
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


CLOSE_CALL = 0.03       # a router choice nearer than this (relative to the largest logit) may fall either way in bfloat16


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
