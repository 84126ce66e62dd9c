"""Pirisun without a GPU: the configuration and its errors, the order of layer runs with a loop, tensor names and
shapes, the cache and state each run asks for, the rows of routed experts with identity experts left out, random model
folders, and the plain implementation's mechanisms against closed forms."""
import copy
import dataclasses
import math

import numpy as np
import pytest
import torch

import pirisun_helpers as H
import plain_pirisun as P


def test_configuration_reads_every_key_and_round_trips():
    import zinfer_b200 as z
    for name, d in H.CONFIGS.items():
        c = z.config_from_dict(d)
        assert c.architecture == "Pirisun" and c.vocab_size == d["vocab"] and c.hidden_size == d["width"]
        assert c.norm_eps == d["norm"]["eps"] and len(c.layers) == len(d["layers"])
        assert c.logit_scale == d.get("logit_scale", 1.0)
        assert dataclasses.replace(z.config_from_dict(c.to_json_dict()), raw={}) == dataclasses.replace(c, raw={})
        again = c.to_json_dict()
        again.pop("logit_scale", None) if "logit_scale" not in d else None
        for L, La in zip(d["layers"], again["layers"]):      # what a file leaves out reads back as absent or as its default
            if L["mlp"] is not None:
                assert La["mlp"]["router"] == {**{"identity": 0}, **L["mlp"]["router"]} and La["mlp"].get("shared") == L["mlp"].get("shared")
            assert La["mixer"] == L["mixer"], name
    c = z.config_from_dict(H.CONFIGS["pa"])
    a, r = c.layers[0].left, c.layers[0].right
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.softcap, a.q_temp_coef, a.q_temp_every) == (4, 2, 16, 12, 0.3, 2.0, 0.4, 7)
    assert (r.heads, r.dim, r.vdim, r.decay, r.rot_base, r.rot_dims) == (3, 8, 10, (0.9, 0.97, 0.995), 100.0, 4)
    assert c.layers[2].mlp is None and c.layers[2].left.softcap == 0.0 and c.layers[2].right.rot_dims == 0
    assert c.layers[0].mlp.identity == 1 and c.layers[0].mlp.shared_ff == 16 and c.layers[1].mlp.shared_ff == 0
    assert c.layers[1].latent.kv_rank == 24 and c.layers[1].latent.rot_dim == 4 and c.loop.times == 2 and c.logit_scale == 0.5
    assert z.config_from_dict(H.CONFIGS["pb"]).logit_scale == 1.0 and z.config_from_dict(H.CONFIGS["pb"]).loop is None


@pytest.mark.parametrize("change,message", [
    (lambda d: d["layers"][0].update(type="mamba"), "known types"),
    (lambda d: d["layers"][0]["mixer"]["left"].update(kv_heads=3), "not a multiple"),
    (lambda d: d["layers"][0]["mixer"]["right"]["rot"].update(dims=3), "even"),
    (lambda d: d["layers"][0]["mixer"]["right"]["rot"].update(dims=10), "at most dim"),
    (lambda d: d["layers"][0]["mixer"]["right"].update(decay=[0.9]), "decays"),
    (lambda d: d["layers"][0]["mixer"]["left"].pop("scale"), "scale"),
    (lambda d: d["layers"][0]["mixer"]["left"]["q_temp"].pop("every"), "every"),
    (lambda d: d["layers"][0]["mixer"].pop("right"), "mixer.right"),
    (lambda d: d["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda d: d["layers"][1]["mixer"]["rot"].update(dims=2), "must equal rot_dim"),
    (lambda d: d["layers"][0]["mlp"]["router"].update(top=8), "experts per token"),
    (lambda d: d["layers"][1]["mlp"].update(kind="dense"), "moe"),
    (lambda d: d["loop"].update(stop=4), "stretch"),
    (lambda d: d["loop"].update(times=0), "times"),
    (lambda d: d.pop("vocab"), "vocab"),
])
def test_configuration_errors_name_the_key(change, message):
    import zinfer_b200 as z
    d = copy.deepcopy(H.CONFIGS["pa"])
    change(d)
    with pytest.raises(z.ConfigError, match=message):
        z.config_from_dict(d)


def test_layer_runs_follow_the_loop():
    import zinfer_b200 as z
    runs = {n: z.config_from_dict(d).layer_runs() for n, d in H.CONFIGS.items()}
    assert runs["pa"] == [0, 1, 0, 1, 2]
    assert runs["pb"] == [0, 1]
    assert runs["pc"] == [0, 1, 2, 1, 2, 3]
    assert runs["pd"] == [0]
    assert runs["pe"] == [0, 1, 1, 1]
    for n, d in H.CONFIGS.items():
        assert P.layer_runs(d) == runs[n]


def test_model_asks_for_the_tensors_of_the_design_and_storage_per_run():
    import zinfer_b200 as z
    from zinfer_b200.config.registry import build_model
    m = build_model(z.config_from_dict(H.CONFIGS["pa"]))
    specs = m.weight_specs()
    want = {"embed": (101, 48), "head": (101, 48), "final.norm": (48,), "final.norm.b": (48,), "l0.norm1": (48,), "l0.norm1.b": (48,),
            "l0.mix.left.q": (64, 48), "l0.mix.left.k": (32, 48), "l0.mix.left.v": (24, 48), "l0.mix.left.o": (48, 48),
            "l0.mix.right.q": (24, 48), "l0.mix.right.k": (24, 48), "l0.mix.right.v": (30, 48), "l0.mix.right.g": (30, 48),
            "l0.mix.right.o": (48, 30), "l0.mix.left.out": (48,), "l0.mix.right.out": (48,), "l0.mlp.router": (7, 48),
            "l0.mlp.correction": (7,), "l0.mlp.e5.gate": (24, 48), "l0.mlp.e0.down": (48, 24), "l0.mlp.shared.up": (16, 48),
            "l0.mlp.shared.down": (48, 16), "l1.mix.q": (36, 48), "l1.mix.dkv": (28, 48), "l1.mix.dkv.norm": (24,),
            "l1.mix.uk": (24, 24), "l1.mix.uv": (30, 24), "l1.mix.sink": (3,), "l1.mix.g": (30, 48), "l1.mix.o": (48, 30),
            "l1.mlp.router": (4, 48), "l2.mix.right.g": (20, 48)}
    for name, shape in want.items():
        assert specs[name].shape == shape, name
    assert not any(n.startswith("l2.mlp") or n.startswith("l1.mlp.shared") or n.startswith("l0.mlp.e6") for n in specs)
    assert len(specs) == 4 + (2 + 11 + 2 + 18 + 3) + (2 + 8 + 2 + 12) + (2 + 11)
    cs = m.cache_specs()
    assert len(cs) == 5                                       # storage per run: layers 0 and 1 run twice
    assert cs[0].kv == cs[2].kv and cs[0].kv.n_kv_heads == 2 and cs[0].kv.head_dim == 16 and cs[0].kv.v_dim == 12 and cs[0].kv.window == 0
    assert cs[0].state.shape == (3 * 8 * 10,) and cs[0].state.dtype == torch.float32 and cs[4].state.shape == (12 * 20,)
    assert cs[1].kv.n_kv_heads == 1 and cs[1].kv.head_dim == 24 + 4 and cs[1].kv.v_dim == 0 and cs[1].state is None


def test_expert_rows_leave_identity_pairs_out():
    from zinfer_b200.parts.moe import expert_rows
    ids = np.array([0, 3, 2, 2, 4, 1, 0, 0])            # 4 tokens x top 2; experts 0..2 have weights, 3 and 4 are identity
    row_token, pair_row, bounds = expert_rows(ids, 3, 2, tile=4)
    assert pair_row[1] == -1 and pair_row[4] == -1 and bounds.tolist() == [0, 4, 8, 12]
    for i, e in enumerate(ids):
        if e < 3:
            assert bounds[e] <= pair_row[i] < bounds[e + 1] and row_token[pair_row[i]] == i // 2
    assert sorted(row_token[row_token >= 0].tolist()) == [0, 1, 1, 2, 3, 3]
    row_token, pair_row, bounds = expert_rows(np.array([1, 0, 1, 2]), 3, 2)          # none: as before
    assert pair_row.tolist() == [1, 0, 2, 3] and row_token.tolist() == [0, 0, 1, 1]


def test_random_model_folders_load_back(tmp_path):
    import zinfer_b200 as z
    from zinfer_b200.weights.safetensors_io import SafetensorsFile
    cfg = z.config_from_dict(H.CONFIGS["pe"])
    folder = z.write_random_model(tmp_path / "m", cfg, seed=3)
    assert dataclasses.replace(z.config_from_folder(folder), raw={}) == dataclasses.replace(cfg, raw={})
    with SafetensorsFile(folder / "model.safetensors") as f:
        from zinfer_b200.config.registry import build_model
        assert sorted(f.names()) == sorted(build_model(cfg).weight_specs())


# ------------------------------------------------------------------------------- the plain implementation's own mechanisms

def test_plain_retention_is_its_closed_form():
    """o_t = sum_{j <= t} decay^(t-j) (q_t . k_j) v_j, before the unit norm and the gate."""
    rng = np.random.default_rng(0)
    n, D, d, e, g = 9, 6, 4, 3, 0.9
    W = {"q": rng.normal(size=(d, D)), "k": rng.normal(size=(d, D)), "v": rng.normal(size=(e, D)), "g": rng.normal(size=(e, D)),
         "o": np.eye(e)}
    h = rng.normal(size=(n, D))
    got = P.retention(h, W, {"heads": 1, "dim": d, "vdim": e, "decay": [g]}, 1e-6)
    q, k, v = h @ W["q"].T, h @ W["k"].T * d ** -0.5, h @ W["v"].T
    o = np.stack([sum(g ** (t - j) * (q[t] @ k[j]) * v[j] for j in range(t + 1)) for t in range(n)])
    assert np.allclose(got, P.rms(o, 1e-6) * P.silu(h @ W["g"].T))


def test_plain_rotations_pair_as_they_say():
    v = np.arange(1.0, 9.0)
    a = P.rotate(v, 3, 100.0, 4, True)
    b = P.rotate(v, 3, 100.0, 4, False)
    c0, s0, c1, s1 = math.cos(3.0), math.sin(3.0), math.cos(0.3), math.sin(0.3)
    assert np.allclose(a[:4], [1 * c0 - 2 * s0, 2 * c0 + 1 * s0, 3 * c1 - 4 * s1, 4 * c1 + 3 * s1]) and np.array_equal(a[4:], v[4:])
    assert np.allclose(b[:4], [1 * c0 - 3 * s0, 2 * c1 - 4 * s1, 3 * c0 + 1 * s0, 4 * c1 + 2 * s1]) and np.array_equal(b[4:], v[4:])
    assert np.array_equal(P.rotate(v, 0, 100.0, 8, True), v)


def test_plain_router_chooses_by_corrected_score_and_weighs_by_score():
    z = np.log(np.array([0.4, 0.3, 0.2, 0.1]))
    chosen, w, margin = P.route(z, np.array([0.0, 0.0, 0.0, 0.25]), 2)
    assert chosen == [0, 3] and np.allclose(w, [0.8, 0.2]) and abs(margin - 0.05) < 1e-12
    chosen, w, margin = P.route(z, None, 4)
    assert chosen == [0, 1, 2, 3] and margin == np.inf and abs(sum(w) - 1) < 1e-12


def test_plain_identity_expert_hands_its_input_on():
    rng = np.random.default_rng(1)
    h = rng.normal(size=(5, 6))
    W = {"router": np.zeros((2, 6)), "correction": np.array([0.0, 1.0]), "e0.gate": rng.normal(size=(3, 6)),
         "e0.up": rng.normal(size=(3, 6)), "e0.down": rng.normal(size=(6, 3))}
    out = P.experts(h, W, {"router": {"experts": 1, "identity": 1, "top": 1}})
    assert np.allclose(out, h)                                # the identity expert alone, weight 0.5 / 0.5
    both = P.experts(h, W, {"router": {"experts": 1, "identity": 1, "top": 2}})
    assert np.allclose(both, 0.5 * h + 0.5 * P.gated_unit(h, W["e0.gate"], W["e0.up"], W["e0.down"]))


def test_plain_query_temperature_steps_where_it_should():
    """Scores of position p carry the factor 1 + coef * ln(floor((p + 1) / every) + 1): with one key the softmax hides
    it, so compare the single-head output for two keys at the positions around a step."""
    D = 4
    W = {"q": np.eye(D), "k": np.eye(D), "v": np.eye(D), "o": np.eye(D)}
    m = {"heads": 1, "kv_heads": 1, "dim": D, "vdim": D, "scale": 1.0, "q_temp": {"coef": 1.0, "every": 3}}
    h = np.zeros((4, D))
    h[0, 0] = h[1, 1] = h[2, 2] = 1.0
    h[3] = [1.0, 0, 0, 0]
    out = P.capped_attention(h, W, m)
    temp = 1.0 + math.log(math.floor(4 / 3) + 1.0)           # position 3
    e = math.exp(temp)
    w0 = (e + e) / (2 * e + 2)                               # keys 0 and 3 both score temp, keys 1 and 2 score 0
    assert abs(out[3, 0] - w0) < 1e-12
    assert abs(P.capped_attention(h[:2], W, m)[1, 1] - math.e / (math.e + 1)) < 1e-12       # position 1: factor 1
