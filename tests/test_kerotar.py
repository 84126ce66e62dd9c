"""Kerotar without a GPU: the configuration and its errors, the order of layer runs with a loop, tensor names and
shapes, the cache each run asks for, kept first pages in the cache, the rows of routed experts, and the plain
implementation's mechanisms against closed forms."""
import copy
import dataclasses

import numpy as np
import pytest
import torch

import kerotar_helpers as H
import plain_kerotar as P


def test_configuration_reads_every_key_and_round_trips():
    import zinfer_b200 as z
    for name, d in H.CONFIGS.items():
        c = z.config_from_dict(d)
        assert c.architecture == "Kerotar" and c.vocab_size == d["vocab"] and c.hidden_size == d["width"]
        assert c.norm_eps == d["norm"]["eps"] and len(c.layers) == len(d["layers"])
        assert c.embedding_scale == d["embedding"]["scale"]
        assert c.to_json_dict() == d, name
        assert dataclasses.replace(z.config_from_dict(c.to_json_dict()), raw={}) == dataclasses.replace(c, raw={})
    c = z.config_from_dict(H.CONFIGS["kc"])
    assert c.layers[2].mixer.window == 0 and c.layers[1].mixer.keep_first == 5 and c.layers[1].mixer.window == 112
    assert c.layers[3].mlp is None and c.layers[2].mlp.top == 1 and c.layers[0].mlp.limit == 1.0
    assert c.layers[0].mixer.kv_rank == 64 and c.layers[3].mixer.rot_dim == 16 and c.loop.times == 2
    d = copy.deepcopy(H.CONFIGS["kb"])
    del d["embedding"]
    assert z.config_from_dict(d).embedding_scale == 1.0


@pytest.mark.parametrize("change,message", [
    (lambda d: d["layers"][0].update(type="mamba"), "known types"),
    (lambda d: d["layers"][0]["mixer"].update(kv_heads=3), "not a multiple"),
    (lambda d: d["layers"][0]["mixer"]["rot"].update(dims=7), "even"),
    (lambda d: d["layers"][0]["mixer"]["rot"].update(dims=18), "at most dim"),
    (lambda d: d["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda d: d["layers"][0]["mixer"]["mask"].pop("size"), "size"),
    (lambda d: d["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda d: d["layers"][1]["mixer"]["rot"].update(dims=2), "must equal rot_dim"),
    (lambda d: d["layers"][1]["mlp"].pop("limit"), "limit"),
    (lambda d: d["layers"][0]["mlp"]["router"].update(top=7), "experts per token"),
    (lambda d: d["layers"][1]["mlp"].update(kind="sparse"), "known kinds"),
    (lambda d: d["loop"].update(stop=4), "stretch"),
    (lambda d: d["loop"].update(times=0), "times"),
    (lambda d: d.pop("vocab"), "vocab"),
])
def test_configuration_errors_name_the_key(change, message):
    import zinfer_b200 as z
    d = copy.deepcopy(H.CONFIGS["ka"])
    change(d)
    with pytest.raises(z.ConfigError, match=message):
        z.config_from_dict(d)


def test_layer_runs_follow_the_loop():
    import zinfer_b200 as z
    runs = {n: z.config_from_dict(d).layer_runs() for n, d in H.CONFIGS.items()}
    assert runs["ka"] == [(0, 0), (1, None), (0, 1), (1, None), (2, None)]
    assert runs["kb"] == [(0, None), (1, None)]
    assert runs["kc"] == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (3, None)]
    assert runs["kd"] == [(0, 0)]
    assert runs["ke"] == [(0, None), (1, 0), (1, 1), (1, 2)]
    for n, d in H.CONFIGS.items():
        assert P.run_order(d) == runs[n]


def test_model_asks_for_the_tensors_of_the_design_and_a_cache_per_run():
    import zinfer_b200 as z
    from zinfer_b200.config.registry import build_model
    m = build_model(z.config_from_dict(H.CONFIGS["ka"]))
    specs = m.weight_specs()
    want = {"embed": (101, 48), "head": (101, 48), "final.norm": (48,), "loop.in": (48, 96), "loop.step": (2, 48),
            "l0.norm1": (48,), "l0.mix.q": (64, 48), "l0.mix.k": (32, 48), "l0.mix.v": (24, 48), "l0.mix.o": (48, 48),
            "l0.mix.q.norm": (64,), "l0.mix.k.norm": (32,), "l0.mix.sink": (4,), "l0.mlp.router": (6, 48),
            "l0.mlp.e5.gate": (24, 48), "l0.mlp.e0.down": (48, 24), "l1.mix.dq": (20, 48), "l1.mix.dq.norm": (20,),
            "l1.mix.uq": (36, 20), "l1.mix.dkv": (28, 48), "l1.mix.dkv.norm": (24,), "l1.mix.uk": (24, 24),
            "l1.mix.uv": (30, 24), "l1.mix.g": (3, 48), "l1.mix.o": (48, 30), "l1.mlp.gate": (56, 48),
            "l1.mlp.down": (48, 56), "l2.mix.sink": (2,)}
    for name, shape in want.items():
        assert specs[name].shape == shape, name
    assert not any(n.startswith("l2.mlp") for n in specs) and "l0.norm2" not in specs
    assert len(specs) == 5 + (1 + 7 + 1 + 18) + (1 + 9 + 3) + (1 + 7)
    cs = m.cache_specs()
    assert len(cs) == 5                                       # a cache per run: layers 0 and 1 run twice
    assert cs[0].kv == cs[2].kv and cs[0].kv.window == 20 and cs[0].kv.keep_first == 3 and cs[0].kv.v_dim == 12
    assert cs[1].kv.n_kv_heads == 1 and cs[1].kv.head_dim == 24 + 4 and cs[1].kv.v_dim == 0      # one row per token
    assert cs[4].kv.keep_first == 0 and cs[4].kv.window == 40
    assert all(c.state is None for c in cs)


def test_the_cache_keeps_the_pages_of_kept_first_tokens():
    from zinfer_b200.cache import CacheManager, CallCacheSpec
    from zinfer_b200.parts.base import KVRequest
    c = CacheManager([CallCacheSpec(kv=KVRequest(2, 8, 20, keep_first=18)), CallCacheSpec(kv=KVRequest(2, 8, 20))],
                     2, 16 * 16, 400, 16, torch.float32, "cpu")
    kept, plain = c.groups
    assert kept.kept_pages == 2 and plain.kept_pages == 0
    s = c.alloc_slots(1)[0]
    c.reserve([s], [100])
    c.advance([s], [100])
    first = [int(p) for p in kept.table_host[s, :2]]
    assert all(p >= 0 for p in first)
    assert [int(p) for p in kept.table_host[s, 2:5]] == [-1, -1, -1] and kept.table_host[s, 5] >= 0    # 81.. is seen
    assert [int(p) for p in plain.table_host[s, :5]] == [-1] * 5
    for _ in range(150):                                       # single tokens: pages go round, the first two stay
        c.reserve([s], [1])
        c.advance([s], [1])
    assert [int(p) for p in kept.table_host[s, :2]] == first
    assert len(kept.pages_held(s)) == 2 + 2 and len(plain.pages_held(s)) == 2
    c.check_consistency()
    c.free_slots([s])
    c.check_consistency()
    assert c.free_page_count() == [16, 16]
    s2 = c.alloc_slots(1)[0]                                   # a short sequence never reaches the kept pages' end
    c.reserve([s2], [5])
    c.advance([s2], [5])
    c.free_slots([s2])
    c.check_consistency()


def test_rows_of_routed_experts():
    from zinfer_b200.parts.moe import expert_rows
    chosen = np.array([2, 0, 1, 2, 2, 1, 0, 2])                # 4 tokens, 2 experts each
    row_token, pair_row, bounds = expert_rows(chosen, 4, 2, tile=4)
    assert bounds.tolist() == [0, 4, 8, 12, 12]                # expert 3 has no rows, the others one tile each
    assert row_token.tolist() == [0, 3, -1, -1, 1, 2, -1, -1, 0, 1, 2, 3]
    for pair, e in enumerate(chosen):
        r = pair_row[pair]
        assert bounds[e] <= r < bounds[e + 1] and row_token[r] == pair // 2


def test_plain_window_keeps_the_first_tokens():
    assert [j for j in range(12) if P.visible(11, j, 4, 2)] == [0, 1, 8, 9, 10, 11]
    assert [j for j in range(12) if P.visible(3, j, 4, 2)] == [0, 1, 2, 3]
    assert [j for j in range(12) if P.visible(5, j, 0, 0)] == [0, 1, 2, 3, 4, 5]
    assert [j for j in range(6) if P.visible(5, j, 2, 9)] == [0, 1, 2, 3, 4, 5]


def test_plain_sink_only_enlarges_the_denominator():
    sc = [0.3, -1.0, 2.0]
    w0, w1 = P.softmax_rows(sc), P.softmax_rows(sc, sink=1.5)
    z0 = sum(np.exp(sc))
    assert np.allclose(w0, np.exp(sc) / z0) and np.allclose(w1, np.exp(sc) / (z0 + np.exp(1.5)))
    assert abs(sum(w1) - z0 / (z0 + np.exp(1.5))) < 1e-12
    assert np.allclose(P.softmax_rows([0.0], sink=800.0), [0.0]) and np.allclose(P.softmax_rows([800.0], sink=0.0), [1.0])


def test_plain_rotation_pairs_the_halves_and_leaves_the_rest():
    v = np.arange(1.0, 9.0)
    r = P.rotate_half(v, 3, 100.0, 4)
    assert np.array_equal(r[4:], v[4:])
    for i in range(2):
        a = 3 * 100.0 ** (-2.0 * i / 4)
        assert np.isclose(r[i], v[i] * np.cos(a) - v[i + 2] * np.sin(a)) and np.isclose(r[i + 2], v[i + 2] * np.cos(a) + v[i] * np.sin(a))
    assert np.array_equal(P.rotate_half(v, 0, 100.0, 8), v)
    q, k = np.random.default_rng(0).normal(size=(2, 6))          # a score depends on the distance alone
    s1 = P.rotate_half(q, 9, 50.0, 6) @ P.rotate_half(k, 4, 50.0, 6)
    s2 = P.rotate_half(q, 105, 50.0, 6) @ P.rotate_half(k, 100, 50.0, 6)
    assert np.isclose(s1, s2)


def test_plain_latent_attention_equals_attention_over_the_latents():
    """The form a cache of latents allows (queries carried into the latent's space, weights applied to the latents,
    values expanded afterwards) gives what the plain function computes with expanded keys and values."""
    rng = np.random.default_rng(5)
    D, H, d, p, e, r, s, n = 20, 3, 4, 2, 5, 6, 7, 9
    m = {"heads": H, "dim": d, "rot_dim": p, "vdim": e, "kv_rank": r, "q_rank": s, "scale": 0.3, "rot": {"base": 30.0, "dims": p}}
    W = {"dq": rng.normal(size=(s, D)), "dq.norm": rng.normal(1, 0.1, s), "uq": rng.normal(size=(H * (d + p), s)) * 0.4,
         "dkv": rng.normal(size=(r + p, D)) * 0.3, "dkv.norm": rng.normal(1, 0.1, r), "uk": rng.normal(size=(H * d, r)) * 0.4,
         "uv": rng.normal(size=(H * e, r)), "g": rng.normal(size=(H, D)) * 0.2, "o": rng.normal(size=(D, H * e))}
    h = rng.normal(size=(n, D))
    ref = P.latent_attention(h, W, m, 1e-5)
    cq = P.rmsnorm(h @ W["dq"].T, W["dq.norm"], 1e-5)
    q = (cq @ W["uq"].T).reshape(n, H, d + p)
    dkv = h @ W["dkv"].T
    rows = np.concatenate([P.rmsnorm(dkv[:, :r], W["dkv.norm"], 1e-5),
                           np.stack([P.rotate_half(dkv[t, r:], t, 30.0, p) for t in range(n)])], axis=1)
    out = np.zeros((n, H, e))
    for t in range(n):
        for a in range(H):
            qa = np.concatenate([W["uk"][a * d:(a + 1) * d].T @ q[t, a, :d], P.rotate_half(q[t, a, d:], t, 30.0, p)])
            w = P.softmax_rows([float(qa @ rows[j]) * 0.3 for j in range(t + 1)])
            lat = sum(wj * rows[j, :r] for j, wj in enumerate(w))
            out[t, a] = P.sigmoid(W["g"][a] @ h[t]) * (W["uv"][a * e:(a + 1) * e] @ lat)
    assert np.allclose(out.reshape(n, -1) @ W["o"].T, ref, atol=1e-10)


def test_plain_experts_and_gated_unit():
    rng = np.random.default_rng(1)
    h = rng.normal(size=(5, 8))
    W = {"router": rng.normal(size=(3, 8)), **{f"e{i}.{n}": rng.normal(size=s) for i in range(3)
                                              for n, s in (("gate", (4, 8)), ("up", (4, 8)), ("down", (8, 4)))}}
    one = P.routed_experts(h, W, 3, 1)
    for t in range(5):
        e = int(np.argmax(W["router"] @ h[t]))
        g, u = W[f"e{e}.gate"] @ h[t], W[f"e{e}.up"] @ h[t]
        assert np.allclose(one[t], W[f"e{e}.down"] @ (g / (1 + np.exp(-g)) * u))       # one expert: weight 1
    margins = [np.inf] * 5
    P.routed_experts(h, W, 3, 2, margins)
    assert all(0 <= m < np.inf for m in margins)
    Wd = {"gate": np.eye(3) * 10, "up": np.eye(3) * 10, "down": np.eye(3)}
    y = P.clamped_glu(np.array([[1.0, -1.0, 0.01]]), Wd, 2.0)[0]
    assert np.isclose(y[0], 2.0 * P.sigmoid(1.702 * 2.0) * 3.0)                         # both capped at the limit
    assert np.isclose(y[1], -10.0 * P.sigmoid(-17.02) * (-2.0 + 1.0))                   # gate not capped from below
    assert np.isclose(y[2], 0.1 * P.sigmoid(0.1702) * 1.1)


def test_random_model_folder_loads_by_name(tmp_path):
    import zinfer_b200 as z
    from zinfer_b200.weights.safetensors_io import SafetensorsFile
    cfg = z.config_from_dict(H.CONFIGS["ke"])
    folder = z.write_random_model(tmp_path / "ke", cfg, seed=3)
    with SafetensorsFile(folder / "model.safetensors") as f:
        names = set(f.names())
    from zinfer_b200.config.registry import build_model
    assert names == set(build_model(cfg).weight_specs())
    assert z.config_from_folder(folder).to_json_dict() == H.CONFIGS["ke"]
