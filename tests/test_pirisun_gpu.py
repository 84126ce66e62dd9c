"""Pirisun models through the engine, against the plain implementation: whole prompts, prompt then single tokens,
portions of several sizes, batches of unequal requests, slots, pages and states used again, long decoding over page
borders and temperature periods, the engine's own chunking, greedy generation through `Engine.generate` (recorded
single-token steps), the command line and the replay program.

In bfloat16 a token whose expert choice is a close call may take another expert than the plain implementation; the
comparison then covers the positions before the first such token (`H.plain_logits` says how many), in 32-bit all.
Two configurations choose every router output or have no experts: they compare everywhere in bfloat16 too."""
import dataclasses
import json
import subprocess
import sys

import numpy as np
import pytest

import pirisun_helpers as H

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
PAGE = {"pc": 64, "pf": 64, "pe": 64}      # "pe": heads of 10 / 7 values, padded up to the tensor-core kernels' 64 in bfloat16


@pytest.fixture(scope="module")
def zoo(tmp_path_factory):
    """name -> (config dict, weights, folder)."""
    root = tmp_path_factory.mktemp("pirisun_models")
    out = {}
    for i, (name, cfg) in enumerate(H.CONFIGS.items()):
        W = H.make_weights(cfg, 700 + i)
        out[name] = (cfg, W, H.write_folder(root / name, cfg, W))
    return out


_plain_cache = {}


def plain(zoo, name, tokens):
    key = (name, tuple(tokens))
    if key not in _plain_cache:
        cfg, W, _ = zoo[name]
        _plain_cache[key] = H.plain_logits(cfg, W, tokens)
    return _plain_cache[key]


def engine_for(zoo, name, dtype, **kw):
    import zinfer_b200 as z
    model = z.load(zoo[name][2], dtype=dtype)
    kw.setdefault("max_batch", 4)
    kw.setdefault("max_seq_len", 320)
    kw.setdefault("page_size", PAGE.get(name, 16))
    return z.Engine(model, **kw)


def feed(engine, slot, tokens, cuts):
    """Feeds `tokens` to one sequence in portions of the sizes `cuts` (the rest one by one); logits of every position."""
    rows, at = [], 0
    sizes = list(cuts)
    while at < len(tokens):
        n = sizes.pop(0) if sizes else 1
        part = tokens[at:at + n]
        rows.append(engine.step([slot], [part], [list(range(len(part)))]).cpu().numpy())
        at += len(part)
    return np.concatenate(rows)


def check(got, ref_safe, dtype, what, least=1):
    """Compares with the plain logits: all positions in 32-bit, in bfloat16 those before the first close call."""
    ref, safe = ref_safe
    n = len(ref) if dtype == "float32" else safe
    if n < least:
        return 0
    e = H.rel_err(got[:n], ref[:n])
    assert e <= H.TOL[dtype], f"{what}: error {e:.3e} over {n} positions (tolerance {H.TOL[dtype]:.0e})"
    return n


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(H.CONFIGS))
def test_whole_prompts(zoo, name, dtype):
    """Every position of prompts of 1, 2, 3 and many tokens, each prompt alone in one step: the first tokens of a
    sequence, keys in other pages, positions on both sides of a temperature step."""
    cfg = zoo[name][0]
    eng = engine_for(zoo, name, dtype)
    for n in (1, 2, 3, 19, 130):
        toks = H.tokens_for(cfg, n, n)
        s = eng.start(1)
        got = feed(eng, s[0], toks, [n])
        eng.finish(s)
        check(got, plain(zoo, name, toks), dtype, f"{name} prompt of {n}")
    eng.cache.check_consistency()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,cuts", [("pa", [30]), ("pb", [1]), ("pc", [100]), ("pe", [2]), ("pa", [2, 2, 5, 1, 17, 3, 2, 16, 16]),
                                       ("pb", [64, 2, 30, 2]), ("pc", [3, 61, 64, 2, 70]), ("pd", [5, 2]), ("pe", [7, 2, 40]),
                                       ("pf", [64, 2, 62, 3]), ("pf", [1])])
def test_portions_and_single_tokens_give_what_the_whole_prompt_gives(zoo, name, dtype, cuts):
    """A sequence fed in portions (down to two tokens, across page borders) and then token by token: keys, latents and
    the recurrence's state must pass from step to step as if the sequence were whole."""
    cfg = zoo[name][0]
    n = sum(cuts) + (110 if name in PAGE else 75)
    toks = H.tokens_for(cfg, 7 + len(cuts), n)
    eng = engine_for(zoo, name, dtype)
    s = eng.start(1)
    got = feed(eng, s[0], toks, cuts)
    eng.finish(s)
    check(got, plain(zoo, name, toks), dtype, f"{name} cut {cuts}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["pa", "pb", "pc", "pe", "pf"])
def test_unequal_requests_together_and_slots_used_again(zoo, name, dtype):
    """Requests of unequal length in one batch, decoded together while the shorter ones leave; then new requests in
    the slots, pages and states the first ones gave back, with a cache so small that pages must be reused: a state that
    is not zeroed when its slot is handed out again would show in the second round."""
    cfg = zoo[name][0]
    eng = engine_for(zoo, name, dtype, max_batch=3, max_seq_len=192 if name in PAGE else 160, max_tokens=3 * (192 if name in PAGE else 128))
    for round_ in range(2):
        lens = [(1, 9), (40, 61), (23, 95)] if round_ == 0 else [(33, 80), (2, 4), (64, 90)]
        toks = [H.tokens_for(cfg, 50 + 10 * round_ + b, total) for b, (_, total) in enumerate(lens)]
        slots = eng.start(3)
        got = [[] for _ in lens]
        out = eng.step(slots, [t[:p] for t, (p, _) in zip(toks, lens)], [list(range(p)) for p, _ in lens]).cpu().numpy()
        at = 0
        for b, (p, _) in enumerate(lens):
            got[b].append(out[at:at + p])
            at += p
        pos = [p for p, _ in lens]
        live = list(range(3))
        while live:
            out = eng.step([slots[b] for b in live], [[toks[b][pos[b]]] for b in live]).cpu().numpy()
            for i, b in enumerate(live):
                got[b].append(out[i:i + 1])
                pos[b] += 1
            ended = [b for b in live if pos[b] == lens[b][1]]
            if ended:
                eng.finish([slots[b] for b in ended])
                live = [b for b in live if b not in ended]
        for b in range(3):
            check(np.concatenate(got[b]), plain(zoo, name, toks[b]), dtype, f"{name} round {round_} request {b}")
        eng.cache.check_consistency()
    assert eng.cache.free_slot_count() == 3 and all(n == eng.cache.num_pages for n in eng.cache.free_page_count())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["pb", "pd", "pe"])
def test_long_decoding(zoo, name, dtype):
    """300 tokens, all but five of them one at a time, over many page borders and temperature periods; the
    recurrence's state is carried through 295 single-token steps."""
    cfg = zoo[name][0]
    toks = H.tokens_for(cfg, 3, 300)
    eng = engine_for(zoo, name, dtype, max_batch=1)
    s = eng.start(1)
    got = feed(eng, s[0], toks, [5])
    eng.finish(s)
    check(got, plain(zoo, name, toks), dtype, "300 tokens one by one")
    eng.cache.check_consistency()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["pc", "pf"])
def test_the_engines_own_chunking(zoo, name, dtype):
    """A prompt step larger than max_step_tokens runs as packed chunks; so does a batch of them."""
    cfg = zoo[name][0]
    eng = engine_for(zoo, name, dtype, max_step_tokens=48)
    toks = [H.tokens_for(cfg, 70 + b, n) for b, n in enumerate((130, 50, 7))]
    slots = eng.start(3)
    out = eng.step(slots, toks, [list(range(len(t))) for t in toks]).cpu().numpy()
    eng.finish(slots)
    at = 0
    for b, t in enumerate(toks):
        check(out[at:at + len(t)], plain(zoo, name, t), dtype, f"chunked request {b}")
        at += len(t)


def test_bfloat16_comparisons_cover_positions(zoo):
    """The close-call rule must not hollow the bfloat16 tests out: the configurations without a choice to make are
    compared everywhere."""
    for name in ("pb", "pd", "pf"):
        assert plain(zoo, name, H.tokens_for(zoo[name][0], 130, 130))[1] == 130


@pytest.mark.parametrize("name", ["pa", "pc", "pe", "pf"])
def test_greedy_generation_through_the_engines_own_loop(zoo, name):
    """`Engine.generate` (scheduler, recorded single-token steps, device arg-max) against the plain implementation's
    greedy choice, in 32-bit so that no near-tie decides; batches of unequal prompts."""
    cfg = zoo[name][0]
    eng = engine_for(zoo, name, "float32", max_batch=2)
    assert eng.use_graphs, "every mixer of the model must be recordable"
    prompts = [H.tokens_for(cfg, 90 + b, n) for b, n in enumerate((5, 17, 1))]
    results = eng.generate(prompts, max_new_tokens=10, temperature=0.0, stop_ids=[])
    for p, r in zip(prompts, results):
        seq = list(p)
        for _ in range(10):
            lg = plain(zoo, name, seq)[0][-1]
            top2 = np.sort(lg)[-2:]
            if top2[1] - top2[0] < 1e-3 * np.abs(lg).max():
                break                     # a near-tie: both choices are right, stop comparing this request
            seq.append(int(np.argmax(lg)))
        n = len(seq) - len(p)
        assert r.tokens[:n] == seq[len(p):], (name, r.tokens, seq[len(p):])
        assert len(r.tokens) == 10 and r.finish_reason == "length"


@pytest.mark.parametrize("name", ["pb", "pf"])
def test_recorded_single_token_steps_equal_unrecorded_ones(zoo, name):
    """`Engine.decode` replays a CUDA graph from its second call on: the logits must be those of `step`; the
    recurrence's state and the positions behind the rotation and the temperature move on under the recording."""
    cfg = zoo[name][0]
    toks = [H.tokens_for(cfg, 120 + b, 30) for b in range(2)]
    outs = []
    for graphs in (True, False):
        eng = engine_for(zoo, name, "bfloat16", max_batch=2, use_graphs=graphs)
        slots = eng.start(2)
        eng.step(slots, [t[:6] for t in toks])
        rows = []
        for i in range(6, 30):
            rows.append(eng.decode(slots, [t[i] for t in toks]).clone().cpu().numpy())
        eng.check_status()
        eng.finish(slots)
        outs.append(np.stack(rows))
    assert np.array_equal(outs[0], outs[1])
    ref, safe = plain(zoo, name, toks[0])
    check(outs[0][:, 0], (ref[6:], safe - 6), "bfloat16", "recorded steps")


def test_command_line_and_replay_program(zoo, tmp_path):
    """The architecture is found by config.json's name; the command line generates and the replay program writes the
    logits of the wanted places."""
    name = "pe"
    cfg, W, folder = zoo[name]
    from helpers import ROOT
    r = subprocess.run([sys.executable, "-m", "zinfer_b200", "-m", str(folder), "-p", "3,9,27", "-n", "5", "--temp", "0",
                        "--dtype", "fp32", "--stop", ""], capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
    seq = [3, 9, 27]
    for _ in range(5):
        seq.append(int(np.argmax(plain(zoo, name, seq)[0][-1])))
    assert r.stdout.split("[")[0].split() == [str(t) for t in seq[3:]], r.stdout
    toks = H.tokens_for(cfg, 5, 20)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[:12], "want": [0, 11]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": toks[12:14], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": toks[14:], "want": [5]}], "end": ["a"]}]
    out = tmp_path / "out"
    r = subprocess.run([str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "64"], input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True,
                       text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    ref = plain(zoo, name, toks)[0]
    got0 = np.fromfile(out / "0.f32", dtype="<f4").reshape(2, -1)
    got2 = np.fromfile(out / "2.f32", dtype="<f4").reshape(1, -1)
    assert not (out / "1.f32").exists()
    assert H.rel_err(np.concatenate([got0, got2]), ref[[0, 11, 19]]) <= H.TOL["float32"]


def test_config_of_a_folder_round_trips(zoo):
    import zinfer_b200 as z
    for name, (cfg, _, folder) in zoo.items():
        c = z.config_from_folder(folder)
        again = z.config_from_dict(c.to_json_dict())
        assert c.architecture == "Pirisun" and dataclasses.replace(again, raw={}) == dataclasses.replace(c, raw={}), name
