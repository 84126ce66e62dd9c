"""The mechanisms the Kerotar design brought, each alone against its plain function: the gated unit with clamps and the
gate per head, the router and the routed experts both ways they run, the map of rows and embedding rows at the start
of a pass, the parallel block, windowed attention with kept first tokens and a sink (inputs made so that ONE marked key
decides the last query: the first token, the last kept token and the one behind it, both sides of the window's edge
and of page borders, in prompt steps and in single-token steps), and attention through a latent (with scores so sharp
that every query hangs on one or two keys somewhere in the sequence)."""
import numpy as np
import pytest
import torch

import plain_kerotar as P
from test_parts_gpu import Bench, close, load, rnd, run_mixer

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def k():
    from zinfer_b200 import kernels
    kernels.require_cuda()
    return kernels


def f64(t):
    return t.numpy().astype(np.float64)


class Ctx:
    """The little of a step context that a feed-forward reads."""

    def __init__(self, k, dtype, n, decode=False):
        self.dtype, self.device, self.status = dtype, torch.device("cuda"), k.status_word(torch.device("cuda"))
        self.n_tokens, self.is_decode, self._memo = n, decode, {}

    def memo(self, key, make):
        if key not in self._memo:
            self._memo[key] = make()
        return self._memo[key]


# ------------------------------------------------------------------------------- row kernels

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("F,il", [(50, 0), (96, 16), (320, 16)])
def test_clamped_gated_unit_and_head_gate(k, dtype, F, il):
    from zinfer_b200.parts.linear import interleave_rows
    g, u = rnd((9, F), 1, dtype, 2.0), rnd((9, F), 2, dtype, 2.0)
    gu = torch.cat([g, u], dim=1) if not il else interleave_rows([g.T.contiguous(), u.T.contiguous()], il).T.contiguous()
    for limit, alpha in ((1.5, 1.702), (0.25, 1.0)):
        gg, uu = np.minimum(f64(g), limit), np.clip(f64(u), -limit, limit)
        close(k.clamped_glu(gu.to(dtype).cuda(), limit, alpha, il), gg * P.sigmoid(alpha * gg) * (uu + 1), dtype, "gated unit")
    H, w = 5, F // 5 if F % 5 == 0 else 7
    rows, gate = rnd((9, H * w), 3, dtype), rnd((9, H + 3), 4, torch.float32, 2.0)
    ref = (f64(rows).reshape(9, H, w) * P.sigmoid(f64(gate)[:, 1:1 + H, None])).reshape(9, -1)
    close(k.head_gate(rows.to(dtype).cuda(), gate.cuda()[:, 1:1 + H], H), ref, dtype, "gate per head")


# ------------------------------------------------------------------------------- feed-forwards

def expert_tensors(D, F, E, dtype, seed):
    t = {"router": rnd((E, D), seed, torch.bfloat16, 2.0 * D ** -0.5)}
    for e in range(E):
        t[f"e{e}.gate"], t[f"e{e}.up"] = rnd((F, D), seed + 3 * e + 1, dtype, D ** -0.5), rnd((F, D), seed + 3 * e + 2, dtype, D ** -0.5)
        t[f"e{e}.down"] = rnd((D, F), seed + 3 * e + 3, dtype, F ** -0.5)
    return t


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D,F,E,top,rows", [(48, 24, 6, 2, 7), (64, 16, 4, 4, 33), (128, 64, 8, 2, 300), (128, 128, 3, 1, 200),
                                            (38, 10, 5, 3, 130), (256, 96, 16, 2, 1), (128, 64, 8, 2, 700), (38, 10, 5, 2, 515)])
def test_router_and_routed_experts_both_ways(k, dtype, D, F, E, top, rows):
    """The streaming kernels (few rows, single-token steps) and the grouped contractions (many rows), against the plain
    function; the router's ids and weights against the plain choice; rows alone against rows in a batch.  Rows whose
    choice is a close call are left out of the bfloat16 comparison (they are independent of one another here)."""
    from zinfer_b200.parts import RoutedMoE
    t = expert_tensors(D, F, E, dtype, 20)
    ff = load(RoutedMoE(D, F, E, top, "router", lambda e: (f"e{e}.gate", f"e{e}.up", f"e{e}.down")), t, dtype)
    x = rnd((rows, D), 5, dtype)
    W = {n: f64(a) for n, a in t.items()}
    margins = [np.inf] * rows
    ref = P.routed_experts(f64(x), W, E, top, margins)
    keep = np.array([m > (0.03 if dtype == torch.bfloat16 else 1e-5) for m in margins])
    assert keep.sum() >= max(1, rows // 2)
    ids, wts = k.moe_router(x.to(dtype).cuda(), ff.w_router, top)
    z = f64(x) @ W["router"].T
    s = np.exp(z - z.max(1, keepdims=True))
    s /= s.sum(1, keepdims=True)
    order = np.argsort(-s, axis=1, kind="stable")[:, :top]
    assert np.array_equal(ids.cpu().numpy()[keep], order[keep])
    chosen = np.take_along_axis(s, order, 1)
    close(wts[torch.from_numpy(keep).cuda()], (chosen / chosen.sum(1, keepdims=True))[keep], dtype, "router weights")
    outs = {}
    for decode in (False, True):
        out = torch.full((rows, D), 0.5, device="cuda")
        ff.forward(Ctx(k, dtype, rows, decode), x.to(dtype).cuda(), out, True)
        outs[decode] = out - 0.5
        close(outs[decode][torch.from_numpy(keep).cuda()], ref[keep], dtype, "decode" if decode else "prompt")
    i = int(np.flatnonzero(keep)[-1])
    ids1, wts1 = k.moe_router(x[i:i + 1].to(dtype).cuda(), ff.w_router, top)     # a row's choice is the same bits alone
    assert torch.equal(ids1[0], ids[i]) and torch.equal(wts1[0], wts[i])
    alone = torch.zeros((1, D), device="cuda")
    ff.forward(Ctx(k, dtype, 1, True), x[i:i + 1].to(dtype).cuda(), alone, False)
    assert torch.equal(alone[0], (outs[True][i] + 0.5) - 0.5) or torch.allclose(alone[0], outs[True][i], atol=1e-6)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D,F,rows,limit", [(48, 56, 5, 2.0), (128, 256, 40, 1.0), (38, 50, 130, 0.75), (256, 320, 1, 1.5),
                                            (128, 256, 300, 1.0), (64, 48, 200, 0.5), (128, 384, 20, 0.8)])
def test_clamped_glu_part(k, dtype, D, F, rows, limit):
    from zinfer_b200.parts import ClampedGLU
    t = {"gate": rnd((F, D), 1, dtype, 2 * D ** -0.5), "up": rnd((F, D), 2, dtype, 2 * D ** -0.5), "down": rnd((D, F), 3, dtype, F ** -0.5)}
    ff = load(ClampedGLU(D, F, "gate", "up", "down", limit), t, dtype)
    x = rnd((rows, D), 4, dtype)
    out = torch.full((rows, D), 0.25, device="cuda")
    ff.forward(Ctx(k, dtype, rows), x.to(dtype).cuda(), out, True)
    close(out - 0.25, P.clamped_glu(f64(x), {n: f64(a) for n, a in t.items()}, limit), dtype, "clamped GLU")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D,rows", [(48, 1), (64, 23), (38, 5), (128, 200)])
def test_pass_input_maps_rows_and_embedding_rows(k, dtype, D, rows):
    from zinfer_b200.parts import PassInput
    t = {"in": rnd((D, 2 * D), 1, dtype, (2 * D) ** -0.5), "step": rnd((3, D), 2, dtype, 0.5)}
    part = load(PassInput("step", 3, D, {0: 0, 4: 1, 7: 2}, in_name="in"), t, dtype)
    assert part.needs_embedding and part.starts_at(4) and not part.starts_at(5)
    x, x0 = rnd((rows, D), 3, torch.float32), rnd((rows, D), 4, torch.float32)
    ctx = Ctx(k, dtype, rows)
    rd = (lambda a: a.to(dtype).float()) if dtype == torch.bfloat16 else (lambda a: a)
    for call, tt in ((0, 0), (4, 1), (7, 2), (5, None)):
        xd = x.clone().cuda()
        part.before(ctx, call, xd, x0.cuda())
        ref = f64(x) if tt is None else np.concatenate([f64(rd(x)), f64(rd(x0))], 1) @ f64(t["in"]).T + f64(t["step"])[tt]
        close(xd, ref, dtype, f"before call {call}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows", [1, 23, 130])
def test_parallel_block_feeds_both_sublayers_the_rows_as_they_were(k, dtype, rows):
    """Both sublayers read the norm of the rows as they were BEFORE the mixer summed into them, whichever contraction
    kernel the row count selects (some apply the norm themselves, when they run)."""
    from zinfer_b200.parts import ClampedGLU, GqaAttention, ParallelBlock, RMSNorm
    D, H, d, F, eps = 64, 4, 16, 96, 1e-5
    t = {"norm": 1.0 + rnd((D,), 1, dtype, 0.2), "q": rnd((H * d, D), 2, dtype, D ** -0.5), "k": rnd((H * d, D), 3, dtype, D ** -0.5),
         "v": rnd((H * d, D), 4, dtype, D ** -0.5), "o": rnd((D, H * d), 5, dtype, (H * d) ** -0.5), "qn": 1.0 + rnd((H * d,), 6, dtype, 0.1),
         "kn": 1.0 + rnd((H * d,), 7, dtype, 0.1), "sink": rnd((H,), 8, dtype), "gate": rnd((F, D), 9, dtype, D ** -0.5),
         "up": rnd((F, D), 10, dtype, D ** -0.5), "down": rnd((D, F), 11, dtype, F ** -0.5)}
    mixer = GqaAttention(D, H, H, d, "q", "k", "v", "o", "qn", "kn", eps, None, window=8, scale=0.25, qk_norm_span="all",
                         keep_first=2, sink_name="sink")
    block = load(ParallelBlock(RMSNorm(D, eps, "norm"), mixer, ClampedGLU(D, F, "gate", "up", "down", 1.0)), t, dtype)
    bench = Bench(k, mixer, dtype, n_slots=max(2, rows), max_seq=16)
    x = rnd((rows, D), 12, torch.float32, 3.0)
    W = {n: f64(a) for n, a in t.items()}
    h = P.rmsnorm(f64(x), W["norm"], eps)
    m = {"heads": H, "kv_heads": H, "dim": d, "vdim": d, "scale": 0.25, "mask": {"size": 8, "keep_first": 2}}
    Wm = {"q": W["q"], "k": W["k"], "v": W["v"], "o": W["o"], "q.norm": W["qn"], "k.norm": W["kn"], "sink": W["sink"]}
    ref = f64(x) + np.concatenate([P.window_attention(h[i:i + 1], Wm, m, eps) for i in range(rows)]) \
        + P.clamped_glu(h, {"gate": W["gate"], "up": W["up"], "down": W["down"]}, 1.0)
    slots = bench.cache.alloc_slots(rows)                       # every row a sequence of its own: one token each
    ctx = bench.step(slots, [1] * rows)
    xd = x.clone().cuda()
    block.forward(ctx, bench.call, xd)
    bench.done(slots, [1] * rows)
    close(xd, ref, dtype, f"{rows} rows")


# ------------------------------------------------------------------------------- windowed attention

def window_tensors(D, H, G, d, vd, dtype, seed, split=False):
    t = {"q": rnd((H * d, D), seed, dtype, D ** -0.5), "k": rnd((G * d, D), seed + 1, dtype, D ** -0.5),
         "v": rnd((G * vd, D), seed + 2, dtype, D ** -0.5), "o": rnd((D, H * vd), seed + 3, dtype, (H * vd) ** -0.5),
         "qn": 1.0 + rnd((H * d,), seed + 4, dtype, 0.2), "kn": 1.0 + rnd((G * d,), seed + 5, dtype, 0.2),
         "sink": rnd((H,), seed + 6, dtype, 1.5)}
    if split:       # q and k read the first half of the input only, v the second half only
        t["q"][:, D // 2:] = 0
        t["k"][:, D // 2:] = 0
        t["v"][:, :D // 2] = 0
    return t


def make_window_attention(D, H, G, d, vd, scale, rot, mask, t, dtype, eps=2e-6):
    from zinfer_b200.parts import GqaAttention, RotaryEncoding
    pos = RotaryEncoding(d, rot[0], n_rot=rot[1]) if rot else None
    return load(GqaAttention(D, H, G, d, "q", "k", "v", "o", "qn", "kn", eps, pos, window=mask[0] if mask else 0, scale=scale,
                             value_dim=vd, qk_norm_span="all", keep_first=mask[1] if mask else 0, sink_name="sink"), t, dtype)


def plain_window(x, t, H, G, d, vd, scale, rot, mask, eps=2e-6):
    m = {"heads": H, "kv_heads": G, "dim": d, "vdim": vd, "scale": scale}
    if rot:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    if mask:
        m["mask"] = {"size": mask[0], "keep_first": mask[1]}
    p = {"q": t["q"], "k": t["k"], "v": t["v"], "o": t["o"], "q.norm": t["qn"], "k.norm": t["kn"], "sink": t["sink"]}
    return P.window_attention(f64(x), {n: f64(a) for n, a in p.items()}, m, eps)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D,H,G,d,vd,scale,rot,mask,page", [
    (40, 4, 2, 16, 12, 0.3, (100.0, 8), (20, 3), 16),          # window over a page border, three kept tokens
    (64, 6, 6, 8, 16, 0.35, (30.0, 4), (7, 20), 16),           # more kept tokens than the window is long, in two pages
    (128, 8, 2, 64, 64, 0.12, (300000.0, 32), (112, 5), 64),   # head widths the tensor cores take
    (128, 4, 4, 64, 64, 0.11, (500.0, 64), None, 64),          # no window at all: the sink alone
    (38, 5, 5, 10, 7, 0.3, (20.0, 6), (33, 1), 16),            # odd sizes, one kept token
    (64, 2, 1, 32, 32, 0.2, None, (40, 0), 32),                # a window without kept tokens and without rotation
    (96, 3, 1, 128, 48, 0.09, (10000.0, 128), (16, 16), 16),   # the window as long as a page, a page of kept tokens
])
def test_windowed_attention_alone(k, dtype, D, H, G, d, vd, scale, rot, mask, page):
    t = window_tensors(D, H, G, d, vd, dtype, 70)
    mixer = make_window_attention(D, H, G, d, vd, scale, rot, mask, t, dtype)
    req = mixer.kv_request()
    assert (req.n_kv_heads, req.head_dim, req.v_dim, req.keep_first) == (G, d, vd, mask[1] if mask else 0)
    xs = [rnd((n, D), 80 + n, dtype) for n in (150, 37, 45)]
    outs = run_mixer(k, mixer, dtype, xs, [100, 17, 1], page=page)
    for b, x in enumerate(xs):
        close(outs[b], plain_window(x, t, H, G, d, vd, scale, rot, mask), dtype, f"sequence {b}")


T_MARK, WINDOW, KEEP = 200, 50, 18


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,d,page", [(4, 2, 16, 16), (4, 2, 64, 64)])
@pytest.mark.parametrize("mark,seen", [(0, True), (15, True), (16, True), (KEEP - 1, True), (KEEP, False), (63, False), (64, False),
                                       (T_MARK - 1 - WINDOW, False), (T_MARK - WINDOW, True), (T_MARK - WINDOW + 1, True),
                                       (159, True), (160, True), (T_MARK - 2, True)])
def test_one_marked_key_decides_or_is_out_of_sight(k, dtype, H, G, d, page, mark, seen):
    """The last token's query is made to match the key of token `mark` alone (same first half of the input, a sharp
    scale), while the values come from the second half.  A marked key in sight decides the output; one out of sight
    (behind the kept tokens, before the window) must not move it at all.  The last token comes in a prompt step, and
    then as a single token behind a prompt."""
    marked_key(k, dtype, H, G, d, page, mark, seen, T_MARK, WINDOW, KEEP, (T_MARK, T_MARK - 1, 150))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("mark,seen", [(0, True), (63, True), (64, True), (69, True), (70, False), (128, False), (519, False),
                                       (520, True), (575, True), (576, True)])
def test_kept_keys_over_a_tile_border_far_behind_the_window(k, dtype, mark, seen):
    """600 tokens, a window of 80 and 70 kept tokens (more than a key tile of 64), pages of 64: the kept keys and the
    window lie in different pages, tiles and chunks of the keys, in a prompt step and in single-token steps."""
    marked_key(k, dtype, 4, 2, 64, 64, mark, seen, 600, 80, 70, (600, 599, 560))


def marked_key(k, dtype, H, G, d, page, mark, seen, T_MARK, WINDOW, KEEP, prompts):
    D, vd, T = 2 * d, d, T_MARK
    t = window_tensors(D, H, G, d, vd, dtype, 90, split=True)
    t["q"] = t["k"].reshape(G, 1, d, D).expand(G, H // G, d, D).reshape(H * d, D).clone()
    t["qn"] = t["kn"].reshape(G, 1, d).expand(G, H // G, d).reshape(H * d).clone()
    t["sink"] = torch.full((H,), -2.0)
    scale = 6.0 / d ** 0.5 * (H / G) ** 0.5          # the q norm runs over H*d entries, the k norm over G*d
    mask = (WINDOW, KEEP)
    mixer = make_window_attention(D, H, G, d, vd, scale, None, mask, t, dtype)
    x = rnd((T, D), 91, dtype)
    x[T - 1, :D // 2] = x[mark, :D // 2]
    ref = plain_window(x, t, H, G, d, vd, scale, None, mask)
    other = x.clone()
    other[mark, D // 2:] = rnd((D // 2,), 92, dtype)            # another value at the marked token
    moved = plain_window(other, t, H, G, d, vd, scale, None, mask)
    if seen:
        assert np.abs(ref[-1] - moved[-1]).max() > 0.1 * np.abs(ref).max(), "the marked key does not decide the last query"
    else:
        assert np.abs(ref[-1] - moved[-1]).max() == 0.0
    for prompt in prompts:
        outs = run_mixer(k, mixer, dtype, [x], [prompt], page=page)
        close(outs[0], ref, dtype, f"prompt of {prompt}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_heavy_sink_takes_the_weight(k, dtype):
    """With a sink far above every score the output all but vanishes; with one far below it is plain softmax."""
    D, H, G, d = 32, 2, 1, 16
    t = window_tensors(D, H, G, d, d, dtype, 40)
    x = rnd((30, D), 41, dtype)
    for sink in (30.0, -30.0):
        t["sink"] = torch.full((H,), sink)
        mixer = make_window_attention(D, H, G, d, d, 0.25, None, (12, 2), t, dtype)
        ref = plain_window(x, t, H, G, d, d, 0.25, None, (12, 2))
        outs = run_mixer(k, mixer, dtype, [x], [20], page=16)
        if sink > 0:
            assert np.abs(ref).max() < 1e-8 and float(outs[0].abs().max()) < 1e-6
        else:
            close(outs[0], ref, dtype, "sink far below")


# ------------------------------------------------------------------------------- attention through a latent

def latent_tensors(D, H, d, p, e, r, s, dtype, seed):
    return {"dq": rnd((s, D), seed, dtype, D ** -0.5), "dqn": 1.0 + rnd((s,), seed + 1, dtype, 0.2),
            "uq": rnd((H * (d + p), s), seed + 2, dtype, s ** -0.5), "dkv": rnd((r + p, D), seed + 3, dtype, D ** -0.5),
            "dkvn": 1.0 + rnd((r,), seed + 4, dtype, 0.2), "uk": rnd((H * d, r), seed + 5, dtype, r ** -0.5),
            "uv": rnd((H * e, r), seed + 6, dtype, r ** -0.5), "g": rnd((H, D), seed + 7, dtype, D ** -0.5),
            "o": rnd((D, H * e), seed + 8, dtype, (H * e) ** -0.5)}


def make_latent(D, H, d, p, e, r, s, scale, base, t, dtype, eps=2e-6):
    from zinfer_b200.parts import LatentAttention
    return load(LatentAttention(D, H, d, p, e, r, s, scale, base, "dq", "dqn", "uq", "dkv", "dkvn", "uk", "uv", "o", gate_name="g",
                                norm_eps=eps), t, dtype)


def plain_latent(x, t, H, d, p, e, r, s, scale, base, eps=2e-6):
    m = {"heads": H, "dim": d, "rot_dim": p, "vdim": e, "kv_rank": r, "q_rank": s, "scale": scale, "rot": {"base": base, "dims": p}}
    W = {"dq": t["dq"], "dq.norm": t["dqn"], "uq": t["uq"], "dkv": t["dkv"], "dkv.norm": t["dkvn"], "uk": t["uk"], "uv": t["uv"],
         "g": t["g"], "o": t["o"]}
    return P.latent_attention(f64(x), {n: f64(a) for n, a in W.items()}, m, eps)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D,H,d,p,e,r,s,scale,base,page", [
    (48, 3, 8, 4, 10, 24, 20, 0.3, 50.0, 16),
    (64, 2, 16, 8, 16, 32, 40, 0.2, 10000.0, 16),
    (128, 4, 32, 32, 64, 64, 64, 0.12, 10000.0, 64),
    (32, 1, 4, 2, 4, 8, 8, 0.4, 20.0, 16),                    # one head
    (38, 3, 6, 6, 5, 18, 14, 0.3, 40.0, 16),                  # odd sizes
    (128, 8, 32, 16, 32, 320, 96, 0.1, 1000.0, 32),           # a latent wider than 256: rows of 336 values
    (64, 2, 16, 8, 16, 32, 40, 2.5, 100.0, 16),               # scores so sharp that one or two far keys decide a query
    (128, 4, 32, 32, 64, 64, 64, 1.5, 10000.0, 64),
    (128, 4, 48, 16, 40, 96, 64, 0.12, 10000.0, 64),          # values narrower than the kernel's value rows
    (128, 2, 64, 32, 64, 160, 64, 0.1, 10000.0, 64),          # keys of 96 entries in rows of 128, values of 64
    (128, 2, 96, 32, 128, 160, 64, 0.09, 10000.0, 128),       # keys and values of 128
    (128, 3, 32, 16, 96, 80, 64, 0.14, 500.0, 64),            # values wider than the keys
    (128, 20, 16, 32, 16, 512, 48, 0.1, 10000.0, 64),         # rows of 544 values, heads in two groups of sixteen
    (64, 17, 16, 16, 32, 272, 32, 0.15, 100.0, 64),           # rows of 288 values, one head beyond the first group
    (96, 3, 20, 12, 28, 40, 36, 0.18, 300.0, 64),             # pages of 64 with widths that are no multiples of 8 or 16
    (80, 5, 10, 6, 70, 24, 30, 0.25, 50.0, 64),               # values of 70 in rows of 128, keys of 16 in rows of 128
])
def test_latent_attention_alone(k, dtype, D, H, d, p, e, r, s, scale, base, page):
    t = latent_tensors(D, H, d, p, e, r, s, dtype, 70)
    mixer = make_latent(D, H, d, p, e, r, s, scale, base, t, dtype)
    req = mixer.kv_request()
    assert (req.n_kv_heads, req.head_dim, req.v_dim, req.window) == (1, r + p, 0, 0)
    xs = [rnd((n, D), 80 + n, dtype) for n in (200, 37, 45)]
    outs = run_mixer(k, mixer, dtype, xs, [130, 17, 1], page=page)
    for b, x in enumerate(xs):
        ref = plain_latent(x, t, H, d, p, e, r, s, scale, base)
        if scale > 1 and dtype == torch.bfloat16:
            continue            # sharp scores amplify the rounding of the scores themselves; the 32-bit run decides
        close(outs[b], ref, dtype, f"sequence {b}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D,H,d,p,e,r,s,page", [(128, 4, 32, 32, 64, 64, 64, 64), (128, 2, 64, 32, 64, 160, 64, 64),
                                                (64, 3, 16, 8, 20, 48, 40, 16), (96, 3, 20, 12, 28, 40, 36, 64)])
def test_latent_attention_in_portions_of_a_prompt(k, dtype, D, H, d, p, e, r, s, page):
    """Two sequences whose prompts come in portions of unequal sizes (a long later portion, which expands the cached
    latents once more; a short one behind a long prefix; portions of two tokens; a portion that ends on a page border)."""
    t = latent_tensors(D, H, d, p, e, r, s, dtype, 170)
    mixer = make_latent(D, H, d, p, e, r, s, 0.12, 10000.0, t, dtype)
    xs = [rnd((192, D), 171, dtype), rnd((150, D), 172, dtype)]
    portions = [[70, 58, 2, 60, 2], [20, 100, 3, 2, 25]]
    bench = Bench(k, mixer, dtype, n_slots=3, max_seq=256, page=page)
    held = bench.cache.alloc_slots(3)
    slots = held[1:]
    outs = [torch.zeros(x.shape[0], D) for x in xs]
    done = [0, 0]
    for step in range(5):
        lens = [portions[b][step] for b in range(2)]
        ctx = bench.step(slots, lens)
        xn = torch.cat([xs[b][done[b]:done[b] + lens[b]] for b in range(2)]).to(dtype).cuda()
        out = torch.full((xn.shape[0], D), 7.0, device="cuda")
        mixer.forward(ctx, bench.call, xn, out, False)
        bench.done(slots, lens)
        o = 0
        for b in range(2):
            outs[b][done[b]:done[b] + lens[b]] = out[o:o + lens[b]].cpu()
            o += lens[b]
            done[b] += lens[b]
    bench.cache.free_slots(held)
    for b, x in enumerate(xs):
        close(outs[b], plain_latent(x, t, H, d, p, e, r, s, 0.12, 10000.0), dtype, f"sequence {b}")
