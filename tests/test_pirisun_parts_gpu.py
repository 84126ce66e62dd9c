"""The mechanisms the Pirisun design brought, each alone against its plain function: the layer norm, the gate per value
and the unit norm with its gate, retention (rotated or not, decays up to 1, prompt steps against single tokens, unequal
sequences together, an input made so that the FIRST token decides an output 250 tokens later), softmax attention with a
query temperature and capped scores (every kernel that takes it; inputs made so that ONE marked key decides the last
query: the first token, both sides of page borders, a far key, in a prompt step and as a single token), the pair of
mixers, latent attention with a sink, interleaved pairs and a gate per value (both of its forms, in portions), and the
router with a correction, identity experts and a shared expert both ways the experts run."""
import numpy as np
import pytest
import torch

import plain_pirisun as P
from test_parts_gpu import close, load, rnd, run_mixer

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
    """The little of a step context that a norm or a feed-forward reads."""

    def __init__(self, k, dtype, n, decode=False):
        self.dtype, self.device, self.status = dtype, torch.device("cuda"), k.status_word(torch.device("cuda"))
        self.n_tokens, self.is_decode, self._memo = n, decode, {}

    def memo(self, key, make):
        if key not in self._memo:
            self._memo[key] = make()
        return self._memo[key]


# ------------------------------------------------------------------------------- row kernels

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("dim,eps,bias", [(38, 1e-4, True), (192, 1e-6, True), (1000, 3e-6, False), (5000, 1e-5, True)])
def test_layer_norm_part(k, dtype, dim, eps, bias):
    """Rows with a large common offset, so that a variance taken as E[x^2] - mean^2 or a forgotten mean shows; all rows
    and a chosen few."""
    from zinfer_b200.parts import LayerNorm
    t = {"w": 1.0 + rnd((dim,), 1, dtype, 0.3), "w.b": rnd((dim,), 2, dtype, 0.5)}
    norm = load(LayerNorm(dim, eps, "w", "w.b" if bias else None), t, dtype)
    x = rnd((9, dim), 3, torch.float32, 2.0) + torch.linspace(-30.0, 50.0, 9)[:, None]
    ref = P.layer_norm(f64(x), f64(t["w"]), f64(t["w.b"]) if bias else 0.0, eps)
    ctx = Ctx(k, dtype, 9)
    close(norm.forward(ctx, x.cuda()), ref, dtype, "all rows")
    rows = torch.tensor([7, 0, 3], dtype=torch.int32)
    close(norm.forward(ctx, x.cuda(), rows=rows.cuda()), ref[[7, 0, 3]], dtype, "chosen rows")
    assert norm.pending(ctx, x.cuda()) is None


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,width,valid,skip", [(4, 64, 64, 96), (3, 128, 64, 100), (5, 7, 7, 3), (2, 16, 10, 1)])
def test_gate_per_value(k, dtype, H, width, valid, skip):
    """rows[t, h, j] *= sigmoid(gate[t, h * valid + j]); columns of a head behind `valid` are padding and stay."""
    rows, gate = rnd((11, H * width), 1, dtype), rnd((11, skip + H * valid), 2, torch.float32, 2.0)
    ref = f64(rows).reshape(11, H, width).copy()
    ref[:, :, :valid] *= P.sigmoid(f64(gate)[:, skip:].reshape(11, H, valid))
    got = k.value_gate(rows.to(dtype).cuda(), gate.cuda()[:, skip:], H, valid)
    close(got, ref.reshape(11, -1), dtype, "gate per value")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,e", [(6, 32), (1, 5), (3, 100), (2, 64)])
def test_unit_norm_with_gate(k, dtype, H, e):
    o, gate = rnd((13, H * e), 1, torch.float32, 3.0), rnd((13, 5 + H * e), 2, torch.float32, 2.0)
    ref = (P.rms(f64(o).reshape(13, H, e), 1e-5).reshape(13, -1)) * P.silu(f64(gate)[:, 5:])
    close(k.unit_norm_gate(o.cuda(), gate.cuda()[:, 5:], H, 1e-5, dtype), ref, dtype, "unit norm and gate")


@pytest.mark.parametrize("scale", [0.5, 1.0])
def test_sum_of_a_share_of_normalised_rows(k, scale):
    m, w, x = rnd((7, 200), 1, torch.float32, 2.0), 1.0 + rnd((200,), 2, torch.float32, 0.2), rnd((7, 200), 3, torch.float32)
    got = k.rmsnorm_add(m.cuda(), w.cuda(), 1e-6, x.clone().cuda(), scale)
    close(got, f64(x) + scale * P.rms(f64(m), 1e-6) * f64(w), torch.float32, "share of a norm")


@pytest.mark.parametrize("dim", [38, 200, 2048, 5000])
def test_sum_of_two_normalised_rows(k, dim):
    a, b, x = rnd((7, dim), 1, torch.float32, 2.0), rnd((7, dim), 2, torch.float32, 0.1), rnd((7, dim), 3, torch.float32)
    wa, wb = 1.0 + rnd((dim,), 4, torch.float32, 0.2), 1.0 + rnd((dim,), 5, torch.float32, 0.2)
    got = k.rmsnorm_pair_add(a.cuda(), b.cuda(), wa.cuda(), wb.cuda(), 1e-6, x.clone().cuda(), 0.5)
    close(got, f64(x) + 0.5 * (P.rms(f64(a), 1e-6) * f64(wa) + P.rms(f64(b), 1e-6) * f64(wb)), torch.float32, "pair of norms")


# ------------------------------------------------------------------------------- retention

def retention_tensors(D, H, d, e, dtype, seed):
    return {"q": rnd((H * d, D), seed, dtype, D ** -0.5), "k": rnd((H * d, D), seed + 1, dtype, D ** -0.5),
            "v": rnd((H * e, D), seed + 2, dtype, D ** -0.5), "g": rnd((H * e, D), seed + 3, dtype, D ** -0.5),
            "o": rnd((D, H * e), seed + 4, dtype, (H * e) ** -0.5)}


def make_retention(D, H, d, e, decay, rot, t, dtype, eps=1e-5):
    from zinfer_b200.parts import Retention, RotaryEncoding
    position = RotaryEncoding(d, rot[0], n_rot=rot[1]) if rot else None
    return load(Retention(D, H, d, e, decay, "q", "k", "v", "g", "o", position=position, norm_eps=eps), t, dtype)


def plain_retention(x, t, H, d, e, decay, rot, eps=1e-5):
    m = {"heads": H, "dim": d, "vdim": e, "decay": list(decay)}
    if rot:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    return P.retention(f64(x), {n: f64(a) for n, a in t.items()}, m, eps)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D,H,d,e,decay,rot", [(48, 3, 8, 10, (0.9, 0.97, 0.995), (100.0, 4)), (32, 1, 12, 20, (1.0,), None),
                                               (128, 4, 32, 32, (0.96, 0.98, 0.99, 0.999), (300000.0, 32)),
                                               (38, 2, 6, 5, (0.93, 0.999), (20.0, 2)), (64, 2, 64, 40, (0.8, 0.99), (500.0, 32)),
                                               (64, 1, 160, 33, (0.97,), (1000.0, 160))])
def test_retention_alone(k, dtype, D, H, d, e, decay, rot):
    """Three sequences of unequal length in one batch: a long prompt then single tokens, a short prompt, one token; the
    state passes from the prompt step to the single-token steps, and the rotation goes by each token's own position."""
    t = retention_tensors(D, H, d, e, dtype, 10)
    mixer = make_retention(D, H, d, e, decay, rot, t, dtype)
    xs = [rnd((n, D), 20 + b, dtype) for b, n in enumerate((90, 37, 12))]
    outs = run_mixer(k, mixer, dtype, xs, [70, 17, 1], page=16)
    for b, x in enumerate(xs):
        close(outs[b], plain_retention(x, t, H, d, e, decay, rot), dtype, f"sequence {b}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("prompt", [260, 100, 2, 1])
def test_retention_keeps_the_first_token_for_hundreds_of_steps(k, dtype, prompt):
    """Keys of all tokens but the first are made tiny, so every output is the first token's value as far as the decay
    lets it through: a state that is lost, zeroed or decayed wrongly between steps changes everything."""
    D, H, d, e, decay = 32, 2, 8, 8, (0.999, 0.99)
    t = retention_tensors(D, H, d, e, dtype, 30)
    t["k"][:, D // 2:] = 0.0                               # keys read the first half of the input only
    mixer = make_retention(D, H, d, e, decay, (50.0, 8), t, dtype)
    x = rnd((260, D), 31, dtype)
    x[1:, :D // 2] *= 1e-3
    ref = plain_retention(x, t, H, d, e, decay, (50.0, 8))
    without = x.clone()
    without[0, :D // 2] = x[1, :D // 2]
    assert np.abs(ref[-1] - plain_retention(without, t, H, d, e, decay, (50.0, 8))[-1]).max() > 0.1 * np.abs(ref).max()
    outs = run_mixer(k, mixer, dtype, [x], [prompt], page=16)
    close(outs[0], ref, dtype, f"prompt of {prompt}")


# ------------------------------------------------------------------------------- attention with a temperature and a cap

def capped_tensors(D, H, G, d, e, dtype, seed):
    return {"q": rnd((H * d, D), seed, dtype, D ** -0.5), "k": rnd((G * d, D), seed + 1, dtype, D ** -0.5),
            "v": rnd((G * e, D), seed + 2, dtype, D ** -0.5), "o": rnd((D, H * e), seed + 3, dtype, (H * e) ** -0.5)}


def make_capped(D, H, G, d, e, scale, cap, q_temp, t, dtype, pad=False):
    from zinfer_b200.parts import GqaAttention
    return load(GqaAttention(D, H, G, d, "q", "k", "v", "o", scale=scale, value_dim=e, softcap=cap, query_temperature=q_temp,
                             pad_heads=pad), t, dtype)


def plain_capped(x, t, H, G, d, e, scale, cap, q_temp):
    m = {"heads": H, "kv_heads": G, "dim": d, "vdim": e, "scale": scale}
    if cap:
        m["softcap"] = cap
    if q_temp:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return P.capped_attention(f64(x), {n: f64(a) for n, a in t.items()}, m)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D,H,G,d,e,scale,cap,q_temp,page", [
    (48, 4, 2, 16, 12, 0.6, 2.0, (0.4, 7), 16), (64, 6, 6, 8, 16, 0.7, None, None, 16), (38, 5, 1, 10, 7, 0.6, 4.0, (0.25, 3), 16),
    (128, 8, 2, 64, 64, 0.25, 3.0, (0.35, 16), 64), (128, 4, 4, 64, 64, 0.2, 50.0, None, 64), (128, 2, 1, 128, 128, 0.15, 2.5, (1.0, 50), 64),
    (64, 2, 1, 64, 128, 0.2, 3.0, (0.35, 96), 64), (32, 1, 1, 4, 6, 1.0, 1.0, (0.2, 1), 16), (128, 8, 2, 64, 64, 0.25, None, (0.5, 10), 64)])
@pytest.mark.parametrize("pad", [False, True])
def test_capped_attention_alone(k, dtype, D, H, G, d, e, scale, cap, q_temp, page, pad):
    """Three unequal sequences: a prompt step then single tokens, over several periods of the temperature and several
    pages; caps low enough to bend most scores.  The shapes include those of the two mma.sync kernels; with `pad`, heads
    of other widths are padded up to them in a bfloat16 run (pages of 64 tokens, which those kernels want)."""
    t = capped_tensors(D, H, G, d, e, dtype, 40)
    mixer = make_capped(D, H, G, d, e, scale, cap, q_temp, t, dtype, pad)
    padded = pad and dtype == torch.bfloat16 and not (d == e and d in (64, 128))
    assert (mixer.run_head_dim, mixer.run_value_dim) == ((64, 64) if padded and max(d, e) <= 64 else (128, 128) if padded else (d, e))
    assert mixer.kv_request().head_dim == mixer.run_head_dim and mixer.kv_request().v_dim == mixer.run_value_dim
    xs = [rnd((n, D), 50 + b, dtype, 1.5) for b, n in enumerate((150, 40, 9))]
    outs = run_mixer(k, mixer, dtype, xs, [130, 17, 1], page=64 if pad else page)
    for b, x in enumerate(xs):
        close(outs[b], plain_capped(x, t, H, G, d, e, scale, cap, q_temp), dtype, f"sequence {b}")


def test_a_low_cap_changes_the_result():
    """The oracle's own cap: scores far above it all weigh the same."""
    t = capped_tensors(16, 1, 1, 8, 8, torch.float32, 60)
    x = rnd((6, 16), 61, torch.float32, 4.0)
    a, b = plain_capped(x, t, 1, 1, 8, 8, 5.0, None, None), plain_capped(x, t, 1, 1, 8, 8, 5.0, 0.01, None)
    v = f64(x) @ f64(t["v"]).T
    mean = np.stack([v[:i + 1].mean(0) for i in range(6)]) @ f64(t["o"]).T
    assert np.abs(a - b).max() > 0.05 and np.abs(b - mean).max() < 1e-2 * np.abs(mean).max() + 1e-3


T_MARK = 300


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,d,page", [(4, 2, 16, 16), (4, 2, 64, 64)])
@pytest.mark.parametrize("mark", [0, 1, 15, 16, 63, 64, 127, 128, 255, 256, T_MARK - 2])
def test_one_marked_key_decides_the_last_query(k, dtype, H, G, d, page, mark):
    """The last token's query is made to match the key of token `mark` alone (same first half of the input, a sharp
    scale, a cap high enough to leave the match standing), while the values come from the second half.  The last token
    comes in a prompt step, and then as a single token behind prompts of two lengths."""
    D, T = 2 * d, T_MARK
    t = capped_tensors(D, H, G, d, d, dtype, 70)
    t["k"][:, D // 2:] = 0.0
    t["v"][:, :D // 2] = 0.0
    t["q"] = t["k"].reshape(G, 1, d, D).expand(G, H // G, d, D).reshape(H * d, D).clone()
    scale, cap, q_temp = 8.0 / d, 60.0, (0.35, 64)
    mixer = make_capped(D, H, G, d, d, scale, cap, q_temp, t, dtype)
    x = rnd((T, D), 71, dtype)
    x[mark, :D // 2] *= 2.0                                    # a long key, so that its match with itself stands out
    x[T - 1, :D // 2] = x[mark, :D // 2]
    ref = plain_capped(x, t, H, G, d, d, scale, cap, q_temp)
    other = x.clone()
    other[mark, D // 2:] = rnd((D // 2,), 72, dtype)
    moved = plain_capped(other, t, H, G, d, d, scale, cap, q_temp)
    assert np.abs(ref[-1] - moved[-1]).max() > 0.1 * np.abs(ref).max(), "the marked key does not decide the last query"
    for prompt in (T, T - 1, 200):
        outs = run_mixer(k, mixer, dtype, [x], [prompt], page=page)
        close(outs[0], ref, dtype, f"prompt of {prompt}")


# ------------------------------------------------------------------------------- two mixers side by side

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D,left,right", [(48, (4, 2, 16, 12, 0.3, 2.0, (0.4, 7)), (3, 8, 10, (0.9, 0.97, 0.995), (100.0, 4))),
                                          (128, (8, 2, 64, 64, 0.12, 8.0, (0.35, 16)), (4, 32, 32, (0.96, 0.98, 0.99, 0.999), (3e5, 32)))])
def test_mixer_pair(k, dtype, D, left, right):
    """Half the sum of the two normalised results; the attention side takes the call's cache and the recurrence its
    state, through prompt steps and single-token steps of unequal sequences."""
    from zinfer_b200.parts import GqaAttention, MixerPair, Retention, RotaryEncoding
    H, G, d, e, scale, cap, qt = left
    Hr, dr, er, decay, rot = right
    tl, tr = capped_tensors(D, H, G, d, e, dtype, 80), retention_tensors(D, Hr, dr, er, dtype, 90)
    t = {**{"left." + n: a for n, a in tl.items()}, **{"right." + n: a for n, a in tr.items()},
         "left.out": 1.0 + rnd((D,), 5, dtype, 0.2), "right.out": 1.0 + rnd((D,), 6, dtype, 0.2)}
    a = GqaAttention(D, H, G, d, "left.q", "left.k", "left.v", "left.o", scale=scale, value_dim=e, softcap=cap, query_temperature=qt)
    b = Retention(D, Hr, dr, er, decay, "right.q", "right.k", "right.v", "right.g", "right.o",
                  position=RotaryEncoding(dr, rot[0], n_rot=rot[1]), norm_eps=1e-5)
    pair = load(MixerPair(D, a, b, "left.out", "right.out", norm_eps=1e-5), t, dtype)
    assert pair.kv_request() == a.kv_request() and pair.state_request() == b.state_request() and pair.capture_safe
    m = {"left": {"heads": H, "kv_heads": G, "dim": d, "vdim": e, "scale": scale, "softcap": cap, "q_temp": {"coef": qt[0], "every": qt[1]}},
         "right": {"heads": Hr, "dim": dr, "vdim": er, "decay": list(decay), "rot": {"base": rot[0], "dims": rot[1]}}}
    xs = [rnd((n, D), 100 + i, dtype) for i, n in enumerate((80, 30, 5))]
    outs = run_mixer(k, pair, dtype, xs, [64, 17, 1], page=64 if D == 128 else 16)
    for i, x in enumerate(xs):
        close(outs[i], P.mixer_pair(f64(x), {n: f64(v) for n, v in t.items()}, m, 1e-5), dtype, f"sequence {i}")
    with pytest.raises(ValueError):
        MixerPair(D, a, a, "left.out", "right.out")


# ------------------------------------------------------------------------------- attention through a latent

def latent_tensors(D, H, d, p, e, r, dtype, seed, sink=(0.5, 1.5)):
    return {"q": rnd((H * (d + p), D), seed, dtype, D ** -0.5), "dkv": rnd((r + p, D), seed + 1, dtype, D ** -0.5),
            "dkv.norm": 1.0 + rnd((r,), seed + 2, dtype, 0.2), "uk": rnd((H * d, r), seed + 3, dtype, r ** -0.5),
            "uv": rnd((H * e, r), seed + 4, dtype, r ** -0.5), "g": rnd((H * e, D), seed + 5, dtype, 2 * D ** -0.5),
            "o": rnd((D, H * e), seed + 6, dtype, (H * e) ** -0.5), "sink": sink[0] + rnd((H,), seed + 7, dtype, sink[1])}


def make_latent(D, H, d, p, e, r, scale, base, t, dtype, eps=2e-6):
    from zinfer_b200.parts import LatentAttention
    return load(LatentAttention(D, H, d, p, e, r, None, scale, base, None, None, "q", "dkv", "dkv.norm", "uk", "uv", "o",
                                gate_name="g", norm_eps=eps, gate_per_value=True, sink_name="sink", interleaved=True), t, dtype)


def plain_latent(x, t, H, d, p, e, r, scale, base, eps=2e-6):
    m = {"heads": H, "dim": d, "rot_dim": p, "vdim": e, "kv_rank": r, "scale": scale, "rot": {"base": base, "dims": p}}
    return P.latent_attention(f64(x), {n: f64(a) for n, a in t.items()}, m, eps)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D,H,d,p,e,r,scale,base,page", [
    (48, 3, 8, 4, 10, 24, 0.5, 50.0, 16), (64, 2, 16, 8, 16, 32, 0.4, 1e4, 16), (128, 4, 32, 32, 64, 64, 0.25, 1e4, 64),
    (128, 2, 64, 16, 32, 128, 0.2, 1e3, 64), (38, 3, 6, 6, 5, 18, 0.5, 40.0, 16), (128, 20, 16, 16, 16, 48, 0.3, 1e5, 64),
    (64, 1, 4, 2, 4, 8, 0.8, 20.0, 16), (256, 2, 64, 32, 128, 96, 0.2, 1e4, 64)])
def test_latent_attention_with_sink_and_value_gate(k, dtype, D, H, d, p, e, r, scale, base, page):
    """Unequal sequences, a prompt step (keys and values expanded) then single tokens (queries carried into the
    latent's space): both forms must agree with the plain function, the sink in either one's denominator."""
    t = latent_tensors(D, H, d, p, e, r, dtype, 110)
    mixer = make_latent(D, H, d, p, e, r, scale, base, t, dtype)
    xs = [rnd((n, D), 120 + b, dtype, 1.5) for b, n in enumerate((140, 33, 6))]
    outs = run_mixer(k, mixer, dtype, xs, [120, 17, 1], page=page)
    for b, x in enumerate(xs):
        close(outs[b], plain_latent(x, t, H, d, p, e, r, scale, base), dtype, f"sequence {b}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sink", [30.0, -30.0])
def test_latent_sink_far_above_and_far_below(k, dtype, sink):
    D, H, d, p, e, r = 128, 4, 32, 32, 64, 64
    t = latent_tensors(D, H, d, p, e, r, dtype, 130, sink=(sink, 0.0))
    mixer = make_latent(D, H, d, p, e, r, 0.2, 1e4, t, dtype)
    x = rnd((90, D), 131, dtype)
    ref = plain_latent(x, t, H, d, p, e, r, 0.2, 1e4)
    outs = run_mixer(k, mixer, dtype, [x], [70], page=64)
    if sink > 0:
        assert np.abs(ref).max() < 1e-6 and float(outs[0].abs().max()) < 1e-5
    else:
        close(outs[0], ref, dtype, "sink far below")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D,H,d,p,e,r,page,cuts", [(128, 4, 32, 32, 64, 64, 64, (64, 2, 30, 100, 3)), (48, 3, 8, 4, 10, 24, 16, (2, 2, 5, 40, 2))])
def test_latent_attention_in_portions(k, dtype, D, H, d, p, e, r, page, cuts):
    """A prompt fed in portions (long ones, and short ones behind a long prefix), then single tokens."""
    from test_parts_gpu import Bench
    t = latent_tensors(D, H, d, p, e, r, dtype, 140)
    mixer = make_latent(D, H, d, p, e, r, 0.3, 1e4, t, dtype)
    T = sum(cuts) + 5
    x = rnd((T, D), 141, dtype)
    bench = Bench(k, mixer, dtype, n_slots=2, max_seq=256, page=page)
    slot = bench.cache.alloc_slots(2)[1:]
    got, at = [], 0
    for n in list(cuts) + [1] * 5:
        ctx = bench.step(slot, [n])
        out = torch.zeros((n, D), device="cuda")
        mixer.forward(ctx, bench.call, x[at:at + n].to(dtype).cuda(), out, False)
        bench.done(slot, [n])
        got.append(out.cpu())
        at += n
    close(torch.cat(got), plain_latent(x, t, H, d, p, e, r, 0.3, 1e4), dtype, f"portions {cuts}")


# ------------------------------------------------------------------------------- router and experts

def expert_tensors(D, F, E, ident, shared, dtype, seed):
    t = {"router": rnd((E + ident, D), seed, torch.bfloat16, 3.0 * D ** -0.5), "correction": rnd((E + ident,), seed + 1, torch.bfloat16, 0.1)}
    for e in range(E):
        t[f"e{e}.gate"], t[f"e{e}.up"] = rnd((F, D), seed + 3 * e + 2, dtype, D ** -0.5), rnd((F, D), seed + 3 * e + 3, dtype, D ** -0.5)
        t[f"e{e}.down"] = rnd((D, F), seed + 3 * e + 4, dtype, F ** -0.5)
    if shared:
        t["shared.gate"], t["shared.up"] = rnd((shared, D), seed + 900, dtype, D ** -0.5), rnd((shared, D), seed + 901, dtype, D ** -0.5)
        t["shared.down"] = rnd((D, shared), seed + 902, dtype, shared ** -0.5)
    return t


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D,F,E,ident,top,shared,rows", [(48, 24, 6, 1, 2, 16, 7), (64, 16, 3, 1, 4, 0, 33), (128, 64, 8, 2, 2, 128, 300),
                                                         (128, 64, 8, 1, 3, 0, 200), (38, 10, 3, 3, 2, 12, 130), (256, 96, 16, 2, 4, 64, 3),
                                                         (128, 64, 8, 2, 3, 128, 700), (38, 10, 5, 0, 3, 0, 515), (64, 32, 2, 2, 4, 32, 120)])
def test_router_with_correction_identity_and_shared_experts(k, dtype, D, F, E, ident, top, shared, rows):
    """The streaming kernels (few rows, single-token steps) and the grouped contractions (many rows) against the plain
    function; the router's ids and weights against the plain choice (by score + correction, weighed by score alone).
    Rows whose choice is a close call are left out of the bfloat16 comparison (they are independent of one another)."""
    from zinfer_b200.parts import RoutedMoE, SwiGLU
    t = expert_tensors(D, F, E, ident, shared, dtype, 20)
    sh = SwiGLU(D, shared, "shared.gate", "shared.up", "shared.down") if shared else None
    ff = load(RoutedMoE(D, F, E, top, "router", lambda e: (f"e{e}.gate", f"e{e}.up", f"e{e}.down"), correction_name="correction",
                        n_identity=ident, shared=sh), t, dtype)
    x = rnd((rows, D), 5, dtype)
    W = {n: f64(a) for n, a in t.items()}
    ml = {"router": {"experts": E, "identity": ident, "top": top}}
    margins = [np.inf] * rows
    ref = P.experts(f64(x), W, ml, margins)
    keep = np.array([m > (0.02 if dtype == torch.bfloat16 else 1e-6) for m in margins])
    assert keep.sum() >= max(1, rows // 2)
    ids, wts = k.moe_router(x.to(dtype).cuda(), ff.w_router, top, ff.correction)
    z = f64(x) @ W["router"].T
    for i in np.flatnonzero(keep)[:40]:
        chosen, w, _ = P.route(z[i], W["correction"], top)
        assert ids[i].tolist() == chosen, (i, ids[i].tolist(), chosen)
        assert np.allclose(wts[i].cpu().numpy(), w, rtol=1e-4, atol=1e-6)
    if ident:
        assert bool((ids >= E).any()), "no row chose an identity expert: the test shows nothing of them"
    sel = torch.from_numpy(keep).cuda()
    outs = {}
    for decode in (False, True):
        out = torch.full((rows, D), 0.5, device="cuda")
        ff.forward(Ctx(k, dtype, rows, decode), x.to(dtype).cuda(), out, True)
        outs[decode] = out - 0.5
        close(outs[decode][sel], ref[keep], dtype, "decode" if decode else "prompt")
    i = int(np.flatnonzero(keep)[-1])
    alone = torch.zeros((1, D), device="cuda")
    ff.forward(Ctx(k, dtype, 1, True), x[i:i + 1].to(dtype).cuda(), alone, False)
    assert torch.allclose(alone[0], outs[True][i], atol=2e-6 * float(outs[True][i].abs().max()) + 1e-6)
