"""The mechanisms the Zosurax design brought, each alone against its plain function: the row kernels (layer
scale, pass input, squared relu), the token shift with its state, the HGRN2 recurrence with its state
(also with gates that forget so slowly that the first tokens still decide the last), attention with a
weighted norm before a partial half-split rotation, and attention with an interleaved rotation, a unit
norm behind it and weights mixed across the heads (inputs made so that ONE far key decides a query:
the first token, both sides of page borders, in prompt steps and in single-token steps)."""
import numpy as np
import pytest
import torch

import plain_zosurax as P
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


# ------------------------------------------------------------------------------- row kernels

@pytest.mark.parametrize("dim", [38, 256, 1000])
def test_layer_scale_pass_input_and_squared_relu(k, dim):
    m, x, s = rnd((7, dim), 1, torch.float32, 3.0), rnd((7, dim), 2, torch.float32), rnd((dim,), 3, torch.float32)
    close(k.scale_add(m.cuda(), s.cuda(), x.clone().cuda()), f64(x) + f64(m) * f64(s), torch.float32, "scale")
    base, vec = rnd((7, dim), 4, torch.float32), rnd((dim,), 5, torch.float32)
    close(k.rows_add(x.clone().cuda(), vec.cuda(), base.cuda()), f64(x) + f64(base) + f64(vec), torch.float32, "pass input")
    close(k.rows_add(x.clone().cuda(), vec.cuda()), f64(x) + f64(vec), torch.float32, "first pass")
    for dtype in DTYPES:
        z = rnd((5, dim), 6, dtype, 2.0)
        close(k.activation(z.to(dtype).cuda(), "relu_squared"), np.maximum(f64(z), 0) ** 2, dtype, "squared relu")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows", [3, 16, 40, 200])
@pytest.mark.parametrize("N,K", [(256, 128), (96, 72), (512, 256)])
def test_contractions_with_an_activation_or_a_scaled_sum(k, dtype, rows, N, K):
    """`linear(act=...)` and `linear(out=ScaledSink(...))` whichever kernel runs the product: the few-row kernel's
    epilogue, the persistent tcgen05 forms' epilogue, or kernels of their own behind any other contraction."""
    from zinfer_b200.parts.linear import ScaledSink, linear
    a, w = rnd((rows, K), 10, dtype), rnd((N, K), 11, dtype, K ** -0.5)
    x, sc = rnd((rows, N), 12, torch.float32), rnd((N,), 13, torch.float32)
    y = f64(a) @ f64(w).T
    got = linear(a.to(dtype).cuda(), w.to(dtype).cuda(), act="relu_squared")
    assert got.dtype == dtype
    close(got, np.maximum(y, 0) ** 2, dtype, "activated")
    rows_dev = x.clone().cuda()
    linear(a.to(dtype).cuda(), w.to(dtype).cuda(), out=ScaledSink(rows_dev, sc.cuda()), accumulate=True)
    ref = f64(x) + y * f64(sc)
    close(rows_dev, ref, dtype, "scaled sum")


# ------------------------------------------------------------------------------- token shift

class Passthrough:
    """An inner mixer that returns what it reads, so that the shift in front of it can be seen."""
    capture_safe = True

    def __init__(self, state_shape=None):
        self.state_shape, self.seen_dtype, self.seen_state = state_shape, None, None

    def kv_request(self):
        return None

    def state_request(self):
        from zinfer_b200.parts import StateRequest
        return None if self.state_shape is None else StateRequest(self.state_shape)

    def forward(self, ctx, call, h, out, accumulate):
        self.seen_dtype, self.seen_state = h.dtype, call.state
        out.copy_(out + h.float() if accumulate else h.float())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D,normed,inner_state", [(40, True, None), (64, False, (3, 5)), (38, True, (7,)), (1000, True, None)])
def test_token_shift_with_state(k, dtype, D, normed, inner_state):
    """Portions of 1, 2 and more tokens, then single tokens, for three sequences at once; with the norm
    still pending (the kernel applies it) and with plain float32 rows; then a slot that is used again."""
    from zinfer_b200.parts import TokenShift
    from zinfer_b200.parts.linear import NormedRows
    inner = Passthrough(inner_state)
    mu, w, eps = rnd((D,), 20, dtype, 0.3) + 0.5, 1.0 + rnd((D,), 21, dtype, 0.2), 1e-5
    shift = TokenShift(inner, D, "mu")
    shift.load({"mu": mu.cuda()}, dtype, torch.device("cuda"))
    extra = int(np.prod(inner_state)) if inner_state else 0
    assert shift.state_request().shape == (D + extra,) and shift.takes_pending_norm
    xs = [rnd((n, D), 30 + n, torch.float32, 2.0) for n in (41, 17, 26)]
    bench = Bench(k, shift, dtype, n_slots=4)
    held = bench.cache.alloc_slots(4)
    slots = held[1:][::-1]
    outs, at = [[] for _ in xs], [0, 0, 0]
    plan = [[2, 1, 5], [1, 1, 2], [9, 2, 3], [1, 1, 1], [1, 1, 1]]

    def run(slots_, rows):
        ctx = bench.step(slots_, [r.shape[0] for r in rows])
        x = torch.cat(rows).cuda()
        out = torch.empty_like(x)
        shift.forward(ctx, bench.call, NormedRows(x, w.cuda(), eps, dtype) if normed else x, out, False)
        bench.done(slots_, [r.shape[0] for r in rows])
        return out.cpu()

    while any(a < x.shape[0] for a, x in zip(at, xs)):
        sizes = plan.pop(0) if plan else [1, 1, 1]
        live = [b for b in range(3) if at[b] < xs[b].shape[0]]
        take = [min(sizes[b], xs[b].shape[0] - at[b]) for b in live]
        out = run([slots[b] for b in live], [xs[b][at[b]:at[b] + n] for b, n in zip(live, take)])
        o = 0
        for b, n in zip(live, take):
            outs[b].append(out[o:o + n])
            o += n
            at[b] += n
    assert inner.seen_dtype == dtype
    if inner_state:
        assert tuple(inner.seen_state.shape[1:]) == inner_state and not bool(inner.seen_state.any())

    def plain(x):
        h = P.rms(f64(x), eps) * f64(w) if normed else f64(x)
        return P.token_shift(h, f64(mu))

    for b, x in enumerate(xs):
        close(torch.cat(outs[b]), plain(x), dtype, f"sequence {b}")
    bench.cache.free_slots(held)
    again = bench.cache.alloc_slots(4)
    close(run([again[2]], [xs[0][:3]]), plain(xs[0][:3]), dtype, "slot used again")


# ------------------------------------------------------------------------------- HGRN2

def hgrn2_tensors(D, H, d, e, dtype, seed, slow=False):
    lower = torch.rand((H * d,), generator=torch.Generator().manual_seed(seed + 9))
    lower = (0.95 + 0.049 * lower) if slow else 0.9 * lower
    return {"q": rnd((H * d, D), seed, dtype, D ** -0.5), "f": rnd((H * d, D), seed + 1, dtype, D ** -0.5),
            "fb": rnd((H * d,), seed + 2, dtype, 1.0), "lo": lower.to(dtype).float(),
            "v": rnd((H * e, D), seed + 3, dtype, D ** -0.5), "n": 1.0 + rnd((e,), seed + 4, dtype, 0.2),
            "o": rnd((D, H * e), seed + 5, dtype, (H * e) ** -0.5)}


def plain_hgrn2(x, t, H, d, e, eps):
    p = {"q": t["q"], "f": t["f"], "f.b": t["fb"], "lower": t["lo"], "v": t["v"], "norm": t["n"], "o": t["o"]}
    return P.hgrn2(f64(x), {n: f64(a) for n, a in p.items()}, {"heads": H, "dim": d, "vdim": e}, eps)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D,H,d,e", [(40, 2, 8, 12), (32, 1, 4, 4), (38, 3, 5, 9), (128, 2, 64, 64), (64, 1, 128, 32),
                                     (48, 1, 160, 16), (64, 2, 16, 200), (32, 1, 300, 40)])
def test_hgrn2_part(k, dtype, D, H, d, e):
    """Three sequences: a prompt step of unequal portions, then single tokens; slots other than the batch index."""
    from zinfer_b200.parts import Hgrn2
    eps = 1e-5
    t = hgrn2_tensors(D, H, d, e, dtype, 40)
    mixer = load(Hgrn2(D, H, d, e, "q", "f", "fb", "lo", "v", "n", "o", norm_eps=eps), t, dtype)
    assert mixer.kv_request() is None and mixer.state_request().shape == (H * d * e,)
    xs = [rnd((n, D), 50 + n, dtype) for n in (45, 21, 30)]
    outs = run_mixer(k, mixer, dtype, xs, [40, 1, 9])
    for b, x in enumerate(xs):
        close(outs[b], plain_hgrn2(x, t, H, d, e, eps), dtype, f"sequence {b}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_hgrn2_remembers_over_hundreds_of_tokens(k, dtype):
    """Gates of 0.95 to 0.999: what the first tokens wrote still decides the output 250 tokens later, whether
    they came in a prompt step, in portions or one by one.  A state that is lost or zeroed between steps shows."""
    from zinfer_b200.parts import Hgrn2
    D, H, d, e, eps = 48, 2, 16, 24, 1e-5
    t = hgrn2_tensors(D, H, d, e, dtype, 60, slow=True)
    mixer = load(Hgrn2(D, H, d, e, "q", "f", "fb", "lo", "v", "n", "o", norm_eps=eps), t, dtype)
    x = rnd((250, D), 61, dtype)
    x[:3] *= 30.0                                   # the first tokens write large values
    ref = plain_hgrn2(x, t, H, d, e, eps)
    forgot = plain_hgrn2(x[3:], t, H, d, e, eps)    # what a state that lost the first tokens would give
    assert np.abs(ref[3:] - forgot)[-40:].max() > 0.2 * np.abs(ref).max()
    for prompt in (250, 5, 171):
        outs = run_mixer(k, mixer, dtype, [x, x[:50]], [prompt, 2])
        close(outs[0], ref, dtype, f"prompt of {prompt}")
        close(outs[1], ref[:50], dtype, "the short one beside it")


# ------------------------------------------------------------------------------- attention

def attention_tensors(D, H, G, d, vd, dtype, seed, split=False):
    """split: q and k read the first half of the input only and v the second half only, so that a test can
    give two tokens the same key and different values."""
    t = {"q": rnd((H * d, D), seed, dtype, D ** -0.5), "k": rnd((G * d, D), seed + 1, dtype, D ** -0.5),
         "v": rnd((G * vd, D), seed + 2, dtype, D ** -0.5), "o": rnd((D, H * vd), seed + 3, dtype, (H * vd) ** -0.5),
         "qn": 1.0 + rnd((d,), seed + 4, dtype, 0.2), "kn": 1.0 + rnd((d,), seed + 5, dtype, 0.2),
         "talk": (0.7 * torch.eye(H) + rnd((H, H), seed + 6, dtype, 0.35)).to(dtype).float()}
    if split:
        t["q"][:, D // 2:] = 0
        t["k"][:, D // 2:] = 0
        t["v"][:, :D // 2] = 0
    return t


def make_attention(kind, D, H, G, d, vd, scale, rot, t, dtype, eps=2e-6):
    from zinfer_b200.parts import GqaAttention, RotaryEncoding
    talking = kind == "attention_2"
    pos = RotaryEncoding(d, rot[0], n_rot=rot[1], interleaved=talking) if rot else None
    return load(GqaAttention(D, H, G, d, "q", "k", "v", "o", None if talking else "qn", None if talking else "kn", eps, pos,
                             scale=scale, value_dim=vd, unit_norm_after_rotation=talking,
                             talk_name="talk" if talking else None), t, dtype)


def plain_attention(kind, x, t, H, G, d, vd, scale, rot, eps=2e-6):
    m = {"heads": H, "kv_heads": G, "dim": d, "vdim": vd, "scale": scale}
    if rot:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    p = {"q": t["q"], "k": t["k"], "v": t["v"], "o": t["o"], "q.norm": t["qn"], "k.norm": t["kn"], "talk": t["talk"]}
    fn = P.attention_talking if kind == "attention_2" else P.attention_normed
    return fn(f64(x), {n: f64(a) for n, a in p.items()}, m, eps, np.arange(x.shape[0]))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind,D,H,G,d,vd,scale,rot,page", [
    ("attention", 40, 3, 1, 16, 24, 0.3, (100.0, 8), 16),        # three heads on one key/value head, values wider, half a head rotated
    ("attention", 64, 4, 4, 8, 8, 0.4, None, 16),                # no rotation at all
    ("attention", 128, 8, 2, 64, 64, 0.12, (10000.0, 64), 64),   # what the tensor-core kernels take, whole head rotated
    ("attention", 128, 4, 2, 64, 64, 0.2, (10000.0, 32), 64),    # the same kernels behind a partial rotation
    ("attention", 96, 2, 2, 128, 128, 0.09, (10000.0, 64), 64),
    ("attention", 64, 2, 1, 64, 32, 0.15, (500.0, 64), 64),      # values narrower than keys at a head width the tensor cores take
    ("attention_2", 40, 4, 2, 10, 6, 0.35, (50.0, 10), 16),      # values narrower, the whole head rotated in interleaved pairs
    ("attention_2", 64, 2, 1, 32, 32, 0.2, (10000.0, 16), 16),   # all heads on ONE key/value head
    ("attention_2", 38, 5, 5, 10, 7, 0.3, (20.0, 6), 16),        # a head per key/value head, odd value width
    ("attention_2", 128, 4, 4, 64, 64, 0.11, (500.0, 32), 64),
    ("attention_2", 64, 1, 1, 16, 16, 0.25, None, 16),           # a single head: the mix is one number
    ("attention_2", 96, 6, 2, 48, 40, 0.14, (10000.0, 48), 32),
    ("attention", 64, 4, 2, 32, 32, 0.18, (10000.0, 16), 32),    # head widths that the one-lane-per-key single-token kernel takes
    ("attention", 96, 2, 1, 96, 96, 0.1, (300.0, 96), 32),
    ("attention_2", 128, 4, 2, 128, 128, 0.09, (10000.0, 64), 64),   # mixed heads on the mma.sync kernels of width 128
    ("attention_2", 64, 8, 8, 64, 64, 0.12, None, 64),               # eight value heads for every head's weights
])
def test_attention_kinds_alone(k, dtype, kind, D, H, G, d, vd, scale, rot, page):
    t = attention_tensors(D, H, G, d, vd, dtype, 70)
    mixer = make_attention(kind, D, H, G, d, vd, scale, rot, t, dtype)
    req = mixer.kv_request()
    assert (req.n_kv_heads, req.head_dim, req.v_dim) == (G, d, vd)
    xs = [rnd((n, D), 80 + n, dtype) for n in (70, 37, 45)]
    outs = run_mixer(k, mixer, dtype, xs, [65, 17, 1], page=page)
    for b, x in enumerate(xs):
        close(outs[b], plain_attention(kind, x, t, H, G, d, vd, scale, rot), dtype, f"sequence {b}")


def marked_tensors(D, H, G, d, vd, dtype):
    """Every query head projects like its key head, and the norms' weights agree: two tokens with the same first
    half of the input then have a query and a key that point the same way."""
    t = attention_tensors(D, H, G, d, vd, dtype, 90, split=True)
    t["q"] = t["k"].reshape(G, 1, d, D).expand(G, H // G, d, D).reshape(H * d, D).clone()
    t["qn"] = t["kn"].clone()
    t["talk"] = (torch.eye(H) * 0.8 + 0.1).to(dtype).float()
    return t


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind,H,G,d,page", [("attention_2", 4, 2, 16, 16), ("attention", 4, 2, 64, 64), ("attention_2", 2, 2, 64, 64)])
@pytest.mark.parametrize("mark", [0, 1, 15, 16, 17, 63, 64, 65, 127, 128, 129, 190])
def test_one_far_key_decides(k, dtype, kind, H, G, d, page, mark):
    """The last token's query is made to match the key of token `mark` alone (same first half of the input, a
    sharp scale), while the values come from the second half: the output is then token `mark`'s value, and a
    kernel that loses that key (a page border, the first token, a chunk's edge) is far off.  The last token comes
    in a prompt step, and then as a single token behind a prompt."""
    D, vd, T = 2 * d, d, 200
    t = marked_tensors(D, H, G, d, vd, dtype)
    scale = 6.0 / d ** 0.5 if kind == "attention" else 6.0 / d         # unit-normed heads have length sqrt(d)
    mixer = make_attention(kind, D, H, G, d, vd, scale, None, t, dtype)
    x = rnd((T, D), 91, dtype)
    x[T - 1, :D // 2] = x[mark, :D // 2]
    ref = plain_attention(kind, x, t, H, G, d, vd, scale, None)
    other = x.clone()
    other[mark, D // 2:] = rnd((D // 2,), 92, dtype)            # another value at the marked token
    moved = plain_attention(kind, other, t, H, G, d, vd, scale, None)
    assert np.abs(ref[-1] - moved[-1]).max() > 0.1 * np.abs(ref).max(), "the marked key does not decide the last query"
    for prompt in (T, T - 1, 150):
        outs = run_mixer(k, mixer, dtype, [x], [prompt], page=page)
        close(outs[0], ref, dtype, f"prompt of {prompt}")
