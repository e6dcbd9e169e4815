"""The mechanisms the Ponusun design brought, each alone against its plain function: the row kernels,
the input convolution with its state, attention with whole-projection norms, a value width of its own,
the log-distance bias and windows (inputs made so that ONE key decides a query's output: far keys, keys at
page borders, keys just inside and just outside the window, in prompt steps and single-token steps), a
reader of another call's cache, the table-routed experts, and the block that normalises sublayer outputs."""
import math

import numpy as np
import pytest
import torch

import plain_ponusun as P
from test_parts_gpu import Bench, close, load, rnd, run_mixer

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def k():
    from zinfer_b200 import kernels
    kernels.require_cuda()
    return kernels


def context(k, dtype, cache, slots, token_lists, host=True):
    """A step context for `token_lists` continuing the sequences in `slots` of `cache`; `host`: the context
    also carries the ids on the host, as a prompt step's does."""
    from zinfer_b200.engine.context import StepContext, pack_batch
    lens = [len(t) for t in token_lists]
    starts = [int(cache.lengths[s]) for s in slots]
    cache.reserve(slots, lens)
    cache.sync()
    buf = torch.from_numpy(pack_batch(slots, starts, token_lists)).cuda()
    return StepContext(dtype, torch.device("cuda"), k.status_word("cuda"), buf, sum(lens), len(slots), lens,
                       max(s + n for s, n in zip(starts, lens)),
                       host_tokens=np.concatenate([np.asarray(t, dtype=np.int32) for t in token_lists]) if host else None)


# ------------------------------------------------------------------------------- row kernels

@pytest.mark.parametrize("dim", [40, 256, 5000])
def test_norm_of_a_sublayer_output_is_summed_into_the_rows(k, dim):
    m, x, w = rnd((7, dim), 1, torch.float32, 3.0), rnd((7, dim), 2, torch.float32), 1.0 + rnd((dim,), 3, torch.float32, 0.3)
    got = k.rmsnorm_add(m.cuda(), w.cuda(), 1e-5, x.clone().cuda())
    ref = x.numpy().astype(np.float64) + P.rms_unit(m.numpy().astype(np.float64), 1e-5) * w.numpy()
    close(got, ref, torch.float32)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(5, 333), (6, 64)])      # a count that is no multiple of 8 (one value at a time) and one that is
def test_activations(k, dtype, shape):
    z = rnd(shape, 4, dtype, 2.5)
    close(k.activation(z.to(dtype).cuda(), "gelu_erf"), P.gelu_erf(z.numpy().astype(np.float64)), dtype, "erf")
    close(k.activation(z.to(dtype).cuda(), "gelu_tanh"), P.gelu_tanh(z.numpy().astype(np.float64)), dtype, "tanh")
    close(k.activation(z.to(dtype).cuda(), "silu"), P.silu(z.numpy().astype(np.float64)), dtype, "silu")
    # the two gelus differ by more than the tolerance somewhere, so the test tells them apart
    assert np.abs(P.gelu_erf(z.numpy().astype(np.float64)) - P.gelu_tanh(z.numpy().astype(np.float64))).max() > 1e-4


def test_softcap_weighted_sum_and_gate(k):
    z = rnd((3, 1001), 5, torch.float32, 40.0)
    close(k.softcap(z.clone().cuda(), 17.0), P.softcap(z.numpy().astype(np.float64), 17.0), torch.float32, "cap")
    planes = rnd((6, 9, 50), 6, torch.float32)
    w = rnd((5,), 7, torch.float32)
    dev = planes.clone().cuda()
    k.weighted_sum(dev, w.cuda(), 5, dev[5])
    ref = P.depth_average([planes[j].numpy().astype(np.float64) for j in range(5)], w.numpy())
    close(dev[5], ref, torch.float32, "mix")
    assert torch.equal(dev[:5].cpu(), planes[:5])
    k.weighted_sum(dev, None, 1, dev[1])
    assert torch.equal(dev[1].cpu(), planes[0])
    x, g, s, m = rnd((4, 70), 8, torch.float32), rnd((70,), 9, torch.float32, 0.3), rnd((4, 33), 10, torch.float32), rnd((4, 33), 11, torch.float32)
    got = k.gate_add(x.cuda(), g.cuda(), s.cuda(), m.clone().cuda())
    gate = 1.0 / (1.0 + np.exp(-(x.numpy().astype(np.float64) @ g.numpy())))
    close(got, m.numpy() + gate[:, None] * s.numpy(), torch.float32, "gate")


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_with_learned_positions_and_capped_head(k, dtype):
    from zinfer_b200.cache import CacheManager, CallCacheSpec
    from zinfer_b200.parts import LMHead, TokenEmbedding
    vocab, dim, npos = 77, 40, 30
    t = {"e": rnd((vocab, dim), 12, dtype), "p": rnd((npos, dim), 13, dtype), "h": rnd((vocab, dim), 14, dtype, 0.5)}
    emb = load(TokenEmbedding(vocab, dim, "e", position_name="p", max_positions=npos), t, dtype)
    head = load(LMHead(vocab, dim, "h", softcap=3.0), t, dtype)
    cache = CacheManager([CallCacheSpec()], 2, 64, 32, 16, dtype, "cuda")
    slots = cache.alloc_slots(2)
    cache.lengths[slots[1]] = 9                       # the second sequence goes on at position 9
    toks = [[5, 76, 0], [33, 2]]
    ctx = context(k, dtype, cache, slots, toks)
    x = emb.forward(ctx, ctx.tokens)
    ref = np.concatenate([P.embed_with_positions(toks[0], t["e"].numpy(), t["p"].numpy()),
                          t["e"].numpy()[toks[1]].astype(np.float64) + t["p"].numpy()[9:11]])
    close(x, ref, torch.float32, "embedding")
    logits = head.forward(ctx, x.to(dtype))
    close(logits, P.softcap(x.to(dtype).double().cpu().numpy() @ t["h"].numpy().astype(np.float64).T, 3.0), dtype, "head")
    assert int(ctx.status.item()) == 0
    cache.lengths[slots[1]] = 29                      # positions 29, 30: the second lies outside the table
    ctx = context(k, dtype, cache, [slots[1]], [[1, 2]])
    emb.forward(ctx, ctx.tokens)
    assert int(ctx.status.item()) == 3
    ctx.status.zero_()


# ------------------------------------------------------------------------------- input convolution

class Passthrough:
    """An inner mixer that returns what it reads, so that the convolution in front of it can be seen."""
    capture_safe = True

    def __init__(self):
        self.seen_dtype = None

    def kv_request(self):
        return None

    def state_request(self):
        return None

    def forward(self, ctx, call, h, out, accumulate):
        self.seen_dtype = h.dtype
        out.copy_(out + h.float() if accumulate else h.float())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D,K", [(40, 3), (64, 1), (200, 4), (72, 7)])
def test_input_convolution_with_state(k, dtype, D, K):
    """Portions of 1, 2, K-1, K and more tokens, then single tokens, for three sequences at once."""
    from zinfer_b200.parts import InputConv
    inner = Passthrough()
    taps = rnd((D, K), 20, dtype, 0.5)
    conv = InputConv(inner, D, K, "c")
    conv.load({"c": taps.cuda()}, dtype, torch.device("cuda"))
    assert conv.state_request().shape == (max(K - 1, 1), D) and conv.takes_residual_rows
    xs = [rnd((n, D), 30 + n, torch.float32) for n in (41, 17, 26)]
    bench = Bench(k, conv, dtype, n_slots=4)
    held = bench.cache.alloc_slots(4)
    slots = held[1:][::-1]
    outs = [[] for _ in xs]
    at = [0, 0, 0]
    plan = [[2, 1, max(K - 1, 1)], [K, 1, 1], [9, 2, K + 1], [1, 1, 1], [1, 1, 1]]
    while any(a < x.shape[0] for a, x in zip(at, xs)):
        sizes = plan.pop(0) if plan else [1, 1, 1]
        live = [b for b in range(3) if at[b] < xs[b].shape[0]]
        take = [min(sizes[b], xs[b].shape[0] - at[b]) for b in live]
        ctx = bench.step([slots[b] for b in live], take)
        x = torch.cat([xs[b][at[b]:at[b] + n] for b, n in zip(live, take)]).cuda()
        out = torch.empty_like(x)
        conv.forward(ctx, bench.call, x, out, False)
        bench.done([slots[b] for b in live], take)
        o = 0
        for b, n in zip(live, take):
            outs[b].append(out[o:o + n].cpu())
            o += n
            at[b] += n
    assert inner.seen_dtype == dtype
    for b, x in enumerate(xs):
        close(torch.cat(outs[b]), P.input_conv(x.numpy().astype(np.float64), taps.numpy().astype(np.float64)), dtype, f"sequence {b}")
    # a slot that is handed out again starts from zeros
    bench.cache.free_slots(held)
    again = bench.cache.alloc_slots(4)
    ctx = bench.step([again[2]], [3])
    out = torch.empty((3, D), device="cuda")
    conv.forward(ctx, bench.call, xs[0][:3].cuda(), out, False)
    close(out, P.input_conv(xs[0][:3].numpy().astype(np.float64), taps.numpy().astype(np.float64)), dtype, "slot used again")


# ------------------------------------------------------------------------------- attention

def attention_tensors(D, H, G, d, vd, dtype, seed, split=False):
    """split: q and k read the first half of the input only and v the second half only, so that a test can
    give two tokens the same key and different values."""
    t = {"q": rnd((H * d, D), seed, dtype, D ** -0.5), "k": rnd((G * d, D), seed + 1, dtype, D ** -0.5),
         "v": rnd((G * vd, D), seed + 2, dtype, D ** -0.5), "o": rnd((D, H * vd), seed + 3, dtype, (H * vd) ** -0.5),
         "qn": 1.0 + rnd((H * d,), seed + 4, dtype, 0.2), "kn": 1.0 + rnd((G * d,), seed + 5, dtype, 0.2),
         "r1": rnd((H,), seed + 6, dtype, 0.5).abs() + 0.2, "r2": rnd((H,), seed + 7, dtype, 0.7).abs() + 0.05}
    if split:
        t["q"][:, D // 2:] = 0
        t["k"][:, D // 2:] = 0
        t["v"][:, :D // 2] = 0
    return t


def make_attention(D, H, G, d, vd, scale, window, t, dtype, own_kv=True):
    from zinfer_b200.parts import GqaAttention
    return load(GqaAttention(D, H, G, d, "q", "k", "v", "o", "qn", "kn", 2e-6, None, window, scale, value_dim=vd,
                             qk_norm_span="all", distance_bias=("r1", "r2"), own_kv=own_kv), t, dtype)


def plain_mixer(x, t, H, G, d, vd, scale, window, kv=None):
    f = lambda n: t[n].numpy().astype(np.float64)
    return P.log_distance_attention(np.asarray(x, dtype=np.float64), f("q"), f("k"), f("v"), f("o"), f("qn"), f("kn"), H, G, d, vd,
                                    scale, f("r1"), f("r2"), window, 2e-6, kv=kv)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D,H,G,d,vd,scale,window,page", [
    (40, 3, 1, 16, 24, 0.3, 11, 16),        # three heads on one key/value head, values wider than keys
    (64, 4, 4, 8, 8, 0.5, 0, 16),           # one head per key/value head, no window
    (96, 4, 2, 32, 16, 0.2, 33, 32),        # values narrower than keys, a window longer than a page
    (128, 8, 2, 64, 64, 0.11, 16, 16),     # the widths the tensor-core kernels take; a window of one page
    (72, 6, 2, 24, 40, 0.15, 1, 16),        # a window of ONE token: every query sees itself only
    (128, 8, 2, 64, 64, 0.11, 40, 64),     # pages of 64: in bfloat16 the tensor-core kernels run
    (96, 2, 1, 128, 128, 0.1, 70, 64),      # heads of 128, a window over a page border
    (64, 16, 1, 64, 64, 0.2, 0, 64),        # sixteen heads on one key/value head, no window
])
def test_log_distance_attention_part(k, dtype, D, H, G, d, vd, scale, window, page):
    t = attention_tensors(D, H, G, d, vd, dtype, 40)
    mixer = make_attention(D, H, G, d, vd, scale, window, t, dtype)
    req = mixer.kv_request()
    assert (req.n_kv_heads, req.head_dim, req.v_dim, req.window) == (G, d, vd, window)
    xs = [rnd((n, D), 50 + n, dtype) for n in (70, 37, 45)]
    outs = run_mixer(k, mixer, dtype, xs, [70 - 5, 37 - 20, 1], page=page)
    for b, x in enumerate(xs):
        close(outs[b], plain_mixer(x.numpy(), t, H, G, d, vd, scale, window)[0], dtype, f"sequence {b}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d", [16, 64])      # heads of 64 with pages of 64: the tensor-core kernels in bfloat16
@pytest.mark.parametrize("window,page,prompt", [(0, 16, 150), (0, 64, 40), (48, 16, 120), (64, 64, 70), (37, 32, 3),
                                                (65, 64, 130), (128, 64, 2)])
def test_one_key_decides(k, dtype, window, page, prompt, d):
    """Rows are made so that a few MARKED tokens carry the key direction of the queries that follow, each
    with a value of its own; everything else scores ten lower.  Marked: the first token, the tokens on both
    sides of every page border, and for each probing query the tokens just inside (distance window - 1) and
    just outside (distance window) its window.  A kernel that misses a marked key, sees one it must not, or
    reads another page or row gives another value: an error of order one."""
    D, H, G, vd, scale, T = 64, 2, 1, d, 32.0 / d, 200
    t = attention_tensors(D, H, G, d, vd, dtype, 60, split=True)
    for h in range(H):                  # every head's query projection is the key projection, norm weights are 1:
        t["q"][h * d:(h + 1) * d] = t["k"]      # a query that follows key_dir scores scale * d = 32 on a marked key
    t["qn"][:] = 1.0
    t["kn"][:] = 1.0
    t["r1"][:] = 0.25
    rng = np.random.default_rng(window + page)
    x = rng.normal(0, 1.0, (T, D)).astype(np.float32)
    key_dir = rng.normal(0, 1.0, D // 2).astype(np.float32)
    probes = [T - 1, T - 2, prompt - 1, prompt, prompt + 1, 130, 77] if prompt > 3 else [T - 1, 100, 63, 64, 2, 3]
    marked = {0, 1}
    for b in range(page, T, page):
        marked |= {b - 1, b}
    for i in probes:
        x[i, :D // 2] = key_dir                     # a probing query: its q and k follow key_dir
        if window:
            marked |= {j for j in (i - window + 1, i - window) if j >= 0}
    for j in marked:
        x[j, :D // 2] = key_dir
    x = torch.from_numpy(x).to(dtype).float()
    mixer = make_attention(D, H, G, d, vd, scale, window, t, dtype)
    ref = plain_mixer(x.numpy(), t, H, G, d, vd, scale, window)[0]
    # the construction works: a marked key dominates its query's softmax
    out = run_mixer(k, mixer, dtype, [x], [prompt], page=page)[0]
    close(out, ref, dtype, f"window {window} page {page}")
    if window:       # and the oracle itself tells inside from outside: one token more in the window changes the probes
        other = plain_mixer(x.numpy(), t, H, G, d, vd, scale, window + 1)[0]
        assert max(np.abs(other[i] - ref[i]).max() for i in probes if i >= window) > 0.03 * np.abs(ref).max()


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_reader_of_another_calls_cache_with_a_window_of_its_own(k, dtype):
    """Two schedule entries: the second has no key/value weights, reads the first one's cache and looks
    further back than its owner does; pages stay while the wider window needs them."""
    from zinfer_b200.cache import CacheManager, CallCacheSpec
    from zinfer_b200.engine.context import CallContext
    D, H, G, d, vd, scale, page = 48, 4, 2, 8, 12, 0.4, 16
    ta, tb = attention_tensors(D, H, G, d, vd, dtype, 70), attention_tensors(D, H, G, d, vd, dtype, 80)
    for n in ("k", "v", "kn"):
        del tb[n]
    owner = make_attention(D, H, G, d, vd, scale, 9, ta, dtype)
    reader = make_attention(D, H, G, d, vd, scale, 40, tb, dtype, own_kv=False)
    assert {s.name for s in reader.weight_specs()} == {"q", "o", "qn", "r1", "r2"}
    cache = CacheManager([CallCacheSpec(kv=owner.kv_request()), CallCacheSpec(kv=reader.kv_request(), kv_owner=0)], 2, 96, 128,
                         page, dtype, "cuda")
    calls = [CallContext(c, c, cache.kv_view(c), cache.writes_kv(c), None) for c in range(2)]
    assert calls[0].kv.window == 9 and calls[1].kv.window == 40 and not calls[1].writes_kv
    xa, xb = rnd((90, D), 90, dtype), rnd((90, D), 91, dtype)
    slot = cache.alloc_slots(2)[1]
    got_a, got_b, at = [], [], 0
    for n in [30, 2, 17] + [1] * 41:
        ctx = context(k, dtype, cache, [slot], [[0] * n])
        oa, ob = torch.empty((n, D), device="cuda"), torch.empty((n, D), device="cuda")
        owner.forward(ctx, calls[0], xa[at:at + n].to(dtype).cuda(), oa, False)
        reader.forward(ctx, calls[1], xb[at:at + n].to(dtype).cuda(), ob, False)
        cache.advance([slot], [n])
        got_a.append(oa.cpu())
        got_b.append(ob.cpu())
        at += n
    assert int(k.status_word("cuda").item()) == 0
    ref_a, kv = plain_mixer(xa.numpy(), ta, H, G, d, vd, scale, 9)
    tb_full = dict(tb, k=ta["k"], v=ta["v"], kn=ta["kn"])
    ref_b = plain_mixer(xb.numpy(), tb_full, H, G, d, vd, scale, 40, kv=kv)[0]
    close(torch.cat(got_a), ref_a, dtype, "owner")
    close(torch.cat(got_b), ref_b, dtype, "reader")
    assert len(cache.groups[0].pages_held(slot)) == 3        # the next query (position 90) sees keys 51..90: pages 3, 4, 5


# ------------------------------------------------------------------------------- experts

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D,F,E,top,shared,rows", [(40, 24, 5, 3, 40, 7), (64, 16, 3, 1, 0, 1), (128, 64, 8, 2, 64, 40),
                                                  (72, 20, 4, 4, 12, 3), (256, 96, 6, 2, 32, 200),
                                                  (256, 128, 5, 2, 0, 200)])     # widths of whole 256-wide tiles: the persistent grouped form
def test_table_routed_experts(k, dtype, D, F, E, top, shared, rows):
    from zinfer_b200.cache import CacheManager, CallCacheSpec
    from zinfer_b200.parts import SwiGLU, TableMoE
    vocab = 53
    rng = np.random.default_rng(D + top)
    t = {"table": torch.from_numpy(np.stack([rng.permutation(E)[:top] for _ in range(vocab)]).astype(np.int32))}
    for e in range(E):
        t[f"e{e}.g"], t[f"e{e}.u"], t[f"e{e}.d"] = (rnd((F, D), 100 + 3 * e, dtype, D ** -0.5), rnd((F, D), 101 + 3 * e, dtype, D ** -0.5),
                                                    rnd((D, F), 102 + 3 * e, dtype, F ** -0.5))
    sh = None
    if shared:
        t.update({"s.g": rnd((shared, D), 200, dtype, D ** -0.5), "s.u": rnd((shared, D), 201, dtype, D ** -0.5),
                  "s.d": rnd((D, shared), 202, dtype, shared ** -0.5), "s.sg": rnd((1, D), 203, dtype, 0.3)})
        sh = SwiGLU(D, shared, "s.g", "s.u", "s.d")
    moe = TableMoE(D, F, E, top, vocab, "table", lambda e: (f"e{e}.g", f"e{e}.u", f"e{e}.d"), shared=sh,
                   shared_gate_name="s.sg" if shared else None)
    given = {}
    for part in [moe] + moe.parts():
        for spec in part.weight_specs():
            v = t[spec.name]
            given[spec.name] = v.cuda() if spec.role == "table" else v.to(dtype if spec.role == "matrix" else torch.float32).cuda().contiguous()
    for part in [moe] + moe.parts():
        part.load(given, dtype, torch.device("cuda"))
    toks = rng.integers(0, vocab, size=rows).tolist()
    cache = CacheManager([CallCacheSpec()], 1, 256, 256, 16, dtype, "cuda")
    ctx = context(k, dtype, cache, cache.alloc_slots(1), [toks])
    x = rnd((rows, D), 300, dtype)
    out = torch.full((rows, D), 9.0, device="cuda")
    moe.forward(ctx, x.cuda(), out, False)
    from zinfer_b200.parts.moe import GROUPED_MIN_TOKENS
    assert (rows >= GROUPED_MIN_TOKENS) == (rows == 200), "the test means to run both ways"
    f = lambda n: t[n].numpy().astype(np.float64)
    ref = P.table_experts(x.numpy().astype(np.float64), toks, t["table"].numpy(), [(f(f"e{e}.g"), f(f"e{e}.u"), f(f"e{e}.d")) for e in range(E)],
                          (f("s.g"), f("s.u"), f("s.d")) if shared else None, f("s.sg").reshape(-1) if shared else None)
    close(out, ref, dtype, "experts")
    assert int(ctx.status.item()) == 0
    if rows >= GROUPED_MIN_TOKENS:       # the same step without the ids on the host: the streaming kernels, added into `out`
        cache2 = CacheManager([CallCacheSpec()], 1, 256, 256, 16, dtype, "cuda")
        ctx2 = context(k, dtype, cache2, cache2.alloc_slots(1), [toks], host=False)
        base = torch.full((rows, D), 0.25, device="cuda")
        both = base.clone()
        moe.forward(ctx2, x.cuda(), both, True)
        close(both - base, ref, dtype, "experts, streamed")
    # a row's result does not depend on the rows beside it
    one = torch.empty((1, D), device="cuda")
    cache1 = CacheManager([CallCacheSpec()], 1, 256, 256, 16, dtype, "cuda")
    ctx1 = context(k, dtype, cache1, cache1.alloc_slots(1), [toks[-1:]])
    moe.forward(ctx1, x[-1:].cuda(), one, False)
    if dtype == torch.float32 and rows < GROUPED_MIN_TOKENS:       # the same kernels ran: the same bits
        assert torch.equal(one[0], out[-1])
    else:
        close(one, ref[-1:], dtype, "alone")


# ------------------------------------------------------------------------------- block

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("with_ffn", [True, False])
def test_block_that_normalises_what_its_sublayers_return(k, dtype, with_ffn):
    from zinfer_b200.parts import ActMlp, InputConv, RMSNorm, SublayerNormBlock
    D, H, G, d, vd, scale, window, K, F, eps = 48, 3, 3, 8, 8, 0.35, 13, 3, 80, 2e-6
    t = attention_tensors(D, H, G, d, vd, dtype, 400)
    t.update({"c": rnd((D, K), 410, dtype, 0.4), "n1": 1.0 + rnd((D,), 411, dtype, 0.2), "n2": 1.0 + rnd((D,), 412, dtype, 0.2),
              "up": rnd((F, D), 413, dtype, D ** -0.5), "down": rnd((D, F), 414, dtype, F ** -0.5)})
    mixer = InputConv(make_attention(D, H, G, d, vd, scale, window, t, dtype), D, K, "c")
    block = SublayerNormBlock(mixer, RMSNorm(D, eps, "n1"), ActMlp(D, F, "up", "down") if with_ffn else None,
                              RMSNorm(D, eps, "n2") if with_ffn else None)
    load(block, t, dtype)
    x0 = rnd((50, D), 420, torch.float32)
    bench = Bench(k, mixer, dtype, n_slots=2)
    slot = bench.cache.alloc_slots(2)[1:]
    got, at = [], 0
    for n in [20, 2] + [1] * 28:
        ctx = bench.step(slot, [n])
        x = x0[at:at + n].clone().cuda()
        block.forward(ctx, bench.call, x)
        bench.done(slot, [n])
        got.append(x.cpu())
        at += n
    f = lambda n: t[n].numpy().astype(np.float64)
    x = x0.numpy().astype(np.float64)
    y = plain_mixer(P.input_conv(x, f("c")), t, H, G, d, vd, scale, window)[0]
    x = x + P.rms_unit(y, eps) * f("n1")
    if with_ffn:
        x = x + P.rms_unit(P.dense_ff(x, f("up"), f("down")), eps) * f("n2")
    close(torch.cat(got), x, dtype, "block")
